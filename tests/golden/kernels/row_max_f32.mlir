// Row maxima of an [m, 128] f32 tensor: each warp takes 4 rows.
#global = #kapy.encoding<global_memory>
#values = #kapy.encoding<register_file>
module attributes {kapy.num_warps = 2 : i64, kapy.nvidia_cc = 100 : i64} {
  kapy.func public @row_max(%src: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %dst: !kapy.ptr<1> {kapy.alignment = 16 : i64}, %m: i32 {kapy.alignment = 8 : i64}) {
    %c0 = arith.constant 0 : i32
    %c1 = arith.constant 1 : i32
    %c4 = arith.constant 4 : i32
    %c8 = arith.constant 8 : i32
    %c128 = arith.constant 128 : i32
    %g = kapy.mk_global %src[%c0] [%m, %c128] [%c128, %c1] : !kapy.ptr<1> -> tensor<?x?xf32, #global>
    %pid = kapy.program_id {axis = 0 : i32} : i32
    %wid = kapy.warp_id : i32
    %a = arith.muli %pid, %c8 : i32
    %b = arith.muli %wid, %c4 : i32
    %r0 = arith.addi %a, %b : i32
    %r1 = arith.addi %r0, %c4 : i32
    %v = kapy.sv_global %g[%r0 : %r1, %c0 : %c128] : tensor<?x?xf32, #global> -> tensor<4x128xf32, #global>
    %t = kapy.ld_global %v : tensor<4x128xf32, #global> -> tensor<4x128xf32, #values>
    %r = kapy.reduce %t {axis = 1 : i32} lambda(%p: f32, %q: f32) {
      %mx = arith.maximumf %p, %q : f32
      kapy.return %mx : f32
    } : tensor<4x128xf32, #values> -> tensor<4x1xf32, #values>
    %go = kapy.mk_global %dst[%c0] [%m, %c1] [%c1, %m] : !kapy.ptr<1> -> tensor<?x?xf32, #global>
    %vo = kapy.sv_global %go[%r0 : %r1, %c0 : %c1] : tensor<?x?xf32, #global> -> tensor<4x1xf32, #global>
    kapy.st_global %r, %vo : tensor<4x1xf32, #values>, tensor<4x1xf32, #global>
    kapy.return
  }
}
