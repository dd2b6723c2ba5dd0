// y = truncf(fma(extf(x), s, b)) over a [1, n] bf16 tensor; one program covers
// 1024 elements, each of its 4 warps a [1, 256] tile.
#global = #kapy.encoding<global_memory>
#values = #kapy.encoding<register_file>
module attributes {kapy.num_warps = 4 : i64, kapy.nvidia_cc = 100 : i64} {
  kapy.func public @scale_shift(%x: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %y: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %n: i32 {kapy.alignment = 1024 : i64}) {
    %c0 = arith.constant 0 : i32
    %c1 = arith.constant 1 : i32
    %c256 = arith.constant 256 : i32
    %c1024 = arith.constant 1024 : i32
    %s = arith.constant dense<5.000000e-01> : tensor<1x256xf32, #values>
    %b = arith.constant dense<1.000000e-01> : tensor<1x256xf32, #values>
    %gx = kapy.mk_global %x[%c0] [%c1, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16, #global>
    %gy = kapy.mk_global %y[%c0] [%c1, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16, #global>
    %pid = kapy.program_id {axis = 0 : i32} : i32
    %wid = kapy.warp_id : i32
    %p0 = arith.muli %pid, %c1024 : i32
    %w0 = arith.muli %wid, %c256 : i32
    %lo = arith.addi %p0, %w0 : i32
    %hi = arith.addi %lo, %c256 : i32
    %vx = kapy.sv_global %gx[%c0 : %c1, %lo : %hi] : tensor<?x?xbf16, #global> -> tensor<1x256xbf16, #global>
    %vy = kapy.sv_global %gy[%c0 : %c1, %lo : %hi] : tensor<?x?xbf16, #global> -> tensor<1x256xbf16, #global>
    %t = kapy.ld_global %vx : tensor<1x256xbf16, #global> -> tensor<1x256xbf16, #values>
    %tf = arith.extf %t : tensor<1x256xbf16, #values> to tensor<1x256xf32, #values>
    %u = math.fma %tf, %s, %b : tensor<1x256xf32, #values>
    %o = arith.truncf %u : tensor<1x256xf32, #values> to tensor<1x256xbf16, #values>
    kapy.st_global %o, %vy : tensor<1x256xbf16, #values>, tensor<1x256xbf16, #global>
    kapy.return
  }
}
