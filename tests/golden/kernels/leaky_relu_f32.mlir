// y = select(x > 0, x, 0.1 * x) over a [1, n] f32 tensor (arith.cmpf feeding
// arith.select); one program covers 512 elements, each of its 2 warps a
// [1, 256] tile.
#global = #kapy.encoding<global_memory>
#values = #kapy.encoding<register_file>
module attributes {kapy.num_warps = 2 : i64, kapy.nvidia_cc = 100 : i64} {
  kapy.func public @leaky_relu(%x: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %y: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %n: i32 {kapy.alignment = 512 : i64}) {
    %c0 = arith.constant 0 : i32
    %c1 = arith.constant 1 : i32
    %c256 = arith.constant 256 : i32
    %c512 = arith.constant 512 : i32
    %zero = arith.constant dense<0.000000e+00> : tensor<1x256xf32, #values>
    %slope = arith.constant dense<1.000000e-01> : tensor<1x256xf32, #values>
    %gx = kapy.mk_global %x[%c0] [%c1, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xf32, #global>
    %gy = kapy.mk_global %y[%c0] [%c1, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xf32, #global>
    %pid = kapy.program_id {axis = 0 : i32} : i32
    %wid = kapy.warp_id : i32
    %p0 = arith.muli %pid, %c512 : i32
    %w0 = arith.muli %wid, %c256 : i32
    %lo = arith.addi %p0, %w0 : i32
    %hi = arith.addi %lo, %c256 : i32
    %vx = kapy.sv_global %gx[%c0 : %c1, %lo : %hi] : tensor<?x?xf32, #global> -> tensor<1x256xf32, #global>
    %vy = kapy.sv_global %gy[%c0 : %c1, %lo : %hi] : tensor<?x?xf32, #global> -> tensor<1x256xf32, #global>
    %t = kapy.ld_global %vx : tensor<1x256xf32, #global> -> tensor<1x256xf32, #values>
    %pos = arith.cmpf ogt, %t, %zero : tensor<1x256xf32, #values>
    %neg = arith.mulf %t, %slope : tensor<1x256xf32, #values>
    %o = arith.select %pos, %t, %neg : tensor<1x256xi1, #values>, tensor<1x256xf32, #values>
    kapy.st_global %o, %vy : tensor<1x256xf32, #values>, tensor<1x256xf32, #global>
    kapy.return
  }
}
