// C[M,N] = A[M,K] . B[K,N], bf16 operands, f32 accumulator, bf16 result.
// One warp per program owns a 32x32 output tile and walks K in steps of 16
// through a single shared-memory buffer pair (copy, wait, ld_matrix, matmul).
#global = #kapy.encoding<global_memory>
#shared = #kapy.encoding<shared_memory>
#values = #kapy.encoding<register_file>
module attributes {kapy.num_warps = 1 : i64, kapy.nvidia_cc = 100 : i64} {
  kapy.func public @gemm_ring(%pa: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %pb: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %pc: !kapy.ptr<1> {kapy.alignment = 128 : i64}, %m: i32, %k: i32, %n: i32) {
    %zero = arith.constant dense<0.000000e+00> : tensor<32x32xf32, #values>
    %za = arith.constant dense<0.000000e+00> : tensor<32x16xbf16, #values>
    %zb = arith.constant dense<0.000000e+00> : tensor<16x32xbf16, #values>
    %c0 = arith.constant 0 : i32
    %c1 = arith.constant 1 : i32
    %c16 = arith.constant 16 : i32
    %c32 = arith.constant 32 : i32
    %ga = kapy.mk_global %pa[%c0] [%m, %k] [%k, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16, #global>
    %gb = kapy.mk_global %pb[%c0] [%k, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16, #global>
    %gc = kapy.mk_global %pc[%c0] [%m, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16, #global>
    %sa = kapy.mk_shared {kapy.row_major = true} : tensor<32x16xbf16, #shared>
    %sb = kapy.mk_shared {kapy.row_major = true} : tensor<16x32xbf16, #shared>
    %px = kapy.program_id {axis = 0 : i32} : i32
    %py = kapy.program_id {axis = 1 : i32} : i32
    %r0 = arith.muli %px, %c32 : i32
    %r1 = arith.addi %r0, %c32 : i32
    %q0 = arith.muli %py, %c32 : i32
    %q1 = arith.addi %q0, %c32 : i32
    %steps = arith.divui %k, %c16 : i32
    %acc = scf.for %i = %c0 to %steps step %c1 iter_args(%cur = %zero) -> (tensor<32x32xf32, #values>)  : i32 {
      %k0 = arith.muli %i, %c16 : i32
      %k1 = arith.addi %k0, %c16 : i32
      %va = kapy.sv_global %ga[%r0 : %r1, %k0 : %k1] : tensor<?x?xbf16, #global> -> tensor<32x16xbf16, #global>
      %vb = kapy.sv_global %gb[%k0 : %k1, %q0 : %q1] : tensor<?x?xbf16, #global> -> tensor<16x32xbf16, #global>
      kapy.cp_async_global_to_shared %va, %sa, %za : tensor<32x16xbf16, #global>, tensor<32x16xbf16, #shared>, tensor<32x16xbf16, #values>
      kapy.cp_async_global_to_shared %vb, %sb, %zb : tensor<16x32xbf16, #global>, tensor<16x32xbf16, #shared>, tensor<16x32xbf16, #values>
      kapy.cp_async_wait_group {num_pending = 0 : i32}
      %fa = kapy.ld_matrix %sa, %za : tensor<32x16xbf16, #shared>, tensor<32x16xbf16, #values> -> tensor<32x16xbf16, #values>
      %fb = kapy.ld_matrix %sb, %zb : tensor<16x32xbf16, #shared>, tensor<16x32xbf16, #values> -> tensor<16x32xbf16, #values>
      %nxt = kapy.matmul mma_m16n8k16_f16 %fa, %fb, %cur : tensor<32x16xbf16, #values>, tensor<16x32xbf16, #values> -> tensor<32x32xf32, #values>
      scf.yield %nxt : tensor<32x32xf32, #values>
    }
    %out = arith.truncf %acc : tensor<32x32xf32, #values> to tensor<32x32xbf16, #values>
    %vc = kapy.sv_global %gc[%r0 : %r1, %q0 : %q1] : tensor<?x?xbf16, #global> -> tensor<32x32xbf16, #global>
    kapy.st_global %out, %vc : tensor<32x32xbf16, #values>, tensor<32x32xbf16, #global>
    kapy.return
  }
}
