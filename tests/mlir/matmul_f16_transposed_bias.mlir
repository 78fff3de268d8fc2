// f16 GEMMs with the operand layouts and result types of the reference's
// larger GEMM tests (test/Integration/Dialect/XeGPU/WG/gemm_4kx4kx4k_transpose_b.mlir:
// B stored [N,K]; gemm_4kx4kx4k_transpose_a.mlir: A stored [K,M];
// gemm_4kx4kx4k_f16_f16_f32_bias.mlir: + bias; gemm_4kx4kx4k_f16_f16_f16.mlir: f16
// result), written at the linalg level: each function becomes ONE fused launch.
// RUN: imex_runner.py -i %s -f linalg-to-gpu.pp -e main --entry-point-result=void --filecheck
#id = affine_map<(d0, d1) -> (d0, d1)>
#row = affine_map<(d0, d1) -> (d1)>
#a_nt = affine_map<(d0, d1, d2) -> (d0, d2)>
#a_t = affine_map<(d0, d1, d2) -> (d2, d0)>
#b_nt = affine_map<(d0, d1, d2) -> (d2, d1)>
#b_t = affine_map<(d0, d1, d2) -> (d1, d2)>
#c = affine_map<(d0, d1, d2) -> (d0, d1)>
module @matmul_f16_layouts {
  // C[8,16] f16 = relu(A[8,64] . B^T + bias), B stored [16,64]
  func.func @gemm_bt_bias_relu_f16(%a: tensor<8x64xf16>, %b: tensor<16x64xf16>, %bias: tensor<16xf32>) -> tensor<8x16xf16> {
    %zero = arith.constant 0.0 : f32
    %ec = tensor.empty() : tensor<8x16xf32>
    %c0 = linalg.fill ins(%zero : f32) outs(%ec : tensor<8x16xf32>) -> tensor<8x16xf32>
    %c = linalg.generic {indexing_maps = [#a_nt, #b_t, #c], iterator_types = ["parallel", "parallel", "reduction"]}
         ins(%a, %b : tensor<8x64xf16>, tensor<16x64xf16>) outs(%c0 : tensor<8x16xf32>) {
    ^bb0(%x: f16, %y: f16, %acc: f32):
      %xf = arith.extf %x : f16 to f32
      %yf = arith.extf %y : f16 to f32
      %p = arith.mulf %xf, %yf : f32
      %s = arith.addf %acc, %p : f32
      linalg.yield %s : f32
    } -> tensor<8x16xf32>
    %eb = tensor.empty() : tensor<8x16xf32>
    %bb = linalg.generic {indexing_maps = [#row, #id], iterator_types = ["parallel", "parallel"]} ins(%bias : tensor<16xf32>) outs(%eb : tensor<8x16xf32>) {
    ^bb0(%in: f32, %out: f32):
      linalg.yield %in : f32
    } -> tensor<8x16xf32>
    %es = tensor.empty() : tensor<8x16xf32>
    %sum = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]} ins(%c, %bb : tensor<8x16xf32>, tensor<8x16xf32>) outs(%es : tensor<8x16xf32>) {
    ^bb0(%in: f32, %in_0: f32, %out: f32):
      %s = arith.addf %in, %in_0 : f32
      linalg.yield %s : f32
    } -> tensor<8x16xf32>
    %er = tensor.empty() : tensor<8x16xf32>
    %r = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%sum : tensor<8x16xf32>) outs(%er : tensor<8x16xf32>) {
    ^bb0(%in: f32, %out: f32):
      %g = arith.cmpf ugt, %in, %zero : f32
      %s = arith.select %g, %in, %zero : f32
      linalg.yield %s : f32
    } -> tensor<8x16xf32>
    %et = tensor.empty() : tensor<8x16xf16>
    %t = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%r : tensor<8x16xf32>) outs(%et : tensor<8x16xf16>) {
    ^bb0(%in: f32, %out: f16):
      %h = arith.truncf %in : f32 to f16
      linalg.yield %h : f16
    } -> tensor<8x16xf16>
    return %t : tensor<8x16xf16>
  }
  // C[8,16] f32 = A^T . B, A stored [64,8]
  func.func @gemm_at(%a: tensor<64x8xf16>, %b: tensor<64x16xf16>) -> tensor<8x16xf32> {
    %zero = arith.constant 0.0 : f32
    %ec = tensor.empty() : tensor<8x16xf32>
    %c0 = linalg.fill ins(%zero : f32) outs(%ec : tensor<8x16xf32>) -> tensor<8x16xf32>
    %c = linalg.generic {indexing_maps = [#a_t, #b_nt, #c], iterator_types = ["parallel", "parallel", "reduction"]}
         ins(%a, %b : tensor<64x8xf16>, tensor<64x16xf16>) outs(%c0 : tensor<8x16xf32>) {
    ^bb0(%x: f16, %y: f16, %acc: f32):
      %xf = arith.extf %x : f16 to f32
      %yf = arith.extf %y : f16 to f32
      %p = arith.mulf %xf, %yf : f32
      %s = arith.addf %acc, %p : f32
      linalg.yield %s : f32
    } -> tensor<8x16xf32>
    return %c : tensor<8x16xf32>
  }
  func.func private @printMemrefF16(tensor<*xf16>)
  func.func private @printMemrefF32(tensor<*xf32>)
  func.func @main() {
    %a = arith.constant dense<0.5> : tensor<8x64xf16>
    %at = arith.constant dense<0.5> : tensor<64x8xf16>
    %bt = arith.constant dense<0.25> : tensor<16x64xf16>
    %bm = arith.constant dense<-0.25> : tensor<16x64xf16>
    %b = arith.constant dense<0.25> : tensor<64x16xf16>
    %bias = arith.constant dense<[0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, -1.0, -2.0, -3.0, -4.0, -5.0, -6.0, -7.0, -9.0]> : tensor<16xf32>
    // every element of A.B^T is 64 * 0.125 = 8; + bias[j]; relu; f16
    %r0 = call @gemm_bt_bias_relu_f16(%a, %bt, %bias) : (tensor<8x64xf16>, tensor<16x64xf16>, tensor<16xf32>) -> tensor<8x16xf16>
    %u0 = tensor.cast %r0 : tensor<8x16xf16> to tensor<*xf16>
    call @printMemrefF16(%u0) : (tensor<*xf16>) -> ()
    // CHECK: sizes = [8, 16] strides = [16, 1] data =
    // CHECK-NEXT: {{\[}}[8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0],
    // CHECK-NEXT: [8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0],
    // CHECK-NEXT: [8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0],
    // CHECK-NEXT: [8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0],
    // CHECK-NEXT: [8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0],
    // CHECK-NEXT: [8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0],
    // CHECK-NEXT: [8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0],
    // CHECK-NEXT: [8, 9, 10, 11, 12, 13, 14, 15, 7, 6, 5, 4, 3, 2, 1, 0]]
    // -8 + bias[j] <= 0 everywhere: relu leaves zeros
    %r1 = call @gemm_bt_bias_relu_f16(%a, %bm, %bias) : (tensor<8x64xf16>, tensor<16x64xf16>, tensor<16xf32>) -> tensor<8x16xf16>
    %u1 = tensor.cast %r1 : tensor<8x16xf16> to tensor<*xf16>
    call @printMemrefF16(%u1) : (tensor<*xf16>) -> ()
    // CHECK: [0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0]
    %r2 = call @gemm_at(%at, %b) : (tensor<64x8xf16>, tensor<64x16xf16>) -> tensor<8x16xf32>
    %u2 = tensor.cast %r2 : tensor<8x16xf32> to tensor<*xf32>
    call @printMemrefF32(%u2) : (tensor<*xf32>) -> ()
    // CHECK: {{\[}}[8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8, 8],
    return
  }
}
