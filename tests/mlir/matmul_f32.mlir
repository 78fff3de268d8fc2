// linalg.matmul (named op) and the matmul-shaped generic with an initial C,
// f32: the bit-exact SIMT GEMM.  Expected values from the CPU oracle.
// RUN: imex_runner.py -i %s -f linalg-to-gpu.pp -e main --entry-point-result=void --filecheck
#map0 = affine_map<(d0, d1, d2) -> (d0, d2)>
#map1 = affine_map<(d0, d1, d2) -> (d2, d1)>
#map2 = affine_map<(d0, d1, d2) -> (d0, d1)>
module @matmul_f32 {
  func.func @named(%a: tensor<4x3xf32>, %b: tensor<3x2xf32>) -> tensor<4x2xf32> {
    %zero = arith.constant 0.0 : f32
    %e = tensor.empty() : tensor<4x2xf32>
    %c0 = linalg.fill ins(%zero : f32) outs(%e : tensor<4x2xf32>) -> tensor<4x2xf32>
    %c = linalg.matmul ins(%a, %b : tensor<4x3xf32>, tensor<3x2xf32>) outs(%c0 : tensor<4x2xf32>) -> tensor<4x2xf32>
    return %c : tensor<4x2xf32>
  }
  func.func @with_init(%a: tensor<4x3xf32>, %b: tensor<3x2xf32>, %c0: tensor<4x2xf32>) -> tensor<4x2xf32> {
    %c = linalg.generic {indexing_maps = [#map0, #map1, #map2], iterator_types = ["parallel", "parallel", "reduction"]}
         ins(%a, %b : tensor<4x3xf32>, tensor<3x2xf32>) outs(%c0 : tensor<4x2xf32>) {
    ^bb0(%x: f32, %y: f32, %acc: f32):
      %p = arith.mulf %x, %y : f32
      %s = arith.addf %acc, %p : f32
      linalg.yield %s : f32
    } -> tensor<4x2xf32>
    return %c : tensor<4x2xf32>
  }
  func.func private @printMemrefF32(tensor<*xf32>)
  func.func @main() {
    %a = arith.constant dense<[[-2.0, -1.5, -1.0], [-0.5, 0.0, 0.5], [1.0, 1.5, 2.0], [2.5, 3.0, 3.5]]> : tensor<4x3xf32>
    %b = arith.constant dense<[[1.0, -1.0], [2.0, 0.5], [-3.0, 4.0]]> : tensor<3x2xf32>
    %ten = arith.constant dense<10.0> : tensor<4x2xf32>
    %r0 = call @named(%a, %b) : (tensor<4x3xf32>, tensor<3x2xf32>) -> tensor<4x2xf32>
    %u0 = tensor.cast %r0 : tensor<4x2xf32> to tensor<*xf32>
    call @printMemrefF32(%u0) : (tensor<*xf32>) -> ()
    // CHECK: Unranked Memref base@ = {{(0x)?[-9a-f]*}}
    // CHECK-SAME: rank = 2 offset = 0 sizes = [4, 2] strides = [2, 1] data =
    // CHECK-NEXT: [-2, -2.75],
    // CHECK-NEXT: [-2, 2.5],
    // CHECK-NEXT: [-2, 7.75],
    // CHECK-NEXT: [-2, 13]
    %r1 = call @with_init(%a, %b, %ten) : (tensor<4x3xf32>, tensor<3x2xf32>, tensor<4x2xf32>) -> tensor<4x2xf32>
    %u1 = tensor.cast %r1 : tensor<4x2xf32> to tensor<*xf32>
    call @printMemrefF32(%u1) : (tensor<*xf32>) -> ()
    // CHECK: [8, 7.25],
    // CHECK-NEXT: [8, 12.5],
    // CHECK-NEXT: [8, 17.75],
    // CHECK-NEXT: [8, 23]
    return
  }
}
