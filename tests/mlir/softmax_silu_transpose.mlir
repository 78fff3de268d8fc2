// The benchmark forms of softmax (with its dead arg-max output), silu and the
// 2-D transpose, plus the leading-dim reduction.  Expected values from the
// CPU oracle, printed with six significant digits.
// RUN: imex_runner.py -i %s -f linalg-to-gpu.pp -e main --entry-point-result=void --filecheck
#map = affine_map<(d0, d1) -> (d0, d1)>
#map1 = affine_map<(d0, d1) -> (d0, 0)>
#mapt = affine_map<(d0, d1) -> (d1, d0)>
module attributes {torch.debug_module_name = "Softmax"} {
  func.func @softmax(%arg0: tensor<3x4xf32>) -> tensor<3x4xf32> {
    %c0_i64 = arith.constant 0 : i64
    %cst = arith.constant -3.40282347E+38 : f32
    %cst_0 = arith.constant 0.000000e+00 : f32
    %0 = tensor.empty() : tensor<3x1xi64>
    %1 = linalg.fill ins(%c0_i64 : i64) outs(%0 : tensor<3x1xi64>) -> tensor<3x1xi64>
    %2 = tensor.empty() : tensor<3x1xf32>
    %3 = linalg.fill ins(%cst : f32) outs(%2 : tensor<3x1xf32>) -> tensor<3x1xf32>
    %4:2 = linalg.generic {indexing_maps = [#map, #map1, #map1], iterator_types = ["parallel", "reduction"]} ins(%arg0 : tensor<3x4xf32>) outs(%3, %1 : tensor<3x1xf32>, tensor<3x1xi64>) {
    ^bb0(%in: f32, %out: f32, %out_1: i64):
      %11 = linalg.index 1 : index
      %12 = arith.index_cast %11 : index to i64
      %13 = arith.maximumf %in, %out : f32
      %14 = arith.cmpf ogt, %in, %out : f32
      %15 = arith.select %14, %12, %out_1 : i64
      linalg.yield %13, %15 : f32, i64
    } -> (tensor<3x1xf32>, tensor<3x1xi64>)
    %5 = tensor.empty() : tensor<3x4xf32>
    %6 = linalg.generic {indexing_maps = [#map, #map1, #map], iterator_types = ["parallel", "parallel"]} ins(%arg0, %4#0 : tensor<3x4xf32>, tensor<3x1xf32>) outs(%5 : tensor<3x4xf32>) {
    ^bb0(%in: f32, %in_1: f32, %out: f32):
      %11 = arith.subf %in, %in_1 : f32
      linalg.yield %11 : f32
    } -> tensor<3x4xf32>
    %7 = linalg.generic {indexing_maps = [#map, #map], iterator_types = ["parallel", "parallel"]} ins(%6 : tensor<3x4xf32>) outs(%5 : tensor<3x4xf32>) {
    ^bb0(%in: f32, %out: f32):
      %11 = math.exp %in : f32
      linalg.yield %11 : f32
    } -> tensor<3x4xf32>
    %8 = linalg.fill ins(%cst_0 : f32) outs(%2 : tensor<3x1xf32>) -> tensor<3x1xf32>
    %9 = linalg.generic {indexing_maps = [#map, #map1], iterator_types = ["parallel", "reduction"]} ins(%7 : tensor<3x4xf32>) outs(%8 : tensor<3x1xf32>) {
    ^bb0(%in: f32, %out: f32):
      %11 = arith.addf %in, %out : f32
      linalg.yield %11 : f32
    } -> tensor<3x1xf32>
    %10 = linalg.generic {indexing_maps = [#map, #map1, #map], iterator_types = ["parallel", "parallel"]} ins(%7, %9 : tensor<3x4xf32>, tensor<3x1xf32>) outs(%5 : tensor<3x4xf32>) {
    ^bb0(%in: f32, %in_1: f32, %out: f32):
      %11 = arith.divf %in, %in_1 : f32
      linalg.yield %11 : f32
    } -> tensor<3x4xf32>
    return %10 : tensor<3x4xf32>
  }
  func.func @silu(%arg0: tensor<1x4xf32>) -> tensor<1x4xf32> {
    %cst = arith.constant 1.000000e+00 : f32
    %0 = tensor.empty() : tensor<1x4xf32>
    %1 = linalg.generic {indexing_maps = [#map, #map], iterator_types = ["parallel", "parallel"]} ins(%arg0 : tensor<1x4xf32>) outs(%0 : tensor<1x4xf32>) {
    ^bb0(%in: f32, %out: f32):
      %3 = arith.negf %in : f32
      %4 = math.exp %3 : f32
      %5 = arith.addf %4, %cst : f32
      %6 = arith.divf %cst, %5 : f32
      linalg.yield %6 : f32
    } -> tensor<1x4xf32>
    %2 = linalg.generic {indexing_maps = [#map, #map, #map], iterator_types = ["parallel", "parallel"]} ins(%1, %arg0 : tensor<1x4xf32>, tensor<1x4xf32>) outs(%0 : tensor<1x4xf32>) {
    ^bb0(%in: f32, %in_0: f32, %out: f32):
      %3 = arith.mulf %in, %in_0 : f32
      linalg.yield %3 : f32
    } -> tensor<1x4xf32>
    return %2 : tensor<1x4xf32>
  }
  func.func @transpose(%arg0: tensor<3x4xf32>) -> tensor<4x3xf32> {
    %0 = tensor.empty() : tensor<4x3xf32>
    %1 = linalg.generic {indexing_maps = [#map, #mapt], iterator_types = ["parallel", "parallel"]} ins(%arg0 : tensor<3x4xf32>) outs(%0 : tensor<4x3xf32>) {
    ^bb0(%in: f32, %out: f32):
      linalg.yield %in : f32
    } -> tensor<4x3xf32>
    return %1 : tensor<4x3xf32>
  }
  func.func @reduce_leading(%arg0: tensor<3x4xf32>) -> tensor<4xf32> {
    %zero = arith.constant 0.0 : f32
    %0 = tensor.empty() : tensor<4xf32>
    %1 = linalg.fill ins(%zero : f32) outs(%0 : tensor<4xf32>) -> tensor<4xf32>
    %2 = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d1, d0)>, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]} ins(%arg0 : tensor<3x4xf32>) outs(%1 : tensor<4xf32>) {
    ^bb0(%in: f32, %out: f32):
      %3 = arith.addf %out, %in : f32
      linalg.yield %3 : f32
    } -> tensor<4xf32>
    return %2 : tensor<4xf32>
  }
  func.func private @printMemrefF32(tensor<*xf32>)
  func.func @main() {
    %x = arith.constant dense<[[1.0, 2.0, 3.0, 4.0], [0.0, 0.0, 0.0, 0.0], [-1.5, 0.25, 2.0, -3.0]]> : tensor<3x4xf32>
    %y = call @softmax(%x) : (tensor<3x4xf32>) -> tensor<3x4xf32>
    %uy = tensor.cast %y : tensor<3x4xf32> to tensor<*xf32>
    call @printMemrefF32(%uy) : (tensor<*xf32>) -> ()
    // CHECK: sizes = [3, 4] strides = [4, 1] data =
    // CHECK-NEXT: [0.0320586, 0.0871443, 0.236883, 0.643914],
    // CHECK-NEXT: [0.25, 0.25, 0.25, 0.25],
    // CHECK-NEXT: [0.0249419, 0.143531, 0.825962, 0.00556529]
    %v = arith.constant dense<[[1.3, -2.0, 0.0, 4.5]]> : tensor<1x4xf32>
    %s = call @silu(%v) : (tensor<1x4xf32>) -> tensor<1x4xf32>
    %us = tensor.cast %s : tensor<1x4xf32> to tensor<*xf32>
    call @printMemrefF32(%us) : (tensor<*xf32>) -> ()
    // CHECK: [1.02159, -0.238406, 0, 4.45056]
    %r = arith.constant dense<[[1.0, 2.0, 3.0, 4.5], [0.25, 0.25, 0.25, 0.25], [-1.0, 1.0, -1.0, 1.0]]> : tensor<3x4xf32>
    %t = call @transpose(%r) : (tensor<3x4xf32>) -> tensor<4x3xf32>
    %ut = tensor.cast %t : tensor<4x3xf32> to tensor<*xf32>
    call @printMemrefF32(%ut) : (tensor<*xf32>) -> ()
    // CHECK: sizes = [4, 3] strides = [3, 1]
    // CHECK-NEXT: [1, 0.25, -1],
    // CHECK-NEXT: [2, 0.25, 1],
    // CHECK-NEXT: [3, 0.25, -1],
    // CHECK-NEXT: [4.5, 0.25, 1]
    %l = call @reduce_leading(%r) : (tensor<3x4xf32>) -> tensor<4xf32>
    %ul = tensor.cast %l : tensor<4xf32> to tensor<*xf32>
    call @printMemrefF32(%ul) : (tensor<*xf32>) -> ()
    // CHECK: [0.25, 3.25, 2.25, 5.75]
    return
  }
}
