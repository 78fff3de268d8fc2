// A linalg op in buffer form (no results, the output is written in place): the runner works
// on tensors and must say so instead of binding nothing and printing stale data.
#map = affine_map<(d0) -> (d0)>
module {
  func.func @main() {
    %x = arith.constant dense<2.0> : tensor<4xf32>
    %m = bufferization.to_memref %x : tensor<4xf32> to memref<4xf32>
    linalg.generic {indexing_maps = [#map, #map], iterator_types = ["parallel"]} ins(%m : memref<4xf32>) outs(%m : memref<4xf32>) {
    ^bb0(%in: f32, %out: f32):
      %s = arith.addf %in, %in : f32
      linalg.yield %s : f32
    }
    return
  }
}
