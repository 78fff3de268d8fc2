// An elementwise op outside the hot path: the runner must refuse it (there is
// no CPU fallback), naming the line and the body it could not match.
#map = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @main() {
    %x = arith.constant dense<2.0> : tensor<2x2xf32>
    %0 = tensor.empty() : tensor<2x2xf32>
    %1 = linalg.generic {indexing_maps = [#map, #map], iterator_types = ["parallel", "parallel"]} ins(%x : tensor<2x2xf32>) outs(%0 : tensor<2x2xf32>) {
    ^bb0(%in: f32, %out: f32):
      %s = math.erf %in : f32
      linalg.yield %s : f32
    } -> tensor<2x2xf32>
    return
  }
}
