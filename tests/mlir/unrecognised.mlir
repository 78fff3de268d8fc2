// An op that is neither a hot-path kernel nor expressible as a loop-nest kernel (the body
// uses an operation without a translation): the runner must refuse it, naming the line and
// the reason; there is no CPU fallback.
#map = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @main() {
    %x = arith.constant dense<2> : tensor<2x2xi32>
    %0 = tensor.empty() : tensor<2x2xi32>
    %1 = linalg.generic {indexing_maps = [#map, #map], iterator_types = ["parallel", "parallel"]} ins(%x : tensor<2x2xi32>) outs(%0 : tensor<2x2xi32>) {
    ^bb0(%in: i32, %out: i32):
      %s = math.ctlz %in : i32
      linalg.yield %s : i32
    } -> tensor<2x2xi32>
    return
  }
}
