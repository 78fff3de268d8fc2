// Row sharding through the reference's annotation surface (shard.grid / shard.sharding /
// shard.shard, test/Dialect/NDArray/Extensions/sharding_propagation.mlir:4-12): a matmul with
// its bias and relu, a softmax and a row sum on arrays whose rows are split over four ranks.
// Started with --shard-rank R --shard-count 4 the runner holds and computes rank R's rows
// only (9 rows: blocks of 2, 2, 2, 3 by the partition rule); the four outputs together are
// the output of the unsharded program.
#id = affine_map<(d0, d1) -> (d0, d1)>
#row = affine_map<(d0, d1) -> (d0)>
#col = affine_map<(d0, d1) -> (d1)>
module {
shard.grid @mesh4(shape = 4)
func.func private @printMemrefF32(tensor<*xf32>)

func.func @main() {
  %a = arith.constant dense<[[1.0, 2.0, 0.5], [0.0, -1.0, 2.0], [3.0, 1.0, 1.0], [-2.0, 0.5, 0.25], [1.5, 1.5, -1.5],
                             [4.0, 0.0, -3.0], [0.25, 0.75, 1.25], [-1.0, -2.0, -3.0], [2.0, 2.0, 2.0]]> : tensor<9x3xf32>
  %w = arith.constant dense<[[1.0, -1.0], [0.5, 2.0], [-2.0, 0.25]]> : tensor<3x2xf32>
  %bias = arith.constant dense<[0.5, -0.5]> : tensor<2xf32>
  %s = shard.sharding @mesh4 split_axes = [[0]] : !shard.sharding
  %as = shard.shard %a to %s : tensor<9x3xf32>
  %zero = arith.constant 0.0 : f32
  %e = tensor.empty() : tensor<9x2xf32>
  %c0 = linalg.fill ins(%zero : f32) outs(%e : tensor<9x2xf32>) -> tensor<9x2xf32>
  %c = linalg.matmul ins(%as, %w : tensor<9x3xf32>, tensor<3x2xf32>) outs(%c0 : tensor<9x2xf32>) -> tensor<9x2xf32>
  %be = tensor.empty() : tensor<9x2xf32>
  %bb = linalg.generic {indexing_maps = [#col, #id], iterator_types = ["parallel", "parallel"]} ins(%bias : tensor<2xf32>) outs(%be : tensor<9x2xf32>) {
  ^bb0(%in: f32, %out: f32):
    linalg.yield %in : f32
  } -> tensor<9x2xf32>
  %se = tensor.empty() : tensor<9x2xf32>
  %sum = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]} ins(%c, %bb : tensor<9x2xf32>, tensor<9x2xf32>) outs(%se : tensor<9x2xf32>) {
  ^bb0(%x: f32, %y: f32, %out: f32):
    %r = arith.addf %x, %y : f32
    linalg.yield %r : f32
  } -> tensor<9x2xf32>
  %re = tensor.empty() : tensor<9x2xf32>
  %relu = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%sum : tensor<9x2xf32>) outs(%re : tensor<9x2xf32>) {
  ^bb0(%x: f32, %out: f32):
    %p = arith.cmpf ugt, %x, %zero : f32
    %r = arith.select %p, %x, %zero : f32
    linalg.yield %r : f32
  } -> tensor<9x2xf32>
  %u = tensor.cast %relu : tensor<9x2xf32> to tensor<*xf32>
  call @printMemrefF32(%u) : (tensor<*xf32>) -> ()
  // row sum of the sharded input: one value per row this rank holds
  %ye = tensor.empty() : tensor<9xf32>
  %y0 = linalg.fill ins(%zero : f32) outs(%ye : tensor<9xf32>) -> tensor<9xf32>
  %y = linalg.generic {indexing_maps = [#id, #row], iterator_types = ["parallel", "reduction"]} ins(%as : tensor<9x3xf32>) outs(%y0 : tensor<9xf32>) {
  ^bb0(%x: f32, %acc: f32):
    %r = arith.addf %x, %acc : f32
    linalg.yield %r : f32
  } -> tensor<9xf32>
  %yu = tensor.cast %y : tensor<9xf32> to tensor<*xf32>
  call @printMemrefF32(%yu) : (tensor<*xf32>) -> ()
  return
}
}
