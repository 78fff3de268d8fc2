// Chains of elementwise generics in the shape of the reference's fusion benchmarks
// (benchmarks/kLoopFusion/kLoopFusion.mlir.in:4-30, benchmarks/kInputFusion/
// kInputFusion.mlir.in:6-41): each function becomes ONE launch.  f16 arithmetic
// rounds after every operation, as the IR's element type says.
// RUN: imex_runner.py -i %s -f linalg-to-gpu.pp -e main --entry-point-result=void --filecheck
#id = affine_map<(d0, d1) -> (d0, d1)>
#rowv = affine_map<(d0, d1) -> (d1)>
#tr = affine_map<(d0, d1) -> (d1, d0)>
#red = affine_map<(d0, d1) -> (d0)>
module @fused_elementwise {
  // (log(x) + |y|) - x
  func.func @loop_fusion_f32(%x: tensor<4x8xf32>, %y: tensor<4x8xf32>) -> tensor<4x8xf32> {
    %e = tensor.empty() : tensor<4x8xf32>
    %l = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%x : tensor<4x8xf32>) outs(%e : tensor<4x8xf32>) {
    ^bb0(%in: f32, %out: f32):
      %v = math.log %in : f32
      linalg.yield %v : f32
    } -> tensor<4x8xf32>
    %a = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%y : tensor<4x8xf32>) outs(%e : tensor<4x8xf32>) {
    ^bb0(%in: f32, %out: f32):
      %v = math.absf %in : f32
      linalg.yield %v : f32
    } -> tensor<4x8xf32>
    %s = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]} ins(%l, %a : tensor<4x8xf32>, tensor<4x8xf32>) outs(%e : tensor<4x8xf32>) {
    ^bb0(%in: f32, %in_0: f32, %out: f32):
      %v = arith.addf %in, %in_0 : f32
      linalg.yield %v : f32
    } -> tensor<4x8xf32>
    %d = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]} ins(%s, %x : tensor<4x8xf32>, tensor<4x8xf32>) outs(%e : tensor<4x8xf32>) {
    ^bb0(%in: f32, %in_0: f32, %out: f32):
      %v = arith.subf %in, %in_0 : f32
      linalg.yield %v : f32
    } -> tensor<4x8xf32>
    return %d : tensor<4x8xf32>
  }
  // the same chain in f16: every operation rounds to f16
  func.func @loop_fusion_f16(%x: tensor<4x8xf16>, %y: tensor<4x8xf16>) -> tensor<4x8xf16> {
    %e = tensor.empty() : tensor<4x8xf16>
    %l = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%x : tensor<4x8xf16>) outs(%e : tensor<4x8xf16>) {
    ^bb0(%in: f16, %out: f16):
      %v = math.log %in : f16
      linalg.yield %v : f16
    } -> tensor<4x8xf16>
    %a = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%y : tensor<4x8xf16>) outs(%e : tensor<4x8xf16>) {
    ^bb0(%in: f16, %out: f16):
      %v = math.absf %in : f16
      linalg.yield %v : f16
    } -> tensor<4x8xf16>
    %s = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]} ins(%l, %a : tensor<4x8xf16>, tensor<4x8xf16>) outs(%e : tensor<4x8xf16>) {
    ^bb0(%in: f16, %in_0: f16, %out: f16):
      %v = arith.addf %in, %in_0 : f16
      linalg.yield %v : f16
    } -> tensor<4x8xf16>
    %d = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]} ins(%s, %x : tensor<4x8xf16>, tensor<4x8xf16>) outs(%e : tensor<4x8xf16>) {
    ^bb0(%in: f16, %in_0: f16, %out: f16):
      %v = arith.subf %in, %in_0 : f16
      linalg.yield %v : f16
    } -> tensor<4x8xf16>
    return %d : tensor<4x8xf16>
  }
  // column sums of (|x| + row vector): the chain feeds the reduce, nothing is stored in between
  func.func @input_fusion(%x: tensor<4x8xf32>, %r: tensor<8xf32>) -> tensor<8xf32> {
    %zero = arith.constant 0.0 : f32
    %e = tensor.empty() : tensor<4x8xf32>
    %a = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%x : tensor<4x8xf32>) outs(%e : tensor<4x8xf32>) {
    ^bb0(%in: f32, %out: f32):
      %v = math.absf %in : f32
      linalg.yield %v : f32
    } -> tensor<4x8xf32>
    %s = linalg.generic {indexing_maps = [#id, #rowv, #id], iterator_types = ["parallel", "parallel"]} ins(%a, %r : tensor<4x8xf32>, tensor<8xf32>) outs(%e : tensor<4x8xf32>) {
    ^bb0(%in: f32, %in_0: f32, %out: f32):
      %v = arith.addf %in, %in_0 : f32
      linalg.yield %v : f32
    } -> tensor<4x8xf32>
    %ey = tensor.empty() : tensor<8xf32>
    %y0 = linalg.fill ins(%zero : f32) outs(%ey : tensor<8xf32>) -> tensor<8xf32>
    %y = linalg.generic {indexing_maps = [#tr, #red], iterator_types = ["parallel", "reduction"]} ins(%s : tensor<4x8xf32>) outs(%y0 : tensor<8xf32>) {
    ^bb0(%in: f32, %out: f32):
      %v = arith.addf %out, %in : f32
      linalg.yield %v : f32
    } -> tensor<8xf32>
    return %y : tensor<8xf32>
  }
  func.func private @printMemrefF32(tensor<*xf32>)
  func.func private @printMemrefF16(tensor<*xf16>)
  func.func @main() {
    %x = arith.constant dense<1.0> : tensor<4x8xf32>
    %y = arith.constant dense<-2.5> : tensor<4x8xf32>
    // (log 1 + 2.5) - 1
    %r0 = call @loop_fusion_f32(%x, %y) : (tensor<4x8xf32>, tensor<4x8xf32>) -> tensor<4x8xf32>
    %u0 = tensor.cast %r0 : tensor<4x8xf32> to tensor<*xf32>
    call @printMemrefF32(%u0) : (tensor<*xf32>) -> ()
    // CHECK: sizes = [4, 8] strides = [8, 1] data =
    // CHECK-NEXT: {{\[}}[1.5, 1.5, 1.5, 1.5, 1.5, 1.5, 1.5, 1.5],
    %xh = arith.constant dense<3.0> : tensor<4x8xf16>
    %yh = arith.constant dense<-0.6> : tensor<4x8xf16>
    // log 3 -> f16 1.09863; + 0.600098 -> f16 1.69922; - 3 = -1.30078
    // (one rounding at the end would give -1.30176)
    %r1 = call @loop_fusion_f16(%xh, %yh) : (tensor<4x8xf16>, tensor<4x8xf16>) -> tensor<4x8xf16>
    %u1 = tensor.cast %r1 : tensor<4x8xf16> to tensor<*xf16>
    call @printMemrefF16(%u1) : (tensor<*xf16>) -> ()
    // CHECK: sizes = [4, 8] strides = [8, 1] data =
    // CHECK-NEXT: {{\[}}[-1.30078, -1.30078,
    %z = arith.constant dense<-0.25> : tensor<4x8xf32>
    %rv = arith.constant dense<[0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0]> : tensor<8xf32>
    // 4 rows of (0.25 + j)
    %r2 = call @input_fusion(%z, %rv) : (tensor<4x8xf32>, tensor<8xf32>) -> tensor<8xf32>
    %u2 = tensor.cast %r2 : tensor<8xf32> to tensor<*xf32>
    call @printMemrefF32(%u2) : (tensor<*xf32>) -> ()
    // CHECK: sizes = [8] strides = [1] data =
    // CHECK-NEXT: [1, 5, 9, 13, 17, 21, 25, 29]
    return
  }
}
