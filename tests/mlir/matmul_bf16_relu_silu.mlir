// bf16 operands extended to f32, f32 multiply-add, then the relu / silu
// generics of the benchmarks: one fused tensor-core GEMM per call.
// RUN: imex_runner.py -i %s -f linalg-to-gpu.pp -e main --entry-point-result=void --filecheck
#id = affine_map<(d0, d1) -> (d0, d1)>
#map0 = affine_map<(d0, d1, d2) -> (d0, d2)>
#map1 = affine_map<(d0, d1, d2) -> (d2, d1)>
#map2 = affine_map<(d0, d1, d2) -> (d0, d1)>
module @matmul_bf16 {
  func.func @gemm_relu(%a: tensor<256x64xbf16>, %b: tensor<64x16xbf16>) -> tensor<256x16xf32> {
    %zero = arith.constant 0.0 : f32
    %ea = tensor.empty() : tensor<256x64xf32>
    %af = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%a : tensor<256x64xbf16>) outs(%ea : tensor<256x64xf32>) {
    ^bb0(%x: bf16, %o: f32):
      %e = arith.extf %x : bf16 to f32
      linalg.yield %e : f32
    } -> tensor<256x64xf32>
    %eb = tensor.empty() : tensor<64x16xf32>
    %bf = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%b : tensor<64x16xbf16>) outs(%eb : tensor<64x16xf32>) {
    ^bb0(%x: bf16, %o: f32):
      %e = arith.extf %x : bf16 to f32
      linalg.yield %e : f32
    } -> tensor<64x16xf32>
    %ec = tensor.empty() : tensor<256x16xf32>
    %c0 = linalg.fill ins(%zero : f32) outs(%ec : tensor<256x16xf32>) -> tensor<256x16xf32>
    %c = linalg.generic {indexing_maps = [#map0, #map1, #map2], iterator_types = ["parallel", "parallel", "reduction"]}
         ins(%af, %bf : tensor<256x64xf32>, tensor<64x16xf32>) outs(%c0 : tensor<256x16xf32>) {
    ^bb0(%x: f32, %y: f32, %acc: f32):
      %p = arith.mulf %x, %y : f32
      %s = arith.addf %acc, %p : f32
      linalg.yield %s : f32
    } -> tensor<256x16xf32>
    %er = tensor.empty() : tensor<256x16xf32>
    %r = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%c : tensor<256x16xf32>) outs(%er : tensor<256x16xf32>) {
    ^bb0(%in: f32, %out: f32):
      %g = arith.cmpf ugt, %in, %zero : f32
      %s = arith.select %g, %in, %zero : f32
      linalg.yield %s : f32
    } -> tensor<256x16xf32>
    return %r : tensor<256x16xf32>
  }
  func.func @gemm_silu(%a: tensor<256x64xbf16>, %b: tensor<64x16xbf16>) -> tensor<256x16xf32> {
    %zero = arith.constant 0.0 : f32
    %one = arith.constant 1.0 : f32
    %ec = tensor.empty() : tensor<256x16xf32>
    %c0 = linalg.fill ins(%zero : f32) outs(%ec : tensor<256x16xf32>) -> tensor<256x16xf32>
    %c = linalg.generic {indexing_maps = [#map0, #map1, #map2], iterator_types = ["parallel", "parallel", "reduction"]}
         ins(%a, %b : tensor<256x64xbf16>, tensor<64x16xbf16>) outs(%c0 : tensor<256x16xf32>) {
    ^bb0(%x: bf16, %y: bf16, %acc: f32):
      %xf = arith.extf %x : bf16 to f32
      %yf = arith.extf %y : bf16 to f32
      %p = arith.mulf %xf, %yf : f32
      %s = arith.addf %acc, %p : f32
      linalg.yield %s : f32
    } -> tensor<256x16xf32>
    %e1 = tensor.empty() : tensor<256x16xf32>
    %sg = linalg.generic {indexing_maps = [#id, #id], iterator_types = ["parallel", "parallel"]} ins(%c : tensor<256x16xf32>) outs(%e1 : tensor<256x16xf32>) {
    ^bb0(%in: f32, %out: f32):
      %n = arith.negf %in : f32
      %e = math.exp %n : f32
      %d = arith.addf %e, %one : f32
      %q = arith.divf %one, %d : f32
      linalg.yield %q : f32
    } -> tensor<256x16xf32>
    %r = linalg.generic {indexing_maps = [#id, #id, #id], iterator_types = ["parallel", "parallel"]} ins(%sg, %c : tensor<256x16xf32>, tensor<256x16xf32>) outs(%e1 : tensor<256x16xf32>) {
    ^bb0(%in: f32, %in_0: f32, %out: f32):
      %m = arith.mulf %in, %in_0 : f32
      linalg.yield %m : f32
    } -> tensor<256x16xf32>
    return %r : tensor<256x16xf32>
  }
  func.func @row_sum(%x: tensor<256x16xf32>) -> tensor<256xf32> {
    %zero = arith.constant 0.0 : f32
    %e = tensor.empty() : tensor<256xf32>
    %z = linalg.fill ins(%zero : f32) outs(%e : tensor<256xf32>) -> tensor<256xf32>
    %s = linalg.generic {indexing_maps = [#id, affine_map<(d0, d1) -> (d0)>], iterator_types = ["parallel", "reduction"]} ins(%x : tensor<256x16xf32>) outs(%z : tensor<256xf32>) {
    ^bb0(%in: f32, %out: f32):
      %a = arith.addf %in, %out : f32
      linalg.yield %a : f32
    } -> tensor<256xf32>
    return %s : tensor<256xf32>
  }
  func.func @total(%x: tensor<256xf32>) -> tensor<f32> {
    %zero = arith.constant 0.0 : f32
    %e = tensor.empty() : tensor<f32>
    %z = linalg.fill ins(%zero : f32) outs(%e : tensor<f32>) -> tensor<f32>
    %s = linalg.generic {indexing_maps = [affine_map<(d0) -> (d0)>, affine_map<(d0) -> ()>], iterator_types = ["reduction"]} ins(%x : tensor<256xf32>) outs(%z : tensor<f32>) {
    ^bb0(%in: f32, %out: f32):
      %a = arith.addf %out, %in : f32
      linalg.yield %a : f32
    } -> tensor<f32>
    return %s : tensor<f32>
  }
  func.func private @printMemrefF32(tensor<*xf32>)
  func.func @main() {
    %a = arith.constant dense<0.5> : tensor<256x64xbf16>
    %bp = arith.constant dense<0.25> : tensor<64x16xbf16>
    %bn = arith.constant dense<-0.25> : tensor<64x16xbf16>
    // every element of A.Bp is 64 * 0.125 = 8, of A.Bn is -8
    %r0 = call @gemm_relu(%a, %bp) : (tensor<256x64xbf16>, tensor<64x16xbf16>) -> tensor<256x16xf32>
    %s0 = call @row_sum(%r0) : (tensor<256x16xf32>) -> tensor<256xf32>
    %t0 = call @total(%s0) : (tensor<256xf32>) -> tensor<f32>
    %u0 = tensor.cast %t0 : tensor<f32> to tensor<*xf32>
    call @printMemrefF32(%u0) : (tensor<*xf32>) -> ()
    // 256 * 16 * 8
    // CHECK: rank = 0 offset = 0 sizes = [] strides = [] data =
    // CHECK-NEXT: [32768]
    %r1 = call @gemm_relu(%a, %bn) : (tensor<256x64xbf16>, tensor<64x16xbf16>) -> tensor<256x16xf32>
    %s1 = call @row_sum(%r1) : (tensor<256x16xf32>) -> tensor<256xf32>
    %t1 = call @total(%s1) : (tensor<256xf32>) -> tensor<f32>
    %u1 = tensor.cast %t1 : tensor<f32> to tensor<*xf32>
    call @printMemrefF32(%u1) : (tensor<*xf32>) -> ()
    // CHECK: [0]
    // silu(8) = 7.99732, silu(-8) = -0.00268276; times 256 * 16
    %r2 = call @gemm_silu(%a, %bp) : (tensor<256x64xbf16>, tensor<64x16xbf16>) -> tensor<256x16xf32>
    %s2 = call @row_sum(%r2) : (tensor<256x16xf32>) -> tensor<256xf32>
    %t2 = call @total(%s2) : (tensor<256xf32>) -> tensor<f32>
    %u2 = tensor.cast %t2 : tensor<f32> to tensor<*xf32>
    call @printMemrefF32(%u2) : (tensor<*xf32>) -> ()
    // CHECK: [3275{{[0-9.]*}}]
    %r3 = call @gemm_silu(%a, %bn) : (tensor<256x64xbf16>, tensor<64x16xbf16>) -> tensor<256x16xf32>
    %s3 = call @row_sum(%r3) : (tensor<256x16xf32>) -> tensor<256xf32>
    %t3 = call @total(%s3) : (tensor<256xf32>) -> tensor<f32>
    %u3 = tensor.cast %t3 : tensor<f32> to tensor<*xf32>
    call @printMemrefF32(%u3) : (tensor<*xf32>) -> ()
    // CHECK: [-10.98{{[0-9]*}}]
    return
  }
}
