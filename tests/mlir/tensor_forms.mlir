// Tensor-level forms beside the hot path, each as the reference's tests write them: a
// concatenation as scf.if over tensor.dim / tensor.extract inside a region
// (test/Jax/janet/jit_prim_fun.50_linalg.mlir:21-40), extents the IR leaves dynamic
// (test/PlaidML/OpTest.EltwiseAdd.dynamic.mlir:12-28), a static slice and a pad
// (test/PlaidML/CppEdsl.Convolution.mlir:26-29), and scf.while over tensors on the host
// (test/Jax/janet/jit__get_age_weights_from_tables.8_linalg.mlir:389-591).
#map1 = affine_map<(d0) -> (d0)>
#map2 = affine_map<(d0, d1) -> (d0, d1)>
#map0 = affine_map<() -> ()>
module {
  func.func private @printMemrefF32(tensor<*xf32>)
  func.func private @printMemrefI32(tensor<*xi32>)

  // [a ; b] along dim 0
  func.func @concat(%a: tensor<3xf32>, %b: tensor<2xf32>) -> tensor<5xf32> {
    %c0 = arith.constant 0 : index
    %0 = tensor.empty() : tensor<5xf32>
    %1 = linalg.generic {indexing_maps = [#map1], iterator_types = ["parallel"]} outs(%0 : tensor<5xf32>) {
    ^bb0(%out: f32):
      %i = linalg.index 0 : index
      %n = tensor.dim %a, %c0 : tensor<3xf32>
      %first = arith.cmpi ult, %i, %n : index
      %v = scf.if %first -> (f32) {
        %x = tensor.extract %a[%i] : tensor<3xf32>
        scf.yield %x : f32
      } else {
        %j = arith.subi %i, %n : index
        %x = tensor.extract %b[%j] : tensor<2xf32>
        scf.yield %x : f32
      }
      linalg.yield %v : f32
    } -> tensor<5xf32>
    return %1 : tensor<5xf32>
  }

  // x + x for whatever extents x has
  func.func @twice(%x: tensor<?x?xf32>) -> tensor<?x?xf32> {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %d0 = tensor.dim %x, %c0 : tensor<?x?xf32>
    %d1 = tensor.dim %x, %c1 : tensor<?x?xf32>
    %0 = tensor.empty(%d0, %d1) : tensor<?x?xf32>
    %1 = linalg.generic {indexing_maps = [#map2, #map2], iterator_types = ["parallel", "parallel"]}
         ins(%x : tensor<?x?xf32>) outs(%0 : tensor<?x?xf32>) {
    ^bb0(%e: f32, %o: f32):
      %s = arith.addf %e, %e : f32
      linalg.yield %s : f32
    } -> tensor<?x?xf32>
    return %1 : tensor<?x?xf32>
  }

  // counts up to 5 in a tensor<i32>, doubling a tensor<2xi32> every round: [3, 5] * 2^5
  func.func @loop(%start: tensor<2xi32>) -> tensor<2xi32> {
    %zero = arith.constant dense<0> : tensor<i32>
    %r:2 = scf.while (%n = %zero, %acc = %start) : (tensor<i32>, tensor<2xi32>) -> (tensor<i32>, tensor<2xi32>) {
      %five = arith.constant dense<5> : tensor<i32>
      %0 = tensor.empty() : tensor<i1>
      %1 = linalg.generic {indexing_maps = [#map0, #map0, #map0], iterator_types = []} ins(%n, %five : tensor<i32>, tensor<i32>) outs(%0 : tensor<i1>) {
      ^bb0(%p: i32, %q: i32, %o: i1):
        %lt = arith.cmpi slt, %p, %q : i32
        linalg.yield %lt : i1
      } -> tensor<i1>
      %go = tensor.extract %1[] : tensor<i1>
      scf.condition(%go) %n, %acc : tensor<i32>, tensor<2xi32>
    } do {
    ^bb0(%n: tensor<i32>, %acc: tensor<2xi32>):
      %one = arith.constant dense<1> : tensor<i32>
      %0 = tensor.empty() : tensor<i32>
      %1 = linalg.generic {indexing_maps = [#map0, #map0, #map0], iterator_types = []} ins(%n, %one : tensor<i32>, tensor<i32>) outs(%0 : tensor<i32>) {
      ^bb0(%p: i32, %q: i32, %o: i32):
        %s = arith.addi %p, %q : i32
        linalg.yield %s : i32
      } -> tensor<i32>
      %2 = tensor.empty() : tensor<2xi32>
      %3 = linalg.generic {indexing_maps = [#map1, #map1], iterator_types = ["parallel"]} ins(%acc : tensor<2xi32>) outs(%2 : tensor<2xi32>) {
      ^bb0(%p: i32, %o: i32):
        %s = arith.addi %p, %p : i32
        linalg.yield %s : i32
      } -> tensor<2xi32>
      scf.yield %1, %3 : tensor<i32>, tensor<2xi32>
    }
    return %r#1 : tensor<2xi32>
  }

  func.func @main() {
    %a = arith.constant dense<[1.0, 2.0, 3.0]> : tensor<3xf32>
    %b = arith.constant dense<[4.0, 5.0]> : tensor<2xf32>
    %c = call @concat(%a, %b) : (tensor<3xf32>, tensor<2xf32>) -> tensor<5xf32>
    %cu = tensor.cast %c : tensor<5xf32> to tensor<*xf32>
    call @printMemrefF32(%cu) : (tensor<*xf32>) -> ()
    // CHECK: sizes = [5] strides = [1] data =
    // CHECK-NEXT: [1, 2, 3, 4, 5]

    // the middle three, then one element of padding either side
    %s = tensor.extract_slice %c[1] [3] [1] : tensor<5xf32> to tensor<3xf32>
    %pv = arith.constant -1.0 : f32
    %p = tensor.pad %s low[1] high[1] {
    ^bb0(%i: index):
      tensor.yield %pv : f32
    } : tensor<3xf32> to tensor<5xf32>
    %pu = tensor.cast %p : tensor<5xf32> to tensor<*xf32>
    call @printMemrefF32(%pu) : (tensor<*xf32>) -> ()
    // CHECK: sizes = [5] strides = [1] data =
    // CHECK-NEXT: [-1, 2, 3, 4, -1]

    %m = arith.constant dense<[[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]> : tensor<2x3xf32>
    %md = tensor.cast %m : tensor<2x3xf32> to tensor<?x?xf32>
    %t = call @twice(%md) : (tensor<?x?xf32>) -> tensor<?x?xf32>
    %tu = tensor.cast %t : tensor<?x?xf32> to tensor<*xf32>
    call @printMemrefF32(%tu) : (tensor<*xf32>) -> ()
    // CHECK: sizes = [2, 3] strides = [3, 1] data =
    // CHECK-NEXT: {{\[}}[2, 4, 6],
    // CHECK-NEXT: [8, 10, 12]]

    %st = arith.constant dense<[3, 5]> : tensor<2xi32>
    %l = call @loop(%st) : (tensor<2xi32>) -> tensor<2xi32>
    %lu = tensor.cast %l : tensor<2xi32> to tensor<*xi32>
    call @printMemrefI32(%lu) : (tensor<*xi32>) -> ()
    // CHECK: sizes = [2] strides = [1] data =
    // CHECK-NEXT: [96, 160]
    return
  }
}
