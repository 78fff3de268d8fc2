// GPU-dialect host code around hand-written XeGPU device code, in the style of the
// reference's integration tests (test/Integration/Dialect/XeGPU/WG/gemm_4kx4kx4k_f16_f16_f32_bias.mlir,
// gemm_4kx4kx4k_transpose_b.mlir): memref.alloc'ed host arrays filled by runner-utils calls and
// scf.for nests, gpu.alloc / gpu.memcpy / gpu.launch_func / gpu.wait, a CPU reference through
// gemmF16F16F32 and printAllcloseF32.  The device code cannot run on a B200; the runner
// recognises WHAT each gpu.func computes from its data flow and serves it with its own GEMM.
// Two kernels: C = A.B + bias (C read as the initial accumulator), and C = A.B^T with B stored [N,K].
module @gemm attributes {gpu.container_module} {
  func.func @run_bias(%A: memref<384x256xf16>, %B: memref<256x512xf16>, %C: memref<384x512xf32>, %bias: memref<512xf32>) {
    %c1 = arith.constant 1 : index
    %c2 = arith.constant 2 : index
    %c3 = arith.constant 3 : index
    %c256 = arith.constant 256 : index
    %A_gpu = gpu.alloc () : memref<384x256xf16>
    gpu.memcpy %A_gpu, %A : memref<384x256xf16>, memref<384x256xf16>
    %B_gpu = gpu.alloc () : memref<256x512xf16>
    gpu.memcpy %B_gpu, %B : memref<256x512xf16>, memref<256x512xf16>
    %C_gpu = gpu.alloc () : memref<384x512xf32>
    gpu.memcpy %C_gpu, %C : memref<384x512xf32>, memref<384x512xf32>
    %bias_gpu = gpu.alloc () : memref<512xf32>
    gpu.memcpy %bias_gpu, %bias : memref<512xf32>, memref<512xf32>
    gpu.launch_func @kernels::@gemm_bias blocks in (%c2, %c3, %c1) threads in (%c256, %c1, %c1) args(%bias_gpu : memref<512xf32>, %C_gpu : memref<384x512xf32>, %A_gpu : memref<384x256xf16>, %B_gpu : memref<256x512xf16>)
    gpu.wait
    gpu.memcpy %C, %C_gpu : memref<384x512xf32>, memref<384x512xf32>
    gpu.dealloc %A_gpu : memref<384x256xf16>
    gpu.dealloc %B_gpu : memref<256x512xf16>
    gpu.dealloc %C_gpu : memref<384x512xf32>
    gpu.dealloc %bias_gpu : memref<512xf32>
    return
  }

  func.func @run_transpose_b(%A: memref<384x256xf16>, %Bt: memref<512x256xf16>, %C: memref<384x512xf32>) {
    %c1 = arith.constant 1 : index
    %c2 = arith.constant 2 : index
    %c3 = arith.constant 3 : index
    %c256 = arith.constant 256 : index
    %A_gpu = gpu.alloc () : memref<384x256xf16>
    gpu.memcpy %A_gpu, %A : memref<384x256xf16>, memref<384x256xf16>
    %B_gpu = gpu.alloc () : memref<512x256xf16>
    gpu.memcpy %B_gpu, %Bt : memref<512x256xf16>, memref<512x256xf16>
    %C_gpu = gpu.alloc () : memref<384x512xf32>
    gpu.launch_func @kernels::@gemm_bt blocks in (%c2, %c3, %c1) threads in (%c256, %c1, %c1) args(%A_gpu : memref<384x256xf16>, %B_gpu : memref<512x256xf16>, %C_gpu : memref<384x512xf32>)
    gpu.wait
    gpu.memcpy %C, %C_gpu : memref<384x512xf32>, memref<384x512xf32>
    return
  }

  gpu.module @kernels {
    // C[128-row block, 256-column block] = C + A.B, then + bias[column]
    gpu.func @gemm_bias(%bias: memref<512xf32>, %C: memref<384x512xf32>, %A: memref<384x256xf16>, %B: memref<256x512xf16>) kernel {
      %c0 = arith.constant 0 : index
      %c32 = arith.constant 32 : index
      %c128 = arith.constant 128 : index
      %c256 = arith.constant 256 : index
      %mask = arith.constant dense<true> : vector<256xi1>
      %bx = gpu.block_id x
      %by = gpu.block_id y
      %col0 = arith.muli %bx, %c256 : index
      %row0 = arith.muli %by, %c128 : index
      %lanes = vector.step : vector<256xindex>
      %colv = vector.broadcast %col0 : index to vector<256xindex>
      %cols = arith.addi %colv, %lanes : vector<256xindex>
      %bias_ptr = memref.extract_aligned_pointer_as_index %bias : memref<512xf32> -> index
      %bias_i64 = arith.index_cast %bias_ptr : index to i64
      %bias_row = xegpu.load %bias_i64[%cols], %mask : i64, vector<256xindex>, vector<256xi1> -> vector<256xf32>
      %bias_tile = vector.broadcast %bias_row : vector<256xf32> to vector<128x256xf32>
      %c_desc = xegpu.create_nd_tdesc %C : memref<384x512xf32> -> !xegpu.tensor_desc<128x256xf32>
      %c_init = xegpu.load_nd %c_desc[%row0, %col0] : !xegpu.tensor_desc<128x256xf32> -> vector<128x256xf32>
      %a_desc = xegpu.create_nd_tdesc %A : memref<384x256xf16> -> !xegpu.tensor_desc<128x32xf16>
      %b_desc = xegpu.create_nd_tdesc %B : memref<256x512xf16> -> !xegpu.tensor_desc<32x256xf16>
      %acc = scf.for %k = %c0 to %c256 step %c32 iter_args(%c_val = %c_init) -> (vector<128x256xf32>) {
        %a_val = xegpu.load_nd %a_desc[%row0, %k] : !xegpu.tensor_desc<128x32xf16> -> vector<128x32xf16>
        %b_val = xegpu.load_nd %b_desc[%k, %col0] : !xegpu.tensor_desc<32x256xf16> -> vector<32x256xf16>
        %c_new = xegpu.dpas %a_val, %b_val, %c_val : vector<128x32xf16>, vector<32x256xf16>, vector<128x256xf32> -> vector<128x256xf32>
        scf.yield %c_new : vector<128x256xf32>
      }
      %out = arith.addf %bias_tile, %acc : vector<128x256xf32>
      xegpu.store_nd %out, %c_desc[%row0, %col0] : vector<128x256xf32>, !xegpu.tensor_desc<128x256xf32>
      gpu.return
    }
    // C = A . B^T with B stored [N, K]: the B tile is transposed in registers before the product
    gpu.func @gemm_bt(%A: memref<384x256xf16>, %B: memref<512x256xf16>, %C: memref<384x512xf32>) kernel {
      %c0 = arith.constant 0 : index
      %c32 = arith.constant 32 : index
      %c128 = arith.constant 128 : index
      %c256 = arith.constant 256 : index
      %zero = arith.constant dense<0.0> : vector<128x256xf32>
      %bx = gpu.block_id x
      %by = gpu.block_id y
      %col0 = arith.muli %bx, %c256 : index
      %row0 = arith.muli %by, %c128 : index
      %a_desc = xegpu.create_nd_tdesc %A : memref<384x256xf16> -> !xegpu.tensor_desc<128x32xf16>
      %b_desc = xegpu.create_nd_tdesc %B : memref<512x256xf16> -> !xegpu.tensor_desc<256x32xf16>
      %c_desc = xegpu.create_nd_tdesc %C : memref<384x512xf32> -> !xegpu.tensor_desc<128x256xf32>
      %acc = scf.for %k = %c0 to %c256 step %c32 iter_args(%c_val = %zero) -> (vector<128x256xf32>) {
        %a_val = xegpu.load_nd %a_desc[%row0, %k] : !xegpu.tensor_desc<128x32xf16> -> vector<128x32xf16>
        %b_val = xegpu.load_nd %b_desc[%col0, %k] : !xegpu.tensor_desc<256x32xf16> -> vector<256x32xf16>
        %b_t = vector.transpose %b_val, [1, 0] : vector<256x32xf16> to vector<32x256xf16>
        %c_new = xegpu.dpas %a_val, %b_t, %c_val : vector<128x32xf16>, vector<32x256xf16>, vector<128x256xf32> -> vector<128x256xf32>
        scf.yield %c_new : vector<128x256xf32>
      }
      xegpu.store_nd %acc, %c_desc[%row0, %col0] : vector<128x256xf32>, !xegpu.tensor_desc<128x256xf32>
      gpu.return
    }
  }

  func.func @main() attributes {llvm.emit_c_interface} {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %c256 = arith.constant 256 : index
    %c384 = arith.constant 384 : index
    %c512 = arith.constant 512 : index
    %lo = arith.constant -0.5 : f32
    %hi = arith.constant 0.5 : f32
    %frac = arith.constant 0 : i1
    %zero = arith.constant 0.0 : f32
    %A = memref.alloc() : memref<384x256xf16>
    %B = memref.alloc() : memref<256x512xf16>
    %Bt = memref.alloc() : memref<512x256xf16>
    %C = memref.alloc() : memref<384x512xf32>
    %C2 = memref.alloc() : memref<384x512xf32>
    %C_ref = memref.alloc() : memref<384x512xf32>
    %bias = memref.alloc() : memref<512xf32>
    %A_u = memref.cast %A : memref<384x256xf16> to memref<*xf16>
    call @fillResource1DRandomF16(%A_u, %lo, %hi, %frac) : (memref<*xf16>, f32, f32, i1) -> ()
    %B_u = memref.cast %B : memref<256x512xf16> to memref<*xf16>
    call @fillResource1DRandomF16(%B_u, %lo, %hi, %frac) : (memref<*xf16>, f32, f32, i1) -> ()
    %bias_u = memref.cast %bias : memref<512xf32> to memref<*xf32>
    call @fillResource1DRandomF32(%bias_u, %lo, %hi, %frac) : (memref<*xf32>, f32, f32, i1) -> ()
    // C = C2 = C_ref = 0 ; Bt[n, k] = B[k, n]
    scf.for %i = %c0 to %c384 step %c1 {
      scf.for %j = %c0 to %c512 step %c1 {
        memref.store %zero, %C[%i, %j] : memref<384x512xf32>
        memref.store %zero, %C2[%i, %j] : memref<384x512xf32>
        memref.store %zero, %C_ref[%i, %j] : memref<384x512xf32>
      }
    }
    scf.for %k = %c0 to %c256 step %c1 {
      scf.for %n = %c0 to %c512 step %c1 {
        %v = memref.load %B[%k, %n] : memref<256x512xf16>
        memref.store %v, %Bt[%n, %k] : memref<512x256xf16>
      }
    }
    // CPU reference: C_ref = A.B
    %C_ref_u = memref.cast %C_ref : memref<384x512xf32> to memref<*xf32>
    call @gemmF16F16F32(%A_u, %B_u, %C_ref_u) : (memref<*xf16>, memref<*xf16>, memref<*xf32>) -> ()
    // kernel 2: C2 = A.Bt^T, against the reference without the bias
    call @run_transpose_b(%A, %Bt, %C2) : (memref<384x256xf16>, memref<512x256xf16>, memref<384x512xf32>) -> ()
    %C2_u = memref.cast %C2 : memref<384x512xf32> to memref<*xf32>
    // CHECK: [ALLCLOSE: TRUE]
    call @printAllcloseF32(%C2_u, %C_ref_u) : (memref<*xf32>, memref<*xf32>) -> ()
    // kernel 1: C = A.B + bias, against the reference with the bias added on the host
    call @run_bias(%A, %B, %C, %bias) : (memref<384x256xf16>, memref<256x512xf16>, memref<384x512xf32>, memref<512xf32>) -> ()
    scf.for %i = %c0 to %c384 step %c1 {
      scf.for %j = %c0 to %c512 step %c1 {
        %c = memref.load %C_ref[%i, %j] : memref<384x512xf32>
        %b = memref.load %bias[%j] : memref<512xf32>
        %s = arith.addf %c, %b : f32
        memref.store %s, %C_ref[%i, %j] : memref<384x512xf32>
      }
    }
    %C_u = memref.cast %C : memref<384x512xf32> to memref<*xf32>
    // CHECK: [ALLCLOSE: TRUE]
    call @printAllcloseF32(%C_u, %C_ref_u) : (memref<*xf32>, memref<*xf32>) -> ()
    // the bias must have made a difference: without it the same comparison fails
    // CHECK: [ALLCLOSE: FALSE]
    call @printAllcloseF32(%C2_u, %C_ref_u) : (memref<*xf32>, memref<*xf32>) -> ()
    %row = memref.subview %C_ref[0, 0][1, 512][1, 1] : memref<384x512xf32> to memref<1x512xf32, strided<[512, 1], offset: 0>>
    %row_u = memref.cast %row : memref<1x512xf32, strided<[512, 1], offset: 0>> to memref<*xf32>
    // CHECK: sizes = [1, 512]
    call @printMemrefF32(%row_u) : (memref<*xf32>) -> ()
    vector.print str "done\n"
    // CHECK: done
    memref.dealloc %A : memref<384x256xf16>
    return
  }
  func.func private @printMemrefF32(memref<*xf32>) attributes {llvm.emit_c_interface}
  func.func private @printAllcloseF32(memref<*xf32>, memref<*xf32>) attributes {llvm.emit_c_interface}
  func.func private @fillResource1DRandomF16(memref<*xf16>, f32, f32, i1) attributes {llvm.emit_c_interface}
  func.func private @fillResource1DRandomF32(memref<*xf32>, f32, f32, i1) attributes {llvm.emit_c_interface}
  func.func private @gemmF16F16F32(memref<*xf16>, memref<*xf16>, memref<*xf32>) attributes {llvm.emit_c_interface}
}
