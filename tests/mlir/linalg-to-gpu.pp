// Pipeline file in the reference's .pp format; names the reference's GPU
// pipeline stages this runner stands in for (benchmarks/pipelines/linalg-to-gpu.pp).
builtin.module(
    func.func(convert-linalg-to-parallel-loops)
    func.func(imex-add-outer-parallel-loop)
    insert-gpu-allocs{client-api=opencl}
    gpu-kernel-outlining
    convert-gpu-to-gpux
    convert-gpux-to-llvm)
// End
