"""In-tree build of the native libraries (nvcc for sm_100a, g++ for host code).

    python mlir-extensions_b200/build.py [--force]

Outputs (git-ignored, shipped with the working tree):
    lib/libimex_cuda_runtime.so   GPU runtime-wrapper C ABI + all CUDA kernels
    lib/libimex_runner_utils.so   host runner utilities (fill / print / allclose / ...)
    bin/imex-b200-runner          MLIR-text front end: recognises the hot-path ops and runs them
Objects are rebuilt only when a source or header is newer.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "lib")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include")]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-I" + os.path.join(ROOT, "include")]

RUNTIME_SOURCES = [
    "kernels/gemm_simt.cu",
    "kernels/gemm_tcgen05.cu",
    "kernels/gemm_tcgen05_2cta.cu",
    "kernels/softmax.cu",
    "kernels/reduce.cu",
    "kernels/reduce_all_static.cu",
    "kernels/transpose.cu",
    "kernels/eltwise_fill.cu",
    "kernels/eltwise_expr.cu",
    "kernels/expr_jit.cu",
    "kernels/loopnest_jit.cu",
    "kernels/flash_attention.cu",
    "kernels/wait_selftest.cu",
    "runtime/cuda_runtime_wrappers.cu",
    "runtime/peer_copy.cu",
    "runtime/stats.cpp",
]
UTILS_SOURCES = ["utils/runner_utils.cpp"]
FRONTEND_SOURCES = ["frontend/mlir_text.cpp", "frontend/recognise.cpp", "frontend/loopnest.cpp",
                    "frontend/gpu_kernels.cpp", "frontend/host_loops.cpp", "frontend/runner_main.cpp"]
BIN = os.path.join(PKG, "bin")


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA toolkit is needed to build the sm_100a kernels")


def _headers():
    out = []
    for base in (CSRC, os.path.join(ROOT, "include")):
        for d, _, files in os.walk(base):
            out += [os.path.join(d, f) for f in files if f.endswith((".h", ".cuh", ".hpp"))]
    return out


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def _compile(sources, force, verbose):
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    objs = []
    for rel in sources:
        src = os.path.join(CSRC, rel)
        obj = os.path.join(OBJ, rel.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            if rel.endswith(".cu"):
                _run([_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj], verbose)
            else:
                _run(["/usr/bin/g++"] + CXX_FLAGS + ["-c", src, "-o", obj], verbose)
    return objs


def build(force=False, verbose=False):
    os.makedirs(LIB, exist_ok=True)
    objs = _compile(RUNTIME_SOURCES, force, verbose)
    rt = os.path.join(LIB, "libimex_cuda_runtime.so")
    if force or _stale(rt, objs):
        _run([_nvcc(), "-shared", "-o", rt] + objs + ["-cudart", "static", "-ldl"], verbose)
    if all(os.path.exists(os.path.join(CSRC, s)) for s in UTILS_SOURCES):
        objs = _compile(UTILS_SOURCES, force, verbose)
        ut = os.path.join(LIB, "libimex_runner_utils.so")
        if force or _stale(ut, objs):
            _run(["/usr/bin/g++", "-shared", "-o", ut] + objs, verbose)
    if all(os.path.exists(os.path.join(CSRC, s)) for s in FRONTEND_SOURCES):
        os.makedirs(BIN, exist_ok=True)
        objs = _compile(FRONTEND_SOURCES, force, verbose)
        exe = os.path.join(BIN, "imex-b200-runner")
        if force or _stale(exe, objs + [rt]):
            _run(["/usr/bin/g++", "-o", exe] + objs +
                 ["-L" + LIB, "-limex_cuda_runtime", "-limex_runner_utils",
                  "-Wl,-rpath,$ORIGIN/../lib", "-ldl", "-lpthread"], verbose)
    return rt


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print("built", LIB)
