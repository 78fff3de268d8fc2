"""imex-b200: the IMEX hot path (tiled linalg.matmul + relu/silu epilogue,
row softmax, row reduce-sum, transpose) on NVIDIA B200, behind the
reference's GPU runtime-wrapper C ABI.

The directory name carries a hyphen; load it with

    from __graft_entry__ import load_package
    pkg = load_package()          # registers sys.modules["mlir_extensions_b200"]

Importing it loads lib/libimex_cuda_runtime.so and raises ImportError when
the library has not been built — there is no CPU or PyTorch fallback."""
from . import blob, runtime  # noqa: F401  (runtime raises when the .so is missing)
from .session import Session  # noqa: F401

__all__ = ["blob", "runtime", "Session"]
