"""libortho_b200 -- the OrthoLinear forward for NVIDIA B200 (sm_100a).

One operator: ``Y = X . dequant(W_base_int4)^T + alpha . X . W_ortho^T`` behind the reference's
``OrthoLinear`` / ``set_alpha`` API, executed by hand-written CUDA kernels reached through a
C ABI (``include/ortho_b200.h``).  Importing the package does not load the CUDA library; the
first operator call does, and fails loudly if it has not been built.
"""
from .ortho_linear import OrthoLinear  # noqa: F401
from . import _C_ops  # noqa: F401
from .convert import set_alpha_all, swap_linear  # noqa: F401

__all__ = ["OrthoLinear", "_C_ops", "swap_linear", "set_alpha_all"]
__version__ = "0.1.0"
