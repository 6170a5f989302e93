"""Import shim for the reference's module path ``torch_bind.ortho_linear``."""
from libortho_b200.ortho_linear import OrthoLinear  # noqa: F401

HAS_C_OPS = True

__all__ = ["OrthoLinear", "HAS_C_OPS"]
