"""Import shim: ``from torch_bind.ortho_linear import OrthoLinear`` (the reference's import path,
``README.md:76-84``) resolves to the B200 implementation."""
from libortho_b200.ortho_linear import OrthoLinear  # noqa: F401

__all__ = ["OrthoLinear"]
