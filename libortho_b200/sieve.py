"""Producers of the layer's inputs (not on the hot path): host-side torch code, and for FP32 weights that
already live on the GPU the device-side sieve (``csrc/sieve.cu``) with bit-identical results.

Same call surface as the reference's ``tools/sieve.py`` so that callers can switch imports:
``quantize_int4`` (``tools/sieve.py:13-23``), ``hessian_sieve`` (``:25-76``),
``compute_hessian_diag_approx`` (``:79-95``) and ``pack_ortho_sparse`` (``:98-177``).  The CSR
contract -- unique coordinates, row-major order, int32 indices, ``row_ptr`` of length N+1 -- is
what the kernels and the plan rely on.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def quantize_int4(weight: torch.Tensor) -> torch.Tensor:
    """Per-output-row symmetric INT4 fake-quantisation: scale = rowmax|w| / 7 (floored at
    1e-8 / 7), round to nearest even, clamp to [-8, 7], multiply back; non-finite results
    become zero."""
    amax = weight.abs().amax(dim=1, keepdim=True).clamp(min=1e-8)
    scale = amax / 7.0
    deq = torch.clamp(torch.round(weight / scale), -8, 7) * scale
    return torch.where(torch.isfinite(deq), deq, torch.zeros_like(deq))


def hessian_sieve(weight: torch.Tensor, H_inv: torch.Tensor, curvature_thresh: float = 10.0,
                  sparsity_target: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Splits ``weight`` [N,K] into the quantised base and the sparse residual.

    score = residual^2 / (diag(H_inv) + 1e-6), broadcast over rows; a 2-D ``H_inv`` is reduced
    to its diagonal.  The residual is kept where score > threshold, the threshold being
    ``curvature_thresh`` or, when ``sparsity_target`` is given, the k-th largest score with
    k = int(sparsity_target * numel) ("keep the top fraction"; k == 0 keeps nothing)."""
    d = torch.diag(H_inv) if H_inv.dim() > 1 else H_inv
    if weight.is_cuda and weight.dtype == torch.float32 and weight.dim() == 2 and weight.shape[1] % 4 == 0:
        # weights already on the GPU: the device-side sieve produces the same bits as the chain below
        from . import _C_ops
        k = -1 if sparsity_target is None else int(sparsity_target * weight.numel())
        return _C_ops.hessian_sieve(weight, d, curvature_thresh, k)
    w_base = quantize_int4(weight)
    residual = weight - w_base
    score = residual.pow(2) / (d + 1e-6).unsqueeze(0)
    if sparsity_target is None:
        thresh = curvature_thresh
    else:
        k = int(sparsity_target * score.numel())
        thresh = torch.topk(score.flatten(), k).values[-1] if k > 0 else score.max() + 1.0
    return w_base, residual * (score > thresh)


def compute_hessian_diag_approx(inputs: torch.Tensor, outputs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """diag(X^T X) / n + 1e-6 for calibration inputs X [n, K]."""
    return inputs.pow(2).sum(dim=0) / inputs.shape[0] + 1e-6


def pack_ortho_sparse(w_ortho: torch.Tensor, format: str = "csr"):
    """CSR: ``(row_ptr int32 [N+1], col_indices int32 [nnz], values [nnz])`` in row-major order.
    COO (legacy): ``(flat uint16 indices, values, None)``; only meaningful while N*K <= 65536."""
    if format not in ("csr", "coo"):
        raise ValueError(f"Unsupported format: {format}. Use 'csr' or 'coo'")
    n_rows, n_cols = w_ortho.shape
    # torch.nonzero walks a contiguous tensor in row-major order, which is the required order
    coords = torch.nonzero(w_ortho != 0, as_tuple=False)
    rows, cols = coords[:, 0], coords[:, 1]
    values = w_ortho[rows, cols]
    if format == "coo":
        return (rows * n_cols + cols).to(torch.uint16), values, None
    counts = torch.bincount(rows, minlength=n_rows)
    row_ptr = torch.zeros(n_rows + 1, dtype=torch.int32, device=w_ortho.device)
    row_ptr[1:] = torch.cumsum(counts, dim=0).to(torch.int32)
    return row_ptr, cols.to(torch.int32), values
