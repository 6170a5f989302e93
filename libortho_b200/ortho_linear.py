"""``OrthoLinear`` -- drop-in for the reference module of the same name.

Mirrors ``torch_bind/ortho_linear.py:30-168``: same constructor, the same registered buffers
(``base_weight`` u8 [N, K//2], ``base_scales`` f16 [N], ``ortho_values`` f16 [nnz],
``ortho_col_indices`` i32 [nnz], ``ortho_row_ptr`` i32 [N+1]; the three ortho buffers are
zero-length until weights are loaded), the plain ``alpha`` attribute (default 1.0, not part of
the ``state_dict``), ``set_alpha``, ``load_from_weights`` and ``forward``.

Differences, all deliberate:
* the forward runs the sm_100a kernels through the C ABI; a non-CUDA input raises (the reference
  returns uninitialised memory on that branch, ``ortho_linear.py:152-162``);
* the GPU-side re-layout of the sparse component (the plan) and the tensor-core workspace are
  non-persistent caches rebuilt on the first forward after the buffers change;
* ``load_state_dict`` accepts ortho buffers of any length (the reference's zero-length
  placeholders would otherwise reject every saved layer).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _C_ops as _C
from .sieve import pack_ortho_sparse

_ORTHO_BUFFERS = ("ortho_values", "ortho_col_indices", "ortho_row_ptr")


class OrthoLinear(nn.Module):
    """Y = X . dequant(W_base)^T + alpha . X . W_ortho^T with ``alpha`` as the kill switch."""

    def __init__(self, in_features: int, out_features: int, q_bits: int = 4, bias: bool = False,
                 device=None, dtype=None):
        super().__init__()
        if q_bits != 4:
            raise ValueError("only q_bits=4 is supported")
        self.in_features = in_features
        self.out_features = out_features
        self.q_bits = q_bits
        self.register_buffer("base_weight", torch.zeros(out_features, in_features // 2, dtype=torch.uint8, device=device))
        self.register_buffer("base_scales", torch.zeros(out_features, dtype=torch.float16, device=device))
        self.register_buffer("ortho_values", torch.tensor([], dtype=torch.float16, device=device))
        self.register_buffer("ortho_col_indices", torch.tensor([], dtype=torch.int32, device=device))
        self.register_buffer("ortho_row_ptr", torch.tensor([], dtype=torch.int32, device=device))
        self.alpha = 1.0
        if bias:
            self.register_parameter("bias", nn.Parameter(torch.zeros(out_features, dtype=dtype or torch.float32, device=device)))
        else:
            self.register_parameter("bias", None)
        self._plan: Optional[_C.Plan] = None
        self._plan_key = None
        self._ws_need = {}
        self._workspace: Optional[torch.Tensor] = None

    def set_alpha(self, alpha: float):
        self.alpha = alpha

    # -- packing (host-side torch code; follows ortho_linear.py:79-128) -------------------------
    def load_from_weights(self, base_weight: torch.Tensor, ortho_weight: torch.Tensor,
                          base_scales: Optional[torch.Tensor] = None):
        """Quantises ``base_weight`` [N,K] to packed INT4 and packs ``ortho_weight`` [N,K] as CSR.

        scales = rowmax|W| / 7 floored at 1e-6 unless given; w_int = round-half-even(W / scale)
        clamped to [-8, 7], the division using the FP32 scale while the stored scale is FP16;
        two elements per byte, even flat index in the low nibble."""
        device = ortho_weight.device
        if (base_weight.is_cuda and ortho_weight.is_cuda and base_weight.dtype == torch.float32
                and ortho_weight.dtype == torch.float32 and self.in_features % 8 == 0):
            # weights already on the GPU: the device-side packer produces the same bits as the chain below
            self.base_weight.data, self.base_scales.data = _C.pack_base(base_weight, base_scales)
            self.ortho_row_ptr, self.ortho_col_indices, self.ortho_values = _C.pack_ortho_csr(ortho_weight)
            self._invalidate()
            return
        if base_scales is None:
            scales = (base_weight.abs().max(dim=1)[0] / 7.0).clamp(min=1e-6)
        else:
            scales = base_scales
        self.base_scales.data = scales.to(dtype=torch.float16, device=device)
        w_int = (base_weight / scales.unsqueeze(1)).round().clamp(-8, 7).to(torch.int8)
        flat = w_int.flatten()
        if flat.numel() % 2 != 0:
            flat = torch.cat([flat, torch.zeros(1, dtype=torch.int8, device=flat.device)])
        packed = ((flat[0::2] & 0x0F) | ((flat[1::2] & 0x0F) << 4)).to(torch.uint8)
        self.base_weight.data = packed.view(self.out_features, -1).to(device)
        row_ptr, col_indices, values = pack_ortho_sparse(ortho_weight, format="csr")
        self.ortho_row_ptr = row_ptr.to(device=device, dtype=torch.int32)
        self.ortho_col_indices = col_indices.to(device=device, dtype=torch.int32)
        self.ortho_values = values.to(device=device, dtype=torch.float16)
        self._invalidate()

    # -- caches ----------------------------------------------------------------------------------
    def _invalidate(self):
        self._plan = None
        self._plan_key = None
        self._ws_need = {}

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        self._invalidate()
        self._workspace = None
        return out

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        for name in _ORTHO_BUFFERS:
            key = prefix + name
            if key in state_dict:
                cur = getattr(self, name)
                src = state_dict[key]
                if cur.shape != src.shape:
                    setattr(self, name, torch.empty(src.shape, dtype=cur.dtype, device=cur.device))
        self._invalidate()
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def _get_plan(self) -> Optional[_C.Plan]:
        nnz = int(self.ortho_values.numel())
        if nnz == 0:
            return None
        key = (self.ortho_values.data_ptr(), self.ortho_col_indices.data_ptr(),
               self.ortho_row_ptr.data_ptr(), nnz, self.ortho_values._version,
               self.ortho_col_indices._version, self.ortho_row_ptr._version)
        if self._plan is None or self._plan_key != key:
            self._plan = _C.Plan(self.ortho_row_ptr, self.ortho_col_indices, self.ortho_values,
                                 self.in_features, self.out_features)
            self._plan_key = key
            self._ws_need = {}
        return self._plan

    def _get_workspace(self, M: int) -> Optional[torch.Tensor]:
        sparse = self.alpha > 0 and self.ortho_values.numel() > 0
        if not sparse and M <= 24:
            return None
        plan = self._get_plan() if sparse else None
        key = (M, id(plan))
        need = self._ws_need.get(key)
        if need is None:                       # one size query per (token count, plan), not per forward
            need = _C.workspace_bytes(M, self.in_features, self.out_features, plan)
            if len(self._ws_need) > 64:
                self._ws_need.clear()
            self._ws_need[key] = need
        if need == 0:
            return None
        if (self._workspace is None or self._workspace.numel() < need
                or self._workspace.device != self.base_weight.device):
            self._workspace = torch.empty(need, dtype=torch.uint8, device=self.base_weight.device)
        return self._workspace

    # -- forward ---------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("OrthoLinear (libortho_b200) runs on CUDA only; there is no CPU fallback")
        original_shape = x.shape
        x_flat = x.reshape(-1, self.in_features)
        if x_flat.dtype != torch.float16:
            x_flat = x_flat.to(torch.float16)
        x_flat = x_flat.contiguous()
        M = x_flat.shape[0]
        output = torch.empty(M, self.out_features, device=x.device, dtype=torch.float16)
        if M:
            _C.forward(self.base_weight, self.base_scales, self.ortho_values, self.ortho_col_indices,
                       self.ortho_row_ptr, x_flat, output, self.alpha,
                       plan=self._get_plan() if self.alpha > 0 else None,
                       workspace=self._get_workspace(M))
        if self.bias is not None:
            output += self.bias
        if output.dtype != x.dtype:
            output = output.to(x.dtype)
        return output.view(*original_shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, q_bits={self.q_bits}, "
                f"nnz={self.ortho_values.numel()}, alpha={self.alpha}, bias={self.bias is not None}")
