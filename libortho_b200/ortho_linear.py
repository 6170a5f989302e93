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
from . import _lib
from .sieve import pack_ortho_sparse

# raw handle of the current stream without building a torch.cuda.Stream object per call
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _current_stream_handle(dev: torch.device) -> int:
    if _raw_stream is not None:
        return _raw_stream(dev.index)
    return torch.cuda.current_stream(dev).cuda_stream

_ORTHO_BUFFERS = ("ortho_values", "ortho_col_indices", "ortho_row_ptr")
_WATCHED = frozenset(("base_weight", "base_scales", "bias") + _ORTHO_BUFFERS)


class _SharedWorkspace:
    """One grow-on-demand scratch buffer per device, shared by every module on it (a model with hundreds of
    layers runs them one at a time).  Forwards that use it must be issued on one stream at a time."""
    _by_device = {}

    def __init__(self):
        self.tensor: Optional[torch.Tensor] = None
        self.gen = 0

    @classmethod
    def get(cls, device: torch.device, nbytes: int) -> "_SharedWorkspace":
        w = cls._by_device.get(device)
        if w is None:
            w = cls._by_device[device] = cls()
        if nbytes > 0 and (w.tensor is None or w.tensor.numel() < nbytes):
            w.tensor = torch.empty(nbytes, dtype=torch.uint8, device=device)
            w.gen += 1
        return w


class _Bound:
    """Everything about one (module, token count) forward that does not change from call to call: the C
    argument record with all buffer pointers, the plan, the workspace.  Built (and validated) once."""
    __slots__ = ("descs", "ws", "ws_gen", "ws_ptr", "ws_bytes", "key", "fused_bias")


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
        self._bound = {}

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
        self._bound = {}

    def __setattr__(self, name, value):
        super().__setattr__(name, value)
        if name in _WATCHED and "_bound" in self.__dict__:     # a buffer was replaced: cached pointers are stale
            self._invalidate()

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        self._invalidate()
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

    def _workspace_bytes(self, M: int) -> int:
        sparse = self.alpha > 0 and self.ortho_values.numel() > 0
        plan = self._get_plan() if sparse else None
        key = (M, id(plan))
        need = self._ws_need.get(key)
        if need is None:                       # one size query per (token count, plan), not per forward
            need = _C.workspace_bytes(M, self.in_features, self.out_features, plan)
            if len(self._ws_need) > 64:
                self._ws_need.clear()
            self._ws_need[key] = need
        return need

    def _get_workspace(self, M: int) -> Optional[torch.Tensor]:
        """The device's shared scratch buffer, grown to what a forward of M tokens needs (None if nothing)."""
        need = self._workspace_bytes(M)
        if need == 0:
            return None
        return _SharedWorkspace.get(self.base_weight.device, need).tensor

    def _versions(self):
        """What a cached call record depends on besides the token count: the storage of every buffer (a
        ``.data =`` assignment swaps it without going through ``__setattr__``) and the contents of the CSR
        buffers (in-place edits show up in their version counters)."""
        ov, oc, orp, b = self.ortho_values, self.ortho_col_indices, self.ortho_row_ptr, self.bias
        return (self.base_weight.data_ptr(), self.base_scales.data_ptr(), ov.data_ptr(), oc.data_ptr(), orp.data_ptr(),
                ov._version, oc._version, orp._version, (b.data_ptr(), b.dtype) if b is not None else None)

    def _bind(self, M: int, dev: torch.device) -> _Bound:
        N, K = self.out_features, self.in_features
        bw, bs = self.base_weight, self.base_scales
        if bw.dtype != torch.uint8 or bs.dtype != torch.float16:
            raise TypeError("base_weight must be uint8 (packed INT4) and base_scales float16")
        if tuple(bw.shape) != (N, K // 2) or bs.numel() != N or not bw.is_contiguous() or not bs.is_contiguous():
            raise ValueError("base_weight / base_scales do not match (out_features, in_features // 2) / (out_features,)")
        nnz = int(self.ortho_values.numel())
        sparse = self.alpha > 0 and nnz > 0
        tensors = [bw, bs] + ([self.ortho_values, self.ortho_col_indices, self.ortho_row_ptr] if nnz else [])
        if any(t.device != dev for t in tensors):
            raise RuntimeError("all buffers must live on the input's device")
        if nnz:
            if (self.ortho_values.dtype != torch.float16 or self.ortho_col_indices.dtype != torch.int32
                    or self.ortho_row_ptr.dtype != torch.int32):
                raise TypeError("ortho buffers must be float16 / int32 / int32")
            if self.ortho_row_ptr.numel() != N + 1 or self.ortho_col_indices.numel() != nnz:
                raise ValueError("CSR arrays have inconsistent sizes")
        b = _Bound()
        plan = self._get_plan() if sparse else None
        need = self._workspace_bytes(M)
        b.ws = _SharedWorkspace.get(dev, need)
        b.ws_gen = b.ws.gen
        b.ws_ptr = b.ws.tensor.data_ptr() if need else None
        b.ws_bytes = b.ws.tensor.numel() if need else 0
        b.fused_bias = (self.bias is not None and self.bias.dtype == torch.float32 and self.bias.device == dev
                        and self.bias.is_contiguous())
        descs = (_lib.LayerDesc * 1)()
        d = descs[0]
        d.q_weight, d.q_scales_f16 = bw.data_ptr(), bs.data_ptr()
        d.ortho_values_f16 = self.ortho_values.data_ptr() if nnz else None
        d.ortho_col_indices = self.ortho_col_indices.data_ptr() if nnz else None
        d.ortho_row_ptr = self.ortho_row_ptr.data_ptr() if nnz else None
        d.nnz = nnz
        d.plan = plan.handle if plan is not None else None
        d.bias_f32 = self.bias.data_ptr() if b.fused_bias else None
        d.N, d.ldy, d.reserved = N, 0, 0
        b.descs = descs
        b.key = (self.alpha > 0, self._versions())
        if len(self._bound) > 32:
            self._bound.clear()
        self._bound[M] = b
        return b

    # -- forward ---------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`out` (optional, not in the reference's signature): a contiguous FP16 CUDA tensor of `M * out_features`
        elements that receives the result instead of a fresh allocation, e.g. a slice of a serving loop's
        staging buffer."""
        if not x.is_cuda:
            raise RuntimeError("OrthoLinear (libortho_b200) runs on CUDA only; there is no CPU fallback")
        original_shape = x.shape
        x_flat = x.reshape(-1, self.in_features)
        if x_flat.dtype != torch.float16:
            x_flat = x_flat.to(torch.float16)
        if not x_flat.is_contiguous():
            x_flat = x_flat.contiguous()
        M = x_flat.shape[0]
        dev = x.device
        if out is None:
            output = torch.empty(M, self.out_features, device=dev, dtype=torch.float16)
        else:
            if (out.dtype != torch.float16 or out.device != dev or not out.is_contiguous()
                    or out.numel() != M * self.out_features):
                raise RuntimeError("out must be a contiguous FP16 tensor of M * out_features elements on the input's device")
            output = out.view(M, self.out_features)
        fused_bias = False
        if M:
            alpha = float(self.alpha)
            b = self._bound.get(M)
            if b is None or b.key != (alpha > 0, self._versions()) or b.ws_gen != b.ws.gen:
                b = self._bind(M, dev)
            d = b.descs[0]
            d.y_f16 = output.data_ptr()
            d.alpha = alpha
            fused_bias = b.fused_bias
            fwd = _lib.lib().ortho_b200_forward_multi
            if torch.cuda.current_device() == dev.index:
                st = fwd(b.descs, 1, x_flat.data_ptr(), M, self.in_features, b.ws_ptr, b.ws_bytes, _current_stream_handle(dev))
            else:
                with torch.cuda.device(dev):
                    st = fwd(b.descs, 1, x_flat.data_ptr(), M, self.in_features, b.ws_ptr, b.ws_bytes,
                             _current_stream_handle(dev))
            if st:
                _lib.check(st, "ortho_b200_forward_multi")
        if self.bias is not None and not fused_bias:
            output += self.bias
        if output.dtype != x.dtype:
            output = output.to(x.dtype)
        return output.view(*original_shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, q_bits={self.q_bits}, "
                f"nnz={self.ortho_values.numel()}, alpha={self.alpha}, bias={self.bias is not None}")
