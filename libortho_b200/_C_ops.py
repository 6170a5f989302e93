"""Function-level operator with the signature of the reference binding.

``forward(q_weight, q_scales, ortho_values, ortho_col_indices, ortho_row_ptr, input, output,
alpha) -> None`` writes ``output`` in place, like ``libortho._C_ops.forward`` declared in
``torch_bind/bindings.cpp:9-18,46-49`` and called from ``torch_bind/ortho_linear.py:142-151``.
Differences, all deliberate: the buffers really are FP16 (the reference binding asks for
``float*`` from FP16 tensors and cannot run), the call is asynchronous on the current CUDA
stream, and any failure raises instead of being dropped.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib


class Plan:
    """Owns one ``ortho_b200_plan`` (GPU-side re-layout of a layer's CSR ortho component)."""

    def __init__(self, row_ptr: torch.Tensor, col_indices: torch.Tensor, values: torch.Tensor,
                 in_features: int, out_features: int):
        import ctypes
        self._h = ctypes.c_void_p()
        nnz = int(values.numel())
        if nnz:
            assert row_ptr.is_cuda and col_indices.is_cuda and values.is_cuda
            assert row_ptr.dtype == torch.int32 and col_indices.dtype == torch.int32
            assert values.dtype == torch.float16
            assert row_ptr.numel() == out_features + 1 and col_indices.numel() == nnz
            row_ptr, col_indices, values = row_ptr.contiguous(), col_indices.contiguous(), values.contiguous()
        dev = values.device if nnz else torch.device("cuda", torch.cuda.current_device())
        with torch.cuda.device(dev):
            st = _lib.lib().ortho_b200_plan_create(
                ctypes.byref(self._h),
                row_ptr.data_ptr() if nnz else None, col_indices.data_ptr() if nnz else None,
                values.data_ptr() if nnz else None, nnz, in_features, out_features,
                torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(st, "ortho_b200_plan_create")
        self.nnz = nnz
        self.device = dev
        self.in_features, self.out_features = in_features, out_features

    @property
    def handle(self):
        return self._h

    @property
    def max_row_nnz(self) -> int:
        return int(_lib.lib().ortho_b200_plan_max_row_nnz(self._h))

    @property
    def rows_ordered(self) -> bool:
        """Every row lists its columns in ascending order (then the tensor-core kernels fold the entries into their
        weight tiles instead of gathering them)."""
        return int(_lib.lib().ortho_b200_plan_rows_ordered(self._h)) == 1

    def decode_dump(self):
        """(rows, cols, values) of every stored entry, decoded on the GPU from the plan."""
        rows = torch.empty(self.nnz, dtype=torch.int32, device=self.device)
        cols = torch.empty(self.nnz, dtype=torch.int32, device=self.device)
        vals = torch.empty(self.nnz, dtype=torch.float16, device=self.device)
        with torch.cuda.device(self.device):
            st = _lib.lib().ortho_b200_plan_decode_dump(
                self._h, rows.data_ptr(), cols.data_ptr(), vals.data_ptr(),
                torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(st, "ortho_b200_plan_decode_dump")
        return rows, cols, vals

    def close(self):
        if self._h is not None and self._h.value:
            _lib.lib().ortho_b200_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def workspace_bytes(M: int, K: int, N: int, plan: Optional["Plan"] = None) -> int:
    if plan is not None:
        return int(_lib.lib().ortho_b200_plan_workspace_bytes(plan.handle, M))
    return int(_lib.lib().ortho_b200_workspace_bytes(M, K, N))


def dequant_dump(q_weight: torch.Tensor, q_scales: torch.Tensor):
    """(w_int int8 [N,K], w_deq float32 [N,K]) produced by the kernels' own INT4 unpack."""
    assert q_weight.is_cuda and q_weight.dtype == torch.uint8 and q_scales.dtype == torch.float16
    q_weight, q_scales = q_weight.contiguous(), q_scales.contiguous()
    N, kh = q_weight.shape
    wi = torch.empty(N, kh * 2, dtype=torch.int8, device=q_weight.device)
    wd = torch.empty(N, kh * 2, dtype=torch.float32, device=q_weight.device)
    with torch.cuda.device(q_weight.device):
        st = _lib.lib().ortho_b200_dequant_dump(
            q_weight.data_ptr(), q_scales.data_ptr(), N, kh * 2, wi.data_ptr(), wd.data_ptr(),
            torch.cuda.current_stream(q_weight.device).cuda_stream)
    _lib.check(st, "ortho_b200_dequant_dump")
    return wi, wd


def forward(q_weight: torch.Tensor, q_scales: torch.Tensor, ortho_values: torch.Tensor,
            ortho_col_indices: torch.Tensor, ortho_row_ptr: torch.Tensor,
            input: torch.Tensor, output: torch.Tensor, alpha: float,
            plan: Optional[Plan] = None, workspace: Optional[torch.Tensor] = None) -> None:
    """In-place ``output[M,N] = input[M,K] @ dequant(q_weight)^T + alpha * input @ W_ortho^T``."""
    if not input.is_cuda:
        raise RuntimeError("libortho_b200 has no CPU path: `input` must be a CUDA tensor")
    if input.dtype != torch.float16 or output.dtype != torch.float16:
        raise TypeError("input and output must be float16")
    if q_weight.dtype != torch.uint8 or q_scales.dtype != torch.float16:
        raise TypeError("q_weight must be uint8 (packed INT4) and q_scales float16")
    if input.dim() != 2 or output.dim() != 2 or not input.is_contiguous() or not output.is_contiguous():
        raise ValueError("input [M,K] and output [M,N] must be contiguous 2-D tensors")
    M, K = input.shape
    N = output.shape[1]
    if output.shape[0] != M or tuple(q_weight.shape) != (N, K // 2) or q_scales.numel() != N:
        raise ValueError("shape mismatch between q_weight/q_scales/input/output")
    dev = input.device
    for t in (q_weight, q_scales, output):
        if t.device != dev:
            raise RuntimeError("all tensors must live on the input's device")
    nnz = int(ortho_values.numel()) if ortho_values is not None else 0
    if nnz and plan is None:
        if (ortho_values.dtype != torch.float16 or ortho_col_indices.dtype != torch.int32
                or ortho_row_ptr.dtype != torch.int32):
            raise TypeError("ortho buffers must be float16 / int32 / int32")
        if ortho_row_ptr.numel() != N + 1 or ortho_col_indices.numel() != nnz:
            raise ValueError("CSR arrays have inconsistent sizes")
    # scratch of the tensor-core regimes (sparse pre-pass, partial sums of split tiles); 0 for the streaming kernels
    need = workspace_bytes(M, K, N, plan)
    ws_ptr, ws_bytes = None, 0
    if need:
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    with torch.cuda.device(dev):
        st = _lib.lib().ortho_b200_forward(
            q_weight.data_ptr(), q_scales.data_ptr(),
            ortho_values.data_ptr() if nnz else None,
            ortho_col_indices.data_ptr() if nnz else None,
            ortho_row_ptr.data_ptr() if nnz else None, nnz,
            input.data_ptr(), output.data_ptr(), M, K, N, float(alpha),
            plan.handle if plan is not None else None, ws_ptr, ws_bytes,
            torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "ortho_b200_forward")


def forward_multi(layers, input: torch.Tensor, outputs, alphas=None, biases=None, plans=None,
                  workspace: Optional[torch.Tensor] = None) -> None:
    """Several layers that read the same ``input`` [M, K] (separate Q / K / V or gate / up projections), each
    with its own alpha and an optional FP32 bias fused into the kernel: ``layers`` is a sequence of
    ``(q_weight, q_scales, ortho_values, ortho_col_indices, ortho_row_ptr)`` tuples, ``outputs`` the matching
    FP16 ``[M, N_l]`` tensors written in place.  Up to 16 tokens (K a multiple of 256) run as ONE kernel launch."""
    n = len(layers)
    if n == 0:
        return
    if n > 4:
        raise ValueError("at most 4 layers per call")
    if not input.is_cuda:
        raise RuntimeError("libortho_b200 has no CPU path: `input` must be a CUDA tensor")
    if input.dtype != torch.float16 or input.dim() != 2 or not input.is_contiguous():
        raise TypeError("input must be a contiguous float16 [M, K] tensor")
    M, K = input.shape
    dev = input.device
    descs = (_lib.LayerDesc * n)()
    keep = []
    for i, (qw, qs, ov, oc, orp) in enumerate(layers):
        y = outputs[i]
        N = y.shape[1]
        if (qw.dtype != torch.uint8 or qs.dtype != torch.float16 or y.dtype != torch.float16 or not y.is_contiguous()
                or tuple(qw.shape) != (N, K // 2) or qs.numel() != N or y.shape[0] != M):
            raise ValueError(f"layer {i}: dtype or shape mismatch")
        nnz = int(ov.numel()) if ov is not None else 0
        plan = plans[i] if plans is not None else None
        if nnz and plan is None and (ov.dtype != torch.float16 or oc.dtype != torch.int32 or orp.dtype != torch.int32
                                     or orp.numel() != N + 1 or oc.numel() != nnz):
            raise ValueError(f"layer {i}: CSR arrays have inconsistent dtypes or sizes")
        b = biases[i] if biases is not None else None
        if b is not None:
            if b.dtype != torch.float32 or b.numel() != N or not b.is_contiguous() or b.device != dev:
                raise ValueError(f"layer {i}: bias must be a contiguous float32 [N] tensor on the input's device")
            keep.append(b)
        d = descs[i]
        d.q_weight, d.q_scales_f16 = qw.data_ptr(), qs.data_ptr()
        d.ortho_values_f16 = ov.data_ptr() if nnz else None
        d.ortho_col_indices = oc.data_ptr() if nnz else None
        d.ortho_row_ptr = orp.data_ptr() if nnz else None
        d.nnz = nnz
        d.plan = plan.handle if plan is not None else None
        d.bias_f32 = b.data_ptr() if b is not None else None
        d.y_f16, d.N, d.ldy = y.data_ptr(), N, 0
        d.alpha = float(alphas[i]) if alphas is not None else 1.0
        d.reserved = 0
    need = int(_lib.lib().ortho_b200_multi_workspace_bytes(descs, n, M, K))
    ws_ptr, ws_bytes = None, 0
    if need > 0:
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    with torch.cuda.device(dev):
        st = _lib.lib().ortho_b200_forward_multi(descs, n, input.data_ptr(), M, K, ws_ptr, ws_bytes,
                                                 torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "ortho_b200_forward_multi")


COMM_HANDLE_BYTES = 64


class _DevicePtr:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


class Comm:
    """Peer-mapped output buffer of one rank (``ortho_b200_comm_*``).

    ``exchange`` is a callable that takes this rank's handle (``bytes``) and returns the list of all
    ranks' handles in rank order; ``Comm.connect_group`` does it with ``torch.distributed``."""

    def __init__(self, rank: int, world: int, nbytes: int, device=None):
        self.rank, self.world, self.nbytes = rank, world, int(nbytes)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ortho_b200_comm_create(rank, world, self.nbytes, ctypes.byref(h)), "ortho_b200_comm_create")
        self.handle = h
        self._buffer = None

    def export(self) -> bytes:
        buf = ctypes.create_string_buffer(COMM_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ortho_b200_comm_export(self.handle, buf), "ortho_b200_comm_export")
        return bytes(buf.raw)

    def connect(self, handles) -> None:
        if len(handles) != self.world or any(len(h) != COMM_HANDLE_BYTES for h in handles):
            raise ValueError("need one 64-byte handle per rank, in rank order")
        blob = ctypes.create_string_buffer(b"".join(handles), COMM_HANDLE_BYTES * self.world)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ortho_b200_comm_connect(self.handle, blob), "ortho_b200_comm_connect")

    def connect_group(self, group=None) -> None:
        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, self.export(), group=group)
        self.connect(handles)
        dist.barrier(group=group)

    def set_timeout_ms(self, ms: int) -> None:
        _lib.check(_lib.lib().ortho_b200_comm_set_timeout_ms(self.handle, int(ms)), "ortho_b200_comm_set_timeout_ms")

    def set_deferred(self, on: bool) -> None:
        """Deferred mode: a forward only signals; the next forward on this comm (or ``wait``) waits."""
        _lib.check(_lib.lib().ortho_b200_comm_set_deferred(self.handle, 1 if on else 0), "ortho_b200_comm_set_deferred")

    def wait(self) -> None:
        """Enqueue the wait for the last exchange on the current stream (deferred mode; no-op otherwise)."""
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ortho_b200_comm_wait(self.handle, torch.cuda.current_stream(self.device).cuda_stream),
                       "ortho_b200_comm_wait")

    def buffer(self) -> torch.Tensor:
        """The local buffer as a uint8 tensor (outputs of ``forward_gather`` appear in it)."""
        if self._buffer is None:
            ptr = _lib.lib().ortho_b200_comm_local(self.handle)
            self._buffer = torch.as_tensor(_DevicePtr(int(ptr), self.nbytes, self), device=self.device)
        return self._buffer

    def output(self, offset_bytes: int, M: int, N_total: int) -> torch.Tensor:
        """View of the FP16 ``[M, N_total]`` matrix that starts ``offset_bytes`` into the local buffer."""
        return self.buffer()[offset_bytes: offset_bytes + 2 * M * N_total].view(torch.float16).view(M, N_total)

    def close(self) -> None:
        if self.handle is not None and self.handle.value:
            self._buffer = None
            with torch.cuda.device(self.device):
                _lib.lib().ortho_b200_comm_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def forward_gather(q_weight: torch.Tensor, q_scales: torch.Tensor, ortho_values: torch.Tensor,
                   ortho_col_indices: torch.Tensor, ortho_row_ptr: torch.Tensor,
                   input: torch.Tensor, alpha: float, comm: Comm, y_offset_bytes: int,
                   N_total: int, n_offset: int,
                   plan: Optional[Plan] = None, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """This rank's shard (``q_weight`` ``[N_local, K/2]`` ...) of an N-sharded layer: computes columns
    ``[n_offset, n_offset + N_local)`` and leaves the complete ``[M, N_total]`` output in every rank's
    ``comm`` buffer at ``y_offset_bytes``.  Returns the local view of that output."""
    if not input.is_cuda:
        raise RuntimeError("libortho_b200 has no CPU path: `input` must be a CUDA tensor")
    if input.dtype != torch.float16 or q_weight.dtype != torch.uint8 or q_scales.dtype != torch.float16:
        raise TypeError("input / q_scales must be float16 and q_weight uint8 (packed INT4)")
    if input.dim() != 2 or not input.is_contiguous():
        raise ValueError("input must be a contiguous [M, K] tensor")
    M, K = input.shape
    N = q_weight.shape[0]
    if N and (tuple(q_weight.shape) != (N, K // 2) or q_scales.numel() != N):
        raise ValueError("shape mismatch between q_weight/q_scales/input")
    dev = input.device
    nnz = int(ortho_values.numel()) if ortho_values is not None else 0
    need = workspace_bytes(M, K, N, plan) if N else 0
    ws_ptr, ws_bytes = None, 0
    if need:
        if workspace is None or workspace.numel() * workspace.element_size() < need:
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    with torch.cuda.device(dev):
        st = _lib.lib().ortho_b200_forward_gather(
            q_weight.data_ptr() if N else None, q_scales.data_ptr() if N else None,
            ortho_values.data_ptr() if nnz else None,
            ortho_col_indices.data_ptr() if nnz else None,
            ortho_row_ptr.data_ptr() if nnz else None, nnz,
            input.data_ptr(), M, K, N, float(alpha),
            plan.handle if plan is not None else None, ws_ptr, ws_bytes,
            comm.handle, int(y_offset_bytes), int(N_total), int(n_offset),
            torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "ortho_b200_forward_gather")
    return comm.output(y_offset_bytes, M, N_total)


def pack_base(weight: torch.Tensor, scales: Optional[torch.Tensor] = None):
    """Device-side INT4 quantise + pack of an FP32 ``[N, K]`` CUDA tensor: ``(q_weight u8 [N, K/2],
    q_scales f16 [N])``, bit-identical to the torch chain of ``OrthoLinear.load_from_weights``."""
    if not weight.is_cuda or weight.dtype != torch.float32 or weight.dim() != 2:
        raise TypeError("weight must be a 2-D float32 CUDA tensor")
    w = weight.contiguous()
    N, K = w.shape
    dev = w.device
    s_in = None
    if scales is not None:
        s_in = scales.to(device=dev, dtype=torch.float32).contiguous()
        if s_in.numel() != N:
            raise ValueError("scales must have one entry per output row")
    q = torch.empty(N, K // 2, dtype=torch.uint8, device=dev)
    qs = torch.empty(N, dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        st = _lib.lib().ortho_b200_pack_base(w.data_ptr(), N, K, s_in.data_ptr() if s_in is not None else None,
                                             q.data_ptr(), qs.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "ortho_b200_pack_base")
    return q, qs


def pack_ortho_csr(w_ortho: torch.Tensor):
    """Device-side CSR build of an FP32 ``[N, K]`` CUDA tensor: ``(row_ptr i32 [N+1], col i32 [nnz],
    values f16 [nnz])`` in row-major order (one host read of nnz between the two passes)."""
    if not w_ortho.is_cuda or w_ortho.dtype != torch.float32 or w_ortho.dim() != 2:
        raise TypeError("w_ortho must be a 2-D float32 CUDA tensor")
    w = w_ortho.contiguous()
    N, K = w.shape
    dev = w.device
    row_ptr = torch.empty(N + 1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(_lib.lib().ortho_b200_csr_count(w.data_ptr(), N, K, row_ptr.data_ptr(), stream), "ortho_b200_csr_count")
        nnz = int(row_ptr[N].item())
        col = torch.empty(nnz, dtype=torch.int32, device=dev)
        val = torch.empty(nnz, dtype=torch.float16, device=dev)
        if nnz:
            _lib.check(_lib.lib().ortho_b200_csr_fill(w.data_ptr(), N, K, row_ptr.data_ptr(), col.data_ptr(), val.data_ptr(),
                                                     stream), "ortho_b200_csr_fill")
    return row_ptr, col, val


def hessian_sieve(weight: torch.Tensor, h_inv_diag: torch.Tensor, curvature_thresh: float = 10.0,
                  keep_top_k: int = -1):
    """Device-side Hessian sieve of an FP32 ``[N, K]`` CUDA tensor: ``(w_base, w_ortho)`` FP32 ``[N, K]``,
    bit-identical to the torch chain of ``libortho_b200.sieve.hessian_sieve``.  ``keep_top_k < 0`` uses the
    curvature threshold, otherwise the ``keep_top_k``-th largest score is the threshold."""
    if not weight.is_cuda or weight.dtype != torch.float32 or weight.dim() != 2:
        raise TypeError("weight must be a 2-D float32 CUDA tensor")
    w = weight.contiguous()
    N, K = w.shape
    dev = w.device
    h = h_inv_diag.to(device=dev, dtype=torch.float32).contiguous()
    if h.dim() != 1 or h.numel() != K:
        raise ValueError("h_inv_diag must hold one entry per input feature")
    wb, wo = torch.empty_like(w), torch.empty_like(w)
    need = int(_lib.lib().ortho_b200_sieve_scratch_bytes(N))
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        st = _lib.lib().ortho_b200_sieve(w.data_ptr(), h.data_ptr(), N, K, float(curvature_thresh), int(keep_top_k),
                                        wb.data_ptr(), wo.data_ptr(), scratch.data_ptr(), need,
                                        torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(st, "ortho_b200_sieve")
    return wb, wo
