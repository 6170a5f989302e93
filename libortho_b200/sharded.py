"""N-sharded OrthoLinear: each rank holds a contiguous slice of output rows, only Y is exchanged.

Output rows are independent (every ``y[m, n]`` depends on weight row ``n`` alone,
``src/ortho.c:354-366,389-396`` in the reference), so rank ``g`` of ``G`` keeps rows
``[n0, n1)``: a contiguous byte slice of ``base_weight``, the matching slice of ``base_scales`` and
the CSR rows with ``row_ptr`` rebased to 0.  ``X`` is replicated.  The only collective is the
all-gather of the ``[M, N/G]`` output shards into ``[M, N]``: either one NCCL
``all_gather_into_tensor`` (any backend works), or -- ``enable_peer_gather`` -- the kernels store
their slice straight into every rank's peer-mapped output buffer (``ortho_b200_forward_gather``).
The reference has no multi-device path; this module is what a tensor-parallel caller would use
in its place.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .ortho_linear import OrthoLinear


def shard_bounds(n_rows: int, world: int, align: int = 16) -> List[Tuple[int, int]]:
    """Contiguous row ranges, one per rank, each starting on a multiple of ``align`` rows (the
    kernels' row-tile height) and as equal as that allows; trailing ranks may be empty."""
    units = (n_rows + align - 1) // align
    bounds = []
    for r in range(world):
        u0, u1 = units * r // world, units * (r + 1) // world
        bounds.append((min(u0 * align, n_rows), min(u1 * align, n_rows)))
    return bounds


def slice_rows(base_weight, base_scales, row_ptr, col, vals, n0: int, n1: int):
    """Buffers of the shard [n0, n1) of a layer given by its full buffers."""
    if vals.numel():
        e0, e1 = int(row_ptr[n0]), int(row_ptr[n1])
        rp = (row_ptr[n0:n1 + 1] - e0).to(torch.int32).contiguous()
        c, v = col[e0:e1].contiguous(), vals[e0:e1].contiguous()
    else:
        rp, c, v = row_ptr[:0], col[:0], vals[:0]
    return base_weight[n0:n1].contiguous(), base_scales[n0:n1].contiguous(), rp, c, v


class ShardedOrthoLinear(nn.Module):
    """Holds this rank's shard as an ``OrthoLinear`` and all-gathers the outputs.

    ``local_forward`` (optional) replaces the shard's forward; the CPU test-suite uses it to run the
    host-side sharding and gathering logic under ``gloo`` without a GPU."""

    def __init__(self, in_features: int, out_features: int, group=None, align: int = 16,
                 local_forward: Optional[Callable] = None, device=None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_features, self.out_features = in_features, out_features
        self.bounds = shard_bounds(out_features, self.world, align)
        self.n0, self.n1 = self.bounds[self.rank]
        self.max_rows = max(b - a for a, b in self.bounds)
        self.local = OrthoLinear(in_features, max(self.n1 - self.n0, 0), device=device)
        self._local_forward = local_forward
        self._comm = None
        self._comm_max_m = 0
        self._slot = 0
        self._peer_bound = {}

    @classmethod
    def from_full(cls, full: OrthoLinear, group=None, align: int = 16, local_forward=None) -> "ShardedOrthoLinear":
        m = cls(full.in_features, full.out_features, group, align, local_forward, device=full.base_weight.device)
        bw, bs, rp, c, v = slice_rows(full.base_weight, full.base_scales, full.ortho_row_ptr, full.ortho_col_indices,
                                      full.ortho_values, m.n0, m.n1)
        m.local.base_weight, m.local.base_scales = bw, bs
        m.local.ortho_row_ptr, m.local.ortho_col_indices, m.local.ortho_values = rp, c, v
        m.local.set_alpha(full.alpha)
        return m

    def set_alpha(self, alpha: float):
        self.local.set_alpha(alpha)

    def enable_peer_gather(self, max_tokens: int, comm=None, offset_bytes: int = 0) -> None:
        """Switch the exchange to peer stores.  Allocates (or adopts: ``comm`` at ``offset_bytes``) a
        peer-mapped buffer with two ``[max_tokens, out_features]`` FP16 regions that alternate
        between forwards: a returned output stays valid until the second next forward."""
        from . import _C_ops as _C
        self._region = (2 * max_tokens * self.out_features + 255) // 256 * 256
        if comm is None:
            comm = _C.Comm(self.rank, self.world, 2 * self._region, device=self.local.base_weight.device)
            if self.world > 1:
                comm.connect_group(self.group)
            offset_bytes = 0
        self._comm, self._comm_off, self._comm_max_m = comm, offset_bytes, max_tokens
        self._peer_bound = {}

    @staticmethod
    def peer_gather_bytes(max_tokens: int, out_features: int) -> int:
        return 2 * ((2 * max_tokens * out_features + 255) // 256 * 256)

    def _forward_peer(self, x2: torch.Tensor) -> torch.Tensor:
        """The shard's forward with the peer-store exchange.  Everything that does not change from call to call (buffer
        pointers, plan, workspace, the two output views) is bound once per token count and reused, like
        ``OrthoLinear`` does for its own forward."""
        from . import _C_ops as _C
        from . import _lib
        from .ortho_linear import _SharedWorkspace, _current_stream_handle
        M = x2.shape[0]
        if M > self._comm_max_m:
            raise ValueError(f"peer gather was sized for {self._comm_max_m} tokens, got {M}")
        if not x2.is_cuda:
            raise RuntimeError("libortho_b200 has no CPU path: the input must be a CUDA tensor")
        if x2.dtype != torch.float16:
            x2 = x2.to(torch.float16)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        loc = self.local
        dev = x2.device
        alpha = float(loc.alpha)
        b = self._peer_bound.get(M)
        if b is None or b["key"] != (alpha > 0, loc._versions(), id(self._comm), self._comm_off) or b["ws_gen"] != b["ws"].gen:
            rows = self.n1 - self.n0
            nnz = int(loc.ortho_values.numel())
            if rows and (loc.base_weight.dtype != torch.uint8 or loc.base_scales.dtype != torch.float16
                         or tuple(loc.base_weight.shape) != (rows, self.in_features // 2)):
                raise ValueError("the shard's base_weight / base_scales do not match its rows")
            plan = loc._get_plan() if (alpha > 0 and nnz > 0) else None
            need = _C.workspace_bytes(M, self.in_features, rows, plan) if rows else 0
            ws = _SharedWorkspace.get(dev, need)
            b = {
                "key": (alpha > 0, loc._versions(), id(self._comm), self._comm_off), "ws": ws, "ws_gen": ws.gen,
                "head": (loc.base_weight.data_ptr() if rows else None, loc.base_scales.data_ptr() if rows else None,
                         loc.ortho_values.data_ptr() if nnz else None, loc.ortho_col_indices.data_ptr() if nnz else None,
                         loc.ortho_row_ptr.data_ptr() if nnz else None, nnz),
                "tail": (plan.handle if plan is not None else None, ws.tensor.data_ptr() if need else None,
                         ws.tensor.numel() if need else 0, self._comm.handle),
                "plan": plan,
                "off": [self._comm_off + s * self._region for s in (0, 1)],
                "out": [self._comm.output(self._comm_off + s * self._region, M, self.out_features) for s in (0, 1)],
            }
            if len(self._peer_bound) > 32:
                self._peer_bound.clear()
            self._peer_bound[M] = b
        slot = self._slot
        self._slot ^= 1
        fwd = _lib.lib().ortho_b200_forward_gather
        args = (*b["head"], x2.data_ptr(), M, self.in_features, self.n1 - self.n0, alpha, *b["tail"],
                b["off"][slot], self.out_features, self.n0)
        if torch.cuda.current_device() == dev.index:
            st = fwd(*args, _current_stream_handle(dev))
        else:
            with torch.cuda.device(dev):
                st = fwd(*args, _current_stream_handle(dev))
        if st:
            _lib.check(st, "ortho_b200_forward_gather")
        return b["out"][slot]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        M = x2.shape[0]
        rows = self.n1 - self.n0
        if self._comm is not None and M > 0:
            return self._forward_peer(x2).reshape(*lead, self.out_features)
        if self._local_forward is not None:
            y_local = self._local_forward(self.local, x2)
        elif rows > 0:
            y_local = self.local(x2)
        else:
            y_local = x2.new_zeros(M, 0)
        if self.world == 1:
            return y_local.reshape(*lead, self.out_features)
        # equal-sized slots so that one all_gather_into_tensor moves everything
        slot = y_local
        if rows != self.max_rows:
            slot = y_local.new_zeros(M, self.max_rows)
            slot[:, :rows] = y_local
        flat = slot.new_empty(self.world * M, self.max_rows)        # rank r's slot lands in rows [r*M, (r+1)*M)
        dist.all_gather_into_tensor(flat, slot.contiguous(), group=self.group)
        gathered = flat.view(self.world, M, self.max_rows)
        if all(b - a == self.max_rows for a, b in self.bounds):
            y = gathered.permute(1, 0, 2).reshape(M, self.out_features)      # one strided copy (free for M == 1)
        else:
            y = torch.cat([gathered[r, :, :b - a] for r, (a, b) in enumerate(self.bounds)], dim=1)
        return y.reshape(*lead, self.out_features)
