"""N-sharded OrthoLinear: each rank holds a contiguous slice of output rows, only Y is exchanged.

Output rows are independent (every ``y[m, n]`` depends on weight row ``n`` alone,
``src/ortho.c:354-366,389-396`` in the reference), so rank ``g`` of ``G`` keeps rows
``[n0, n1)``: a contiguous byte slice of ``base_weight``, the matching slice of ``base_scales`` and
the CSR rows with ``row_ptr`` rebased to 0.  ``X`` is replicated.  The only collective is the
all-gather of the ``[M, N/G]`` output shards into ``[M, N]`` (NCCL on GPUs; any backend works).
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

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        M = x2.shape[0]
        rows = self.n1 - self.n0
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
