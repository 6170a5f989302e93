"""N-sharding + all-gather host logic on 2 CPU ranks (gloo).  The shard's compute is the CPU oracle
here (the product has no CPU path); what is under test is the partition, the CSR rebasing and the
gather/reassembly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT
import workloads as wl
from libortho_b200.sharded import ShardedOrthoLinear, shard_bounds, slice_rows


def test_shard_bounds_cover_rows_and_align():
    for n, w in [(4096, 8), (57344, 8), (10240, 4), (50, 2), (17, 4), (16, 8)]:
        b = shard_bounds(n, w)
        assert b[0][0] == 0 and b[-1][1] == n
        assert all(b[i][1] == b[i + 1][0] for i in range(w - 1))
        assert all(a % 16 == 0 for a, _ in b if a < n)
    assert shard_bounds(57344, 8) == [(i * 7168, (i + 1) * 7168) for i in range(8)]


def test_slice_rows_rebases_csr():
    L = wl.make_layer(128, 80, 0.05, seed=3)
    bw, bs, rp, c, v = slice_rows(L.base_weight, L.base_scales, L.row_ptr, L.col, L.vals, 32, 64)
    assert bw.shape == (32, 64) and int(rp[0]) == 0 and rp.numel() == 33
    e0, e1 = int(L.row_ptr[32]), int(L.row_ptr[64])
    assert torch.equal(c, L.col[e0:e1]) and torch.equal(v, L.vals[e0:e1]) and int(rp[-1]) == e1 - e0


def _oracle_forward(mod, x2):
    import oracle
    if mod.out_features == 0:
        return x2.new_zeros(x2.shape[0], 0)
    nnz = mod.ortho_values.numel()
    y = oracle.forward_csr(mod.base_weight.numpy(), mod.base_scales.float().numpy(),
                           mod.ortho_row_ptr.numpy() if nnz else None, mod.ortho_col_indices.numpy() if nnz else None,
                           mod.ortho_values.float().numpy() if nnz else None, x2.float().numpy(), mod.alpha, threads=1)
    return torch.from_numpy(y).to(torch.float16)


def _worker(rank, world, port, n_rows, M, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layer = wl.make_layer(96, n_rows, 0.05, seed=7)
        full = layer.to_module()
        full.set_alpha(0.5)
        x = wl.make_input(M, 96, seed=7)
        sh = ShardedOrthoLinear.from_full(full, local_forward=_oracle_forward)
        y = sh(x)
        ref = _oracle_forward(full, x)
        ok = torch.equal(y, ref) and y.shape == (M, n_rows)
        # alpha switch reaches the shard
        sh.set_alpha(0.0)
        full.set_alpha(0.0)
        ok = ok and torch.equal(sh(x.reshape(1, M, 96)).reshape(M, n_rows), _oracle_forward(full, x))
        out[rank] = int(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows,M", [(64, 3), (50, 1), (16, 2)])
def test_two_rank_sharded_forward_equals_full(n_rows, M):
    import oracle
    oracle.build()
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, port, n_rows, M, out), nprocs=2, join=True)
    assert out.get(0) == 1 and out.get(1) == 1
