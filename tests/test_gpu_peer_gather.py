"""The gathering forward (ortho_b200_forward_gather): pitched stores on one GPU against the oracle,
and the real exchange between two ranks on two GPUs (skipped where fewer are visible)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, assert_close, layer_oracle
from libortho_b200 import _C_ops
import workloads as wl
from libortho_b200.sharded import shard_bounds, slice_rows

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("M,K,N", [(1, 512, 208), (16, 256, 96), (5, 320, 64), (40, 512, 144), (130, 256, 272)])
def test_world_of_one_writes_its_columns_of_a_wider_matrix(oracle_mod, M, K, N):
    """A shard in the middle of a wider output: only columns [n0, n0+N) of the [M, N_total] matrix
    may change, and they must match the oracle.  Covers the output pitch of every kernel family
    (streaming decode, generic decode, tcgen05 prefill)."""
    layer = wl.make_layer(K, N, 0.02, seed=70 + M).to(DEV)
    x = wl.make_input(M, K, seed=7).to(DEV)
    n0, n_total = 32, N + 32 + 24
    comm = _C_ops.Comm(0, 1, 4096 + 2 * M * n_total)
    buf = comm.buffer()
    buf.fill_(0x3C)                                   # every half reads 1.0039 before the call
    plan = _C_ops.Plan(layer.row_ptr, layer.col, layer.vals, K, N)
    y = _C_ops.forward_gather(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr,
                              x, 1.0, comm, 4096, n_total, n0, plan=plan)
    torch.cuda.synchronize()
    assert _lib_status_ok()
    ref = layer_oracle(oracle_mod, layer, x, 1.0)
    assert_close(y[:, n0:n0 + N].float().cpu().numpy(), ref, f"gather M={M}")
    untouched = torch.full((1,), 0x3C3C, dtype=torch.int16, device=DEV).view(torch.float16)
    assert torch.all(y[:, :n0] == untouched) and torch.all(y[:, n0 + N:] == untouched)
    assert torch.all(buf[:4096] == 0x3C)
    # same bits as the plain forward
    y2 = torch.empty(M, N, dtype=torch.float16, device=DEV)
    _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, x, y2, 1.0, plan=plan)
    assert torch.equal(y[:, n0:n0 + N], y2)
    comm.close()


def _lib_status_ok():
    from libortho_b200 import _lib
    return _lib.lib().ortho_b200_query_kernel_status() == 0


def test_argument_errors():
    from libortho_b200 import _lib
    layer = wl.make_layer(256, 64, 0.0, seed=3).to(DEV)
    x = wl.make_input(2, 256, seed=1).to(DEV)
    comm = _C_ops.Comm(0, 1, 2 * 2 * 64)
    with pytest.raises(_lib.OrthoB200Error):          # matrix does not fit the buffer
        _C_ops.forward_gather(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr,
                              x, 1.0, comm, 0, 128, 0)
    with pytest.raises(_lib.OrthoB200Error):          # slice sticks out of the matrix
        _C_ops.forward_gather(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr,
                              x, 1.0, comm, 0, 64, 8)
    comm.close()
    with pytest.raises(_lib.OrthoB200Error):
        _C_ops.Comm(3, 2, 1024)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("per_cta", [0, 1])
def test_two_ranks_exchange_through_peer_memory(tmp_path, per_cta):
    """Two processes, one per GPU: every rank must end up with the full output of each forward,
    bit-identical to a single-GPU forward of the unsharded layer (checked inside the workers).  Both signalling
    forms of the exchange: the grid's last CTA raises a flag (0), every CTA counts itself in on the peers (1)."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, ORTHO_B200_TEST_PER_CTA=str(per_cta))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(29741 + per_cta),
           os.path.join(ROOT, "tests", "peer_gather_worker.py"), str(tmp_path)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for rank in (0, 1):
        assert (tmp_path / f"ok{rank}").exists(), r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_in_the_same_process(oracle_mod):
    """Function attributes, SM counts and occupancy caches are kept per device: a process that has run every kernel
    family on cuda:0 runs them on cuda:1 as well (streaming, generic decode, tokens-as-M, prefill)."""
    for dev in ("cuda:0", "cuda:1"):
        for (M, K, N) in [(1, 4096, 512), (20, 1024, 208), (40, 1024, 4352), (300, 1024, 520)]:
            layer = wl.make_layer(K, N, 0.01, seed=500 + M)
            x = wl.make_input(M, K, seed=500 + M)
            m = layer.to(dev).to_module()
            y = m(x.to(dev))
            torch.cuda.synchronize(dev)
            with torch.cuda.device(dev):
                from libortho_b200 import _lib
                assert _lib.lib().ortho_b200_query_kernel_status() == 0
            assert_close(y.float().cpu().numpy(), layer_oracle(oracle_mod, layer, x, 1.0), f"{dev} M={M}")
