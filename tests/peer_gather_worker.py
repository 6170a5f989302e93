"""Worker of the two-GPU peer-gather test (launched by torch.distributed.run, one rank per GPU)."""
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from libortho_b200 import OrthoLinear, _lib
import workloads as wl        # noqa: E402
from libortho_b200.sharded import ShardedOrthoLinear               # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    if os.environ.get("ORTHO_B200_TEST_PER_CTA") == "1":      # the signalling form is fixed when a comm is created
        assert _lib.lib().ortho_b200_set_decode_config(-7, 0, 0, 1) == 0
    cases = [(4096, 2048, 1), (1024, 1056, 16), (512, 528, 40), (256, 1024, 200), (2048, 96, 4), (512, 1056, 300)]
    for K, N, M in cases:
        layer = wl.make_layer(K, N, 0.01, seed=K + N + M).to(dev)
        full = OrthoLinear(K, N, device=dev)
        full.base_weight, full.base_scales = layer.base_weight, layer.base_scales
        full.ortho_row_ptr, full.ortho_col_indices, full.ortho_values = layer.row_ptr, layer.col, layer.vals
        full.set_alpha(1.0)
        sh = ShardedOrthoLinear.from_full(full)
        sh.enable_peer_gather(M)
        for it in range(6):                       # both regions, several epochs
            x = wl.make_input(M, K, seed=100 + it).to(dev)
            y = sh(x)
            ref = full(x)
            torch.cuda.synchronize()
            assert _lib.lib().ortho_b200_query_kernel_status() == 0, "a gather wait timed out"
            # the shard and the full layer may split K differently (another FP32 summation order):
            # equal up to FP16 rounding of the same exact sums
            d = (y.float() - ref.float()).abs().max().item()
            rel = ((y.float() - ref.float()).norm() / ref.float().norm()).item()
            assert d <= 2e-2 and rel <= 1e-3, f"rank {rank}: K={K} N={N} M={M} it={it}: max_abs={d} rel={rel}"
        # deferred mode: a forward only signals; the next forward on the comm, or comm.wait(), waits
        sh._comm.set_deferred(True)
        xa, xb = wl.make_input(M, K, seed=301).to(dev), wl.make_input(M, K, seed=302).to(dev)
        for it in range(4):
            ya = sh(xa)                           # region 0
            yb = sh(xb)                           # region 1; its kernel waits for ya's exchange
            sh._comm.wait()                       # yb's exchange
            # every reader of a region must be ordered before this rank's next forward on the comm (which lets the
            # peers store into it again): take copies now, compare afterwards
            ya, yb = ya.clone(), yb.clone()
            ra, rb = full(xa), full(xb)
            torch.cuda.synchronize()
            dist.barrier()
            assert _lib.lib().ortho_b200_query_kernel_status() == 0, "a deferred gather wait timed out"
            for y, ref in ((ya, ra), (yb, rb)):
                d = (y.float() - ref.float()).abs().max().item()
                rel = ((y.float() - ref.float()).norm() / ref.float().norm()).item()
                assert d <= 2e-2 and rel <= 1e-3, f"rank {rank}: deferred K={K} N={N} M={M} it={it}: max_abs={d} rel={rel}"
        sh._comm.set_deferred(False)
        dist.barrier()
    # A peer that does not show up: rank 1 withholds one forward, so the wait of rank 0's kernel for rank 1's flag
    # must run out after the comm's timeout and leave a status for the host, with the context still usable.
    # Nothing faults or hangs: the kernel polls a flag nobody sets, against a clock.  Rank 1 then issues the withheld
    # call (rank 0's flag of that epoch is already there), the epochs are level again and the next exchange works.
    K, N, M = 1024, 1056, 4
    layer = wl.make_layer(K, N, 0.01, seed=77).to(dev)
    full = OrthoLinear(K, N, device=dev)
    full.base_weight, full.base_scales = layer.base_weight, layer.base_scales
    full.ortho_row_ptr, full.ortho_col_indices, full.ortho_values = layer.row_ptr, layer.col, layer.vals
    sh = ShardedOrthoLinear.from_full(full)
    sh.enable_peer_gather(M)
    x = wl.make_input(M, K, seed=401).to(dev)
    y = sh(x)
    torch.cuda.synchronize()
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    dist.barrier()
    sh._comm.set_timeout_ms(50)
    if rank == 0:
        t0 = time.perf_counter()
        sh(x)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        st = _lib.lib().ortho_b200_query_kernel_status()
        assert st == 8, f"rank 0: expected the bounded wait to run out (status 8), got {st}"
        assert 0.03 < waited < 5.0, waited
        try:
            _lib.check(st, "forward_gather")
            raise AssertionError("a kernel status must surface as an exception")
        except _lib.OrthoB200Error as e:
            assert "bounded wait" in str(e)
        assert _lib.lib().ortho_b200_query_kernel_status() == 0      # reading the status clears it
    dist.barrier()
    if rank == 1:
        sh(x)                                      # the withheld call: rank 0's flag of this epoch is already set
        torch.cuda.synchronize()
        assert _lib.lib().ortho_b200_query_kernel_status() == 0
    dist.barrier()
    sh._comm.set_timeout_ms(2000)
    x2 = wl.make_input(M, K, seed=402).to(dev)
    y2, ref2 = sh(x2), full(x2)
    torch.cuda.synchronize()
    assert _lib.lib().ortho_b200_query_kernel_status() == 0, "the exchange after the timed-out one must work"
    assert (y2.float() - ref2.float()).abs().max().item() <= 2e-2
    dist.barrier()
    torch.cuda.synchronize()
    open(os.path.join(sys.argv[1], f"ok{rank}"), "w").write("ok")
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
