"""Benchmark of the OrthoLinear forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``), the same for every N: the Llama-2-70B-style projections in the decode
regime -- four layers (in->out: 8192->10240, 8192->8192, 8192->57344, 28672->8192), one FP16 token each,
INT4 base from W~N(0,0.02^2), 0.3 % uniform FP16 ortho ~N(0,0.05^2), alpha=1, seeded synthetic tensors.
One "step" is one pass over the four layers.  With N > 1 (launched by torch.distributed.run, one rank
per GPU) every layer is sharded over output rows, each rank runs its shard and the kernel itself stores
its output slice into every rank's peer-mapped buffer (``--exchange nccl``: an NCCL all-gather instead);
``scaling`` is "strong" (the layers are fixed, the per-GPU share shrinks).  Steps rotate over as many
distinct copies of the layers as it takes for a GPU's share to exceed the L2 several times.

``value``    decode GB/s = algorithmic bytes of the step (whole layers) / device time (max over ranks),
             inputs resident in HBM, the steps replayed as CUDA graphs (up to --steps-per-graph steps each), timed with CUDA events.
``e2e``      the same metric through ``OrthoLinear.forward`` / ``ShardedOrthoLinear.forward`` with host
             buffers: every step copies its inputs from pinned host memory, runs the four forwards, copies the four
             outputs back and synchronises the stream, all inside the timed region.
``roofline`` HBM roofline of the decode kernel from the same timed region (per GPU).
``cpu_baseline`` the reference's own CPU forward timed on this host (N=1 only).
``regimes``  (extra, every N) the same four layers at M=32 (GB/s) and M=4096 (TFLOP/s) with the exchange
             cost; ``decode_sweep_7b`` and ``prefill`` (extra, N=1) the Llama-7B-style decode sweep
             (M in {1,4,16}, 0.5 % ortho) and the 8192x8192 Zipf-row prefill configuration.
With N > 1 the gathered output of every layer is compared with the unsharded forward and the kernels'
status word is read after the timed loop; a mismatch or a timed-out wait makes the run fail.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "OrthoLinear decode GB/s (% HBM peak) & prefill TFLOP/s at 1/2/4/8 B200"
WORKLOAD = ("70B-style decode: (8192->10240, 8192->8192, 8192->57344, 28672->8192) x M=1, INT4 base + 0.3% ortho, "
            "alpha=1, N-sharded over the GPUs with output gather")
L2_BYTES = 126 << 20

# DRAM bytes moved per algorithmic byte by the streaming decode kernel, from an ncu capture of one launch
# (dram__bytes_read.sum + dram__bytes_write.sum = 245.2 MB for the 243.8 MB 8192->57344 M=1 launch); the
# kernel reads every weight byte once, so traffic grows in proportion to the algorithmic bytes
NCU_TRAFFIC_RATIO = 245.2 / 243.8


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tf_burst": d["bf16_tflops"], "tf_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [s.strip() for s in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for nme, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nme)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _cpu_impl():
    import oracle
    impl, kind = ("reference_fast", "reference") if oracle.available("reference_fast") else ("port", "port")
    if impl == "port":
        oracle.build()
    return oracle, impl, kind


def _cpu_layers():
    """The four layers of the workload as numpy arrays for the CPU forward (seed 0)."""
    import workloads as wl
    out = []
    for (K, N) in wl.CFG3_SHAPES:
        L = wl.make_layer(K, N, wl.CFG3_DENSITY, seed=0)
        out.append((L, (L.base_weight.numpy(), L.base_scales.float().numpy(), L.row_ptr.numpy(), L.col.numpy(),
                        L.vals.float().numpy()), wl.make_input(1, K, seed=1).float().numpy()))
    return out


# ------------------------------------------------------------------------------------------------
def run_reference(args):
    """The reference's own CPU forward (unmodified src/ortho.c behind oracle/_ref, built with the
    reference's flags) on all host threads; each step is one pass over the same four layers at M=1."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle, impl, kind = _cpu_impl()
    threads = oracle.host_threads()
    layers = _cpu_layers()
    step_bytes = sum(L.algorithmic_bytes(1) for L, _, _ in layers)

    def step():
        for _, a, x in layers:
            oracle.forward_csr(*a, x, 1.0, impl=impl, threads=threads)

    for _ in range(max(0, args.warmup)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    val = step_bytes * args.steps / dt / 1e9
    sample = f"{args.steps} full passes over the four layers at M=1, {threads} threads (rows split over threads)"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def cpu_baseline():
    """Reference CPU forward (oracle/_ref, reference flags) on this host: passes over the workload for ~10 s."""
    oracle, impl, kind = _cpu_impl()
    threads = oracle.host_threads()
    layers = _cpu_layers()
    step_bytes = sum(L.algorithmic_bytes(1) for L, _, _ in layers)
    n, t_total = 0, 0.0
    while n < 3 or (t_total < 10.0 and n < 200):
        t0 = time.perf_counter()
        for _, a, x in layers:
            oracle.forward_csr(*a, x, 1.0, impl=impl, threads=threads)
        t_total += time.perf_counter() - t0
        n += 1
    return {"value": step_bytes * n / t_total / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": f"{n} full passes over the four layers at M=1, {t_total:.2f} s wall", "ms_per_step": t_total / n * 1e3}


# ------------------------------------------------------------------------------------------------
class _Timer:
    """CUDA-graph timing helper: a graph of ``n`` calls ``fn(i)`` is replayed; device time per call from CUDA
    events on the launch stream, median over replays, max over ranks."""

    def __init__(self, torch, dist, dev, stream, world):
        self.torch, self.dist, self.dev, self.stream, self.world = torch, dist, dev, stream, world

    def us_per_call(self, fn, n, replays=5, warm=2):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            fn(0)                                   # first call of a kernel variant happens outside the capture
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                for i in range(n):
                    fn(i)
            for _ in range(warm):
                g.replay()
            self.stream.synchronize()
            if self.world > 1:
                self.dist.barrier()
            ts = []
            for _ in range(replays):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                g.replay()
                e1.record(self.stream)
                e1.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3 / n)
        t = torch.tensor([statistics.median(ts)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        del g
        return float(t.item())


def run_ours(args):
    import torch
    import torch.distributed as dist
    from libortho_b200 import _C_ops, _lib
    import workloads as wl
    from libortho_b200.sharded import ShardedOrthoLinear, shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pk = peaks()
    lib = _lib.lib()
    stream = torch.cuda.Stream(dev)
    timer = _Timer(torch, dist, dev, stream, world)
    shapes = wl.CFG3_SHAPES
    failures = []

    # ---- the four layers, sharded over the ranks; enough distinct copies for a GPU's share to exceed L2 -------
    per_gpu_set = sum(K * N // 2 for (K, N) in shapes) // world
    n_copies = max(2, min(8, -(-int(2.5 * L2_BYTES) // per_gpu_set)))
    sets, fulls = [], {}
    for c in range(n_copies):
        layers = {}
        for (K, N) in shapes:
            full = wl.make_layer(K, N, wl.CFG3_DENSITY, seed=c, device=dev)
            n0, n1 = shard_bounds(N, world)[rank]
            L = full.rows(n0, n1) if world > 1 else full
            L._full_bytes = {M: full.algorithmic_bytes(M) for M in wl.CFG3_M}
            L._full_flops = {M: full.algorithmic_flops(M) for M in wl.CFG3_M}
            L._n0 = n0
            if c == 0 and world > 1:
                fulls[(K, N)] = full              # kept for the check of the gathered output
            del full
            layers[(K, N)] = (L, _C_ops.Plan(L.row_ptr, L.col, L.vals, L.K, L.N))
        sets.append(layers)
    torch.cuda.empty_cache()
    step_bytes = sum(sets[0][kn][0]._full_bytes[1] for kn in shapes)
    xs = {(K, M): wl.make_input(M, K, seed=M, device=dev) for (K, N) in shapes for M in wl.CFG3_M}

    # multi-GPU exchange: peer stores issued by the kernels themselves (default), or NCCL
    exchange, comm = "none", None
    max_n = max(N for _, N in shapes)
    region = {M: (2 * M * max_n + 255) // 256 * 256 for M in wl.CFG3_M}
    if world > 1:
        exchange = args.exchange
        if exchange == "peer":
            if args.per_cta_signal:
                assert lib.ortho_b200_set_decode_config(-7, 0, 0, 1) == 0     # before the comms are created
            try:
                comm = _C_ops.Comm(rank, world, 2 * region[max(wl.CFG3_M)], device=dev)
                comm.connect_group()
            except Exception as e:       # no inter-process mapping on this box: the NCCL exchange still measures the path
                print(f"[bench] peer-mapped buffers unavailable ({e}); using the NCCL all-gather", file=sys.stderr)
                exchange, comm = "nccl", None
            flags = torch.tensor([1 if exchange == "peer" else 0], device=dev)
            dist.all_reduce(flags, op=dist.ReduceOp.MIN)
            if int(flags.item()) == 0:
                exchange, comm = "nccl", None
    ys = {}

    def out_buffers(M):
        if M not in ys:
            ys[M] = {kn: torch.empty(M, sets[0][kn][0].N, dtype=torch.float16, device=dev) for kn in shapes}
            if world > 1 and exchange == "nccl":
                ys[(M, "g")] = {kn: torch.empty(world * M, sets[0][kn][0].N, dtype=torch.float16, device=dev) for kn in shapes}
        return ys[M]

    wss = {}

    def workspace(M, kn):
        L, plan = sets[0][kn]
        need = max(_C_ops.workspace_bytes(M, L.K, L.N, p) for (_, p) in (s[kn] for s in sets))
        cur = wss.get("ws")
        if cur is None or cur.numel() < need:
            wss["ws"] = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
        return wss["ws"]

    slot = [0]

    def forward(c, kn, M, gather=True):
        """One forward of layer kn (copy c) at M tokens: the shard's kernel plus, with N > 1, the exchange."""
        L, plan = sets[c][kn]
        K, N = kn
        x = xs[(K, M)]
        ws = workspace(M, kn)
        if world > 1 and gather and exchange == "peer":
            off = slot[0] * region[M]
            slot[0] ^= 1
            return _C_ops.forward_gather(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, 1.0, comm, off, N, L._n0,
                                         plan=plan, workspace=ws)
        y = out_buffers(M)[kn]
        _C_ops.forward(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, y, 1.0, plan=plan, workspace=ws)
        if world > 1 and gather:
            dist.all_gather_into_tensor(ys[(M, "g")][kn], y)
            return ys[(M, "g")][kn]
        return y

    def run_steps(first, count):
        """`count` consecutive steps (step i works on weight copy i % n_copies).  With the deferred peer exchange every
        forward waits for its predecessor's flags, so only the last forward of the sequence needs an explicit wait."""
        for i in range(first, first + count):
            for kn in shapes:
                forward(i % n_copies, kn, 1)
        if exchange == "peer":
            comm.wait()

    for M in wl.CFG3_M:
        out_buffers(M)
        for kn in shapes:
            workspace(M, kn)
    if exchange == "peer":
        comm.set_deferred(not args.no_deferred)

    # ---- headline: the K timed steps are captured as CUDA graphs of up to `chunk` steps each --------------------
    chunk = max(1, min(args.steps, args.steps_per_graph))
    n_chunks, rem = divmod(args.steps, chunk)

    def capture(first, count):
        g = torch.cuda.CUDAGraph()
        l0 = lib.ortho_b200_launch_count()
        with torch.cuda.graph(g, stream=stream):
            run_steps(first, count)
        return g, lib.ortho_b200_launch_count() - l0

    with torch.cuda.stream(stream):
        run_steps(0, 1)                  # first call of every kernel variant happens outside a capture
        stream.synchronize()
        g_chunk, l_chunk = capture(0, chunk)
        g_rem, l_rem = capture(n_chunks * chunk, rem) if rem else (None, 0)
    timed_launches = n_chunks * l_chunk + l_rem
    launches_per_step = timed_launches / args.steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(3, args.warmup)
    with torch.cuda.stream(stream):
        for i in range(-(-warm // chunk)):
            g_chunk.replay()
        barrier()
        sampler = ClockSampler(local) if rank == 0 else None
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            # one untimed exchange right in front of the first event lines the ranks' streams up on the device, so
            # that the host-side skew of the launches after the barrier is not charged to the first timed step
            if exchange == "peer":
                forward(0, shapes[1], 1)
                comm.wait()
            else:
                dist.all_reduce(torch.zeros(1, device=dev))
        ev0.record(stream)
        for i in range(n_chunks):
            g_chunk.replay()
        if g_rem is not None:
            g_rem.replay()
        ev1.record(stream)
        barrier()
        ms = ev0.elapsed_time(ev1)
    tms = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    clocks = sampler.stop() if sampler else None
    value = step_bytes * args.steps / (ms * 1e-3) / 1e9
    status = torch.tensor([lib.ortho_b200_query_kernel_status()], device=dev)
    if world > 1:
        dist.all_reduce(status, op=dist.ReduceOp.MAX)
    if int(status.item()) != 0:
        failures.append("a kernel gave up on a bounded wait inside the timed loop")
    del g_chunk, g_rem
    if exchange == "peer":
        comm.set_deferred(False)

    # ---- N > 1: the gathered output of every layer against the unsharded forward ------------------------------
    gather_checked, gather_max_abs = None, 0.0
    if world > 1:
        ok = True
        for kn in shapes:
            K, N = kn
            full = fulls[kn]
            for M in (1, 32):
                yg = forward(0, kn, M)
                if exchange == "nccl":
                    yg = yg.view(world, M, -1).permute(1, 0, 2).reshape(M, -1)
                yr = torch.empty(M, N, dtype=torch.float16, device=dev)
                _C_ops.forward(full.base_weight, full.base_scales, full.vals, full.col, full.row_ptr, xs[(K, M)], yr, 1.0,
                               workspace=torch.empty(max(256, _C_ops.workspace_bytes(M, K, N)), dtype=torch.uint8, device=dev))
                torch.cuda.synchronize()
                d = float((yg.float() - yr.float()).abs().max().item())
                gather_max_abs = max(gather_max_abs, d)
                # the shard and the whole layer run the same arithmetic per row; a different K split may change the
                # FP32 summation order, so: equal up to FP16 rounding
                if not (d <= 2e-2) or not bool(torch.isfinite(yg).all()):
                    ok = False
                    failures.append(f"gathered output of {K}->{N} at M={M} differs from the unsharded forward by {d}")
                dist.barrier()
        st2 = torch.tensor([lib.ortho_b200_query_kernel_status(), 0 if ok else 1], device=dev)
        dist.all_reduce(st2, op=dist.ReduceOp.MAX)
        gather_checked = bool(int(st2[0].item()) == 0 and int(st2[1].item()) == 0)
        if int(st2[0].item()) != 0:
            failures.append("a kernel gave up on a bounded wait during the gather check")
        fulls.clear()
        torch.cuda.empty_cache()

    # ---- end to end through the module API with host buffers -----------------------------------------------------
    mods = []
    e2e_comm = None
    if exchange == "peer":
        e2e_comm = _C_ops.Comm(rank, world, len(shapes) * ShardedOrthoLinear.peer_gather_bytes(1, max_n), device=dev)
        e2e_comm.connect_group()
    for c in range(n_copies):
        d = {}
        for i, kn in enumerate(shapes):
            m = sets[c][kn][0].to_module()
            if world > 1:
                sh = ShardedOrthoLinear(kn[0], kn[1], device=dev)
                sh.local = m
                if exchange == "peer":
                    sh.enable_peer_gather(1, comm=e2e_comm, offset_bytes=i * ShardedOrthoLinear.peer_gather_bytes(1, max_n))
                m = sh
            d[kn] = m
        mods.append(d)
    # one pinned host buffer and one device buffer hold the step's inputs (one copy in); with one GPU the modules
    # write into slices of one device buffer (forward(x, out=...)), so the results leave with one copy as well
    Ks = sorted({K for (K, N) in shapes})
    hx_all = torch.cat([xs[(K, 1)].reshape(-1).cpu() for K in Ks]).pin_memory()
    xdev_all = torch.empty_like(hx_all, device=dev)
    xdev, o = {}, 0
    for K in Ks:
        xdev[K] = xdev_all[o:o + K].view(1, K)
        o += K
    hy_all = torch.empty(sum(N for (_, N) in shapes), dtype=torch.float16).pin_memory()
    ydev_all = torch.empty_like(hy_all, device=dev)
    hy, ydev, o = {}, {}, 0
    for kn in shapes:
        hy[kn], ydev[kn] = hy_all[o:o + kn[1]], ydev_all[o:o + kn[1]]
        o += kn[1]
    h2d = hx_all.numel() * 2
    d2h = hy_all.numel() * 2

    def e2e_step(c):
        xdev_all.copy_(hx_all, non_blocking=True)           # this step's inputs, from pinned host memory
        if world == 1:
            for kn in shapes:
                mods[c][kn](xdev[kn[0]], out=ydev[kn])
            hy_all.copy_(ydev_all, non_blocking=True)       # and its results back to the host
        else:
            out = [(kn, mods[c][kn](xdev[kn[0]])) for kn in shapes]
            for kn, y in out:
                hy[kn].copy_(y.view(-1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(max(3, n_copies)):       # touches every weight copy once: plans are built on first use
        e2e_step(i % n_copies)
    barrier()
    e2e_steps = max(3, min(args.steps, 50))
    l_before = lib.ortho_b200_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(e2e_steps):
        e2e_step(i % n_copies)
    ev1.record()
    barrier()
    e2e_launches = lib.ortho_b200_launch_count() - l_before
    tms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    e2e_val = step_bytes * e2e_steps / (float(tms.item()) * 1e-3) / 1e9
    del mods

    # ---- the same layers in the other regimes (every N) and per-layer detail -----------------------------------------
    regimes = {}
    if not args.no_regimes:
        for kn in shapes:
            K, N = kn
            for M in wl.CFG3_M:
                n = (2 * n_copies) if M <= 32 else 2
                t_all = timer.us_per_call(lambda i: forward(i % n_copies, kn, M), n, replays=5 if M <= 32 else 3)
                row = {"us": round(t_all, 2)}
                fb, ff = sets[0][kn][0]._full_bytes[M], sets[0][kn][0]._full_flops[M]
                if M <= 32:
                    row["GB/s"] = round(fb / t_all / 1e3, 1)
                    row["frac_hbm_per_gpu"] = round(fb / t_all / 1e3 / world / pk["hbm_gbs"], 3)
                else:
                    row["TFLOP/s"] = round(ff / t_all / 1e6, 1)
                    row["frac_of_measured_sustained_per_gpu"] = round(ff / t_all / 1e6 / world / pk["tf_sustained"], 3)
                if world > 1:
                    t_loc = timer.us_per_call(lambda i: forward(i % n_copies, kn, M, gather=False), n, replays=5 if M <= 32 else 3)
                    row["shard_only_us"] = round(t_loc, 2)
                    row["exchange_us"] = round(t_all - t_loc, 2)
                regimes[f"{K}x{N}:M{M}"] = row
        st3 = torch.tensor([lib.ortho_b200_query_kernel_status()], device=dev)
        if world > 1:
            dist.all_reduce(st3, op=dist.ReduceOp.MAX)
        if int(st3.item()) != 0:
            failures.append("a kernel gave up on a bounded wait in the regime sweep")

    sweep7b, prefill = {}, {}
    if world == 1 and not args.no_extras:
        del sets
        wss.clear(); ys.clear()
        torch.cuda.empty_cache()
        sweep7b = bench_decode_sweep_7b(dev, pk, stream)
        torch.cuda.empty_cache()
        prefill = bench_prefill(dev, pk)

    if rank == 0:
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD},
            "run": {"parallelism": f"N-sharded x{world} + output gather" if world > 1 else "single GPU",
                    "exchange": {"peer": "peer stores issued by the kernels (ortho_b200_forward_gather)" +
                                         ("; every CTA signals the peers" if args.per_cta_signal else "") +
                                         ("" if args.no_deferred else "; each forward waits for its predecessor's flags, the step ends with a wait"),
                                 "nccl": "NCCL all_gather_into_tensor after the kernel", "none": None}[exchange],
                    "l2": f"rotation over {n_copies} distinct copies of the layers ({per_gpu_set * n_copies >> 20} MB per GPU) > 126 MB L2",
                    "timing": f"the {args.steps} steps replayed as CUDA graphs of {chunk} steps, CUDA events on the launch stream, max over ranks"},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "api": ("ShardedOrthoLinear.forward" if world > 1 else "OrthoLinear.forward") +
                                               ", per step: one pinned host buffer with X in, four forwards, Y out to pinned host memory, one stream sync"},
            "gpu_launches": int(timed_launches + e2e_launches),
            "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": per_gpu / pk["hbm_gbs"],
                         "traffic": NCU_TRAFFIC_RATIO * step_bytes / len(shapes) / world,
                         "traffic_source": "ncu capture of one launch of this kernel (DRAM bytes / algorithmic bytes = 1.006), scaled by algorithmic bytes",
                         "peak_source": pk["source"], "kernel": "ob::decode_stream_kernel",
                         "launches_per_step": launches_per_step,
                         "algorithmic_bytes_per_launch": step_bytes / len(shapes) / world},
            "percent_of_nominal_8TBs": per_gpu / 8000.0 * 100.0,
        }
        if world > 1:
            line["gather_checked"] = gather_checked
            line["gather_max_abs_diff"] = gather_max_abs
        if regimes:
            line["regimes"] = regimes
        if sweep7b:
            line["decode_sweep_7b"] = sweep7b
        if prefill:
            line["prefill"] = prefill
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline()
        if failures:
            line["failures"] = failures
        print(json.dumps(line))
    rc = 1 if failures else 0
    if world > 1:
        # tearing the NCCL communicator down while CUDA graphs that hold its kernels exist has hung at exit:
        # meet once more and leave without the collective teardown
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(rc)
    if rc:
        sys.exit(rc)


def bench_decode_sweep_7b(dev, pk, stream):
    """Llama-7B-style decode sweep on one GPU: (4096->12288, 4096->4096, 4096->22016, 11008->4096) x M in {1,4,16},
    0.5 % ortho, alpha=1; the 12 forwards as one CUDA graph rotating over 6 weight copies (~100 MB each), and
    per (layer, M) the fused forward beside the base-only one (alpha=0)."""
    import torch
    from libortho_b200 import _C_ops
    import workloads as wl
    copies = 6
    sets = []
    for c in range(copies):
        d = {}
        for (K, N) in wl.CFG1_SHAPES:
            L = wl.make_layer(K, N, wl.CFG1_DENSITY, seed=c, device=dev)
            d[(K, N)] = (L, _C_ops.Plan(L.row_ptr, L.col, L.vals, K, N))
        sets.append(d)
    items = [(K, N, M) for M in wl.CFG1_M for (K, N) in wl.CFG1_SHAPES]
    xs = {(K, M): wl.make_input(M, K, seed=M, device=dev) for (K, N, M) in items}
    ys = {(K, N, M): torch.empty(M, N, dtype=torch.float16, device=dev) for (K, N, M) in items}
    need = max(_C_ops.workspace_bytes(M, K, N, sets[0][(K, N)][1]) for (K, N, M) in items)
    ws = torch.empty(max(256, need), dtype=torch.uint8, device=dev)
    timer = _Timer(torch, None, dev, stream, 1)

    def fwd(c, K, N, M, alpha=1.0):
        L, plan = sets[c][(K, N)]
        _C_ops.forward(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, xs[(K, M)], ys[(K, N, M)], alpha, plan=plan, workspace=ws)

    def step(i):
        for (K, N, M) in items:
            fwd(i % copies, K, N, M)

    us_step = timer.us_per_call(step, copies, replays=7)
    step_bytes = sum(sets[0][(K, N)][0].algorithmic_bytes(M) for (K, N, M) in items)
    out = {"us_per_step": round(us_step, 2), "GB/s": round(step_bytes / us_step / 1e3, 1),
           "frac_hbm": round(step_bytes / us_step / 1e3 / pk["hbm_gbs"], 4), "forwards_per_step": len(items), "detail": {}}
    for (K, N, M) in items:
        L = sets[0][(K, N)][0]
        us = timer.us_per_call(lambda i: fwd(i % copies, K, N, M), 2 * copies)
        us0 = timer.us_per_call(lambda i: fwd(i % copies, K, N, M, 0.0), 2 * copies)
        gbs = L.algorithmic_bytes(M) / us / 1e3
        out["detail"][f"{K}x{N}:M{M}"] = {"us": round(us, 2), "GB/s": round(gbs, 1), "frac_hbm": round(gbs / pk["hbm_gbs"], 3),
                                          "base_only_us": round(us0, 2), "sparse_cost": round(us / us0 - 1.0, 3)}
    return out


def bench_prefill(dev, pk):
    import torch
    from libortho_b200 import _C_ops
    import workloads as wl
    K, N = wl.CFG2_SHAPE
    L = wl.make_zipf_layer(K, N, wl.CFG2_DENSITY, seed=0, device=dev, alpha=wl.CFG2_ALPHA)
    plan = _C_ops.Plan(L.row_ptr, L.col, L.vals, K, N)
    out = {}
    for M in wl.CFG2_M:
        x = wl.make_input(M, K, seed=M, device=dev)
        y = torch.empty(M, N, dtype=torch.float16, device=dev)
        ws_bytes = _C_ops.workspace_bytes(M, K, N, plan)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        for alpha, tag in ((wl.CFG2_ALPHA, "fused"), (0.0, "base_only")):
            for _ in range(3):
                _C_ops.forward(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, y, alpha, plan=plan, workspace=ws)
            torch.cuda.synchronize()
            reps = 10 if M <= 2048 else 4
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                _C_ops.forward(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, y, alpha, plan=plan, workspace=ws)
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1) / reps
            tf = L.algorithmic_flops(M, alpha) / (ms * 1e-3) / 1e12
            out[f"M{M}:{tag}"] = {"ms": round(ms, 4), "TFLOP/s": round(tf, 1),
                                  "frac_of_measured_sustained": round(tf / pk["tf_sustained"], 3),
                                  "frac_of_nominal_2250": round(tf / 2250.0, 3)}
    out["config"] = "8192x8192, 0.1% ortho with Zipf(1.2) row loads, alpha=0.5; X (M x 8192 FP16) larger than L2 only for M=8192"
    return out


N_COPIES = 6          # weight copies the single-GPU report rotates through (decode-sized forwards)

def run_report(args):
    """All BASELINE.json configurations on one GPU, as a markdown table (``--report PATH``).  Decode-sized
    forwards rotate over enough weight copies to exceed L2; per-forward device time from CUDA graphs."""
    import torch
    from libortho_b200 import _C_ops
    import workloads as wl
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    pk = peaks()
    stream = torch.cuda.Stream(dev)
    rows = []

    def measure(tag, make, Ms, alphas):
        L0 = make(0)
        nbytes = L0.K * L0.N // 2 + 6 * L0.nnz
        ncopies = max(1, min(N_COPIES, -(-(300 << 20) // nbytes)))
        layers = [L0] + [make(c) for c in range(1, ncopies)]
        plans = [_C_ops.Plan(L.row_ptr, L.col, L.vals, L.K, L.N) for L in layers]
        for M in Ms:
            x = wl.make_input(M, L0.K, seed=M, device=dev)
            y = torch.empty(M, L0.N, dtype=torch.float16, device=dev)
            need = _C_ops.workspace_bytes(M, L0.K, L0.N, plans[0])
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
            for alpha in alphas:
                reps = 2 if M <= 64 else 1
                n = reps * ncopies
                with torch.cuda.stream(stream):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        for r in range(n):
                            L = layers[r % ncopies]
                            _C_ops.forward(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, y, alpha,
                                           plan=plans[r % ncopies], workspace=ws)
                    for _ in range(3):
                        g.replay()
                    stream.synchronize()
                    ts = []
                    for _ in range(5 if M <= 2048 else 3):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        g.replay()
                        e1.record(stream)
                        e1.synchronize()
                        ts.append(e0.elapsed_time(e1) * 1e3 / n)
                us = statistics.median(ts)
                gbs = L0.algorithmic_bytes(M, alpha) / us / 1e3
                tf = L0.algorithmic_flops(M, alpha) / us / 1e6
                rows.append(f"| {tag} | {L0.K}->{L0.N} | {M} | {alpha} | {L0.nnz} | {us:.1f} | {M / us * 1e6:.3g} | {gbs:.0f} | "
                            f"{100 * gbs / pk['hbm_gbs']:.1f} | {tf:.1f} | {100 * tf / pk['tf_sustained']:.1f} |")
            del x, y, ws
        del layers, plans
        torch.cuda.empty_cache()

    measure("0", lambda c: wl.make_layer(4096, 4096, 0.01, seed=c, device=dev, ortho="residual10"), [8], [0.0, 1.0])
    for (K, N) in wl.CFG1_SHAPES:
        measure("1", lambda c: wl.make_layer(K, N, wl.CFG1_DENSITY, seed=c, device=dev), wl.CFG1_M, [1.0])
    K, N = wl.CFG2_SHAPE
    measure("2", lambda c: wl.make_zipf_layer(K, N, wl.CFG2_DENSITY, seed=c, device=dev, alpha=wl.CFG2_ALPHA), wl.CFG2_M,
            [wl.CFG2_ALPHA, 0.0])
    for (K, N) in wl.CFG3_SHAPES:
        measure("3", lambda c: wl.make_layer(K, N, wl.CFG3_DENSITY, seed=c, device=dev), wl.CFG3_M, [1.0])
    sieve = wl.make_sieve_layer(device=dev)
    measure("4 (threshold 10: nnz=0)", lambda c: sieve, [1, 2048], [0.0, 1.0])
    sieve1 = wl.make_sieve_layer(device=dev, sparsity_target=0.01)
    measure("4 (supplementary: keep top 1 %)", lambda c: sieve1, [1, 2048], [0.25, 1.0])

    # device-side packer (the producer of the layout): HBM-bound, W read once from DRAM (row re-read from L2)
    pack_rows = []
    for (K, N) in [(4096, 4096), (8192, 8192), (8192, 28672)]:
        w = torch.randn(N, K, device=dev) * 0.02
        wo = torch.where(torch.rand(N, K, device=dev) < 0.003, torch.randn(N, K, device=dev) * 0.05, torch.zeros((), device=dev))
        for name, fn, nbytes in (("pack_base", lambda: _C_ops.pack_base(w), N * K * 4 + N * K // 2 + 2 * N),
                                 ("pack_ortho_csr (count + scan + fill)", lambda: _C_ops.pack_ortho_csr(wo), 2 * N * K * 4)):
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            e1.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / 5
            pack_rows.append(f"| {name} | {N}x{K} FP32 | {us:.0f} | {nbytes / us / 1e3:.0f} | {100 * nbytes / us / 1e3 / pk['hbm_gbs']:.1f} |")
        del w, wo
        torch.cuda.empty_cache()

    # the reference's CPU forward on configuration 0 (1 thread and all threads)
    import oracle
    impl = "reference_fast" if oracle.available("reference_fast") else "port"
    if impl == "port":
        oracle.build()
    L = wl.make_layer(4096, 4096, 0.01, seed=0, ortho="residual10")
    a = (L.base_weight.numpy(), L.base_scales.float().numpy(), L.row_ptr.numpy(), L.col.numpy(), L.vals.float().numpy())
    x = wl.make_input(8, 4096, seed=8).float().numpy()
    cpu = []
    for th in (1, oracle.host_threads()):
        t0 = time.perf_counter()
        oracle.forward_csr(*a, x, 1.0, impl=impl, threads=th)
        dt = time.perf_counter() - t0
        cpu.append(f"| 0 | 4096->4096 | 8 | 1.0 | {L.nnz} | {dt * 1e6:.0f} | {8 / dt:.3g} | {L.algorithmic_bytes(8) / dt / 1e9:.2f} | - | "
                   f"{L.algorithmic_flops(8) / dt / 1e12:.4f} | - | CPU `{impl}`, {th} thread(s) |")
    head = ("| config | shape K->N | M | alpha | nnz | us / forward | tokens/s | GB/s (algorithmic) | % of measured HBM "
            f"({pk['hbm_gbs']:.0f} GB/s) | TFLOP/s | % of measured sustained tensor ({pk['tf_sustained']:.0f} TF) |")
    sep = "|" + "---|" * 11
    out = ["# All configurations, one B200 (`python bench.py --report <path>`)", "", head, sep, *rows, "",
           "CPU rows (host of the same box):", "", head + " note |", sep + "---|", *cpu, "",
           "Device-side packer (algorithmic bytes: W read once + outputs; the CSR build reads W twice; includes the host "
           "read-back of nnz and the output allocations):", "",
           "| step | input | us | GB/s | % of measured HBM |", "|---|---|---|---|---|", *pack_rows, ""]
    with open(args.report, "w") as f:
        f.write("\n".join(out))
    print("\n".join(out))


def run_sharded_report(args):
    """The 70B-style configuration, N-sharded over the ranks of this job with the peer-store gather
    (``--sharded-report PATH`` under torch.distributed.run).  Per (shape, M): device time of the sharded
    forward with and without the exchange, max over ranks; every timed forward is preceded by an L2 flush
    whose own cost is measured separately and subtracted."""
    import torch
    import torch.distributed as dist
    from libortho_b200 import _C_ops
    import workloads as wl
    from libortho_b200.sharded import shard_bounds
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pk = peaks()
    stream = torch.cuda.Stream(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    max_m, max_n = max(wl.CFG3_M), max(n for _, n in wl.CFG3_SHAPES)
    comm = _C_ops.Comm(rank, world, 2 * max_m * max_n, device=dev)
    if world > 1:
        comm.connect_group()
    rows = []

    def timed(fn, n):
        with torch.cuda.stream(stream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for _ in range(n):
                    flush.fill_(1)
                    fn()
            g.replay()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g.replay()
            e1.record(stream)
            e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / n], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_flush = timed(lambda: None, 4)
    for (K, N) in wl.CFG3_SHAPES:
        full = wl.make_layer(K, N, wl.CFG3_DENSITY, seed=0, device=dev)
        n0, n1 = shard_bounds(N, world)[rank]
        L = full.rows(n0, n1) if world > 1 else full
        fb = {M: full.algorithmic_bytes(M) for M in wl.CFG3_M}
        ff = {M: full.algorithmic_flops(M) for M in wl.CFG3_M}
        del full
        torch.cuda.empty_cache()
        plan = _C_ops.Plan(L.row_ptr, L.col, L.vals, L.K, L.N)
        for M in wl.CFG3_M:
            x = wl.make_input(M, K, seed=M, device=dev)
            y = torch.empty(M, L.N, dtype=torch.float16, device=dev)
            ws = torch.empty(max(_C_ops.workspace_bytes(M, K, L.N, plan), 16), dtype=torch.uint8, device=dev)
            n = 4 if M <= 32 else 2
            t_local = timed(lambda: _C_ops.forward(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, y, 1.0,
                                                   plan=plan, workspace=ws), n) - t_flush
            t_gather = timed(lambda: _C_ops.forward_gather(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, 1.0,
                                                           comm, 0, N, n0, plan=plan, workspace=ws), n) - t_flush
            gbs, tf = fb[M] / t_gather / 1e3, ff[M] / t_gather / 1e6
            rows.append(f"| {K}->{N} | {M} | {world} | {t_local:.1f} | {t_gather:.1f} | {t_gather - t_local:.1f} | {M / t_gather * 1e6:.3g} | "
                        f"{gbs:.0f} | {100 * gbs / world / pk['hbm_gbs']:.1f} | {tf:.1f} | {100 * tf / world / pk['tf_sustained']:.1f} |")
            del x, y, ws
        del L, plan
        torch.cuda.empty_cache()
    if rank == 0:
        head = ("| shape K->N | M | GPUs | us, shard forward only | us, forward + output gather | exchange us | tokens/s | aggregate GB/s | "
                "% of measured HBM per GPU | aggregate TFLOP/s | % of measured sustained tensor per GPU |")
        out = [f"# 70B-style layers, N-sharded over {world} B200 with the peer-store output gather "
               "(`torch.distributed.run ... bench.py --sharded-report <path>`)", "",
               f"L2 flushed before every forward (256 MB fill, {t_flush:.1f} us, subtracted); device time, max over ranks.", "",
               head, "|" + "---|" * 11, *rows, ""]
        with open(args.sharded_report, "w") as f:
            f.write("\n".join(out))
        print("\n".join(out))
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_one(args):
    """``--one KxNxM``: a few forwards of one layer through the C ABI and nothing else, for profiler captures of a
    single kernel.  ``--density``, ``--alpha``, ``--zipf`` pick the ortho part."""
    import torch
    from libortho_b200 import _C_ops, _lib
    import workloads as wl
    K, N, M = [int(v) for v in args.one.lower().split("x")]
    dev = torch.device("cuda", 0)
    mk = wl.make_zipf_layer if args.zipf else wl.make_layer
    L = mk(K, N, args.density, seed=0, device=dev)
    plan = _C_ops.Plan(L.row_ptr, L.col, L.vals, K, N)
    x = wl.make_input(M, K, seed=M, device=dev)
    y = torch.empty(M, N, dtype=torch.float16, device=dev)
    ws = torch.empty(max(256, _C_ops.workspace_bytes(M, K, N, plan)), dtype=torch.uint8, device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.repeat + 1)]
    ev[0].record()
    for i in range(args.repeat):
        _C_ops.forward(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr, x, y, args.alpha, plan=plan, workspace=ws)
        ev[i + 1].record()
    torch.cuda.synchronize()
    us = [ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(args.repeat)]
    print(json.dumps({"one": args.one, "alpha": args.alpha, "density": args.density, "zipf": bool(args.zipf), "nnz": L.nnz,
                      "us_per_forward": [round(u, 1) for u in us], "algorithmic_bytes": L.algorithmic_bytes(M, args.alpha),
                      "algorithmic_flops": L.algorithmic_flops(M, args.alpha),
                      "kernel_status": int(_lib.lib().ortho_b200_query_kernel_status())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--steps-per-graph", type=int, default=64,
                    help="the timed steps are captured as CUDA graphs of at most this many steps each")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-regimes", action="store_true", help="skip the M=32 / M=4096 sweep over the same layers")
    ap.add_argument("--no-extras", action="store_true", help="skip the 7B-style decode sweep and the prefill configuration (N=1)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="multi-GPU output exchange: peer stores from the kernels, or an NCCL all-gather")
    ap.add_argument("--per-cta-signal", action="store_true",
                    help="peer exchange: every CTA signals the peers itself instead of the grid's last CTA")
    ap.add_argument("--no-deferred", action="store_true",
                    help="peer exchange: every forward waits for its own exchange instead of the next one waiting for it")
    ap.add_argument("--one", default=None, metavar="KxNxM", help="run a few forwards of one layer and exit (for profiling)")
    ap.add_argument("--density", type=float, default=0.003)
    ap.add_argument("--alpha", type=float, default=1.0)
    ap.add_argument("--zipf", action="store_true", help="--one: Zipf(1.2) row loads instead of uniform positions")
    ap.add_argument("--repeat", type=int, default=4)
    ap.add_argument("--report", default=None, metavar="PATH",
                    help="instead of the benchmark line: time every configuration on one GPU and write a markdown table")
    ap.add_argument("--sharded-report", default=None, metavar="PATH",
                    help="under torch.distributed.run: time the 70B-style layers sharded over the job's ranks, write a table")
    args = ap.parse_args()
    if args.one:
        run_one(args)
    elif args.sharded_report:
        run_sharded_report(args)
    elif args.report:
        run_report(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
