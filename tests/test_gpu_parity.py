"""Parity of the CUDA path (through the C ABI) with the CPU oracle.  All tests need a B200."""
import numpy as np
import pytest
import torch

from conftest import assert_close, errors, golden, layer_oracle
from cases import SMALL_CASES
from libortho_b200 import OrthoLinear, _C_ops, _lib
import workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_layer(layer, x, alpha, plan=True, ws=None):
    """Forward through the C ABI for a workloads.Layer living on the GPU."""
    y = torch.empty(x.shape[0], layer.N, dtype=torch.float16, device=x.device)
    p = _C_ops.Plan(layer.row_ptr, layer.col, layer.vals, layer.K, layer.N) if (plan and layer.nnz) else None
    _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, x, y, alpha,
                   plan=p, workspace=ws)
    torch.cuda.synchronize()
    return y


def test_native_library_is_loaded_and_counts_launches():
    assert _lib.lib().ortho_b200_version() == 100
    n0 = _lib.lib().ortho_b200_launch_count()
    layer = wl.make_layer(64, 64, 0.05, seed=1).to(DEV)
    run_layer(layer, wl.make_input(2, 64, seed=1).to(DEV), 1.0)
    assert _lib.lib().ortho_b200_launch_count() > n0


def test_int4_unpack_and_scale_bit_exact(oracle_mod):
    """Every byte value in every position, and a seeded layer: the kernels' in-register unpack and
    (float)w_int*scale must equal the oracle's integers and FP32 products bit for bit."""
    packed = torch.arange(256, dtype=torch.uint8).repeat(8, 2).reshape(8, 512).contiguous()
    scales = torch.tensor([0.5, 0.013, 1.0, 3e-4, 0.25, 7.1, 0.099, 1e-6], dtype=torch.float16)
    wi, wd = _C_ops.dequant_dump(packed.to(DEV), scales.to(DEV))
    oi, od = oracle_mod.dequant(packed.numpy(), scales.float().numpy())
    assert np.array_equal(wi.cpu().numpy(), oi)
    assert np.array_equal(wd.cpu().numpy().view(np.uint32), od.view(np.uint32))
    layer = wl.make_layer(512, 96, 0.0, seed=21)
    wi, wd = _C_ops.dequant_dump(layer.base_weight.to(DEV), layer.base_scales.to(DEV))
    oi, od = oracle_mod.dequant(layer.base_weight.numpy(), layer.base_scales.float().numpy())
    assert np.array_equal(wi.cpu().numpy(), oi)
    assert np.array_equal(wd.cpu().numpy().view(np.uint32), od.view(np.uint32))


@pytest.mark.parametrize("kind,K,N,d", [("gauss", 256, 300, 0.03), ("zipf", 512, 257, 0.01), ("gauss", 4096, 128, 0.005)])
def test_sparse_index_decode_bit_exact(kind, K, N, d):
    layer = wl.make_layer(K, N, d, seed=31, ortho=kind).to(DEV)
    plan = _C_ops.Plan(layer.row_ptr, layer.col, layer.vals, K, N)
    rows, cols, vals = plan.decode_dump()
    torch.cuda.synchronize()
    counts = (layer.row_ptr[1:] - layer.row_ptr[:-1]).long()
    exp_rows = torch.repeat_interleave(torch.arange(N, device=DEV), counts).to(torch.int32)
    assert torch.equal(rows, exp_rows) and torch.equal(cols, layer.col)
    assert torch.equal(vals.view(torch.int16), layer.vals.view(torch.int16))
    assert plan.max_row_nnz == int(counts.max())


def _kat_csr(g):
    """The reference test's coordinate draw as CSR: duplicates merged by summation (what the
    oracle's one-entry-at-a-time accumulation amounts to)."""
    dense = np.zeros(64 * 64, dtype=np.float32)
    np.add.at(dense, g["idx16"].astype(np.int64), g["vals"])
    w = torch.from_numpy(dense.reshape(64, 64))
    from libortho_b200.sieve import pack_ortho_sparse
    rp, col, val = pack_ortho_sparse(w, "csr")
    return rp, col, val.to(torch.float16)


def test_known_answer_cases_of_the_reference_test(oracle_mod):
    """tests/test_cpu_forward.c replayed through the CUDA path: alpha=1, alpha=0, empty ortho."""
    g = golden("kat_cpu_forward.npz")
    rp, col, val = _kat_csr(g)
    layer = wl.Layer(64, 64, torch.from_numpy(g["packed"]), torch.from_numpy(g["scales"]).to(torch.float16),
                     rp, col, val, 1.0)
    x = torch.from_numpy(g["x"]).to(torch.float16)
    ld = layer.to(DEV)
    for alpha, key in ((1.0, "y_alpha1"), (0.0, "y_alpha0")):
        y = run_layer(ld, x.to(DEV), alpha).float().cpu().numpy()
        # against the oracle fed the same FP16-rounded operands
        assert_close(y, layer_oracle(oracle_mod, layer, x, alpha), key)
        # and against the reference's recorded FP32 outputs (inputs differ by FP16 rounding only)
        rel, mx = errors(y, g[key])
        assert rel <= 2e-3 and mx <= 5e-2, (key, rel, mx)
    empty = wl.Layer(64, 64, ld.base_weight, ld.base_scales, torch.zeros(65, dtype=torch.int32, device=DEV),
                     ld.col[:0], ld.vals[:0], 1.0)
    y_e = run_layer(empty, x.to(DEV), 1.0)
    y_0 = run_layer(ld, x.to(DEV), 0.0)
    assert torch.equal(y_e, y_0)


def test_null_test_base_only(oracle_mod):
    g = golden("null_test_small.npz")
    m = OrthoLinear(128, 128).to(DEV)
    m.base_weight = torch.from_numpy(g["packed"]).to(DEV)
    m.base_scales = torch.from_numpy(g["scales"]).to(torch.float16).to(DEV)
    x = torch.from_numpy(g["x"]).to(torch.float16)
    y = m(x.to(DEV)).float().cpu().numpy()
    ref = oracle_mod.forward_csr(g["packed"], m.base_scales.float().cpu().numpy(), None, None, None,
                                 x.float().numpy(), 0.0)
    assert_close(y, ref, "null test")


@pytest.mark.parametrize("name", list(SMALL_CASES))
@pytest.mark.parametrize("plan", [True, False])
def test_seeded_small_layers_against_golden(name, plan):
    K, N, M, d, kind, seed, alphas = SMALL_CASES[name]
    g = golden("cfg_small.npz")
    layer = wl.make_layer(K, N, d, seed=seed, ortho=kind).to(DEV)
    x = wl.make_input(M, K, seed=seed).to(DEV)
    for a in alphas:
        y = run_layer(layer, x, a, plan=plan)
        assert_close(y.float().cpu().numpy(), g[f"{name}_a{a}"], f"{name} alpha={a} plan={plan}")


def test_single_layer_config_against_golden():
    """4096x4096, M=8, 1 % residual ortho, alpha in {0, 1}: the reference's CPU-runnable case."""
    g = golden("cfg0_y.npz")
    layer = wl.make_layer(4096, 4096, 0.01, seed=0, ortho="residual10").to(DEV)
    x = wl.make_input(8, 4096, seed=0).to(DEV)
    m = layer.to_module()
    for a, key in ((1.0, "y_alpha1"), (0.0, "y_alpha0")):
        m.set_alpha(a)
        assert_close(m(x).float().cpu().numpy(), g[key], key)
    # alpha = 0 must equal the base-only output exactly (bitwise), with or without stored entries
    m.set_alpha(0.0)
    y0 = m(x)
    base_only = wl.Layer(4096, 4096, layer.base_weight, layer.base_scales,
                         torch.zeros(4097, dtype=torch.int32, device=DEV), layer.col[:0], layer.vals[:0], 1.0)
    assert torch.equal(y0, run_layer(base_only, x, 1.0))
    m.set_alpha(-2.0)
    assert torch.equal(y0, m(x))


@pytest.mark.parametrize("cfg", [(1, 8, 4, 1), (1, 8, 2, 2), (2, 4, 4, 4), (4, 2, 2, 8), (8, 1, 4, 2),
                                 (1, 4, 4, 1), (2, 2, 2, 4), (1, 8, 4, 8)])
@pytest.mark.parametrize("M", [1, 5, 16, 33, 64])
def test_every_decode_tiling_agrees_with_the_oracle(oracle_mod, cfg, M):
    K, N = 1184, 210                      # ragged in both directions (K % 128 != 0, N % 16 != 0)
    layer = wl.make_layer(K, N, 0.02, seed=41)
    x = wl.make_input(M, K, seed=41)
    ref = layer_oracle(oracle_mod, layer, x, 0.75)
    try:
        assert _lib.lib().ortho_b200_set_decode_config(-3, 0, 0, 64) == 0      # keep 33 and 64 tokens on this kernel
        assert _lib.lib().ortho_b200_set_decode_config(*cfg) == 0
        y = run_layer(layer.to(DEV), x.to(DEV), 0.75)
    finally:
        _lib.lib().ortho_b200_set_decode_config(0, 0, 0, 0)
        _lib.lib().ortho_b200_set_decode_config(-3, 0, 0, 24)
    assert_close(y.float().cpu().numpy(), ref, f"cfg={cfg} M={M}")


@pytest.mark.parametrize("K,N", wl.CFG1_SHAPES)
def test_decode_sweep_shapes_against_oracle(oracle_mod, K, N):
    """Llama-7B-style shapes at M in {1,4,16}: full output against the oracle for a row sample
    (rows are independent: a row subset of the layer is a smaller layer with the same arithmetic)."""
    layer = wl.make_layer(K, N, wl.CFG1_DENSITY, seed=51, device=DEV)
    rows = sorted({0, 1, 15, 16, 127, N // 2, N - 17, N - 1} | set(range(N // 3, N // 3 + 40)))
    cpu = layer.to("cpu")
    for M in wl.CFG1_M:
        x = wl.make_input(M, K, seed=M, device=DEV)
        y = run_layer(layer, x, 1.0).float().cpu().numpy()
        sub = [cpu.rows(r, r + 1) for r in rows]
        ref = np.concatenate([layer_oracle(oracle_mod, s, x.cpu(), 1.0, threads=1) for s in sub], axis=1)
        assert_close(y[:, rows], ref, f"{K}->{N} M={M}")
        assert np.isfinite(y).all()


def sampled_oracle(oracle_mod, cpu_layer, rows, x_cpu, alpha):
    """Oracle output for the listed rows (rows are independent in the reference, src/ortho.c:354-366:
    a one-row slice of the layer is a smaller layer with the same arithmetic) and the given tokens."""
    sub = [cpu_layer.rows(r, r + 1) for r in rows]
    return np.concatenate([layer_oracle(oracle_mod, s_, x_cpu, alpha, threads=1) for s_ in sub], axis=1)


@pytest.mark.parametrize("K,N", wl.CFG3_SHAPES)
def test_sharded_config_shapes_against_oracle(oracle_mod, K, N):
    """Llama-70B-style shapes (0.3 % ortho) at M in {1, 32, 4096}: a row sample of the output against
    the oracle, for all tokens at M <= 32 and for a seeded token sample at M = 4096 (tokens and rows
    are independent in the reference: src/ortho.c:346-349, 354-366)."""
    layer = wl.make_layer(K, N, wl.CFG3_DENSITY, seed=71, device=DEV)
    rows = sorted({0, 17, 127, 128, N // 2 + 3, N - 129, N - 1} | set(range(N // 5, N // 5 + 24)))
    cpu = layer.to("cpu")
    sub = [cpu.rows(r, r + 1) for r in rows]
    g = torch.Generator().manual_seed(7)
    for M in (1, 32, 4096):
        x = wl.make_input(M, K, seed=M, device=DEV)
        y = run_layer(layer, x, 1.0)
        toks = list(range(M)) if M <= 32 else sorted(torch.randperm(M, generator=g)[:64].tolist())
        xs = x[toks].cpu()
        ref = np.concatenate([layer_oracle(oracle_mod, s_, xs, 1.0, threads=1) for s_ in sub], axis=1)
        got = y[toks][:, rows].float().cpu().numpy()
        assert_close(got, ref, f"{K}->{N} M={M}")
        assert bool(torch.isfinite(y).all())
        del x, y
    torch.cuda.empty_cache()


def test_linearity_and_alpha_properties_at_full_size():
    """Size-independent properties on a full decode-sweep layer: Y(alpha) - Y(0) is linear in alpha,
    and the forward is additive over token rows (each row is computed independently)."""
    layer = wl.make_layer(4096, 12288, wl.CFG1_DENSITY, seed=61, device=DEV)
    x = wl.make_input(16, 4096, seed=61, device=DEV)
    y0 = run_layer(layer, x, 0.0).float()
    y1 = run_layer(layer, x, 1.0).float()
    yh = run_layer(layer, x, 0.5).float()
    d1, dh = (y1 - y0), (yh - y0)
    assert (d1.abs().max() > 0.05)
    assert torch.allclose(dh, 0.5 * d1, atol=1.5e-2, rtol=0)
    for M in (1, 4):
        ym = run_layer(layer, x[:M].contiguous(), 1.0).float()
        assert torch.allclose(ym, y1[:M], atol=4e-3, rtol=2e-3)


def test_module_forward_shapes_bias_and_dtype():
    layer = wl.make_layer(256, 96, 0.05, seed=71, device=DEV)
    m = layer.to_module()
    x = wl.make_input(6, 256, seed=71, device=DEV).reshape(2, 3, 256)
    y = m(x)
    assert y.shape == (2, 3, 96) and y.dtype == torch.float16
    mb = OrthoLinear(256, 96, bias=True).to(DEV)
    mb.load_state_dict({**m.state_dict(), "bias": torch.full((96,), 0.5)})
    assert torch.allclose(mb(x).float(), y.float() + 0.5, atol=2e-3)
    yb = m(x.to(torch.bfloat16))
    assert yb.dtype == torch.bfloat16
    assert m(x[:0]).shape == (0, 3, 96)
    # fresh module (zero-length ortho buffers) is legal: base only, all-zero weights -> zeros
    fresh = OrthoLinear(256, 96).to(DEV)
    assert torch.count_nonzero(fresh(x)) == 0


def test_error_statuses_surface_as_exceptions():
    layer = wl.make_layer(64, 32, 0.05, seed=81, device=DEV)
    x = wl.make_input(2, 64, seed=81, device=DEV)
    y = torch.empty(2, 32, dtype=torch.float16, device=DEV)
    other = _C_ops.Plan(layer.row_ptr[:17].contiguous(), layer.col[:int(layer.row_ptr[16])].contiguous(),
                        layer.vals[:int(layer.row_ptr[16])].contiguous(), 64, 16)
    with pytest.raises(_lib.OrthoB200Error, match="plan"):
        _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, x, y, 1.0, plan=other)
    with pytest.raises(TypeError):
        _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, x.float(), y, 1.0)
    xm = torch.empty(2, 65, dtype=torch.float16, device=DEV)[:, 1:]
    with pytest.raises(ValueError):
        _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, xm, y, 1.0)
    # K not a multiple of 32 is rejected by the library, not silently handled
    st = _lib.lib().ortho_b200_forward(layer.base_weight.data_ptr(), layer.base_scales.data_ptr(), None, None, None, 0,
                                       x.data_ptr(), y.data_ptr(), 2, 48, 32, 1.0, None, None, 0, None)
    assert st == 2
    torch.cuda.synchronize()


@pytest.mark.parametrize("K,N,M", [(384, 200, 200), (1024, 272, 130), (4096, 512, 257), (64, 64, 65), (2048, 1024, 1024)])
def test_tensor_core_path_base_only_against_oracle(oracle_mod, K, N, M):
    """More than 24 tokens on a layer this wide take the tcgen05 kernel.  alpha = 0: base term only, ragged
    tiles in M, N and K."""
    layer = wl.make_layer(K, N, 0.01, seed=91)
    x = wl.make_input(M, K, seed=91)
    y = run_layer(layer.to(DEV), x.to(DEV), 0.0).float().cpu().numpy()
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    assert_close(y, layer_oracle(oracle_mod, layer, x, 0.0), f"prefill base {K}x{N} M={M}")
    # the same rows through the streaming kernel (64-token calls) agree to FP16 rounding
    y64 = run_layer(layer.to(DEV), x[:64].contiguous().to(DEV), 0.0).float().cpu().numpy()
    assert np.abs(y[:64] - y64).max() <= 2e-2


@pytest.mark.parametrize("kind,K,N,M,d,alpha,plan", [
    ("zipf", 2048, 384, 300, 0.02, 0.5, True),      # rows long enough for the plan's tensor-core pre-pass
    ("zipf", 2048, 384, 300, 0.02, 0.5, False),     # same through raw CSR (no plan)
    ("gauss", 1024, 520, 129, 0.01, 1.0, True),
    ("gauss", 4096, 256, 513, 0.003, 0.25, True),
])
def test_tensor_core_path_with_sparse_term_against_oracle(oracle_mod, kind, K, N, M, d, alpha, plan):
    layer = wl.make_layer(K, N, d, seed=93, ortho=kind)
    x = wl.make_input(M, K, seed=93)
    if kind == "zipf":
        assert int((layer.row_ptr[1:] - layer.row_ptr[:-1]).max()) > 512
    y = run_layer(layer.to(DEV), x.to(DEV), alpha, plan=plan).float().cpu().numpy()
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    assert_close(y, layer_oracle(oracle_mod, layer, x, alpha), f"prefill fused {kind} {K}x{N} M={M}")
    # alpha = 0 on the same layer is bit-identical to the layer without any entries
    y0 = run_layer(layer.to(DEV), x.to(DEV), 0.0, plan=plan)
    empty = wl.Layer(K, N, layer.base_weight.to(DEV), layer.base_scales.to(DEV),
                     torch.zeros(N + 1, dtype=torch.int32, device=DEV), layer.col[:0].to(DEV), layer.vals[:0].to(DEV), 1.0)
    assert torch.equal(y0, run_layer(empty, x.to(DEV), 1.0))
    # a missing workspace is an error status, not a silent fallback
    with pytest.raises(_lib.OrthoB200Error, match="workspace"):
        ld = layer.to(DEV)
        yy = torch.empty(M, N, dtype=torch.float16, device=DEV)
        st = _lib.lib().ortho_b200_forward(ld.base_weight.data_ptr(), ld.base_scales.data_ptr(), ld.vals.data_ptr(),
                                           ld.col.data_ptr(), ld.row_ptr.data_ptr(), ld.nnz, x.to(DEV).data_ptr(),
                                           yy.data_ptr(), M, K, N, alpha, None, None, 0, None)
        _lib.check(st, "ortho_b200_forward")


@pytest.mark.parametrize("M", wl.CFG2_M)
def test_prefill_configuration_at_its_own_shape(oracle_mod, M):
    """8192 x 8192, 0.1 % ortho with Zipf(1.2) row loads, alpha = 0.5, exactly as the benchmark builds it, with
    plan and full workspace (the long rows' tensor-core pre-pass and the split-K of the last wave are both live): the longest
    rows, tile-edge rows and a seeded row sample against the oracle for a seeded token sample."""
    K, N = wl.CFG2_SHAPE
    layer = wl.make_zipf_layer(K, N, wl.CFG2_DENSITY, seed=0, device=DEV, alpha=wl.CFG2_ALPHA)
    cpu = layer.to("cpu")
    counts = (cpu.row_ptr[1:] - cpu.row_ptr[:-1]).long()
    assert int(counts.max()) > 4096                      # the head of the Zipf law is really there
    g = torch.Generator().manual_seed(11)
    rows = sorted(set(torch.topk(counts, 8).indices.tolist()) | {0, 127, 128, N - 129, N - 1}
                  | set(torch.randperm(N, generator=g)[:40].tolist()))
    plan = _C_ops.Plan(layer.row_ptr, layer.col, layer.vals, K, N)
    ws = torch.empty(_C_ops.workspace_bytes(M, K, N, plan), dtype=torch.uint8, device=DEV)
    x = wl.make_input(M, K, seed=M, device=DEV)
    y = torch.empty(M, N, dtype=torch.float16, device=DEV)
    _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, x, y, wl.CFG2_ALPHA,
                   plan=plan, workspace=ws)
    torch.cuda.synchronize()
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    toks = sorted({0, 255, 256, M - 1} | set(torch.randperm(M, generator=g)[:60].tolist()))
    ref = sampled_oracle(oracle_mod, cpu, rows, x[toks].cpu(), wl.CFG2_ALPHA)
    assert_close(y[toks][:, rows].float().cpu().numpy(), ref, f"prefill configuration M={M}")
    assert bool(torch.isfinite(y).all())
    # base only: bit-identical to the layer without entries (the kill switch)
    y0 = torch.empty_like(y)
    _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, x, y0, 0.0, plan=plan, workspace=ws)
    ye = torch.empty_like(y)
    _C_ops.forward(layer.base_weight, layer.base_scales, None, None, None, x, ye, 1.0, workspace=ws)
    assert torch.equal(y0, ye)


@pytest.mark.parametrize("variant", ["threshold", "top1pct"])
def test_sieve_derived_layer_alpha_sweep(oracle_mod, variant):
    """Sieve-derived split (W ~ N(0, 0.02^2), low-rank-plus-noise calibration, curvature threshold 10): the
    threshold leaves the ortho part empty, so every alpha must give the same bits; the keep-top-1 % variant
    exercises a sieve-shaped non-empty ortho.  M in {1, 2048}, alpha in {0, 0.25, 0.5, 1} against the oracle."""
    cpu = wl.make_sieve_layer() if variant == "threshold" else wl.make_sieve_layer(sparsity_target=0.01)
    assert (cpu.nnz == 0) == (variant == "threshold")
    layer = cpu.to(DEV)
    K, N = cpu.K, cpu.N
    g = torch.Generator().manual_seed(13)
    rows = sorted({0, 15, 16, 127, 128, N - 1} | set(torch.randperm(N, generator=g)[:40].tolist()))
    for M in (1, 2048):
        x = wl.make_input(M, K, seed=M, device=DEV)
        toks = list(range(M)) if M <= 64 else sorted({0, 255, 256, M - 1} | set(torch.randperm(M, generator=g)[:60].tolist()))
        outs = {}
        for alpha in (0.0, 0.25, 0.5, 1.0):
            y = run_layer(layer, x, alpha)
            assert _lib.lib().ortho_b200_query_kernel_status() == 0
            ref = sampled_oracle(oracle_mod, cpu, rows, x[toks].cpu(), alpha)
            assert_close(y[toks][:, rows].float().cpu().numpy(), ref, f"sieve {variant} M={M} alpha={alpha}")
            outs[alpha] = y
        if cpu.nnz == 0:
            for alpha in (0.25, 0.5, 1.0):
                assert torch.equal(outs[alpha], outs[0.0])
        else:
            d1 = (outs[1.0].float() - outs[0.0].float())
            assert d1.abs().max() > 1e-3
            assert torch.allclose(outs[0.5].float() - outs[0.0].float(), 0.5 * d1, atol=1.5e-2, rtol=0)


@pytest.mark.parametrize("M,K,N", [(1, 512, 208), (7, 1024, 96), (16, 256, 144), (20, 384, 80), (40, 512, 272), (300, 256, 520)])
def test_bias_is_added_inside_the_kernels(oracle_mod, M, K, N):
    """Every kernel family adds the FP32 bias in its FP32 epilogue (one FP16 rounding): against the oracle's
    FP32 output plus the bias (the reference adds it after the kernel, torch_bind/ortho_linear.py:164-166)."""
    layer = wl.make_layer(K, N, 0.02, seed=200 + M)
    x = wl.make_input(M, K, seed=200 + M)
    g = torch.Generator().manual_seed(M)
    bias = torch.randn(N, generator=g)
    m = layer.to(DEV).to_module()
    mb = OrthoLinear(K, N, bias=True).to(DEV)
    mb.load_state_dict({**m.state_dict(), "bias": bias})
    mb.set_alpha(0.75)
    y = mb(x.to(DEV)).detach().float().cpu().numpy()
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    ref = layer_oracle(oracle_mod, layer, x, 0.75) + bias.numpy()[None, :]
    assert_close(y, ref, f"bias M={M}")
    # a bias that is not FP32 still works (added after the kernel, as the reference does)
    mb.bias.data = mb.bias.data.to(torch.float16)
    y16 = mb(x.to(DEV)).detach().float().cpu().numpy()
    assert np.abs(y16 - ref).max() <= 5e-2


@pytest.mark.parametrize("M,K,Ns", [(1, 4096, (512, 128, 128)), (4, 1024, (208, 96)), (16, 512, (144, 272, 80, 48)),
                                    (8, 2048, (1000,)), (40, 512, (144, 96))])
def test_layers_that_share_the_activations_in_one_call(oracle_mod, M, K, Ns):
    """Separate projections over the same input (Q / K / V, gate / up) through ortho_b200_forward_multi: up to 16
    tokens the tiles of all layers are walked by one launch.  Each member against the oracle with its own alpha
    and bias, and bit-identical to its own single-layer forward."""
    layers = [wl.make_layer(K, N, 0.02 if i != 1 else 0.0, seed=300 + i + M).to(DEV) for i, N in enumerate(Ns)]
    alphas = [1.0, 0.5, 0.0, 0.25][:len(Ns)]
    g = torch.Generator().manual_seed(M)
    biases = [torch.randn(N, generator=g).to(DEV) if i % 2 == 0 else None for i, N in enumerate(Ns)]
    x = wl.make_input(M, K, seed=300 + M).to(DEV)
    outs = [torch.empty(M, N, dtype=torch.float16, device=DEV) for N in Ns]
    n0 = _lib.lib().ortho_b200_launch_count()
    _C_ops.forward_multi([(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr) for L in layers], x, outs,
                         alphas=alphas, biases=biases)
    launches = _lib.lib().ortho_b200_launch_count() - n0
    torch.cuda.synchronize()
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    if M <= 16 and K % 256 == 0 and len(Ns) > 1:
        assert launches == 1
    for L, a, b, y in zip(layers, alphas, biases, outs):
        ref = layer_oracle(oracle_mod, L.to("cpu"), x.cpu(), a)
        if b is not None:
            ref = ref + b.cpu().numpy()[None, :]
        assert_close(y.float().cpu().numpy(), ref, f"multi M={M} N={L.N} alpha={a}")
        y1 = torch.empty_like(y)
        _C_ops.forward_multi([(L.base_weight, L.base_scales, L.vals, L.col, L.row_ptr)], x, [y1], alphas=[a], biases=[b])
        assert torch.equal(y1, y)


def test_swapped_model_runs_and_the_kill_switch_works():
    """nn.Linear layers swapped for OrthoLinear: alpha = 1 is close to the dense model (INT4 base + residual),
    alpha = 0 equals the INT4-only model bit for bit whatever the ortho part holds."""
    import torch.nn as nn
    from libortho_b200 import set_alpha_all, swap_linear
    from libortho_b200.convert import base_only_split, sieve_split
    g = torch.Generator().manual_seed(17)
    dense = nn.Sequential(nn.Linear(256, 512, bias=True), nn.GELU(), nn.Linear(512, 128, bias=False)).to(DEV)
    with torch.no_grad():
        for p_ in dense.parameters():
            p_.copy_((torch.randn(p_.shape, generator=g) * 0.02).to(DEV))
    x = wl.make_input(5, 256, seed=17).to(DEV)
    y_dense = dense(x.float())
    import copy
    a, b = copy.deepcopy(dense), copy.deepcopy(dense)
    hd = {"0": torch.ones(256), "2": torch.ones(512)}
    swap_linear(a, sieve_split(hd, sparsity_target=0.05))
    swap_linear(b, base_only_split)
    ya = a(x)
    assert ya.dtype == torch.float16 and (ya.float() - y_dense).abs().max() < 0.1
    # the sieve's base lies on the same INT4 grid as the base-only split (the re-derived FP32 scale may differ in
    # its last bit): with the switch off both models agree to FP16 rounding, whatever the ortho part holds
    set_alpha_all(a, 0.0)
    assert (a(x).float() - b(x).float()).abs().max() < 4e-3
    y_off = a(x)
    for mod in a.modules():
        if isinstance(mod, OrthoLinear):
            mod.ortho_values = mod.ortho_values[:0]
    assert torch.equal(a(x), y_off)


@pytest.mark.parametrize("M,K,N,d,kind,alpha", [
    (1, 256, 256, 0.02, "gauss", 1.0), (16, 4096, 1100, 0.005, "gauss", 1.0), (32, 1024, 300, 0.02, "zipf", 0.5),
    (33, 512, 520, 0.01, "gauss", 0.25), (64, 2048, 96, 0.01, "gauss", 1.0), (128, 384, 272, 0.02, "gauss", 1.0),
    (100, 1184, 210, 0.02, "gauss", 0.75), (9, 8192, 2048, 0.003, "gauss", 1.0), (32, 11008, 512, 0.005, "gauss", 1.0),
    (48, 4096, 4352, 0.003, "gauss", 0.0)])
def test_tokens_as_m_kernel_against_oracle(oracle_mod, M, K, N, d, kind, alpha):
    """The tcgen05 kernel whose M operand is the token block (up to 128 tokens, 256 weight rows per MMA, stream-K
    split with partial sums in the workspace) through the tuning hook: ragged M / N / K, shares that start inside
    a row tile, long Zipf rows, bias, and the kill switch."""
    layer = wl.make_layer(K, N, d, seed=400 + M, ortho=kind)
    x = wl.make_input(M, K, seed=400 + M)
    g = torch.Generator().manual_seed(M)
    bias = torch.randn(N, generator=g)
    ld = layer.to(DEV)
    try:
        assert _lib.lib().ortho_b200_set_decode_config(-4, 0, 0, 128) == 0
        launches = {}
        ys = {}
        for use_bias in (False, True):
            y = torch.empty(M, N, dtype=torch.float16, device=DEV)
            n0 = _lib.lib().ortho_b200_launch_count()
            _C_ops.forward_multi([(ld.base_weight, ld.base_scales, ld.vals, ld.col, ld.row_ptr)], x.to(DEV), [y], alphas=[alpha],
                                 biases=[bias.to(DEV) if use_bias else None])
            torch.cuda.synchronize()
            launches[use_bias] = _lib.lib().ortho_b200_launch_count() - n0
            ys[use_bias] = y
        y0 = run_layer(ld, x.to(DEV), 0.0)
    finally:
        _lib.lib().ortho_b200_set_decode_config(-4, 0, 0, 0)
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    ref = layer_oracle(oracle_mod, layer, x, alpha)
    assert_close(ys[False].float().cpu().numpy(), ref, f"tokens-as-M M={M} {K}->{N}")
    assert_close(ys[True].float().cpu().numpy(), ref + bias.numpy()[None, :], f"tokens-as-M + bias M={M} {K}->{N}")
    assert launches[False] == (3 if (alpha > 0 and layer.nnz) else 1)       # transpose + sparse pre-pass + the MMA kernel
    empty = wl.Layer(K, N, ld.base_weight, ld.base_scales, torch.zeros(N + 1, dtype=torch.int32, device=DEV), ld.col[:0], ld.vals[:0], 1.0)
    try:
        _lib.lib().ortho_b200_set_decode_config(-4, 0, 0, 128)
        ye = run_layer(empty, x.to(DEV), 1.0)
    finally:
        _lib.lib().ortho_b200_set_decode_config(-4, 0, 0, 0)
    assert torch.equal(y0, ye)


def _force_gathers(on: bool):
    """Tuning hook -6: k_split = 0 makes the tensor-core kernels gather the sparse term instead of folding it into
    the weight tile."""
    assert _lib.lib().ortho_b200_set_decode_config(-6, 0, 0, 0 if on else 1) == 0


@pytest.mark.parametrize("K,N,M,d", [(1024, 520, 300, 0.01), (4096, 256, 513, 0.003), (2048, 384, 1500, 0.02),
                                     (1184, 210, 300, 0.02), (96, 130, 257, 0.05)])
def test_sparse_term_folded_into_the_weights_and_as_gathers(oracle_mod, K, N, M, d):
    """With a plan whose rows are in column order the tensor-core kernel adds the sparse entries to its weight tile;
    the same forward with that switched off gathers them from the transposed activations.  Both against the oracle,
    and against each other within FP16 rounding of the weight tile."""
    layer = wl.make_layer(K, N, d, seed=7)
    assert _C_ops.Plan(*(t.to(DEV) for t in (layer.row_ptr, layer.col, layer.vals)), K, N).rows_ordered
    x = wl.make_input(M, K, seed=7)
    ref = layer_oracle(oracle_mod, layer, x, 0.75)
    ya = run_layer(layer.to(DEV), x.to(DEV), 0.75)
    try:
        _force_gathers(True)
        yb = run_layer(layer.to(DEV), x.to(DEV), 0.75)
    finally:
        _force_gathers(False)
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    assert_close(ya.float().cpu().numpy(), ref, f"folded {K}x{N} M={M}")
    assert_close(yb.float().cpu().numpy(), ref, f"gathered {K}x{N} M={M}")
    rel, mx = errors(ya.float().cpu().numpy(), yb.float().cpu().numpy())
    assert rel <= 5e-4, rel


def test_rows_that_cannot_be_folded_keep_the_gather_path(oracle_mod):
    """Rows with a zero or tiny scale and large sparse values (v * alpha / scale outside FP16) are gathered by the
    epilogue warps straight from X; rows with unordered columns make the whole plan take the gather path."""
    K, N, M = 1024, 300, 260
    layer = wl.make_layer(K, N, 0.01, seed=21)
    scales = layer.base_scales.clone()
    scales[5] = 0.0
    scales[130] = 1e-6
    scales[131] = 6e-8
    scales[299] = 1e-6
    layer = wl.Layer(K, N, layer.base_weight, scales, layer.row_ptr, layer.col, layer.vals, 1.0)
    counts = layer.row_ptr[1:] - layer.row_ptr[:-1]
    assert all(int(counts[r]) > 0 for r in (5, 130, 131, 299))
    x = wl.make_input(M, K, seed=21)
    ref = layer_oracle(oracle_mod, layer, x, 1.0)
    y = run_layer(layer.to(DEV), x.to(DEV), 1.0)
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    assert bool(torch.isfinite(y).all())
    assert_close(y.float().cpu().numpy(), ref, "rows outside the FP16 range of the weight tile")
    # the same entries with every row's columns reversed: an unordered plan
    col, vals = layer.col.clone(), layer.vals.clone()
    rp = layer.row_ptr.tolist()
    for n in range(N):
        col[rp[n]:rp[n + 1]] = layer.col[rp[n]:rp[n + 1]].flip(0)
        vals[rp[n]:rp[n + 1]] = layer.vals[rp[n]:rp[n + 1]].flip(0)
    rev = wl.Layer(K, N, layer.base_weight, scales, layer.row_ptr, col, vals, 1.0)
    assert not _C_ops.Plan(*(t.to(DEV) for t in (rev.row_ptr, rev.col, rev.vals)), K, N).rows_ordered
    y2 = run_layer(rev.to(DEV), x.to(DEV), 1.0)
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    assert_close(y2.float().cpu().numpy(), ref, "plan with unordered rows")


@pytest.mark.parametrize("M,K,N,d", [(32, 1024, 520, 0.01), (100, 4096, 300, 0.003), (128, 2048, 1100, 0.02), (48, 8192, 2048, 0.003),
                                     (100, 1184, 210, 0.02), (17, 96, 130, 0.05)])
def test_tokens_as_m_kernel_folds_the_sparse_term(oracle_mod, M, K, N, d):
    """17..128 tokens with a plan and a workspace: the tokens-as-M kernel adds the sparse entries to its weight tile
    (one launch, shares that start inside a row), gathers the rows whose scale is zero or tiny in its epilogue, and
    agrees with the oracle and with the gather form (transpose + sparse pre-pass + the MMA kernel)."""
    layer = wl.make_layer(K, N, d, seed=900 + M)
    scales = layer.base_scales.clone()
    counts = layer.row_ptr[1:] - layer.row_ptr[:-1]
    special = [r for r in (3, 255, 256, N - 1) if r < N and int(counts[r]) > 0]
    assert special
    for i, r in enumerate(special):
        scales[r] = 0.0 if i % 2 == 0 else 1e-6
    layer = wl.Layer(K, N, layer.base_weight, scales, layer.row_ptr, layer.col, layer.vals, 1.0)
    ld = layer.to(DEV)
    x = wl.make_input(M, K, seed=900 + M)
    plan = _C_ops.Plan(ld.row_ptr, ld.col, ld.vals, K, N)
    assert plan.rows_ordered
    ws = torch.empty(_C_ops.workspace_bytes(M, K, N, plan), dtype=torch.uint8, device=DEV)
    ref = layer_oracle(oracle_mod, layer, x, 0.75)

    def run():
        y = torch.empty(M, N, dtype=torch.float16, device=DEV)
        n0 = _lib.lib().ortho_b200_launch_count()
        _C_ops.forward(ld.base_weight, ld.base_scales, ld.vals, ld.col, ld.row_ptr, x.to(DEV), y, 0.75, plan=plan, workspace=ws)
        torch.cuda.synchronize()
        return y, _lib.lib().ortho_b200_launch_count() - n0

    try:
        assert _lib.lib().ortho_b200_set_decode_config(-4, 0, 0, 128) == 0
        ya, la = run()
        _force_gathers(True)
        yb, lb = run()
    finally:
        _force_gathers(False)
        _lib.lib().ortho_b200_set_decode_config(-4, 0, 0, 0)
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    assert (la, lb) == (1, 3)
    assert bool(torch.isfinite(ya).all())
    assert_close(ya.float().cpu().numpy(), ref, f"tokens-as-M folded M={M} {K}->{N}")
    assert_close(yb.float().cpu().numpy(), ref, f"tokens-as-M gathered M={M} {K}->{N}")


def test_forward_into_a_caller_buffer():
    """``OrthoLinear.forward(x, out=...)`` writes into the given FP16 buffer (a slice of a larger one) and returns a
    view of it; the values equal the allocating call's."""
    layer = wl.make_layer(1024, 272, 0.01, seed=5).to(DEV)
    m = layer.to_module()
    x = wl.make_input(7, 1024, seed=5).to(DEV)
    big = torch.zeros(3 * 7 * 272, dtype=torch.float16, device=DEV)
    out = big[7 * 272: 2 * 7 * 272]
    y = m(x, out=out)
    torch.cuda.synchronize()
    assert y.data_ptr() == out.data_ptr() and tuple(y.shape) == (7, 272)
    assert torch.equal(y, m(x))
    assert float(big[:7 * 272].abs().max()) == 0.0 and float(big[2 * 7 * 272:].abs().max()) == 0.0
    with pytest.raises(RuntimeError, match="out must be"):
        m(x, out=big[:10])
