"""Host-side logic: packer and sieve parity with the reference's Python, module surface, the
C-ABI library's exports (no GPU, no compute calls)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT, golden
from libortho_b200 import OrthoLinear, _lib, sieve
import workloads as wl


def test_packer_matches_reference_buffers():
    g = golden("packer_small.npz")
    m = OrthoLinear(64, 48)
    m.load_from_weights(torch.from_numpy(g["w_base"]), torch.from_numpy(g["w_ortho"]))
    assert np.array_equal(m.base_weight.numpy(), g["base_weight"])
    assert np.array_equal(m.base_scales.numpy(), g["base_scales"])
    assert np.array_equal(m.ortho_row_ptr.numpy(), g["ortho_row_ptr"])
    assert np.array_equal(m.ortho_col_indices.numpy(), g["ortho_col_indices"])
    assert np.array_equal(m.ortho_values.numpy(), g["ortho_values"])
    assert m.ortho_row_ptr.dtype == torch.int32 and m.ortho_values.dtype == torch.float16
    # workloads.quantize_pack is the same rule
    p, s, _ = wl.quantize_pack(torch.from_numpy(g["w_base"]))
    assert np.array_equal(p.numpy(), g["base_weight"]) and np.array_equal(s.numpy(), g["base_scales"])


def test_sieve_matches_reference_outputs():
    g = golden("packer_small.npz")
    W, X = torch.from_numpy(g["W"]), torch.from_numpy(g["X"])
    hd = sieve.compute_hessian_diag_approx(X)
    assert np.allclose(hd.numpy(), g["hdiag"], rtol=1e-6, atol=0)
    h_inv = 1.0 / torch.from_numpy(g["hdiag"])
    assert np.array_equal(sieve.quantize_int4(W).numpy(), g["wq"])
    wb, wo = sieve.hessian_sieve(W, h_inv, sparsity_target=0.05)
    assert np.array_equal(wb.numpy(), g["w_base"]) and np.array_equal(wo.numpy(), g["w_ortho"])
    wb, wo = sieve.hessian_sieve(W, torch.diag(h_inv), curvature_thresh=2e-6)
    assert np.array_equal(wb.numpy(), g["w_base_t"]) and np.array_equal(wo.numpy(), g["w_ortho_t"])
    idx, val, none = sieve.pack_ortho_sparse(torch.from_numpy(g["w_ortho"]), format="coo")
    assert none is None and np.array_equal(idx.numpy(), g["coo_idx"]) and np.array_equal(val.numpy(), g["coo_val"])
    # row-major order: strictly increasing flat index (what the reference's Test 7 intends to pin)
    flat = g["coo_idx"].astype(np.int64)
    assert np.all(np.diff(flat) > 0)
    with pytest.raises(ValueError):
        sieve.pack_ortho_sparse(W, format="ell")


def test_module_surface_matches_reference():
    m = OrthoLinear(128, 64)
    sd = m.state_dict()
    assert list(sd.keys()) == ["base_weight", "base_scales", "ortho_values", "ortho_col_indices", "ortho_row_ptr"]
    assert sd["base_weight"].shape == (64, 64) and sd["base_weight"].dtype == torch.uint8
    assert sd["base_scales"].dtype == torch.float16 and sd["ortho_values"].numel() == 0
    assert sd["ortho_row_ptr"].dtype == torch.int32 and sd["ortho_col_indices"].dtype == torch.int32
    assert m.alpha == 1.0 and m.bias is None and m.q_bits == 4
    m.set_alpha(0.25)
    assert m.alpha == 0.25 and "alpha" not in m.state_dict()
    mb = OrthoLinear(128, 64, bias=True)
    assert mb.bias.dtype == torch.float32 and mb.bias.shape == (64,)
    # a saved layer (non-empty ortho buffers) loads into a fresh module
    layer = wl.make_layer(128, 64, 0.05, seed=1)
    src = layer.to_module()
    dst = OrthoLinear(128, 64)
    dst.load_state_dict(src.state_dict())
    assert torch.equal(dst.ortho_col_indices, src.ortho_col_indices) and torch.equal(dst.base_weight, src.base_weight)
    from torch_bind.ortho_linear import OrthoLinear as Shim
    assert Shim is OrthoLinear


def test_cpu_input_raises_instead_of_returning_garbage():
    m = wl.make_layer(64, 32, 0.05, seed=2).to_module()
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(2, 64, dtype=torch.float16))


def test_workloads_are_deterministic_and_well_formed():
    a = wl.make_layer(256, 96, 0.02, seed=5)
    b = wl.make_layer(256, 96, 0.02, seed=5)
    assert torch.equal(a.base_weight, b.base_weight) and torch.equal(a.col, b.col) and torch.equal(a.vals, b.vals)
    assert a.nnz == round(0.02 * 256 * 96)
    flat = (torch.repeat_interleave(torch.arange(96), (a.row_ptr[1:] - a.row_ptr[:-1]).long()) * 256 + a.col.long())
    assert torch.all(flat[1:] > flat[:-1])          # unique, row-major sorted
    z = wl.make_zipf_layer(256, 128, 0.01, seed=6)
    cnt = (z.row_ptr[1:] - z.row_ptr[:-1])
    assert z.nnz == round(0.01 * 256 * 128) and int(cnt.max()) <= 256 and int(cnt.max()) > 20 * int(cnt.median() + 1)
    sh = a.rows(32, 64)
    assert sh.N == 32 and int(sh.row_ptr[0]) == 0 and sh.nnz == int(a.row_ptr[64] - a.row_ptr[32])
    # algorithmic bytes of the decode sweep's 4096x4096 layer at M=1: 8.93 MB
    assert abs(wl.Layer(4096, 4096, None, None, None, None, torch.zeros(83886), 1.0).algorithmic_bytes(1) - 8.93e6) < 1e4


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "ortho_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(ortho_b200_[a-z0-9_]+)\s*\(", header)))
    assert declared == sorted(_lib.EXPORTS)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    l = _lib.lib()
    assert l.ortho_b200_version() == 100
    assert l.ortho_b200_strerror(0) == b"ok" and b"NULL" in l.ortho_b200_strerror(1)
    assert l.ortho_b200_workspace_bytes(8, 4096, 4096) == 0                  # the decode kernels use no global scratch
    assert l.ortho_b200_workspace_bytes(512, 4096, 4096) > 0
    assert l.ortho_b200_launch_count() >= 0
    # argument validation happens on the host, before any CUDA call
    assert l.ortho_b200_forward(None, None, None, None, None, 0, None, None, 1, 64, 64, 1.0, None, None, 0, None) == 1
    assert l.ortho_b200_forward(16, 16, None, None, None, 0, 16, 16, 1, 48, 64, 1.0, None, None, 0, None) == 2
    assert l.ortho_b200_forward(8, 16, None, None, None, 0, 16, 16, 1, 64, 64, 1.0, None, None, 0, None) == 3
    assert l.ortho_b200_forward(None, None, None, None, None, 0, None, None, 0, 64, 64, 1.0, None, None, 0, None) == 0
    assert l.ortho_b200_set_decode_config(3, 3, 3, 3) == 2 and l.ortho_b200_set_decode_config(0, 0, 0, 0) == 0


def test_swap_linear_replaces_modules_and_keeps_bias():
    """Module swap on a two-layer toy model (CPU: packing only, the forward needs a GPU)."""
    import torch.nn as nn
    from libortho_b200 import set_alpha_all, swap_linear
    from libortho_b200.convert import sieve_split
    g = torch.Generator().manual_seed(3)

    class Toy(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = nn.Linear(64, 96, bias=True)
            self.act = nn.GELU()
            self.block = nn.Sequential(nn.Linear(96, 32, bias=False))
            self.lora_A = nn.Linear(64, 4, bias=False)       # adapters are left alone, as in the reference
    toy = Toy()
    with torch.no_grad():
        for p_ in toy.parameters():
            p_.copy_(torch.randn(p_.shape, generator=g) * 0.05)
    w_up, b_up = toy.up.weight.detach().clone(), toy.up.bias.detach().clone()
    hdiag = {"up": torch.rand(64, generator=g) + 0.5, "block.0": torch.rand(96, generator=g) + 0.5}
    swapped = swap_linear(toy, sieve_split(hdiag, sparsity_target=0.05), alpha=0.5)
    assert sorted(swapped) == ["block.0", "up"]
    assert isinstance(toy.up, OrthoLinear) and isinstance(toy.block[0], OrthoLinear) and isinstance(toy.lora_A, nn.Linear)
    assert toy.up.alpha == 0.5 and toy.up.bias.dtype == torch.float32 and torch.equal(toy.up.bias.detach(), b_up)
    assert toy.block[0].bias is None
    # same buffers as packing the sieve's split by hand
    wb, wo = sieve.hessian_sieve(w_up, hdiag["up"], sparsity_target=0.05)
    ref = OrthoLinear(64, 96)
    ref.load_from_weights(wb, wo)
    for name in ("base_weight", "ortho_col_indices", "ortho_row_ptr"):
        assert torch.equal(getattr(toy.up, name), getattr(ref, name))
    assert toy.up.ortho_values.numel() > 0
    assert set_alpha_all(toy, 0.0) == 2 and toy.block[0].alpha == 0.0
    # replacing a buffer drops the cached call state
    toy.up._bound[1] = object()
    toy.up.base_scales = toy.up.base_scales.clone()
    assert toy.up._bound == {}


def test_kernel_status_surfaces_as_runtime_error():
    """Host side of the failure path: a non-zero status (here: a bounded device-side wait that ran out) becomes a
    RuntimeError that names the cause; no GPU is involved."""
    with pytest.raises(RuntimeError, match="bounded wait"):
        _lib.check(8, "ortho_b200_forward_gather")
    with pytest.raises(_lib.OrthoB200Error, match="workspace"):
        _lib.check(5, "ortho_b200_forward")
    _lib.check(0, "ok")
