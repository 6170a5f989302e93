"""Generates the committed golden fixtures in this directory.  Run in the build container only
(it needs the reference tree and ``oracle/_ref``); the fixtures it writes are what travels.

    python tests/golden/make_golden.py [/path/to/reference]

Fixtures
--------
kat_cpu_forward.npz   the reference's own known-answer cases (tests/test_cpu_forward.c:97-145,
                      172-319): DIM=64, batch 4, 204 coordinate entries with possible duplicates,
                      inputs regenerated from glibc rand() after srand(42) in the test's draw
                      order; outputs produced by the reference's unmodified orth_layer_forward
                      (oracle/_ref/libortho_ref.so) for alpha=1, alpha=0 and an empty list.
null_test_small.npz   the reference null test's generator (tests/benchmark_null_test.c:98-131)
                      at 128x128, batch 8: base-only output of the reference forward.
packer_small.npz      buffers produced by the reference's Python packer
                      (torch_bind/ortho_linear.py:79-128 with tools/sieve.py) for a seeded 48x64
                      layer, plus the sieve outputs they were built from.
cfg_small.npz         reference-forward outputs for seeded small layers from
                      workloads (ragged N, Zipf rows, an empty ortho, alpha sweep).
cfg0_y.npz            reference-forward outputs of the single-layer benchmark configuration
                      (4096x4096, M=8, 1 % density, alpha 0 and 1); inputs are regenerated from the
                      seed by workloads.
"""
import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else oracle.reference_root()
if not REF:
    sys.exit("usage: make_golden.py <path of the reference tree>   (or set LIBORTHO_REF)")
import workloads as wl  # noqa: E402

RAND_MAX = 2147483647


def pack_int4(w_int8):
    flat = w_int8.astype(np.int16).reshape(-1)
    lo = (flat[0::2] & 0x0F).astype(np.uint8)
    hi = ((flat[1::2] & 0x0F) << 4).astype(np.uint8)
    return (lo | hi).astype(np.uint8)


def kat_cpu_forward():
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(42)
    rnd = libc.rand
    DIM, B = 64, 4
    f32 = np.float32
    x = np.array([f32(rnd()) / f32(RAND_MAX) * f32(2.0) - f32(1.0) for _ in range(B * DIM)], dtype=f32).reshape(B, DIM)
    w = np.array([rnd() % 16 - 8 for _ in range(DIM * DIM)], dtype=np.int8)
    scales = np.array([f32(0.1) + f32(rnd()) / f32(RAND_MAX) * f32(0.9) for _ in range(DIM)], dtype=f32)
    count = DIM * DIM // 20
    idx = np.empty(count, dtype=np.uint16)
    vals = np.empty(count, dtype=f32)
    for i in range(count):
        idx[i] = rnd() % (DIM * DIM)
        vals[i] = f32(rnd()) / f32(RAND_MAX) * f32(0.1) - f32(0.05)
    packed = pack_int4(w).reshape(DIM, DIM // 2)
    y1 = oracle.forward_coo16(packed, scales, idx, vals, x, 1.0, impl="reference")
    y0 = oracle.forward_coo16(packed, scales, idx, vals, x, 0.0, impl="reference")
    ye = oracle.forward_coo16(packed, scales, idx[:0], vals[:0], x, 1.0, impl="reference")
    np.savez(os.path.join(HERE, "kat_cpu_forward.npz"), x=x, w_int=w.reshape(DIM, DIM), packed=packed,
             scales=scales, idx16=idx, vals=vals, y_alpha1=y1, y_alpha0=y0, y_empty=ye)


def null_test_small():
    libc = ctypes.CDLL("libc.so.6")
    libc.srand(42)
    rnd = libc.rand
    DIM, B = 128, 8
    f32 = np.float32
    x = np.array([f32(rnd()) / f32(RAND_MAX) * f32(2.0) - f32(1.0) for _ in range(B * DIM)], dtype=f32).reshape(B, DIM)
    w = np.array([rnd() % 16 - 8 for _ in range(DIM * DIM)], dtype=np.int8)
    scales = np.array([f32(0.1) + f32(rnd()) / f32(RAND_MAX) * f32(0.9) for _ in range(DIM)], dtype=f32)
    packed = pack_int4(w).reshape(DIM, DIM // 2)
    y = oracle.forward_coo16(packed, scales, np.zeros(0, np.uint16), np.zeros(0, f32), x, 0.0, impl="reference")
    np.savez(os.path.join(HERE, "null_test_small.npz"), x=x, packed=packed, scales=scales, y=y)


def packer_small():
    sys.path.insert(0, REF)
    from tools.sieve import hessian_sieve, quantize_int4, compute_hessian_diag_approx, pack_ortho_sparse
    from torch_bind.ortho_linear import OrthoLinear as RefOrthoLinear
    g = torch.Generator().manual_seed(7)
    N, K = 48, 64
    W = torch.randn(N, K, generator=g) * 0.02
    X = torch.randn(256, K, generator=g)
    hdiag = compute_hessian_diag_approx(X)
    h_inv = 1.0 / hdiag
    wq = quantize_int4(W)
    w_base, w_ortho = hessian_sieve(W, h_inv, sparsity_target=0.05)
    w_base_t, w_ortho_t = hessian_sieve(W, torch.diag(h_inv), curvature_thresh=2e-6)
    m = RefOrthoLinear(K, N)
    m.load_from_weights(w_base, w_ortho)
    coo_idx, coo_val, _ = pack_ortho_sparse(w_ortho, format="coo")
    np.savez(os.path.join(HERE, "packer_small.npz"), W=W.numpy(), X=X.numpy(), hdiag=hdiag.numpy(),
             wq=wq.numpy(), w_base=w_base.numpy(), w_ortho=w_ortho.numpy(),
             w_base_t=w_base_t.numpy(), w_ortho_t=w_ortho_t.numpy(),
             base_weight=m.base_weight.numpy(), base_scales=m.base_scales.numpy(),
             ortho_values=m.ortho_values.numpy(), ortho_col_indices=m.ortho_col_indices.numpy(),
             ortho_row_ptr=m.ortho_row_ptr.numpy(), coo_idx=coo_idx.numpy(), coo_val=coo_val.numpy())


def _ref_y(layer, x, alpha):
    return oracle.forward_csr(layer.base_weight.numpy(), layer.base_scales.float().numpy(),
                              layer.row_ptr.numpy(), layer.col.numpy(), layer.vals.float().numpy(),
                              x.float().numpy(), alpha, impl="reference")


from cases import SMALL_CASES  # noqa: E402  (tests/cases.py)


def cfg_small():
    out = {}
    for name, (K, N, M, d, kind, seed, alphas) in SMALL_CASES.items():
        layer = wl.make_layer(K, N, d, seed=seed, ortho=kind)
        x = wl.make_input(M, K, seed=seed)
        for a in alphas:
            out[f"{name}_a{a}"] = _ref_y(layer, x, a)
    np.savez(os.path.join(HERE, "cfg_small.npz"), **out)


def cfg0():
    layer = wl.make_layer(4096, 4096, 0.01, seed=0, ortho="residual10")
    x = wl.make_input(8, 4096, seed=0)
    np.savez(os.path.join(HERE, "cfg0_y.npz"), y_alpha0=_ref_y(layer, x, 0.0), y_alpha1=_ref_y(layer, x, 1.0))


if __name__ == "__main__":
    oracle.build(REF)
    kat_cpu_forward()
    null_test_small()
    packer_small()
    cfg_small()
    cfg0()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
