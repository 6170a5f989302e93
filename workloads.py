"""Seeded synthetic layers for the benchmark configurations.

No model weights or datasets are used anywhere: every layer is drawn from a
``torch.Generator`` with the stated seed, with the shapes, densities and value laws of the
five benchmark configurations (single 4096x4096 layer; Llama-7B-style decode sweep; 8192x8192
prefill with Zipf row loads; Llama-2-70B-style projections; sieve-derived split).  The packing
rules are the module's own (``OrthoLinear.load_from_weights``: scale = rowmax/7 stored as FP16,
round-half-even, clamp [-8,7], low nibble = even element; CSR row-major, int32, FP16 values).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

CFG1_SHAPES = [(4096, 12288), (4096, 4096), (4096, 22016), (11008, 4096)]   # (K, N)
CFG1_M = [1, 4, 16]
CFG1_DENSITY = 0.005
CFG2_SHAPE = (8192, 8192)
CFG2_M = [512, 2048, 8192]
CFG2_DENSITY = 0.001
CFG2_ALPHA = 0.5
CFG3_SHAPES = [(8192, 10240), (8192, 8192), (8192, 57344), (28672, 8192)]
CFG3_M = [1, 32, 4096]
CFG3_DENSITY = 0.003


@dataclass
class Layer:
    K: int
    N: int
    base_weight: torch.Tensor      # u8  [N, K/2]
    base_scales: torch.Tensor      # f16 [N]
    row_ptr: torch.Tensor          # i32 [N+1]
    col: torch.Tensor              # i32 [nnz]
    vals: torch.Tensor             # f16 [nnz]
    alpha: float = 1.0

    @property
    def nnz(self) -> int:
        return int(self.vals.numel())

    def to(self, device) -> "Layer":
        return Layer(self.K, self.N, self.base_weight.to(device), self.base_scales.to(device),
                     self.row_ptr.to(device), self.col.to(device), self.vals.to(device), self.alpha)

    def rows(self, n0: int, n1: int) -> "Layer":
        """The N-shard [n0, n1): contiguous slice of the base, CSR slice with row_ptr rebased to 0."""
        e0, e1 = int(self.row_ptr[n0]), int(self.row_ptr[n1])
        return Layer(self.K, n1 - n0, self.base_weight[n0:n1].contiguous(), self.base_scales[n0:n1].contiguous(),
                     (self.row_ptr[n0:n1 + 1] - e0).to(torch.int32).contiguous(),
                     self.col[e0:e1].contiguous(), self.vals[e0:e1].contiguous(), self.alpha)

    def to_module(self):
        from libortho_b200.ortho_linear import OrthoLinear
        m = OrthoLinear(self.K, self.N, device=self.base_weight.device)
        m.base_weight = self.base_weight
        m.base_scales = self.base_scales
        m.ortho_row_ptr = self.row_ptr
        m.ortho_col_indices = self.col
        m.ortho_values = self.vals
        m.set_alpha(self.alpha)
        return m

    # ALGORITHMIC bytes / flops of one forward, defined on the operator's own layout:
    # packed base + FP16 scales + (when the ortho term is active) FP16 values, int32 columns and
    # int32 row pointers + X + Y.
    def algorithmic_bytes(self, M: int, alpha: Optional[float] = None) -> int:
        a = self.alpha if alpha is None else alpha
        b = self.N * self.K // 2 + 2 * self.N + 2 * M * self.K + 2 * M * self.N
        if a > 0 and self.nnz > 0:
            b += self.nnz * 6 + 4 * (self.N + 1)
        return b

    def algorithmic_flops(self, M: int, alpha: Optional[float] = None) -> int:
        a = self.alpha if alpha is None else alpha
        f = 2 * M * self.N * self.K
        if a > 0 and self.nnz > 0:
            f += 2 * M * self.nnz
        return f


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def quantize_pack(W: torch.Tensor):
    """(packed u8 [N,K/2], scales f16 [N], w_int int8 [N,K]) by the module's packing rule."""
    scales = (W.abs().amax(dim=1) / 7.0).clamp(min=1e-6)
    w_int = torch.round(W / scales.unsqueeze(1)).clamp_(-8, 7).to(torch.int8)
    lo = w_int[:, 0::2] & 0x0F
    hi = (w_int[:, 1::2] & 0x0F) << 4
    return (lo | hi).to(torch.uint8).contiguous(), scales.to(torch.float16), w_int


def _base(K: int, N: int, g: torch.Generator, device, keep_w: bool = False):
    packed = torch.empty(N, K // 2, dtype=torch.uint8, device=device)
    scales = torch.empty(N, dtype=torch.float16, device=device)
    w_keep = torch.empty(N, K, dtype=torch.float32, device=device) if keep_w else None
    step = max(1, (1 << 26) // K)     # <= 64 Mi elements of FP32 scratch at a time
    for n0 in range(0, N, step):
        n1 = min(N, n0 + step)
        W = torch.randn(n1 - n0, K, generator=g, device=device, dtype=torch.float32) * 0.02
        p, s, _ = quantize_pack(W)
        packed[n0:n1], scales[n0:n1] = p, s
        if keep_w:
            w_keep[n0:n1] = W
    return packed, scales, w_keep


def _csr_from_mask_rows(rows: torch.Tensor, cols: torch.Tensor, N: int):
    counts = torch.bincount(rows, minlength=N)
    row_ptr = torch.zeros(N + 1, dtype=torch.int32, device=rows.device)
    row_ptr[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return row_ptr


def uniform_positions(K: int, N: int, density: float, g: torch.Generator, device):
    """Row-major sorted (rows, cols) of uniformly placed entries without replacement.  Exactly
    round(density*N*K) entries while N*K <= 2^25 (a seeded permutation); beyond that an i.i.d.
    Bernoulli(density) mask per element, drawn in row blocks (count is then binomial)."""
    total = N * K
    if total <= (1 << 25):
        nnz = int(round(density * total))
        flat = torch.randperm(total, generator=g, device=device)[:nnz].sort().values
        return flat // K, flat % K
    rows_l, cols_l = [], []
    step = max(1, (1 << 26) // K)
    for n0 in range(0, N, step):
        n1 = min(N, n0 + step)
        mask = torch.rand(n1 - n0, K, generator=g, device=device) < density
        nz = torch.nonzero(mask, as_tuple=False)
        rows_l.append(nz[:, 0] + n0)
        cols_l.append(nz[:, 1])
    return torch.cat(rows_l), torch.cat(cols_l)


def make_layer(K: int, N: int, density: float, seed: int = 0, device="cpu", alpha: float = 1.0,
               ortho: str = "gauss") -> Layer:
    """``ortho='gauss'``: FP16 values ~ N(0, 0.05^2) at uniform positions (decode sweep and
    70B-style configurations).  ``ortho='residual10'``: value = FP16(10 * (W - dequant(W))) at
    the drawn positions (single-layer configuration).  ``ortho='zipf'``: see ``make_zipf_layer``."""
    if ortho == "zipf":
        return make_zipf_layer(K, N, density, seed, device, alpha)
    g = _gen(seed, device)
    packed, scales, W = _base(K, N, g, device, keep_w=(ortho == "residual10"))
    if density <= 0:
        z = torch.zeros(0, device=device)
        return Layer(K, N, packed, scales, torch.zeros(N + 1, dtype=torch.int32, device=device),
                     z.to(torch.int32), z.to(torch.float16), alpha)
    rows, cols = uniform_positions(K, N, density, g, device)
    row_ptr = _csr_from_mask_rows(rows, cols, N)
    if ortho == "residual10":
        lo = (packed & 0x0F).to(torch.int16)
        hi = (packed >> 4).to(torch.int16)
        w_int = torch.empty(N, K, dtype=torch.int16, device=device)
        w_int[:, 0::2] = lo - ((lo & 8) << 1)
        w_int[:, 1::2] = hi - ((hi & 8) << 1)
        deq = w_int[rows, cols].to(torch.float32) * scales.to(torch.float32)[rows]
        vals = (10.0 * (W[rows, cols] - deq)).to(torch.float16)
    else:
        vals = (torch.randn(rows.numel(), generator=g, device=device, dtype=torch.float32) * 0.05).to(torch.float16)
    return Layer(K, N, packed, scales, row_ptr, cols.to(torch.int32), vals, alpha)


def zipf_row_counts(N: int, K: int, nnz: int, exponent: float, g: torch.Generator) -> torch.Tensor:
    """Per-row entry counts proportional to rank^-exponent (largest-remainder rounding), capped
    at K with the overflow handed to the following ranks, then a seeded row permutation."""
    ranks = torch.arange(1, N + 1, dtype=torch.float64)
    p = ranks.pow(-exponent)
    p = p / p.sum()
    raw = p * nnz
    counts = raw.floor().to(torch.int64)
    rem = nnz - int(counts.sum())
    if rem > 0:
        order = torch.argsort(raw - counts.to(torch.float64), descending=True)
        counts[order[:rem]] += 1
    over = 0
    cl = counts.tolist()
    for i in range(N):
        c = cl[i] + over
        over = max(0, c - K)
        cl[i] = min(c, K)
    counts = torch.tensor(cl, dtype=torch.int64)
    perm = torch.randperm(N, generator=g)
    out = torch.empty(N, dtype=torch.int64)
    out[perm] = counts
    return out


def make_zipf_layer(K: int, N: int, density: float, seed: int = 0, device="cpu", alpha: float = 0.5,
                    exponent: float = 1.2) -> Layer:
    """Prefill configuration: nnz = round(density*N*K) entries spread over rows by a Zipf law
    (exponent 1.2 over rows, shuffled row order), columns uniform without replacement inside a
    row, FP16 values ~ N(0, 0.05^2) (the value law is not stated for this configuration; the
    decode sweep's is reused)."""
    g = _gen(seed, "cpu")
    gd = _gen(seed, device)
    packed, scales, _ = _base(K, N, gd, device)
    nnz = int(round(density * N * K))
    counts = zipf_row_counts(N, K, nnz, exponent, g)
    row_ptr = torch.zeros(N + 1, dtype=torch.int32)
    row_ptr[1:] = torch.cumsum(counts, 0).to(torch.int32)
    cols = torch.empty(int(counts.sum()), dtype=torch.int32)
    nz_rows = torch.nonzero(counts, as_tuple=False).flatten().tolist()
    for n in nz_rows:
        c = int(counts[n])
        e0 = int(row_ptr[n])
        cols[e0:e0 + c] = torch.randperm(K, generator=g)[:c].sort().values.to(torch.int32)
    vals = (torch.randn(cols.numel(), generator=g, dtype=torch.float32) * 0.05).to(torch.float16)
    return Layer(K, N, packed, scales, row_ptr.to(device), cols.to(device), vals.to(device), alpha)


def make_sieve_layer(K: int = 4096, N: int = 4096, n_cal: int = 2048, rank: int = 64, seed: int = 0,
                     device="cpu", curvature_thresh: float = 10.0, sparsity_target: Optional[float] = None,
                     alpha: float = 1.0) -> Layer:
    """Sieve-derived split: W ~ N(0, 0.02^2); calibration X = A[n,rank] B[rank,K] + 0.1 noise;
    H = X^T X / n + 0.01 mean(diag H) I, inverted on the host in FP64; the Hessian sieve splits
    W into base and ortho at the stated threshold (or keeps the top ``sparsity_target``
    fraction); the layer is then packed with ``OrthoLinear.load_from_weights``."""
    from libortho_b200.ortho_linear import OrthoLinear
    from libortho_b200.sieve import hessian_sieve
    g = _gen(seed, "cpu")
    W = torch.randn(N, K, generator=g) * 0.02
    A = torch.randn(n_cal, rank, generator=g)
    B = torch.randn(rank, K, generator=g)
    X = A @ B + 0.1 * torch.randn(n_cal, K, generator=g)
    H = (X.T @ X).double() / n_cal
    H = H + 0.01 * H.diagonal().mean() * torch.eye(K, dtype=torch.float64)
    H_inv = torch.linalg.inv(H).float()
    w_base, w_ortho = hessian_sieve(W, H_inv, curvature_thresh=curvature_thresh, sparsity_target=sparsity_target)
    m = OrthoLinear(K, N)
    m.load_from_weights(w_base, w_ortho)
    return Layer(K, N, m.base_weight.to(device), m.base_scales.to(device), m.ortho_row_ptr.to(device),
                 m.ortho_col_indices.to(device), m.ortho_values.to(device), alpha)


def make_input(M: int, K: int, seed: int = 0, device="cpu") -> torch.Tensor:
    """FP16 activations ~ N(0, 1)."""
    g = _gen(seed + 1000003, device)
    return torch.randn(M, K, generator=g, device=device, dtype=torch.float32).to(torch.float16)
