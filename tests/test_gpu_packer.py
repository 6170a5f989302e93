"""Device-side packer against the reference's torch chain (bit-exact)."""
import pytest
import torch

from libortho_b200 import OrthoLinear, _C_ops
from libortho_b200.sieve import pack_ortho_sparse

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def torch_chain(w, scales=None):
    """OrthoLinear.load_from_weights of the reference (torch_bind/ortho_linear.py:79-128), on the CPU."""
    if scales is None:
        scales = (w.abs().max(dim=1)[0] / 7.0).clamp(min=1e-6)
    w_int = (w / scales.unsqueeze(1)).round().clamp(-8, 7).to(torch.int8)
    flat = w_int.flatten()
    packed = ((flat[0::2] & 0x0F) | ((flat[1::2] & 0x0F) << 4)).to(torch.uint8)
    return packed.view(w.shape[0], -1), scales.to(torch.float16)


@pytest.mark.parametrize("N,K", [(7, 8), (64, 64), (300, 4096), (1030, 264), (2048, 11008)])
def test_base_pack_matches_the_torch_chain_bit_for_bit(N, K):
    g = torch.Generator().manual_seed(N * 131 + K)
    w = torch.randn(N, K, generator=g) * 0.02
    w[0] = 0.0                                        # all-zero row: scale floor 1e-6
    if N > 2:
        w[1, :8] = torch.tensor([7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -3.5, 6.5])     # scale exactly 1: ties round to even
        w[1, 8:] = 0.0
        w[2] *= 1e-20                                 # tiny but non-zero row
    q_ref, s_ref = torch_chain(w)
    q, s = _C_ops.pack_base(w.to(DEV))
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu().view(torch.int16), s_ref.view(torch.int16))
    # given scales (stored FP16 scales up-cast, as a caller re-quantising with known scales would pass)
    given = s_ref.float() * 1.25
    q_ref2, s_ref2 = torch_chain(w, given)
    q2, s2 = _C_ops.pack_base(w.to(DEV), given.to(DEV))
    assert torch.equal(q2.cpu(), q_ref2) and torch.equal(s2.cpu().view(torch.int16), s_ref2.view(torch.int16))


@pytest.mark.parametrize("N,K,density", [(5, 8, 0.5), (257, 1000, 0.01), (4096, 4096, 0.005), (33, 264, 0.0), (16, 64, 1.0)])
def test_csr_build_matches_pack_ortho_sparse(N, K, density):
    g = torch.Generator().manual_seed(N + K)
    w = torch.randn(N, K, generator=g) * 0.05
    w = torch.where(torch.rand(N, K, generator=g) < density, w, torch.zeros(()))
    if N > 4 and density > 0:
        w[3] = 0.0                                    # an empty row in the middle
        w[4, K - 1] = 1e-30                           # non-zero in FP32, rounds to zero in FP16: still an entry
        w[4, 0] = -0.0                                # negative zero is zero
    rp_ref, col_ref, val_ref = pack_ortho_sparse(w, "csr")
    rp, col, val = _C_ops.pack_ortho_csr(w.to(DEV))
    assert torch.equal(rp.cpu(), rp_ref.to(torch.int32))
    assert torch.equal(col.cpu(), col_ref.to(torch.int32))
    assert torch.equal(val.cpu().view(torch.int16), val_ref.to(torch.float16).view(torch.int16))


def test_load_from_weights_on_the_gpu_equals_the_host_path():
    g = torch.Generator().manual_seed(5)
    K, N = 512, 192
    w = torch.randn(N, K, generator=g) * 0.02
    wo = torch.where(torch.rand(N, K, generator=g) < 0.02, torch.randn(N, K, generator=g) * 0.05, torch.zeros(()))
    host = OrthoLinear(K, N)
    host.load_from_weights(w, wo)
    dev = OrthoLinear(K, N, device=DEV)
    dev.load_from_weights(w.to(DEV), wo.to(DEV))
    for name in ("base_weight", "ortho_row_ptr", "ortho_col_indices"):
        assert torch.equal(getattr(dev, name).cpu(), getattr(host, name)), name
    for name in ("base_scales", "ortho_values"):
        assert torch.equal(getattr(dev, name).cpu().view(torch.int16), getattr(host, name).view(torch.int16)), name
    x = torch.randn(4, K, generator=g).to(torch.float16).to(DEV)
    y = dev(x)
    assert torch.isfinite(y).all()
