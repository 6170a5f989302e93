"""Device-side Hessian sieve against the torch chain it restates (tools/sieve.py:13-23, 25-76 of the
reference): both outputs must be bit-identical, for the curvature threshold and for the keep-top-k rule."""
import pytest
import torch

from libortho_b200 import OrthoLinear, _C_ops, sieve

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _torch_chain(w, hdiag, thresh, target):
    """The host-side restatement, forced onto its torch branch by running it on the CPU."""
    return sieve.hessian_sieve(w.cpu(), hdiag.cpu(), curvature_thresh=thresh, sparsity_target=target)


def _bits(t):
    return t.contiguous().view(torch.int32)


@pytest.mark.parametrize("N,K,thresh,target", [(64, 128, 1e-7, None), (200, 256, 3e-6, None), (96, 512, 10.0, None),
                                               (128, 256, 10.0, 0.05), (300, 128, 10.0, 0.01), (64, 64, 10.0, 0.0),
                                               (512, 1024, 10.0, 0.003)])
def test_sieve_matches_the_torch_chain_bit_for_bit(N, K, thresh, target):
    g = torch.Generator().manual_seed(N * 7 + K)
    w = torch.randn(N, K, generator=g) * 0.02
    w[3] = 0.0                                        # an all-zero row: scale floor, zero residual
    w[5, 7] = 3.0                                     # an outlier that stretches its row's scale
    hdiag = torch.rand(K, generator=g) * 2.0 + 0.01
    wb_ref, wo_ref = _torch_chain(w, hdiag, thresh, target)
    wb, wo = sieve.hessian_sieve(w.to(DEV), hdiag.to(DEV), curvature_thresh=thresh, sparsity_target=target)
    torch.cuda.synchronize()
    assert torch.equal(_bits(wb.cpu()), _bits(wb_ref))
    assert torch.equal(_bits(wo.cpu()), _bits(wo_ref))
    if target:
        kept = int((wo != 0).sum())
        assert 0 < kept <= int(target * N * K)
    # a 2-D H_inv is reduced to its diagonal, like the reference does
    wb2, wo2 = sieve.hessian_sieve(w.to(DEV), torch.diag(hdiag).to(DEV), curvature_thresh=thresh, sparsity_target=target)
    assert torch.equal(_bits(wb2), _bits(wb)) and torch.equal(_bits(wo2), _bits(wo))


def test_sieve_then_pack_then_forward_on_the_device():
    """The whole producer chain on the GPU: sieve -> packer -> OrthoLinear, equal to the host chain's buffers."""
    g = torch.Generator().manual_seed(5)
    N, K = 160, 512
    w = torch.randn(N, K, generator=g) * 0.02
    hdiag = torch.rand(K, generator=g) + 0.5
    wb_h, wo_h = _torch_chain(w, hdiag, 10.0, 0.02)
    host = OrthoLinear(K, N)
    host.load_from_weights(wb_h, wo_h)
    wb_d, wo_d = sieve.hessian_sieve(w.to(DEV), hdiag.to(DEV), sparsity_target=0.02)
    devm = OrthoLinear(K, N, device=DEV)
    devm.load_from_weights(wb_d, wo_d)
    for name in ("base_weight", "ortho_col_indices", "ortho_row_ptr"):
        assert torch.equal(getattr(devm, name).cpu(), getattr(host, name)), name
    assert torch.equal(devm.base_scales.cpu().view(torch.int16), host.base_scales.view(torch.int16))
    assert torch.equal(devm.ortho_values.cpu().view(torch.int16), host.ortho_values.view(torch.int16))
    x = torch.randn(3, K, generator=g).to(torch.float16).to(DEV)
    assert torch.isfinite(devm(x)).all()
