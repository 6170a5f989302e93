"""The allocation-free forward (`ortho_b200_forward_static_scratch`).

Callers that may not allocate device memory (a plugin inside a host application that owns the
allocator, a serving loop with a fixed memory budget, code about to be recorded into a CUDA graph)
cannot give the ordinary forward its prefill workspace, nor build a plan.  This entry point keeps
that scratch in a fixed array inside the library.  Here it is called through the C ABI twice in a
row -- the array is shared and keeps the first call's contents -- and both results are compared
with the ordinary entry point, which got a freshly allocated workspace.  The file name sorts last
so that a run stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from conftest import REL_FRO_TOL, MAX_ABS_TOL, assert_close, errors, layer_oracle
from libortho_b200 import _C_ops, _lib
import workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LIMIT = 32 * 1024 * 1024


def _static(layer, x, alpha):
    y = torch.empty(x.shape[0], layer.N, dtype=torch.float16, device=x.device)
    nnz = layer.nnz
    with torch.cuda.device(x.device):
        st = _lib.lib().ortho_b200_forward_static_scratch(
            layer.base_weight.data_ptr(), layer.base_scales.data_ptr(),
            layer.vals.data_ptr() if nnz else None, layer.col.data_ptr() if nnz else None,
            layer.row_ptr.data_ptr() if nnz else None, nnz, x.data_ptr(), y.data_ptr(),
            x.shape[0], layer.K, layer.N, float(alpha), torch.cuda.current_stream(x.device).cuda_stream)
    return st, y


def _ordinary(layer, x, alpha):
    """The ordinary entry point without a plan and with a freshly allocated workspace of the size of the
    built-in array, so that both entries make the same choices and must produce the same bits."""
    y = torch.empty(x.shape[0], layer.N, dtype=torch.float16, device=x.device)
    ws = torch.empty(LIMIT, dtype=torch.uint8, device=x.device)
    _C_ops.forward(layer.base_weight, layer.base_scales, layer.vals, layer.col, layer.row_ptr, x, y, alpha, workspace=ws)
    return y


def _check(y, ref, what):
    rel, mx = errors(y.float().cpu().numpy(), ref.float().cpu().numpy())
    assert rel <= REL_FRO_TOL and mx <= MAX_ABS_TOL, f"{what}: rel_fro={rel:.3e} max_abs={mx:.3e}"


def test_two_calls_in_a_row_match_the_ordinary_forward(oracle_mod):
    # two different layers and token counts back to back: the second call finds the first call's
    # transposed activations and sparse sums still in the shared array and must not be affected
    a = wl.make_layer(1024, 520, 0.01, seed=101, device=DEV)
    b = wl.make_layer(2048, 384, 0.02, seed=102, ortho="zipf", device=DEV)
    xa = wl.make_input(300, 1024, seed=101, device=DEV)
    xb = wl.make_input(129, 2048, seed=102, device=DEV)
    ra, rb = _ordinary(a, xa, 1.0), _ordinary(b, xb, 0.5)
    torch.cuda.synchronize()
    st1, y1 = _static(a, xa, 1.0)
    st2, y2 = _static(b, xb, 0.5)
    torch.cuda.synchronize()
    assert st1 == 0 and st2 == 0
    assert _lib.lib().ortho_b200_query_kernel_status() == 0
    _check(y1, ra, "first call")
    _check(y2, rb, "second call")
    assert torch.equal(y1, ra) and torch.equal(y2, rb)      # both entries are reproducible and route alike
    # and against the CPU oracle, not only against the other CUDA entry
    assert_close(y1.float().cpu().numpy(), layer_oracle(oracle_mod, a, xa, 1.0), "first call vs oracle")
    assert_close(y2.float().cpu().numpy(), layer_oracle(oracle_mod, b, xb, 0.5), "second call vs oracle")
    # same inputs again after the array has been overwritten by the other layer
    st3, y3 = _static(a, xa, 1.0)
    torch.cuda.synchronize()
    assert st3 == 0
    _check(y3, ra, "third call")
    assert torch.equal(y3, y1)


def test_regimes_without_scratch_and_the_size_limit():
    layer = wl.make_layer(1024, 520, 0.01, seed=103, device=DEV)
    # decode regime and alpha = 0 need no scratch at all
    x8 = wl.make_input(8, 1024, seed=103, device=DEV)
    st, y = _static(layer, x8, 1.0)
    torch.cuda.synchronize()
    assert st == 0
    _check(y, _ordinary(layer, x8, 1.0), "decode regime")
    x200 = wl.make_input(200, 1024, seed=104, device=DEV)
    st, y = _static(layer, x200, 0.0)
    torch.cuda.synchronize()
    assert st == 0 and torch.equal(y, _ordinary(layer, x200, 0.0))
    # a shape whose scratch would not fit the built-in array is refused with its own status
    wide = wl.make_layer(4096, 520, 0.01, seed=107, device=DEV)
    big_m = 8192
    assert 2 * 4096 * big_m > LIMIT                       # the transposed activations alone exceed the array
    xbig = torch.zeros(big_m, 4096, dtype=torch.float16, device=DEV)
    st, _ = _static(wide, xbig, 1.0)
    assert st == 10 and b"scratch" in _lib.lib().ortho_b200_strerror(st)
    torch.cuda.synchronize()
