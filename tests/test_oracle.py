"""The CPU restatement against the reference's own vectors (no GPU)."""
import numpy as np
import pytest

from conftest import golden, layer_oracle
import workloads as wl


def test_unpack_rule_matches_numpy_statement(oracle_mod):
    rng = np.random.default_rng(1)
    packed = rng.integers(0, 256, (7, 16), dtype=np.uint8)
    scales = rng.uniform(0.1, 1.0, 7).astype(np.float32)
    w_int, w_deq = oracle_mod.dequant(packed, scales)
    assert np.array_equal(w_int, oracle_mod.unpack_int4_numpy(packed))
    assert w_int.min() >= -8 and w_int.max() <= 7
    # (float)w_int * scale, one FP32 multiply (src/ortho.c:363)
    assert np.array_equal(w_deq, w_int.astype(np.float32) * scales[:, None])
    # every nibble value at both positions
    b = np.arange(256, dtype=np.uint8).reshape(1, 256)
    u = oracle_mod.unpack_int4_numpy(b)[0]
    lo, hi = u[0::2], u[1::2]
    assert np.array_equal(lo, np.array([(v & 15) - 16 * ((v & 15) >> 3) for v in range(256)], dtype=np.int8))
    assert np.array_equal(hi, np.array([(v >> 4) - 16 * ((v >> 4) >> 3) for v in range(256)], dtype=np.int8))


def test_known_answer_cases_of_the_reference_test(oracle_mod):
    """tests/test_cpu_forward.c: alpha=1, alpha=0, empty list -- bit-for-bit."""
    g = golden("kat_cpu_forward.npz")
    args = (g["packed"], g["scales"], g["idx16"], g["vals"], g["x"])
    assert np.array_equal(oracle_mod.forward_coo16(*args, 1.0), g["y_alpha1"])
    assert np.array_equal(oracle_mod.forward_coo16(*args, 0.0), g["y_alpha0"])
    assert np.array_equal(oracle_mod.forward_coo16(g["packed"], g["scales"], g["idx16"][:0], g["vals"][:0],
                                                   g["x"], 1.0), g["y_empty"])
    # alpha = 0 and the empty list are the base-only result (null-test property)
    assert np.array_equal(g["y_alpha0"], g["y_empty"])
    # the packed fixture really is the nibble packing of the drawn integers
    assert np.array_equal(oracle_mod.unpack_int4_numpy(g["packed"]), g["w_int"])


def test_null_test_base_only(oracle_mod):
    g = golden("null_test_small.npz")
    y = oracle_mod.forward_csr(g["packed"], g["scales"], None, None, None, g["x"], 0.0, threads=1)
    assert np.array_equal(y, g["y"])


def test_negative_alpha_is_gated_off(oracle_mod):
    """src/ortho.c:343 gates on alpha > 0, so a negative alpha behaves as 0."""
    layer = wl.make_layer(64, 32, 0.1, seed=3)
    x = wl.make_input(2, 64, seed=3)
    assert np.array_equal(layer_oracle(oracle_mod, layer, x, -1.0), layer_oracle(oracle_mod, layer, x, 0.0))
    assert not np.array_equal(layer_oracle(oracle_mod, layer, x, 1.0), layer_oracle(oracle_mod, layer, x, 0.0))


def test_seeded_small_layers_bit_exact(oracle_mod):
    from cases import SMALL_CASES
    g = golden("cfg_small.npz")
    for name, (K, N, M, d, kind, seed, alphas) in SMALL_CASES.items():
        layer = wl.make_layer(K, N, d, seed=seed, ortho=kind)
        x = wl.make_input(M, K, seed=seed)
        for a in alphas:
            for threads in (1, 3):
                y = layer_oracle(oracle_mod, layer, x, a, threads=threads)
                assert np.array_equal(y, g[f"{name}_a{a}"]), (name, a, threads)


def test_single_layer_config_bit_exact(oracle_mod):
    layer = wl.make_layer(4096, 4096, 0.01, seed=0, ortho="residual10")
    assert layer.nnz == 167772
    x = wl.make_input(8, 4096, seed=0)
    g = golden("cfg0_y.npz")
    assert np.array_equal(layer_oracle(oracle_mod, layer, x, 1.0), g["y_alpha1"])
    assert np.array_equal(layer_oracle(oracle_mod, layer, x, 0.0), g["y_alpha0"])


def test_restatement_equals_compiled_reference_when_present(oracle_mod):
    if not oracle_mod.available("reference"):
        pytest.skip("oracle/_ref not built on this machine")
    assert oracle_mod.lifecycle_check(64, 64, 10) == 0
    for seed, (K, N, M, d) in enumerate([(64, 40, 3, 0.1), (2048, 70, 2, 0.01), (28672, 6, 1, 0.003)]):
        layer = wl.make_layer(K, N, d, seed=seed)
        x = wl.make_input(M, K, seed=seed)
        for a in (0.0, 0.7):
            assert np.array_equal(layer_oracle(oracle_mod, layer, x, a),
                                  layer_oracle(oracle_mod, layer, x, a, impl="reference"))
