"""Pins the CPU oracle (oracle/t81_oracle.c) to the reference: against fixtures
generated from the reference's own code (tests/golden/generate.py), against the
reference's known-answer tests, and — where oracle/_ref is present — against the
compiled reference module directly on fresh random inputs."""

import numpy as np
import pytest

import oracle
from oracle import ref as oracle_ref


def test_pack_fixed_matches_reference_fixtures(golden):
    g = golden("pack_fixed.npz")
    w = g["w"]
    for name, thr in (("t045", 0.45), ("t050", 0.5), ("t100", 1.0), ("t001", 0.01)):
        assert np.array_equal(oracle.pack_dense_matrix(w, thr), g[f"packed_{name}"]), name
        assert np.array_equal(oracle.quantize_to_trits(w, thr), g[f"trits_{name}"]), name
    # the Python packer of the reference produces the same bytes as its C++ packer
    assert np.array_equal(g["from_float_t045"], g["packed_t045"])
    assert np.array_equal(oracle.unpack_packed_limbs(g["packed_t045"], 64, 100), g["unpacked_t045"])
    for cols in (1, 47, 48, 49, 96, 145):
        assert np.array_equal(oracle.pack_dense_matrix(g[f"w_c{cols}"], 0.45), g[f"packed_c{cols}"]), cols


def test_pack_roundtrip_and_tail_is_zero():
    rng = np.random.default_rng(1)
    for cols in (1, 3, 47, 48, 50, 95, 500):
        t = rng.integers(-1, 2, (7, cols)).astype(np.int8)
        p = oracle.pack_trits_rowwise(t)
        assert p.shape == (7, (cols + 47) // 48, 16) and p.max() <= 26
        assert np.array_equal(oracle.unpack_packed_limbs(p, 7, cols), t)
        full = oracle.unpack_packed_limbs(p, 7, p.shape[1] * 48)
        assert not full[:, cols:].any()


def test_unpack_rejects_bytes_above_26():
    p = np.full((1, 1, 16), 13, np.uint8)
    p[0, 0, 5] = 27
    with pytest.raises(ValueError):
        oracle.unpack_packed_limbs(p, 1, 48)


def test_limb_gemm_matches_reference_fixtures(golden):
    g = golden("gemm_limb.npz")
    for tag in ("nz10", "nz30", "nz48"):
        A, B, C0, C = g[f"A_{tag}"], g[f"B_{tag}"], g[f"C0_{tag}"], g[f"C_{tag}"]
        got = oracle.gemm_limb(A, B, C0, 9, 7, 3 * 48, 1.25, 0.5)
        np.testing.assert_allclose(got, C, rtol=2e-7, atol=0)
        # column-wise packer agrees with the reference's _pack_columnwise
        assert np.array_equal(oracle.pack_trits_columnwise(g[f"tb_{tag}"]), B)
    zero = np.full((3, 16), 13, np.uint8)
    assert np.array_equal(oracle.gemm_limb(zero[:2], zero, np.zeros((2, 3), np.float32), 2, 3, 48), g["ka_zero"])
    got = oracle.gemm_limb(zero[:2], zero, np.full((2, 3), 2.0, np.float32), 2, 3, 48, 0.0, 0.5)
    assert np.array_equal(got, g["ka_beta"]) and np.all(got == 1.0)
    for i in range(64):
        got = oracle.gemm_limb(g["prod_a"][i], g["prod_b"][i], np.zeros((1, 1), np.float32), 1, 1, 48, 1e-30, 0.0)
        np.testing.assert_allclose(got[0, 0], g["prod_c_alpha1e-30"][i], rtol=2e-7)


def test_limb_gemm_probe_value():
    # value(1,1,0,...) = 4, value(-1,0,1,0,...) = 8, C = 2, alpha = 1, beta = 0.5 -> 4*8 + 1 = 33
    ta = np.zeros((1, 48), np.int8); ta[0, :2] = 1
    tb = np.zeros((48, 1), np.int8); tb[0, 0] = -1; tb[2, 0] = 1
    got = oracle.gemm_limb(oracle.pack_trits_rowwise(ta), oracle.pack_trits_columnwise(tb),
                           np.full((1, 1), 2.0, np.float32), 1, 1, 48, 1.0, 0.5)
    assert got[0, 0] == 33.0


def test_trit_gemm_matches_reference_dense_form(golden):
    g = golden("gemm_trit.npz")
    assert np.array_equal(oracle.pack_dense_matrix(g["w"], 0.45), g["packed"])
    assert np.array_equal(oracle.unpack_packed_limbs(g["packed"], 24, 130), g["trits"])
    got = oracle.gemm_trit(g["packed"], g["x"], None, 24, 11, 130)
    np.testing.assert_allclose(got, g["y_f64"].astype(np.float32), rtol=0, atol=0)
    # the token-major layout gives the transpose
    got_nk = oracle.gemm_trit(g["packed"], np.ascontiguousarray(g["x"].T), None, 24, 11, 130, b_is_nk=True)
    assert np.array_equal(got_nk, got.T)
    # alpha / beta follow gemm_cpu.cpp's rounding structure
    C0 = np.ones((24, 11), np.float32)
    got = oracle.gemm_trit(g["packed"], g["x"], C0, 24, 11, 130, 2.0, 0.5)
    np.testing.assert_allclose(got, (2.0 * g["y_f64"] + 0.5).astype(np.float32), rtol=1e-6)


def test_linear_forward_is_scaled_gemm_plus_bias():
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, (20, 100)).astype(np.float32)
    packed, scale = oracle.pack_dense_matrix_absmean(w, 0.45)
    x = rng.normal(size=(5, 100)).astype(np.float32)
    bias = rng.normal(size=20).astype(np.float32)
    y = oracle.linear_forward(packed, scale, bias, x, 100)
    trits = oracle.unpack_packed_limbs(packed, 20, 100).astype(np.float64)
    want = x.astype(np.float64) @ (trits * scale[:, None].astype(np.float64)).T + bias
    np.testing.assert_allclose(y, want.astype(np.float32), rtol=1e-6, atol=1e-7)


def test_absmean_rule_definition():
    """The absmean rule is not a reference behaviour; pin it to its own statement."""
    rng = np.random.default_rng(4)
    w = rng.normal(0, 0.02, (6, 1000)).astype(np.float32)
    w[5] = 0.0
    packed, scale = oracle.pack_dense_matrix_absmean(w, 0.45)
    np.testing.assert_allclose(scale, np.abs(w).astype(np.float64).mean(axis=1).astype(np.float32), rtol=2e-7)
    assert scale[5] == 0.0
    trits = oracle.unpack_packed_limbs(packed, 6, 1000)
    for r in range(6):
        cut = np.float32(0.45) * scale[r] if scale[r] > 0 else np.float32(np.inf)
        want = np.where(w[r] <= -cut, -1, np.where(w[r] >= cut, 1, 0))
        assert np.array_equal(trits[r], want)
    # thread count does not change results
    oracle.set_num_threads(4)
    p4, s4 = oracle.pack_dense_matrix_absmean(w, 0.45)
    oracle.set_num_threads(1)
    assert np.array_equal(p4, packed) and np.array_equal(s4, scale)


@pytest.mark.skipif(not oracle_ref.available(), reason="oracle/_ref not built (reference sources absent)")
def test_against_compiled_reference_on_random_inputs():
    t81lib = oracle_ref.load()
    rng = np.random.default_rng(5)
    for rows, cols, sigma, thr in ((33, 257, 0.5, 0.45), (4, 48, 1.0, 0.9), (17, 1000, 0.3, 0.2)):
        w = rng.normal(0, sigma, (rows, cols)).astype(np.float32)
        assert np.array_equal(oracle.pack_dense_matrix(w, thr), np.asarray(t81lib.pack_dense_matrix(w, thr)))
        assert np.array_equal(oracle.quantize_to_trits(w, thr), np.asarray(t81lib.quantize_to_trits(w, thr)))
    M, N, KL = 5, 4, 2
    ta = np.zeros((M, KL * 48), np.int8); tb = np.zeros((KL * 48, N), np.int8)
    for l in range(KL):
        ta[:, l * 48:l * 48 + 20] = rng.integers(-1, 2, (M, 20))
        tb[l * 48:l * 48 + 20] = rng.integers(-1, 2, (20, N))
    A, B = oracle.pack_trits_rowwise(ta), oracle.pack_trits_columnwise(tb)
    C0 = rng.normal(size=(M, N)).astype(np.float32)
    C = C0.copy()
    t81lib.gemm_ternary(A.reshape(-1, 16).view("V16").reshape(M, KL), B.reshape(-1, 16).view("V16").reshape(KL, N),
                        C, M, N, KL * 48, 0.75, -1.5)
    np.testing.assert_allclose(oracle.gemm_limb(A, B, C0, M, N, KL * 48, 0.75, -1.5), C, rtol=2e-7)


@pytest.mark.skipif(not oracle_ref.available(), reason="oracle/_ref not built (reference sources absent)")
def test_trit_mode_oracle_against_the_reference_sparse_product():
    """TRIT mode has no dense counterpart in the reference; its sparse helper computes the same product from
    one COO entry per non-zero trit (include/t81/sparse/simple.hpp:37-94).  It rounds to fp32 after every
    addition, the oracle accumulates in fp64: agreement to accumulated fp32 rounding."""
    t81lib = oracle_ref.load()
    rng = np.random.default_rng(21)
    for M, K, N, alpha, beta in ((7, 48, 5, 1.0, 0.0), (33, 130, 9, 0.75, -1.5), (64, 1000, 16, 1.0, 0.5)):
        trits = rng.integers(-1, 2, (M, K)).astype(np.int8)
        B = rng.normal(size=(K, N)).astype(np.float32)
        C0 = rng.normal(size=(M, N)).astype(np.float32)
        r, c = np.nonzero(trits)
        C = C0.copy()
        t81lib.spmm_simple([int(v) for v in trits[r, c]], r.astype(np.int32).tolist(), c.astype(np.int32).tolist(),
                           M, K, B, C, N, alpha, beta)
        got = oracle.gemm_trit(oracle.pack_trits_rowwise(trits), B, C0, M, N, K, alpha, beta)
        np.testing.assert_allclose(got, C, rtol=1e-4, atol=1e-4 * float(np.abs(C).max()))


def test_elementwise_restatements_match_the_compiled_reference():
    """where / clamp / lerp / addcmul against the reference's CPU code (src/linalg/gemm_dispatch.cpp:147-222)
    compiled from its sources.  The generic build evaluates one float32 operation per operator and must
    agree bit for bit; the -mavx512f build lets the compiler fuse multiply-adds, so lerp and addcmul may
    differ there by one rounding.  One process can hold only one build of the module, hence the child."""
    import subprocess
    import sys
    if not oracle_ref.available():
        pytest.skip("oracle/_ref not built")
    code = r'''
import importlib.util, sys, numpy as np
sys.path.insert(0, sys.argv[2])
import oracle
spec = importlib.util.spec_from_file_location("t81lib", sys.argv[1])
m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)
exact = sys.argv[3] == "exact"
rng = np.random.default_rng(12)
a, b, c = (rng.normal(size=(61, 23)).astype(np.float32) for _ in range(3))
cond = (a > 0).astype(np.float32)
assert np.array_equal(np.asarray(m.where(cond, b, c)), oracle.where(cond, b, c))
assert np.array_equal(np.asarray(m.clamp(a, -0.5, 0.25)), oracle.clamp(a, -0.5, 0.25))
for got, want in ((m.lerp(a, b, c), oracle.lerp(a, b, c)), (m.addcmul(a, b, c, 0.3), oracle.addcmul(a, b, c, 0.3))):
    got = np.asarray(got)
    if exact:
        assert np.array_equal(got, want)
    else:
        assert np.max(np.abs(got - want)) <= 1e-6 * np.max(np.abs(want))
print("ok")
'''
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    variants = [("generic", "exact")] + ([("avx512f", "close")] if oracle_ref.host_has_avx512f() else [])
    for variant, how in variants:
        res = subprocess.run([sys.executable, "-c", code, oracle_ref.path(variant), root, how], capture_output=True, text=True)
        assert res.returncode == 0 and "ok" in res.stdout, f"{variant}: {res.stdout}{res.stderr}"
