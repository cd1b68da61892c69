"""The decode-stream layout ("T2": two bits per trit in tensor-core fragment order) and TRIT mode on it.

The layout is this library's own; its bytes are checked against the oracle's restatement of the layout's
definition, and the products against the CPU oracle's TRIT-mode result on the same packed limbs — the same
check the limb-layout kernel gets."""

import numpy as np
import pytest
import torch

import oracle


def test_oracle_t2_layout_is_a_rearrangement():
    rng = np.random.default_rng(0)
    trits = rng.integers(-1, 2, (70, 400)).astype(np.int8)
    t2 = oracle.pack_t2(trits)
    assert t2.size == 3 * 3 * 1536
    words = t2.view("<u4").reshape(3, 3, 32, 12)
    # read a few trits back by the layout's statement
    for row, col in ((0, 0), (69, 399), (33, 191), (40, 192), (8, 2), (17, 50)):
        c, T = col // 192, row // 32
        k, rr = col % 192, row % 32
        t, m, r_hi, h = k // 48, (k % 48) // 4, (k % 4) // 2, k % 2
        gr, g, r_lo = rr // 16, rr % 8, (rr % 16) // 8
        j = 4 * (m % 2) + 2 * r_hi + r_lo
        code = (int(words[c, T, 4 * g + t, 6 * gr + m // 2]) >> ((30 if h else 14) - 2 * j)) & 3
        assert {0: 0, 1: 1, 3: -1}[code] == trits[row, col]
    # padding is zero
    assert oracle.pack_t2(np.zeros((1, 1), np.int8)).sum() == 0


pytest_gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(lib_built):
    from t81lib_b200 import _capi
    assert _capi.device_available(), _capi.last_error()
    return torch.device("cuda", 0)


def rel_err(got, want):
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want)) / (np.sqrt(np.mean(want ** 2)) + 1e-30))


@pytest_gpu
@pytest.mark.parametrize("rows,cols", [(1, 1), (32, 192), (33, 193), (70, 400), (100, 130), (256, 3072), (129, 4096)])
def test_pack_t2_bytes_match_the_layout_statement(dev, rows, cols):
    from t81lib_b200 import ops
    rng = np.random.default_rng(rows * 1000 + cols)
    trits = rng.integers(-1, 2, (rows, cols)).astype(np.int8)
    packed = torch.from_numpy(oracle.pack_trits_rowwise(trits)).to(dev)
    got = ops.pack_t2(packed, rows, cols)
    assert np.array_equal(got.cpu().numpy(), oracle.pack_t2(trits))


@pytest_gpu
@pytest.mark.parametrize("out_f,in_f", [(16, 48), (100, 130), (256, 3072), (130, 4096), (384, 8192), (64, 14336), (1000, 1000),
                                       (512, 14336), (128, 4096), (1792, 4096)])  # the last three: per-rank shapes of 8 GPUs
@pytest.mark.parametrize("tokens", [1, 4, 8, 9, 16, 17, 40, 128])
def test_t2_product_matches_oracle(dev, out_f, in_f, tokens):
    from t81lib_b200 import _capi, ops
    rng = np.random.default_rng(out_f * 31 + in_f + tokens)
    trits = rng.integers(-1, 2, (out_f, in_f)).astype(np.int8)
    limbs = oracle.pack_trits_rowwise(trits)
    scale = rng.uniform(0.01, 0.03, out_f).astype(np.float32)
    bias = rng.normal(0, 0.01, out_f).astype(np.float32)
    x = torch.from_numpy(rng.normal(size=(tokens, in_f)).astype(np.float32))
    packed = torch.from_numpy(limbs).to(dev)
    t2 = ops.pack_t2(packed, out_f, in_f)
    sd, bd = torch.from_numpy(scale).to(dev), torch.from_numpy(bias).to(dev)
    xb = x.to(dev).to(torch.bfloat16)
    want = oracle.linear_forward(limbs, scale, bias, xb.float().cpu().numpy(), in_f)
    (y32,) = ops.gemm_trit_t2([t2], [out_f], xb, K=in_f, row_scales=[sd], biases=[bd], out_dtype=torch.float32)
    assert rel_err(y32.cpu().numpy(), want) < 2e-5  # exact products, fp32 accumulation: order only
    (y16,) = ops.gemm_trit_t2([t2], [out_f], xb, K=in_f, row_scales=[sd], biases=[bd])
    np.testing.assert_allclose(y16.float().cpu().numpy(), want, rtol=1e-2, atol=1e-2 * float(np.sqrt(np.mean(want ** 2))))
    # fp32 activations (two bf16 planes: 16 mantissa bits), no scale, no bias, alpha
    want = 0.5 * (x.numpy().astype(np.float64) @ trits.T.astype(np.float64))
    (y,) = ops.gemm_trit_t2([t2], [out_f], x.to(dev), K=in_f, alpha=0.5)
    assert rel_err(y.cpu().numpy(), want) < 1e-4
    assert _capi.kernel_status(reset=True) == 0


@pytest_gpu
@pytest.mark.parametrize("members,in_f,tokens", [([4096, 1024, 1024], 4096, 8), ([14336, 14336], 4096, 8),
                                                 ([4096], 14336, 8), ([100, 33, 700], 130, 16), ([64, 64], 1000, 1)])
def test_t2_grouped_equals_limb_layout_kernel(dev, members, in_f, tokens):
    """Same trits, same activations: the two layouts must agree to accumulation order."""
    from t81lib_b200 import _capi, ops
    gen = torch.Generator(device="cpu").manual_seed(sum(members) + tokens)
    x = torch.randn(tokens, in_f, generator=gen).to(dev).to(torch.bfloat16)
    packed, scales, biases, t2 = [], [], [], []
    for i, out_f in enumerate(members):
        w = torch.randn(out_f, in_f, generator=gen) * 0.02
        p, s = ops.quantize_pack(w.to(dev), 0.45, "absmean")
        packed.append(p); scales.append(s); t2.append(ops.pack_t2(p, out_f, in_f))
        biases.append((torch.randn(out_f, generator=gen) * 0.01).to(dev) if i != 1 else None)
    got = ops.gemm_trit_t2(t2, members, x, K=in_f, row_scales=scales, biases=biases, out_dtype=torch.float32)
    want = ops.gemm_trit_grouped(packed, x, K=in_f, row_scales=scales, biases=biases, out_dtype=torch.float32)
    for y, w_ in zip(got, want):
        assert rel_err(y.cpu().numpy(), w_.cpu().numpy()) < 1e-5
    with pytest.raises(ValueError, match="1 to 128 tokens"):
        ops.gemm_trit_t2(t2, members, torch.zeros(129, in_f, device=dev, dtype=torch.bfloat16), K=in_f)
    assert _capi.kernel_status(reset=True) == 0


@pytest_gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_t2_alpha_beta_and_strided_results(dev, dtype):
    """C = alpha * diag(s) T(A) B + bias + beta * C into a column slice of a wider result (ldc > rows), every
    output dtype: the per-element epilogue and the 128-bit one."""
    from t81lib_b200 import _capi, ops
    rng = np.random.default_rng(3)
    out_f, in_f, tokens = 200, 520, 5
    trits = rng.integers(-1, 2, (out_f, in_f)).astype(np.int8)
    t2 = ops.pack_t2(torch.from_numpy(oracle.pack_trits_rowwise(trits)).to(dev), out_f, in_f)
    scale = torch.from_numpy(rng.uniform(0.5, 1.5, out_f).astype(np.float32)).to(dev)
    bias = torch.from_numpy(rng.normal(size=out_f).astype(np.float32)).to(dev)
    x = torch.from_numpy(rng.normal(size=(tokens, in_f)).astype(np.float32)).to(dev).to(torch.bfloat16)
    wide = torch.from_numpy(rng.normal(size=(tokens, out_f + 56)).astype(np.float32)).to(dev).to(dtype)
    before = wide.clone()
    for beta in (0.0, -0.75):
        wide.copy_(before)
        ops.gemm_trit_t2([t2], [out_f], x, K=in_f, row_scales=[scale], biases=[bias], outs=[wide[:, 8:8 + out_f]], alpha=1.5, beta=beta)
        want = 1.5 * (x.float().cpu().numpy().astype(np.float64) @ trits.T) * scale.cpu().numpy() + bias.cpu().numpy()
        want = want + beta * before[:, 8:8 + out_f].float().cpu().numpy()
        got = wide[:, 8:8 + out_f].float().cpu().numpy()
        tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7
        assert np.max(np.abs(got - want)) <= tol * np.max(np.abs(want))
        # nothing outside the slice was touched
        assert torch.equal(wide[:, :8], before[:, :8]) and torch.equal(wide[:, 8 + out_f:], before[:, 8 + out_f:])
    assert _capi.kernel_status(reset=True) == 0
