"""Parity of the tcgen05 tensor-core kernel (prefill-shaped TRIT mode: more than 16
tokens, bf16 activations, token-major layout) with the CPU oracle."""

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(lib_built):
    from t81lib_b200 import _capi
    assert _capi.device_available(), _capi.last_error()
    return torch.device("cuda", 0)


def cuda(a, dev, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t if dtype is None else t.to(dtype)


def rel_err(got, want):
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want)) / (np.sqrt(np.mean(want ** 2)) + 1e-30))


def case(rng, out_f, in_f, tokens):
    w = rng.normal(0, 0.02, (out_f, in_f)).astype(np.float32)
    packed, scale = oracle.pack_dense_matrix_absmean(w, 0.45)
    x = rng.normal(size=(tokens, in_f)).astype(np.float32)
    bias = rng.normal(0, 0.01, out_f).astype(np.float32)
    return packed, scale, x, bias


# one tile; ragged rows / tokens / K; several tiles per CTA; K below one atom; K spanning many super-blocks
SHAPES = [(128, 192, 256), (384, 1000, 200), (100, 130, 33), (130, 70, 300), (512, 512, 512), (257, 4096, 700),
          (1024, 3072, 2048), (64, 48, 17), (300, 14336, 40)]


@pytest.mark.parametrize("out_f,in_f,tokens", SHAPES)
def test_tc_gemm_matches_oracle(dev, out_f, in_f, tokens):
    from t81lib_b200 import _capi, ops
    rng = np.random.default_rng(out_f + 31 * in_f + 977 * tokens)
    packed, scale, x, bias = case(rng, out_f, in_f, tokens)
    xb = cuda(x, dev, torch.bfloat16)
    oracle.set_num_threads(8)
    want = oracle.linear_forward(packed, scale, bias, xb.float().cpu().numpy(), in_f)
    oracle.set_num_threads(1)
    y = ops.gemm_trit(cuda(packed, dev), xb, M=out_f, K=in_f, layout="nk", row_scale=cuda(scale, dev),
                      bias=cuda(bias, dev), out_dtype=torch.float32)
    assert _capi.kernel_status(reset=True) == 0
    # exact bf16 products, fp32 accumulation in TMEM: only the summation order differs
    assert rel_err(y.cpu().numpy(), want) < 2e-5
    yb = ops.gemm_trit(cuda(packed, dev), xb, M=out_f, K=in_f, layout="nk", row_scale=cuda(scale, dev),
                       bias=cuda(bias, dev))
    assert yb.dtype == torch.bfloat16
    np.testing.assert_allclose(yb.float().cpu().numpy(), want, rtol=1e-2, atol=1e-2 * float(np.sqrt(np.mean(want ** 2))))


def test_tc_gemm_alpha_beta_and_column_slice(dev):
    from t81lib_b200 import _capi, ops
    rng = np.random.default_rng(5)
    packed, scale, x, bias = case(rng, 256, 500, 100)
    xb = cuda(x, dev, torch.bfloat16)
    base = oracle.linear_forward(packed, None, None, xb.float().cpu().numpy(), 500)
    c0 = rng.normal(size=(100, 256)).astype(np.float32)
    C = cuda(c0, dev)
    ops.gemm_trit(cuda(packed, dev), xb, M=256, K=500, layout="nk", C=C, alpha=0.5, beta=2.0)
    assert rel_err(C.cpu().numpy(), 0.5 * base + 2.0 * c0) < 2e-5
    wide = torch.zeros(100, 600, device=dev)
    ops.gemm_trit(cuda(packed, dev), xb, M=256, K=500, layout="nk", C=wide[:, 200:456])
    assert rel_err(wide[:, 200:456].cpu().numpy(), base) < 2e-5
    assert not wide[:, :200].any() and not wide[:, 456:].any()
    assert _capi.kernel_status(reset=True) == 0


def test_prefill_shape_linearity_at_full_size(dev):
    """A 2048-token prefill of the Phi-3-mini qkv layer (3072 -> 9216): checked through linearity,
    y(a*x1 + x2) == a*y(x1) + y(x2), and a sampled comparison with the oracle."""
    from t81lib_b200 import _capi, ops
    gen = torch.Generator(device="cpu").manual_seed(4)
    out_f, in_f, tokens = 9216, 3072, 2048
    w = torch.randn(out_f, in_f, generator=gen) * 0.02
    packed, scale = ops.quantize_pack(w.to(dev), 0.45, "absmean")
    x1 = torch.randn(tokens, in_f, generator=gen).to(dev).to(torch.bfloat16)
    x2 = torch.randn(tokens, in_f, generator=gen).to(dev).to(torch.bfloat16)
    # powers of two keep a*x1 exact in bf16; x1 + x2 is rounded, so compare against y of the rounded sum
    xs = (2.0 * x1.float() + x2.float()).to(torch.bfloat16)
    bias = (torch.randn(out_f, generator=gen) * 0.01).to(dev)
    y1 = ops.gemm_trit(packed, x1, M=out_f, K=in_f, layout="nk", row_scale=scale, out_dtype=torch.float32)
    y2 = ops.gemm_trit(packed, x2, M=out_f, K=in_f, layout="nk", row_scale=scale, out_dtype=torch.float32)
    resid = (xs.float() - (2.0 * x1.float() + x2.float())).to(torch.bfloat16)  # exactly representable rounding error
    ys = ops.gemm_trit(packed, xs, M=out_f, K=in_f, layout="nk", row_scale=scale, out_dtype=torch.float32)
    yr = ops.gemm_trit(packed, resid, M=out_f, K=in_f, layout="nk", row_scale=scale, out_dtype=torch.float32)
    lhs, rhs = ys - yr, 2.0 * y1 + y2
    assert float((lhs - rhs).abs().max() / rhs.pow(2).mean().sqrt()) < 1e-4
    # 64 sampled rows x 48 sampled tokens against the oracle, with the bias
    rows = torch.randperm(out_f, generator=gen)[:64]
    toks = torch.randperm(tokens, generator=gen)[:48]
    yb = ops.gemm_trit(packed, x1, M=out_f, K=in_f, layout="nk", row_scale=scale, bias=bias, out_dtype=torch.float32)
    want = oracle.linear_forward(packed[rows.to(dev)].cpu().numpy(), scale[rows.to(dev)].cpu().numpy(),
                                 bias[rows.to(dev)].cpu().numpy(), x1[toks.to(dev)].float().cpu().numpy(), in_f)
    got = yb[toks.to(dev)][:, rows.to(dev)].cpu().numpy()
    assert rel_err(got, want) < 2e-5
    assert _capi.kernel_status(reset=True) == 0


# ---- activations that need the staging pre-pass (scratch workspace): fp32 / fp16 values, (K, N) layout


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("out_f,in_f,tokens", [(384, 1000, 200), (130, 700, 300), (512, 4096, 129)])
def test_tc_gemm_staged_activations_token_major(dev, dtype, out_f, in_f, tokens):
    from t81lib_b200 import _capi, ops
    rng = np.random.default_rng(out_f + in_f + tokens)
    packed, scale, x, bias = case(rng, out_f, in_f, tokens)
    xd = cuda(x, dev, dtype)
    oracle.set_num_threads(8)
    want = oracle.linear_forward(packed, scale, bias, xd.float().cpu().numpy(), in_f)
    oracle.set_num_threads(1)
    assert _capi.lib.t81b200_gemm_trit_workspace_bytes(_capi.F32 if dtype == torch.float32 else _capi.F16,
                                                        _capi.LAYOUT_NK, _capi.F32, out_f, tokens, in_f) > 0
    y = ops.gemm_trit(cuda(packed, dev), xd, M=out_f, K=in_f, layout="nk", row_scale=cuda(scale, dev),
                      bias=cuda(bias, dev), out_dtype=torch.float32)
    assert _capi.kernel_status(reset=True) == 0
    # two bf16 planes carry 16 mantissa bits of each activation: 1e-3 asked for fp32, ~1e-5 achieved
    assert rel_err(y.cpu().numpy(), want) < 1e-3
    assert rel_err(y.cpu().numpy(), want) < 5e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_tc_gemm_reference_argument_order(dev, dtype):
    """(K, N) dense operand and (M, N) result, the layout of t81::linalg::gemm_ternary."""
    from t81lib_b200 import _capi, ops
    rng = np.random.default_rng(77)
    M, N, K = 300, 260, 1000
    trits = rng.integers(-1, 2, (M, K)).astype(np.int8)
    A = oracle.pack_trits_rowwise(trits)
    B = cuda(rng.normal(size=(K, N)).astype(np.float32), dev, dtype)
    C0 = rng.normal(size=(M, N)).astype(np.float32)
    oracle.set_num_threads(8)
    want = oracle.gemm_trit(A, B.float().cpu().numpy(), C0, M, N, K, 1.5, 0.5)
    oracle.set_num_threads(1)
    C = cuda(C0, dev)
    ops.gemm_trit(cuda(A, dev), B, M=M, K=K, layout="kn", C=C, alpha=1.5, beta=0.5)
    assert _capi.kernel_status(reset=True) == 0
    assert rel_err(C.cpu().numpy(), want) < 5e-5


def test_host_pointer_entry_point(dev):
    """t81b200_gemm_trit_host: what the C++ span overload of gemm_ternary binds to."""
    import ctypes
    from t81lib_b200 import _capi
    rng = np.random.default_rng(78)
    M, N, K = 128, 64, 480
    trits = rng.integers(-1, 2, (M, K)).astype(np.int8)
    A = oracle.pack_trits_rowwise(trits)
    B = rng.normal(size=(K, N)).astype(np.float32)
    C = rng.normal(size=(M, N)).astype(np.float32)
    want = oracle.gemm_trit(A, B, C, M, N, K, 2.0, -1.0)
    vp = ctypes.c_void_p
    rc = _capi.lib.t81b200_gemm_trit_host(A.ctypes.data_as(vp), B.ctypes.data_as(vp), C.ctypes.data_as(vp), M, N, K, 2.0, -1.0)
    assert rc == 0, _capi.last_error()
    assert rel_err(C, want) < 5e-5
    rc = _capi.lib.t81b200_gemm_trit_host(A.ctypes.data_as(vp), B.ctypes.data_as(vp), C.ctypes.data_as(vp), -1, N, K, 1.0, 0.0)
    assert rc == _capi.EINVAL and "non-negative" in _capi.last_error()
