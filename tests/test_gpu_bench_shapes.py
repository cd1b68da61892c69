"""Parity of the matmul kernels (both weight layouts of the streaming one) at the shapes the benchmark times, through the C ABI.

The launch shape of the streaming (decode) kernel is picked from the row count and the
contraction length, so small cases do not reach the configurations the large layers run
with.  Every decode-sized shape of the Phi-3-mini sweep (1, 4 and 16 tokens) and of the
Llama-3-8B-shaped stack (8 tokens), and every prefill shape of both, is therefore run at
full size and compared with the CPU oracle on sampled output features (first and last
row tile included) — the oracle is fed only the sampled rows of the packed matrix, which
is exact because packing is row-wise."""

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

PHI3 = [(9216, 3072), (3072, 3072), (16384, 3072), (3072, 8192)]        # (out_features, in_features)
LLAMA = [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)]


@pytest.fixture(scope="module")
def dev(lib_built):
    from t81lib_b200 import _capi
    assert _capi.device_available(), _capi.last_error()
    return torch.device("cuda", 0)


def rel_err(got, want):
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want)) / (np.sqrt(np.mean(want ** 2)) + 1e-30))


_weights = {}
_t2 = {}


def packed_layer(dev, out_f, in_f):
    """Quantised + packed N(0, 0.02^2) weight of one layer, absmean rule, packed on the device
    (its bytes are checked against the oracle elsewhere); cached per shape."""
    from t81lib_b200 import ops
    key = (out_f, in_f)
    if key not in _weights:
        gen = torch.Generator(device="cpu").manual_seed(out_f * 31 + in_f)
        w = torch.randn(out_f, in_f, generator=gen) * 0.02
        _weights[key] = ops.quantize_pack(w.to(dev), 0.45, "absmean")
    return _weights[key]


def sampled_rows(out_f, gen, n=64):
    rows = torch.randperm(out_f, generator=gen)[:n - 34]
    edge = torch.cat([torch.arange(0, 17), torch.arange(out_f - 17, out_f)])  # first and last row tile
    return torch.unique(torch.cat([rows, edge]))


@pytest.mark.parametrize("tokens", [1, 4, 16])
@pytest.mark.parametrize("out_f,in_f", PHI3)
def test_decode_kernel_phi3_shapes(dev, out_f, in_f, tokens):
    _check_decode(dev, out_f, in_f, tokens)


@pytest.mark.parametrize("out_f,in_f", LLAMA)
def test_decode_kernel_llama_shapes(dev, out_f, in_f):
    _check_decode(dev, out_f, in_f, 8)


def _check_decode(dev, out_f, in_f, tokens):
    from t81lib_b200 import _capi, ops
    packed, scale = packed_layer(dev, out_f, in_f)
    gen = torch.Generator(device="cpu").manual_seed(tokens * 7919 + out_f)
    x = torch.randn(tokens, in_f, generator=gen).to(dev).to(torch.bfloat16)
    bias = (torch.randn(out_f, generator=gen) * 0.01).to(dev)
    rows = sampled_rows(out_f, gen).to(dev)
    want = oracle.linear_forward(packed[rows].cpu().numpy(), scale[rows].cpu().numpy(), bias[rows].cpu().numpy(),
                                 x.float().cpu().numpy(), in_f)
    y32 = ops.gemm_trit(packed, x, M=out_f, K=in_f, layout="nk", row_scale=scale, bias=bias, out_dtype=torch.float32)
    assert rel_err(y32[:, rows].cpu().numpy(), want) < 2e-5   # exact products, fp32 accumulation: order only
    y16 = ops.gemm_trit(packed, x, M=out_f, K=in_f, layout="nk", row_scale=scale, bias=bias)  # the benchmark's form
    np.testing.assert_allclose(y16[:, rows].float().cpu().numpy(), want, rtol=1e-2,
                               atol=1e-2 * float(np.sqrt(np.mean(want ** 2))))  # bf16 activations: 1e-2
    # every output element, not only the sampled rows, against the fp32 result of the same kernel
    assert float((y16.float() - y32).abs().max()) <= 2.0 ** -8 * float(y32.abs().max())
    # the same product on the decode-stream layout of the weight (what the benchmark's decode phase and
    # TernaryTensor.matmul_input run): against the oracle on the sampled rows, and every element against the above
    t2 = _t2.get((out_f, in_f))
    if t2 is None:
        t2 = _t2[(out_f, in_f)] = ops.pack_t2(packed, out_f, in_f)
    (z32,) = ops.gemm_trit_t2([t2], [out_f], x, K=in_f, row_scales=[scale], biases=[bias], out_dtype=torch.float32)
    assert rel_err(z32[:, rows].cpu().numpy(), want) < 2e-5
    assert float((z32 - y32).abs().max()) <= 1e-5 * float(y32.abs().max())
    (z16,) = ops.gemm_trit_t2([t2], [out_f], x, K=in_f, row_scales=[scale], biases=[bias])
    assert float((z16.float() - z32).abs().max()) <= 2.0 ** -8 * float(z32.abs().max())
    assert _capi.kernel_status(reset=True) == 0


@pytest.mark.parametrize("out_f,in_f,tokens", [(o, i, 2048) for o, i in PHI3] + [(o, i, 16384) for o, i in LLAMA])
def test_prefill_kernel_bench_shapes(dev, out_f, in_f, tokens):
    from t81lib_b200 import _capi, ops
    packed, scale = packed_layer(dev, out_f, in_f)
    gen = torch.Generator(device="cpu").manual_seed(tokens + out_f)
    x = torch.randn(tokens, in_f, generator=gen).to(dev).to(torch.bfloat16)
    bias = (torch.randn(out_f, generator=gen) * 0.01).to(dev)
    rows = sampled_rows(out_f, gen).to(dev)
    toks = torch.unique(torch.cat([torch.randperm(tokens, generator=gen)[:40], torch.tensor([0, tokens - 1])])).to(dev)
    want = oracle.linear_forward(packed[rows].cpu().numpy(), scale[rows].cpu().numpy(), bias[rows].cpu().numpy(),
                                 x[toks].float().cpu().numpy(), in_f)
    y = ops.gemm_trit(packed, x, M=out_f, K=in_f, layout="nk", row_scale=scale, bias=bias)  # bf16 out: the benchmark's form
    got = y[toks][:, rows].float().cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-2 * float(np.sqrt(np.mean(want ** 2))))
    if tokens == 2048:  # fp32 output too, at the tight tolerance
        y32 = ops.gemm_trit(packed, x, M=out_f, K=in_f, layout="nk", row_scale=scale, bias=bias, out_dtype=torch.float32)
        assert rel_err(y32[toks][:, rows].cpu().numpy(), want) < 2e-5
    assert _capi.kernel_status(reset=True) == 0


@pytest.mark.parametrize("members,in_f,tokens", [([4096, 1024, 1024], 4096, 8), ([14336, 14336], 4096, 8),
                                                 ([9216], 3072, 4), ([100, 33, 700], 130, 16), ([64, 64], 1000, 1)])
def test_grouped_decode_call_equals_the_separate_calls(dev, members, in_f, tokens):
    """One launch for the matrices that share their input (q/k/v, gate/up) must give what one call per
    matrix gives (the same kernel; the launch shape, and with it the order of the partial sums, may differ)."""
    from t81lib_b200 import _capi, ops
    gen = torch.Generator(device="cpu").manual_seed(sum(members) + tokens)
    x = torch.randn(tokens, in_f, generator=gen).to(dev).to(torch.bfloat16)
    packed, scales, biases = [], [], []
    for i, out_f in enumerate(members):
        w = torch.randn(out_f, in_f, generator=gen) * 0.02
        p, s = ops.quantize_pack(w.to(dev), 0.45, "absmean")
        packed.append(p); scales.append(s); biases.append((torch.randn(out_f, generator=gen) * 0.01).to(dev) if i != 1 else None)
    got = ops.gemm_trit_grouped(packed, x, K=in_f, row_scales=scales, biases=biases, out_dtype=torch.float32)
    for p, s, b, y, out_f in zip(packed, scales, biases, got, members):
        want = ops.gemm_trit(p, x, M=out_f, K=in_f, layout="nk", row_scale=s, bias=b, out_dtype=torch.float32)
        assert rel_err(y.cpu().numpy(), want.cpu().numpy()) < 1e-5
    got16 = ops.gemm_trit_grouped(packed, x, K=in_f, row_scales=scales, biases=biases)
    assert all(y.dtype == torch.bfloat16 and y.shape == (tokens, m) for y, m in zip(got16, members))
    for y16, y32 in zip(got16, got):
        assert float((y16.float() - y32).abs().max()) <= 2.0 ** -8 * float(y32.abs().max()) + 1e-30
    assert _capi.kernel_status(reset=True) == 0
