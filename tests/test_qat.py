"""Quantisation-aware-training forward (t81/nn/linear.py:72-99, t81/qat.py:12-57): the numpy restatement and the
package's PyTorch form against fixtures recorded from the reference's own code (tests/golden/generate_qat.py),
and the fused device path — scale update, quantise + pack, packed-trit product, backward — against the same."""

import numpy as np
import pytest
import torch

import oracle


def test_restatement_matches_reference_fixtures(golden):
    g = golden("qat_linear.npz")
    thr = float(g["threshold"])
    scale = None
    for step in (1, 2):
        scale = oracle.qat_update_scale(g[f"w{step}"], scale)
        assert scale == g[f"scale{step}"]                                       # float32, bit for bit
        assert np.array_equal(oracle.qat_quantize(g[f"w{step}"], scale, thr), g[f"trits{step}"])
        y, gx, gw, gb = oracle.qat_linear(g[f"w{step}"], scale, thr, g[f"x{step}"], g[f"b{step}"])(g[f"gy{step}"])
        np.testing.assert_allclose(y, g[f"y{step}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(gx, g[f"grad_x{step}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(gw, g[f"grad_w{step}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(gb, g[f"grad_b{step}"], rtol=1e-5, atol=1e-6)


def _run_layer(golden, device):
    from t81lib_b200.nn import Linear
    g = golden("qat_linear.npz")
    layer = Linear(50, 12, threshold=float(g["threshold"])).to(device)
    layer.train()
    results = []
    for step in (1, 2):
        with torch.no_grad():
            layer.weight.copy_(torch.from_numpy(g[f"w{step}"]))
            layer.bias.copy_(torch.from_numpy(g[f"b{step}"]))
        layer.zero_grad()
        x = torch.from_numpy(g[f"x{step}"]).to(device).requires_grad_(True)
        y = layer(x)
        (y * torch.from_numpy(g[f"gy{step}"]).to(device)).sum().backward()
        results.append((float(layer.training_scale), y.detach().cpu().numpy(), x.grad.cpu().numpy(),
                        layer.weight.grad.cpu().numpy(), layer.bias.grad.cpu().numpy()))
    return g, results


def test_pytorch_training_forward_matches_reference_fixtures(lib_built, golden):
    g, results = _run_layer(golden, "cpu")
    for step, (scale, y, gx, gw, gb) in zip((1, 2), results):
        assert np.float32(scale) == g[f"scale{step}"]
        np.testing.assert_allclose(y, g[f"y{step}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(gx, g[f"grad_x{step}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(gw, g[f"grad_w{step}"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(gb, g[f"grad_b{step}"], rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
def test_fused_training_forward_matches_reference_fixtures(lib_built, golden):
    from t81lib_b200 import _capi
    assert _capi.device_available(), _capi.last_error()
    g, results = _run_layer(golden, "cuda:0")
    for step, (scale, y, gx, gw, gb) in zip((1, 2), results):
        assert np.float32(scale) == g[f"scale{step}"]                           # the device reduction + blend, bit for bit
        rms = float(np.sqrt(np.mean(g[f"y{step}"] ** 2)))
        assert np.max(np.abs(y - g[f"y{step}"])) < 1e-3 * rms                   # fp32 activations: 1e-3
        np.testing.assert_allclose(gx, g[f"grad_x{step}"], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(gw, g[f"grad_w{step}"], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(gb, g[f"grad_b{step}"], rtol=1e-4, atol=1e-6)
    assert _capi.kernel_status(reset=True) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols,dtype", [(1, 1, torch.float32), (33, 100, torch.float32), (256, 4096, torch.float32),
                                             (64, 1000, torch.bfloat16), (4096, 4096, torch.float32)])
def test_qat_kernels_bit_exact_against_oracle(lib_built, rows, cols, dtype):
    from t81lib_b200 import ops
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(rows + cols)
    w = torch.from_numpy(rng.normal(0, 0.03, (rows, cols)).astype(np.float32)).to(dev).to(dtype)
    wf = w.float().cpu().numpy()
    state = torch.zeros(4, device=dev)
    scale = None
    for _ in range(3):                                                           # first call, then two blends
        got = ops.qat_update_scale(w, state)
        scale = oracle.qat_update_scale(wf, scale)
        assert np.float32(got.item()) == scale
        assert state[1].item() == 0.0 and state[2].item() == 0.0                 # scratch words are clean again
    packed, row_scale = ops.qat_quantize_pack(w, 0.45, state[:1])
    want = oracle.pack_trits_rowwise(oracle.qat_quantize(wf, scale, 0.45))
    assert np.array_equal(packed.cpu().numpy(), want)
    assert bool((row_scale == state[0]).all())
    # threshold 0 keeps every non-zero sign and leaves exact zeros zero (sign(0) = 0)
    w0 = w.clone(); w0[0, 0] = 0.0
    packed0, _ = ops.qat_quantize_pack(w0, 0.0, state[:1])
    assert np.array_equal(packed0.cpu().numpy(), oracle.pack_trits_rowwise(oracle.qat_quantize(w0.float().cpu().numpy(), scale, 0.0)))
