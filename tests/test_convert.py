"""Whole-model conversion (t81lib_b200.convert, the counterpart of the reference's t81/convert.py:100-352):
the module walk, bias policy, statistics and the t81_metadata.json round trip on the CPU; packing on the
device, bit-exact against the oracle, and the converted model's forward against the oracle's Linear chain
on the GPU."""

import numpy as np
import pytest
import torch
from torch import nn

import oracle


class Block(nn.Module):
    """Transformer-shaped: attention projections, a gated MLP, norms and an embedding that must stay untouched."""

    def __init__(self, hidden=96, kv=48, ffn=200, bias=True):
        super().__init__()
        self.norm = nn.LayerNorm(hidden)
        self.attn = nn.ModuleDict({"q": nn.Linear(hidden, hidden, bias=bias), "k": nn.Linear(hidden, kv, bias=False),
                                   "v": nn.Linear(hidden, kv, bias=False), "o": nn.Linear(hidden, hidden, bias=bias)})
        self.mlp = nn.Sequential(nn.Linear(hidden, ffn, bias=bias), nn.GELU(), nn.Linear(ffn, hidden, bias=bias))


class Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(50, 96)
        self.layers = nn.ModuleList([Block(), Block(bias=False)])
        self.head = nn.Linear(96, 50, bias=False)


def _linears(model):
    return [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear)]


def test_convert_walks_replaces_and_keeps_parameters(lib_built):
    from t81lib_b200 import convert as t81_convert
    from t81lib_b200.nn import Linear as TernaryLinear
    torch.manual_seed(0)
    model = Tiny()
    before = {n: m.weight for n, m in _linears(model)}
    with pytest.raises(ValueError, match="inplace=True"):
        t81_convert.convert(model)
    out = t81_convert.convert(model, threshold=0.4, inplace=True)
    assert out is model
    after = _linears(model)
    assert len(after) == len(before) == 13 and all(isinstance(m, TernaryLinear) for _, m in after)
    assert all(m.weight is before[n] for n, m in after)          # parameters are taken over, not copied
    assert all(m.ternary_threshold == 0.4 for _, m in after)
    assert isinstance(model.embed, nn.Embedding) and isinstance(model.layers[0].norm, nn.LayerNorm)
    stats = model._t81_compression_stats
    assert stats.replaced == 13 and stats.packed_on_device == 0  # CPU weights are packed lazily, like the reference
    assert stats.float_bytes == sum(w.numel() * 4 for w in before.values())
    assert stats.ternary_bytes == sum(w.shape[0] * ((w.shape[1] + 47) // 48) * 16 for w in before.values())
    assert model._t81_threshold == 0.4 and model._t81_keep_biases_bf16 is True
    # converting again only updates the threshold of what is already ternary (t81/convert.py:106-108)
    t81_convert.convert(model, threshold=0.3, inplace=True)
    assert all(m.ternary_threshold == 0.3 for _, m in _linears(model)) and model._t81_compression_stats.replaced == 0


def test_bias_policy_and_metadata_round_trip(lib_built, tmp_path):
    from t81lib_b200 import convert as t81_convert
    model = Tiny().to(torch.bfloat16)
    t81_convert.convert(model, threshold=0.37, keep_biases_bf16=False, inplace=True, rule="absmean")
    biases = [m.bias for _, m in _linears(model) if m.bias is not None]
    assert biases and all(b.dtype == torch.float32 for b in biases)   # bf16 biases widened (t81/convert.py:124-133)
    saved = {}
    t81_convert.save_pretrained_t81(model, tmp_path, save_fn=lambda m, d: saved.setdefault("state", m.state_dict()))
    assert "state" in saved
    assert t81_convert.read_metadata(tmp_path) == {"threshold": 0.37, "keep_biases_bf16": False, "rule": "absmean"}

    def loader(path):
        fresh = Tiny()
        fresh.load_state_dict({k: v.float() for k, v in saved["state"].items()})
        return fresh
    again = t81_convert.from_pretrained_t81(None, tmp_path, loader=loader)
    assert all(m.ternary_threshold == 0.37 and m.ternary_rule == "absmean" for _, m in _linears(again))
    assert again._t81_keep_biases_bf16 is False


@pytest.mark.gpu
@pytest.mark.parametrize("rule", ["fixed", "absmean"])
def test_convert_on_device_packs_bit_exactly_and_forward_matches_oracle(lib_built, rule):
    from t81lib_b200 import _capi, convert as t81_convert
    assert _capi.device_available(), _capi.last_error()
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    model = Tiny()
    scale = 1.0 if rule == "absmean" else 25.0   # fixed rule: weights must reach the threshold at all
    with torch.no_grad():
        for _, m in _linears(model):
            m.weight.mul_(scale)
    model = model.to(dev).eval()
    weights = {n: m.weight.detach().cpu().numpy().copy() for n, m in _linears(model)}
    t81_convert.convert(model, threshold=0.45, inplace=True, rule=rule)
    stats = model._t81_compression_stats
    assert stats.replaced == 13 and stats.packed_on_device == 13
    for n, m in _linears(model):
        tt = m.ternary_weight
        assert tt is not None and tt.packed.is_cuda
        if rule == "fixed":
            want, want_scale = oracle.pack_dense_matrix(weights[n], 0.45), None
            assert tt.row_scale is None
        else:
            want, want_scale = oracle.pack_dense_matrix_absmean(weights[n], 0.45)
            assert np.array_equal(tt.row_scale.cpu().numpy(), want_scale)
        assert np.array_equal(tt.packed.cpu().numpy(), want), n
    # forward of the gated MLP of layer 0 against the oracle's Linear chain (bf16 activations: 1e-2)
    mlp = model.layers[0].mlp
    x = torch.randn(6, 96, device=dev).to(torch.bfloat16)
    with torch.no_grad():
        h = mlp[0](x)
        y = mlp[2](torch.nn.functional.gelu(h.float()).to(torch.bfloat16))

    def ref_linear(mod, name, inp):
        if rule == "fixed":
            pk, sc = oracle.pack_dense_matrix(weights[name], 0.45), None
        else:
            pk, sc = oracle.pack_dense_matrix_absmean(weights[name], 0.45)
        return oracle.linear_forward(pk, sc, mod.bias.detach().float().cpu().numpy(), inp, weights[name].shape[1])
    h_ref = ref_linear(mlp[0], "layers.0.mlp.0", x.float().cpu().numpy())
    np.testing.assert_allclose(h.float().cpu().numpy(), h_ref, rtol=1e-2, atol=1e-2 * float(np.sqrt(np.mean(h_ref ** 2))))
    mid = torch.nn.functional.gelu(h.float()).to(torch.bfloat16).float().cpu().numpy()  # same intermediate on both sides
    y_ref = ref_linear(mlp[2], "layers.0.mlp.2", mid)
    np.testing.assert_allclose(y.float().cpu().numpy(), y_ref, rtol=1e-2, atol=1e-2 * float(np.sqrt(np.mean(y_ref ** 2))))


@pytest.mark.gpu
def test_release_float_keeps_only_the_packed_weights(lib_built):
    from t81lib_b200 import convert as t81_convert
    dev = torch.device("cuda", 0)
    torch.manual_seed(4)
    model = Tiny().to(dev).eval()
    x = torch.randn(5, 96, device=dev)
    kept = Tiny().to(dev).eval()
    kept.load_state_dict(model.state_dict())
    t81_convert.convert(kept, inplace=True, rule="absmean")
    t81_convert.convert(model, inplace=True, rule="absmean", release_float=True)
    lin, lin_kept = model.layers[1].mlp[0], kept.layers[1].mlp[0]
    assert lin.weight.numel() == 0 and lin_kept.weight.numel() == 96 * 200
    with torch.no_grad():
        assert torch.equal(lin(x), lin_kept(x))
    with pytest.raises(RuntimeError, match="eval mode"):
        lin.train()
