"""GGUF ternary block formats TQ1_0 / TQ2_0: the numpy restatement against fixtures produced by the reference's
own block codecs (tests/golden/generate_tq.py, from t81/gguf.py:518-662), and the device transcoders
packed limbs <-> blocks against the restatement and the fixtures, bit for bit."""

import numpy as np
import pytest

import oracle

CASES = (("a", 5, 512), ("b", 3, 256), ("c", 4, 600))
FORMATS = (("TQ1_0", "tq1"), ("TQ2_0", "tq2"))


def test_block_codecs_match_the_reference_fixtures(golden):
    g = golden("tq_blocks.npz")
    for tag, rows, cols in CASES:
        trits, scale = g[f"trits_{tag}"], g[f"scale_{tag}"]
        for fmt, key in FORMATS:
            want = g[f"{key}_{tag}"]
            assert np.array_equal(oracle.tq_encode(trits, scale, fmt), want), (tag, fmt)
            got_trits, d = oracle.tq_decode(want, rows, cols, fmt)
            assert np.array_equal(got_trits, trits), (tag, fmt)
            # the reference's dequantiser gives d * trit
            deq = got_trits.astype(np.float32) * np.repeat(d, 256, axis=1)[:, :cols]
            assert np.array_equal(deq, g[f"{key}_deq_{tag}"]), (tag, fmt)


def test_block_round_trip_and_padding():
    rng = np.random.default_rng(9)
    for cols in (1, 255, 256, 257, 1000):
        trits = rng.integers(-1, 2, (3, cols)).astype(np.int8)
        for fmt, _ in FORMATS:
            blocks = oracle.tq_encode(trits, None, fmt)
            assert blocks.shape == (3, (cols + 255) // 256, 66 if fmt == "TQ2_0" else 54)
            back, d = oracle.tq_decode(blocks, 3, cols, fmt)
            assert np.array_equal(back, trits) and set(np.unique(d)) <= {0.0, 1.0}


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,key", FORMATS)
def test_device_transcoders_match_fixtures_and_oracle(lib_built, golden, fmt, key):
    import torch
    from t81lib_b200 import _capi, ops
    assert _capi.device_available(), _capi.last_error()
    dev = torch.device("cuda", 0)
    g = golden("tq_blocks.npz")
    for tag, rows, cols in CASES:
        trits, scale = g[f"trits_{tag}"], g[f"scale_{tag}"]
        packed = torch.from_numpy(oracle.pack_trits_rowwise(trits)).to(dev)
        blocks = ops.packed_to_tq(packed, rows, cols, fmt, row_scale=torch.from_numpy(scale).to(dev))
        assert np.array_equal(blocks.cpu().numpy(), g[f"{key}_{tag}"]), tag           # what the reference writes
        back, d = ops.tq_to_packed(torch.from_numpy(g[f"{key}_{tag}"]).to(dev), rows, cols, fmt)
        assert np.array_equal(back.cpu().numpy(), oracle.pack_trits_rowwise(trits)), tag
        assert np.array_equal(d.cpu().numpy(), oracle.tq_decode(g[f"{key}_{tag}"], rows, cols, fmt)[1])
    # a Linear-sized matrix, through the quantiser: export, import, and the imported weights in the matmul
    rng = np.random.default_rng(5)
    rows, cols = 300, 4096
    w = torch.from_numpy(rng.normal(0, 0.02, (rows, cols)).astype(np.float32)).to(dev)
    packed, scale = ops.quantize_pack(w, 0.45, "absmean")
    blocks = ops.packed_to_tq(packed, rows, cols, fmt, row_scale=scale)
    trits = ops.unpack(packed, rows, cols).cpu().numpy()
    assert np.array_equal(blocks.cpu().numpy(), oracle.tq_encode(trits, scale.cpu().numpy(), fmt))
    back, d = ops.tq_to_packed(blocks, rows, cols, fmt)
    assert torch.equal(back, packed)
    d16 = scale.to(torch.float16).float()
    assert torch.equal(d, d16[:, None].expand(-1, cols // 256))                     # scales come back rounded to fp16
    x = torch.randn(4, cols, device=dev).to(torch.bfloat16)
    y_import = ops.gemm_trit(back, x, M=rows, K=cols, layout="nk", row_scale=d[:, 0].contiguous(), out_dtype=torch.float32)
    y_direct = ops.gemm_trit(packed, x, M=rows, K=cols, layout="nk", row_scale=d16, out_dtype=torch.float32)
    assert torch.equal(y_import, y_direct)
    with pytest.raises(ValueError):
        ops.tq_to_packed(blocks[:, :-1], rows, cols, fmt)
