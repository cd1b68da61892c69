"""Regenerate tests/golden/tq_blocks.npz from the reference's GGUF block codecs.

    python tests/golden/generate_tq.py [/path/to/reference]

The block functions of t81/gguf.py (_quantize_blocks_tq1 / _tq2, _dequantize_blocks_tq1 / _tq2 and the two
helpers they call, lines 518-662) are pure numpy; they are taken out of the reference's source file as they
stand (the module itself imports transformers and the whole package) and run on seeded ternary matrices
scaled per row, the way a ternarised Linear looks.  Inputs and outputs are stored; the reference does not travel.
"""

from __future__ import annotations

import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
    "T81_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
WANTED = {"_round_away_from_zero", "_quantize_trits", "_quantize_blocks_tq1", "_quantize_blocks_tq2",
          "_dequantize_blocks_tq1", "_dequantize_blocks_tq2"}


def reference_functions():
    path = os.path.join(REF, "t81", "gguf.py")
    source = open(path).read()
    tree = ast.parse(source)
    ns = {"np": np, "GGUF_QUANT_BLOCK_ROWS": 256}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in WANTED:
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    return ns


def main():
    ns = reference_functions()
    rng = np.random.default_rng(81)
    out = {}
    for tag, rows, cols in (("a", 5, 512), ("b", 3, 256), ("c", 4, 600)):
        trits = rng.integers(-1, 2, (rows, cols)).astype(np.int8)
        trits[1, :256] = 0                                   # an all-zero block
        scale = rng.uniform(0.01, 0.06, rows).astype(np.float32)
        w = trits.astype(np.float32) * scale[:, None]
        bpr = (cols + 255) // 256
        padded = np.zeros((rows, bpr * 256), np.float32)
        padded[:, :cols] = w
        blocks = padded.reshape(rows * bpr, 256)
        out[f"trits_{tag}"], out[f"scale_{tag}"] = trits, scale
        for fmt, quant, dequant in (("tq1", ns["_quantize_blocks_tq1"], ns["_dequantize_blocks_tq1"]),
                                    ("tq2", ns["_quantize_blocks_tq2"], ns["_dequantize_blocks_tq2"])):
            payload = quant(blocks, 0.5).astype(np.uint8)
            out[f"{fmt}_{tag}"] = payload.reshape(rows, bpr, -1)
            out[f"{fmt}_deq_{tag}"] = dequant(payload).reshape(rows, bpr * 256)[:, :cols].astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "tq_blocks.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
