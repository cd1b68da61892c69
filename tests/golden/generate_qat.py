"""Regenerate tests/golden/qat_linear.npz from the reference's quantisation-aware-training code.

    python tests/golden/generate_qat.py [/path/to/reference]

t81/qat.py imports nothing but torch and is executed as it stands; the running-scale update is the method
``_update_training_scale`` taken out of t81/nn/linear.py's source (the module itself pulls in the whole package)
and bound to a stand-in object.  Two training steps of one small layer are recorded: scales, quantised weights,
outputs and the gradients PyTorch's autograd derives through the reference's straight-through function.
"""

from __future__ import annotations

import ast
import os
import sys
import types

import numpy as np
import torch
from torch.nn import functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
    "T81_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))


def load_reference():
    qat = {"__name__": "t81_qat"}
    exec(compile(open(os.path.join(REF, "t81", "qat.py")).read(), "qat.py", "exec"), qat)
    tree = ast.parse(open(os.path.join(REF, "t81", "nn", "linear.py")).read())
    ns = {"torch": torch}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "_update_training_scale":
            exec(compile(ast.Module([node], []), "linear.py", "exec"), ns)
    return qat["ternary"], ns["_update_training_scale"]


def main():
    ternary, update_scale = load_reference()
    gen = torch.Generator().manual_seed(81)
    out_f, in_f, tokens, thr = 12, 50, 5, 0.45
    layer = types.SimpleNamespace(weight=None, training_scale=None)
    out = {"threshold": np.float32(thr)}
    w = torch.randn(out_f, in_f, generator=gen) * 0.05
    w[0, :4] = torch.tensor([0.0, 1e-9, -1e-9, 0.2])
    bias = torch.randn(out_f, generator=gen) * 0.01
    for step in (1, 2):
        w = (w + torch.randn(out_f, in_f, generator=gen) * 0.01 * (step - 1)).detach().requires_grad_(True)
        x = torch.randn(tokens, in_f, generator=gen, requires_grad=True)
        b = bias.clone().requires_grad_(True)
        gy = torch.randn(tokens, out_f, generator=gen)
        layer.weight = w
        scale = update_scale(layer)
        quantized = ternary(w / scale, threshold=thr, stochastic=False)
        y = F.linear(x, quantized * scale, b)
        (y * gy).sum().backward()
        out.update({f"w{step}": w.detach().numpy(), f"x{step}": x.detach().numpy(), f"b{step}": b.detach().numpy(),
                    f"gy{step}": gy.numpy(), f"scale{step}": scale.detach().numpy(),
                    f"trits{step}": quantized.detach().numpy().astype(np.int8), f"y{step}": y.detach().numpy(),
                    f"grad_w{step}": w.grad.numpy(), f"grad_x{step}": x.grad.numpy(), f"grad_b{step}": b.grad.numpy()})
    np.savez_compressed(os.path.join(HERE, "qat_linear.npz"), **out)
    print({k: getattr(v, "shape", v) for k, v in out.items()})


if __name__ == "__main__":
    main()
