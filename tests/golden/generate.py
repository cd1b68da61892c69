"""Regenerate the golden fixtures in this folder from the reference itself.

Run where the reference checkout is mounted and oracle/_ref has been built
(``make -C oracle ref``):

    python tests/golden/generate.py [/path/to/reference]

It imports the reference's compiled ``t81lib`` module (oracle/_ref) and its
``t81.torch`` Python layer, feeds them seeded inputs and stores inputs and
outputs as small ``.npz`` files.  The fixtures travel with the repository; the
reference does not.
"""

from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
    "T81_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))

from oracle import ref as oracle_ref  # noqa: E402

t81lib = oracle_ref.load()
sys.modules["t81lib"] = t81lib
sys.path.insert(0, REF)
import torch  # noqa: E402
import t81.torch as ref_torch  # noqa: E402


def boundary_matrix(rng, rows=64, cols=100, sigma=0.5):
    w = rng.normal(0.0, sigma, (rows, cols)).astype(np.float32)
    thr = np.float32(0.45)
    w[0, :8] = [thr, -thr, np.nextafter(thr, np.float32(0)), -np.nextafter(thr, np.float32(0)),
                np.nextafter(thr, np.float32(1)), 1.5, -2.0, 0.0]
    w[1, :6] = [np.nan, np.inf, -np.inf, -0.0, 1.0, -1.0]
    return w


def limbs_v16(packed_u8, rows, cols):
    return np.ascontiguousarray(packed_u8).reshape(rows * cols, 16).view("V16").reshape(rows, cols)


def main():
    rng = np.random.default_rng(20240611)

    # ---- pack / quantize / unpack (rule "fixed") -------------------------------
    w = boundary_matrix(rng)
    out = {"w": w}
    for name, thr in (("t045", 0.45), ("t050", 0.5), ("t100", 1.0), ("t001", 0.01)):
        out[f"packed_{name}"] = np.asarray(t81lib.pack_dense_matrix(w, thr))
        out[f"trits_{name}"] = np.asarray(t81lib.quantize_to_trits(w, thr))
    tt = ref_torch.TernaryTensor.from_float(torch.from_numpy(w), threshold=0.45)
    out["from_float_t045"] = np.ascontiguousarray(tt._packed).view(np.uint8).reshape(64, -1, 16)
    out["unpacked_t045"] = np.asarray(t81lib.unpack_packed_limbs(out["packed_t045"], 64, 100))
    # threshold 0 through the Python layer (the C++ binding rejects it)
    tt0 = ref_torch.TernaryTensor.from_float(torch.from_numpy(w), threshold=0.0)
    out["from_float_t000"] = np.ascontiguousarray(tt0._packed).view(np.uint8).reshape(64, -1, 16)
    # odd widths: 1, 47, 48, 49, 96, 145 columns
    for cols in (1, 47, 48, 49, 96, 145):
        wc = rng.normal(0.0, 0.6, (5, cols)).astype(np.float32)
        out[f"w_c{cols}"] = wc
        out[f"packed_c{cols}"] = np.asarray(t81lib.pack_dense_matrix(wc, 0.45))
    np.savez_compressed(os.path.join(HERE, "pack_fixed.npz"), **out)

    # ---- LIMB-mode GEMM ---------------------------------------------------------
    g = {}
    M, N, KL = 9, 7, 3

    def small_trits(shape_rows, shape_cols, along_rows, nz):
        """trits with only the first `nz` positions of each limb non-zero"""
        t = np.zeros((shape_rows, shape_cols), np.int8)
        for l in range(KL):
            if along_rows:
                t[:, l * 48:l * 48 + nz] = rng.integers(-1, 2, (shape_rows, nz))
            else:
                t[l * 48:l * 48 + nz, :] = rng.integers(-1, 2, (nz, shape_cols))
        return t

    for tag, nz in (("nz10", 10), ("nz30", 30), ("nz48", 48)):
        ta = small_trits(M, KL * 48, True, nz)
        tb = small_trits(KL * 48, N, False, nz)
        A = np.asarray(t81lib.pack_dense_matrix(ta.astype(np.float32), 0.5))
        B = np.ascontiguousarray(ref_torch._pack_columnwise(tb, KL, KL * 48)).view(np.uint8).reshape(KL, N, 16)
        C0 = rng.normal(size=(M, N)).astype(np.float32)
        C = C0.copy()
        t81lib.gemm_ternary(limbs_v16(A, M, KL), limbs_v16(B, KL, N), C, M, N, KL * 48, 1.25, 0.5)
        g[f"A_{tag}"], g[f"B_{tag}"], g[f"C0_{tag}"], g[f"C_{tag}"] = A, B, C0, C
        g[f"ta_{tag}"], g[f"tb_{tag}"] = ta, tb
    # the reference's known-answer checks (tests/python/test_bindings.py:17-39)
    zero = np.full((6, 16), 13, np.uint8)
    C = np.zeros((2, 3), np.float32)
    t81lib.gemm_ternary(limbs_v16(zero[:2], 2, 1), limbs_v16(zero[:3], 1, 3), C, 2, 3, 48)
    g["ka_zero"] = C.copy()
    C = np.full((2, 3), 2.0, np.float32)
    t81lib.gemm_ternary(limbs_v16(zero[:2], 2, 1), limbs_v16(zero[:3], 1, 3), C, 2, 3, 48, 0.0, 0.5)
    g["ka_beta"] = C.copy()
    # single limb products on random full-range limbs, seed as in tests/unit/test_limb_basic.cpp:106
    r2 = np.random.default_rng(0xDEADBEEF)
    la = r2.integers(0, 27, (64, 16)).astype(np.uint8)
    lb = r2.integers(0, 27, (64, 16)).astype(np.uint8)
    prod = np.zeros(64, np.float64)
    for i in range(64):
        # alpha scales the product into fp32 range so the float32 C keeps 24 bits of it
        C = np.zeros((1, 1), np.float32)
        t81lib.gemm_ternary(limbs_v16(la[i:i + 1], 1, 1), limbs_v16(lb[i:i + 1], 1, 1), C, 1, 1, 48, 1e-30, 0.0)
        prod[i] = C[0, 0]
    g["prod_a"], g["prod_b"], g["prod_c_alpha1e-30"] = la, lb, prod.astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "gemm_limb.npz"), **g)

    # ---- TRIT-mode cross-check owned by the reference: its autograd backward's dense form
    # (t81/torch/__init__.py:292-300): dequantised trits, float matmul ----------------------
    t = {}
    wt = rng.normal(0.0, 0.5, (24, 130)).astype(np.float32)
    tern = ref_torch.TernaryTensor.from_float(torch.from_numpy(wt), threshold=0.45)
    trits = ref_torch._limbs_to_trits(tern._packed, 24, tern._k_limbs)[:, :130].astype(np.float32)
    x = rng.normal(size=(130, 11)).astype(np.float32)
    t["w"], t["packed"], t["x"] = wt, np.ascontiguousarray(tern._packed).view(np.uint8).reshape(24, -1, 16), x
    t["trits"] = trits.astype(np.int8)
    t["y_f64"] = trits.astype(np.float64) @ x.astype(np.float64)
    np.savez_compressed(os.path.join(HERE, "gemm_trit.npz"), **t)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
