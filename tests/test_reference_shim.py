"""The C++ boundary: reference_shim/linalg_cuda_shim.cpp fills the CUDA backend slot the
reference's own headers declare.  ``make -C oracle ref_cuda`` links the reference's unmodified
gemm_dispatch.cpp + gemm_cpu.cpp (and, for the Python module, python/bindings.cpp) with the shim
and libt81_b200.so under -DT81LIB_USE_CUDA=1; the CPU tests check that this build links and
loads, the GPU tests drive the reference's public C++ and pybind entry points through it and
compare with the CPU oracle."""

import os
import struct
import subprocess
import sys

import numpy as np
import pytest

import oracle
from oracle import ref as oracle_ref

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("T81_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))  # beside the repository
DRIVER = os.path.join(oracle_ref.cuda_dir(), "ref_cuda_driver")


def _have_reference():
    return os.path.isdir(os.path.join(REFERENCE, "python"))


def test_shim_links_into_the_unmodified_reference(lib_built):
    """Where the reference sources are mounted, build the integration from scratch; the build
    fails on any duplicate or missing symbol between the shim and the reference's dispatcher."""
    if not _have_reference():
        pytest.skip("reference sources are not mounted here; the prebuilt files are checked below")
    res = subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-B", "ref_cuda", "-j2", f"REF={REFERENCE}"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert os.path.exists(DRIVER)


def test_cuda_enabled_reference_module_loads_and_reports_the_backend(lib_built):
    if not os.path.exists(DRIVER):
        pytest.skip("oracle/_ref/cuda has not been built (needs the reference sources)")
    _run_module_worker("cpu")
    # the driver starts and links against libt81_b200.so wherever the tree lies
    res = subprocess.run([DRIVER], capture_output=True, text=True)
    assert res.returncode == 2 and "usage" in res.stderr


# ------------------------------------------------------------------------------------------ on the GPU


def _run_driver(mode, payload: bytes, tmp_path) -> bytes:
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    fin.write_bytes(payload)
    res = subprocess.run([DRIVER, mode, str(fin), str(fout)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    return fout.read_bytes()


def _finite_limb_operands(rng, M, N, KL, nonzero=10):
    """Limbs with few non-zero trits, so limb values and their products stay finite in fp32."""
    ta = np.zeros((M, KL * 48), np.int8)
    tb = np.zeros((KL * 48, N), np.int8)
    for l in range(KL):
        ta[:, l * 48:l * 48 + nonzero] = rng.integers(-1, 2, (M, nonzero))
        tb[l * 48:l * 48 + nonzero] = rng.integers(-1, 2, (nonzero, N))
    return oracle.pack_trits_rowwise(ta), oracle.pack_trits_columnwise(tb)


@pytest.mark.gpu
def test_cpp_gemm_ternary_limb_mode_through_the_reference_dispatcher(lib_built, tmp_path):
    assert os.path.exists(DRIVER), "oracle/_ref/cuda/ref_cuda_driver missing: run make -C oracle ref_cuda"
    rng = np.random.default_rng(5)
    M, N, KL = 70, 33, 5
    A, B = _finite_limb_operands(rng, M, N, KL)
    C0 = rng.normal(size=(M, N)).astype(np.float32)
    alpha, beta = 1.25, 0.5
    out = _run_driver("limb", struct.pack("<iiiff", M, N, KL, alpha, beta) + A.tobytes() + B.tobytes() + C0.tobytes(), tmp_path)
    got = np.frombuffer(out, np.float32).reshape(5, M, N)
    want = oracle.gemm_limb(A, B, C0, M, N, KL * 48, alpha, beta)
    names = ["span API (Backend::Auto)", "dispatch(Backend::CUDA)", "dispatch(Backend::CPU)", "TensorMetadata host",
             "TensorMetadata device"]
    for g, name in zip(got, names):
        np.testing.assert_allclose(g, want, rtol=1e-6, err_msg=name)  # fp64 accumulation on both sides
    # the device runs agree with one another bit for bit (same kernel), and are not the CPU run relabelled
    assert np.array_equal(got[0], got[1]) and np.array_equal(got[0], got[3]) and np.array_equal(got[0], got[4])


@pytest.mark.gpu
def test_cpp_gemm_ternary_trit_mode_overloads(lib_built, tmp_path):
    assert os.path.exists(DRIVER)
    rng = np.random.default_rng(6)
    M, N, KL = 130, 50, 7
    trits = rng.integers(-1, 2, (M, KL * 48)).astype(np.int8)
    A = oracle.pack_trits_rowwise(trits)
    B = rng.normal(size=(KL * 48, N)).astype(np.float32)
    C0 = rng.normal(size=(M, N)).astype(np.float32)
    out = _run_driver("trit", struct.pack("<iiiff", M, N, KL, 1.5, -0.5) + A.tobytes() + B.tobytes() + C0.tobytes(), tmp_path)
    got = np.frombuffer(out, np.float32).reshape(3, M, N)
    want = oracle.gemm_trit(A, B, C0, M, N, KL * 48, 1.5, -0.5)
    scale = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    for g in got:
        assert np.max(np.abs(g - want)) / scale < 1e-3   # fp32 operands: 1e-3 (achieved ~1e-5)
        assert np.max(np.abs(g - want)) / scale < 5e-5


@pytest.mark.gpu
def test_cpp_elementwise_helpers_host_and_device(lib_built, tmp_path):
    assert os.path.exists(DRIVER)
    rng = np.random.default_rng(7)
    n = 100003  # not a multiple of 4: the vector body and the tail both run
    a = rng.normal(size=n).astype(np.float32)
    a[::5] = 0.0  # zeros for the where condition
    b = rng.normal(size=n).astype(np.float32)
    c = rng.normal(size=n).astype(np.float32)
    lo, hi, value = -0.25, 0.75, 1.7
    out = _run_driver("elementwise", struct.pack("<qfff", n, lo, hi, value) + a.tobytes() + b.tobytes() + c.tobytes(), tmp_path)
    got = np.frombuffer(out, np.float32).reshape(2, 4, n)
    want = [oracle.where(a, b, c), oracle.clamp(a, lo, hi), oracle.lerp(a, b, c), oracle.addcmul(a, b, c, value)]
    for where in range(2):
        for op in range(4):
            assert np.array_equal(got[where, op], want[op]), (where, op)  # one rounding per operator on both sides


@pytest.mark.gpu
def test_cpp_boundary_raises_the_reference_exceptions(lib_built, tmp_path):
    assert os.path.exists(DRIVER)
    lines = _run_driver("errors", b"", tmp_path).decode().splitlines()
    got = {line.split(" ", 1)[0]: line.split(" ", 1)[1] for line in lines}
    assert got["negative"] == "invalid_argument gemm_ternary dimensions must be non-negative"
    assert got["k_not_48"] == "invalid_argument gemm_ternary requires K divisible by 48"
    assert got["a_size"] == "invalid_argument A span size does not match (M, K / 48)"
    assert got["empty"] == "none"
    assert got["dense_b_size"] == "invalid_argument B span size does not match (K, N)"
    assert got["clamp_dtype"] == "invalid_argument CUDA kernels only support float32"
    assert got["where_length"].startswith("invalid_argument")


def _run_module_worker(mode):
    """The module is exercised in a child process: an interpreter can hold only one build of the
    reference's ``t81lib`` extension, and other tests load the CPU build."""
    worker = os.path.join(ROOT, "tests", "_ref_cuda_module_worker.py")
    res = subprocess.run([sys.executable, worker, mode], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "worker ok" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
def test_reference_pybind_module_runs_on_the_gpu_through_the_shim(lib_built):
    """The reference's own python/bindings.cpp, built against the shim: its known-answer test
    (tests/python/test_bindings.py:17-39 of the reference), random operands against the oracle, torch
    CUDA tensors used in place, and the four elementwise bindings."""
    assert os.path.exists(DRIVER)
    _run_module_worker("gpu")
