"""t81b200_gemm_trit_static — the entry point for callers that cannot allocate device
memory (hosts with a frozen memory pool, code inside a stream capture, thin language
bindings): its scratch is a fixed buffer inside the library instead of a workspace the
caller passes.  Through the C ABI, its output must equal that of t81b200_gemm_trit given
a caller-allocated workspace, on two calls in a row that reuse the built-in buffer with
different data, and a call too large for the buffer must be refused without running.

Collected last on purpose (file name): a run that stops at the first failure has then
already executed every other test."""

import ctypes

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


def _run_both(dev, rng, out_f, in_f, tokens, dtype, layout):
    """One problem through both entry points; returns (static result, workspace result, oracle)."""
    from t81lib_b200 import _capi
    lib = _capi.lib
    w = rng.normal(0, 0.02, (out_f, in_f)).astype(np.float32)
    packed_np, scale_np = oracle.pack_dense_matrix_absmean(w, 0.45)
    bias_np = rng.normal(0, 0.01, out_f).astype(np.float32)
    x_np = rng.normal(size=(tokens, in_f)).astype(np.float32)
    packed = torch.from_numpy(packed_np).to(dev)
    scale = torch.from_numpy(scale_np).to(dev)
    bias = torch.from_numpy(bias_np).to(dev)
    x = torch.from_numpy(x_np).to(dev).to(dtype)
    want = oracle.linear_forward(packed_np, scale_np, bias_np, x.float().cpu().numpy(), in_f)
    code = {torch.float32: _capi.F32, torch.float16: _capi.F16, torch.bfloat16: _capi.BF16}[dtype]
    if layout == "nk":
        b, lay, ldb, shape, ldc = x, _capi.LAYOUT_NK, in_f, (tokens, out_f), out_f
    else:
        b, lay, ldb, shape, ldc = x.t().contiguous(), _capi.LAYOUT_KN, tokens, (out_f, tokens), tokens
        want = want.T
    stream = torch.cuda.current_stream(dev).cuda_stream
    need = lib.t81b200_gemm_trit_workspace_bytes(code, lay, _capi.F32, out_f, tokens, in_f)
    assert 0 < need <= _capi.STATIC_SCRATCH_BYTES  # the case must exercise the scratch path
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    c_ws = torch.zeros(shape, dtype=torch.float32, device=dev)
    c_static = torch.zeros(shape, dtype=torch.float32, device=dev)
    rc = lib.t81b200_gemm_trit(packed.data_ptr(), scale.data_ptr(), b.data_ptr(), code, lay, ldb, bias.data_ptr(),
                               c_ws.data_ptr(), _capi.F32, ldc, out_f, tokens, in_f, 1.0, 0.0, ws.data_ptr(), need, stream)
    assert rc == 0, _capi.last_error()
    # Free device memory as the driver reports it (cudaMemGetInfo): unlike torch's own counters it
    # would move if the library called cudaMalloc.  The first static call may load kernels into the
    # context, so the comparison brackets a repeat of the same call.
    def static_call():
        code_ = lib.t81b200_gemm_trit_static(packed.data_ptr(), scale.data_ptr(), b.data_ptr(), code, lay, ldb,
                                             bias.data_ptr(), c_static.data_ptr(), _capi.F32, ldc, out_f, tokens, in_f,
                                             1.0, 0.0, stream)
        assert code_ == 0, _capi.last_error()
        torch.cuda.synchronize(dev)
    static_call()
    free_before, _ = torch.cuda.mem_get_info(dev)
    static_call()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before
    assert _capi.kernel_status(reset=True) == 0
    return c_static.cpu().numpy(), c_ws.cpu().numpy(), want


def _rel_err(got, want):
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want)) / (np.sqrt(np.mean(want ** 2)) + 1e-30))


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row(dev):
    rng = np.random.default_rng(2024)
    # first call: fp32 activations, token-major; second call reuses the built-in buffer with other
    # data, another shape and the (K, N) argument order
    for out_f, in_f, tokens, dtype, layout in ((384, 1000, 200, torch.float32, "nk"),
                                               (512, 2048, 300, torch.float16, "kn")):
        got, ref, want = _run_both(dev, rng, out_f, in_f, tokens, dtype, layout)
        assert np.array_equal(got, ref)          # same kernels, same order of operations
        assert _rel_err(got, want) < 5e-5        # and both agree with the CPU oracle (fp32 tolerance 1e-3)


def test_static_scratch_entry_rejects_sizes_beyond_its_buffer(dev):
    from t81lib_b200 import _capi
    lib = _capi.lib
    out_f, in_f, tokens = 256, 8192, 4096  # 2 planes x 4096 x 8192 x 2 bytes = 128 MiB of scratch
    need = lib.t81b200_gemm_trit_workspace_bytes(_capi.F32, _capi.LAYOUT_NK, _capi.F32, out_f, tokens, in_f)
    assert need > _capi.STATIC_SCRATCH_BYTES
    c = torch.full((8,), 7.0, device=dev)
    # pointers are never dereferenced: the size check comes first
    rc = lib.t81b200_gemm_trit_static(c.data_ptr(), None, c.data_ptr(), _capi.F32, _capi.LAYOUT_NK, in_f, None,
                                      c.data_ptr(), _capi.F32, out_f, out_f, tokens, in_f, 1.0, 0.0, None)
    assert rc == _capi.ELIMIT
    assert "built-in buffer" in _capi.last_error()
    torch.cuda.synchronize(dev)
    assert bool((c == 7.0).all())
