// C ABI glue: error state, device probing and the TRIT-mode dispatcher.
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace t81b200 {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

int check_device() {
    static int cached = 1;  // 1 = unknown, 0 = ok, <0 = error
    static char why[256] = "";
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (cached == 1) {
        int count = 0;
        cudaError_t err = cudaGetDeviceCount(&count);
        if (err != cudaSuccess || count == 0) {
            snprintf(why, sizeof why, "no usable CUDA device (%s); there is no CPU fallback",
                     err != cudaSuccess ? cudaGetErrorString(err) : "device count is 0");
            (void)cudaGetLastError();
            cached = T81B200_ENODEVICE;
        } else {
            int dev = 0, major = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if (major != 10) {
                snprintf(why, sizeof why, "device %d has compute capability %d.x; this library is built for sm_100a only",
                         dev, major);
                cached = T81B200_ENODEVICE;
            } else {
                cached = 0;
            }
        }
    }
    if (cached != 0) set_error("%s", why);
    return cached;
}

int sm_count() {
    static int counts[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (counts[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        counts[dev] = n;
    }
    return counts[dev];
}

int gemv_trit_launch(const uint8_t *A, const float *row_scale, const void *X, int x_dtype, int64_t ldx,
                     const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M, int ntok, int64_t K,
                     float alpha, float beta, cudaStream_t st);
int gemm_trit_simt_launch(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                          int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                          int64_t N, int64_t K, float alpha, float beta, cudaStream_t st);
bool gemm_trit_tc_eligible(int b_dtype, int layout, int c_dtype, int64_t M, int64_t N, int64_t K);
size_t gemm_trit_tc_workspace(int b_dtype, int layout, int c_dtype, int64_t M, int64_t N, int64_t K);
int gemm_trit_tc_launch(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                        int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M, int64_t N,
                        int64_t K, float alpha, float beta, void *workspace, size_t workspace_bytes,
                        cudaStream_t st);

int gemm_trit_tc_status(int reset);
int gemv_trit_status(int reset);

}  // namespace t81b200

using namespace t81b200;

extern "C" int t81b200_kernel_status(int reset) {
    if (int rc = check_device()) return rc;
    const int tc = gemm_trit_tc_status(reset);
    const int gv = gemv_trit_status(reset);
    return tc != 0 ? tc : gv;
}

extern "C" const char *t81b200_last_error(void) { return g_error; }

extern "C" const char *t81b200_version(void) { return "t81_b200 0.1 (sm_100a)"; }

extern "C" int t81b200_device_available(void) { return check_device() == 0 ? 1 : 0; }

static bool valid_dtype(int d) { return d == T81B200_F32 || d == T81B200_BF16 || d == T81B200_F16; }

extern "C" size_t t81b200_gemm_trit_workspace_bytes(int b_dtype, int layout, int c_dtype, int64_t M, int64_t N,
                                                    int64_t K) {
    if (M <= 0 || N <= 0 || K < 0) return 0;
    if (!gemm_trit_tc_eligible(b_dtype, layout, c_dtype, M, N, K)) return 0;
    return gemm_trit_tc_workspace(b_dtype, layout, c_dtype, M, N, K);
}

extern "C" int t81b200_gemm_trit(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                                 int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                                 int64_t N, int64_t K, float alpha, float beta, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    if (M < 0 || N < 0 || K < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (!valid_dtype(b_dtype) || !valid_dtype(c_dtype)) return fail(T81B200_EINVAL, "gemm_trit: unknown dtype");
    if (layout != T81B200_LAYOUT_KN && layout != T81B200_LAYOUT_NK)
        return fail(T81B200_EINVAL, "gemm_trit: unknown layout %d", layout);
    const int64_t min_ldb = layout == T81B200_LAYOUT_KN ? N : K;
    const int64_t min_ldc = layout == T81B200_LAYOUT_KN ? N : M;
    if (ldb < min_ldb) return fail(T81B200_EINVAL, "gemm_trit: ldb (%lld) below the row length (%lld)", (long long)ldb, (long long)min_ldb);
    if (ldc < min_ldc) return fail(T81B200_EINVAL, "gemm_trit: ldc (%lld) below the row length (%lld)", (long long)ldc, (long long)min_ldc);
    if (int rc = check_device()) return rc;
    if (M == 0 || N == 0) return T81B200_OK;
    if (!C || (K > 0 && (!A || !B))) return fail(T81B200_EINVAL, "gemm_trit: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool a_aligned = reinterpret_cast<uintptr_t>(A) % 16 == 0;

    // T81B200_SMALLN_PATH=tc sends token counts <= 16 to the tensor-core kernel too (A/B runs).
    const char *small_n = getenv("T81B200_SMALLN_PATH");
    const bool small_n_tc = small_n && small_n[0] == 't' && b_dtype == T81B200_BF16;
    if (a_aligned && layout == T81B200_LAYOUT_NK && N <= 16 && K > 0 && !small_n_tc)
        return gemv_trit_launch(A, row_scale, B, b_dtype, ldb, bias, C, c_dtype, ldc, M, (int)N, K, alpha, beta, st);

    if (a_aligned && gemm_trit_tc_eligible(b_dtype, layout, c_dtype, M, N, K)) {
        const size_t need = gemm_trit_tc_workspace(b_dtype, layout, c_dtype, M, N, K);
        if (need > 0 && (!workspace || workspace_bytes < need))
            return fail(T81B200_EWORKSPACE, "gemm_trit: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        const int rc = gemm_trit_tc_launch(A, row_scale, B, b_dtype, layout, ldb, bias, C, c_dtype, ldc, M, N, K,
                                           alpha, beta, workspace, workspace_bytes, st);
        if (rc != T81B200_EALIGN) return rc;  // unaligned activations: the general kernel takes them
    }
    return gemm_trit_simt_launch(A, row_scale, B, b_dtype, layout, ldb, bias, C, c_dtype, ldc, M, N, K, alpha, beta, st);
}
