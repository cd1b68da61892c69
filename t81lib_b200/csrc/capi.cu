// C ABI glue: error state, device probing and the TRIT-mode dispatcher.
#include "common.cuh"

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
                     float alpha, float beta, cudaStream_t st, PeerCtx *ctx);
int gemm_trit_simt_launch(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                          int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                          int64_t N, int64_t K, float alpha, float beta, cudaStream_t st);
bool gemm_trit_tc_eligible(int b_dtype, int layout, int c_dtype, int64_t M, int64_t N, int64_t K);
size_t gemm_trit_tc_workspace(int b_dtype, int layout, int c_dtype, int64_t M, int64_t N, int64_t K);
int gemm_trit_tc_launch(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                        int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M, int64_t N,
                        int64_t K, float alpha, float beta, void *workspace, size_t workspace_bytes,
                        cudaStream_t st, int n_peers, void *const *peer_C);

int gemm_trit_tc_status(int reset);
int gemv_trit_status(int reset);
int gemv_trit_lut_status(int reset);
int quantize_pack_status(int reset);
int gemv_trit_lut_launch(int fmt, int n_seg, const uint8_t *const *A, const float *const *row_scale, const float *const *bias,
                         void *const *C, const int64_t *M, const void *X, int x_dtype, int64_t ldx, int c_dtype,
                         int64_t ldc, int ntok, int64_t K, float alpha, float beta, cudaStream_t st, const PeerCtx *ctx);

}  // namespace t81b200

using namespace t81b200;

extern "C" int t81b200_kernel_status(int reset) {
    if (int rc = check_device()) return rc;
    const int tc = gemm_trit_tc_status(reset);
    const int gv = gemv_trit_status(reset);
    const int lut = gemv_trit_lut_status(reset);
    const int qp = quantize_pack_status(reset);
    return tc != 0 ? tc : (gv != 0 ? gv : (lut != 0 ? lut : qp));
}

extern "C" int t81b200_copy_columns(void *dst, int64_t dst_pitch, const void *src, int64_t src_pitch,
                                    int64_t width_bytes, int64_t rows, void *stream) {
    if (int rc = check_device()) return rc;
    if (width_bytes < 0 || rows < 0 || dst_pitch < width_bytes || src_pitch < width_bytes)
        return fail(T81B200_EINVAL, "copy_columns: pitches (%lld, %lld) must cover the row width %lld",
                    (long long)dst_pitch, (long long)src_pitch, (long long)width_bytes);
    if (width_bytes == 0 || rows == 0) return T81B200_OK;
    if (!dst || !src) return fail(T81B200_EINVAL, "copy_columns: null pointer");
    T81_CUDA_TRY(cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width_bytes, (size_t)rows,
                                   cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return T81B200_OK;
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

static int gemm_trit_local(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                           int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                           int64_t N, int64_t K, float alpha, float beta, void *workspace,
                           size_t workspace_bytes, void *stream, PeerCtx *ctx);

extern "C" int t81b200_gemm_trit(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                                 int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                                 int64_t N, int64_t K, float alpha, float beta, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    return gemm_trit_local(A, row_scale, B, b_dtype, layout, ldb, bias, C, c_dtype, ldc, M, N, K, alpha, beta, workspace,
                           workspace_bytes, stream, nullptr);
}

// The peers' results and flag slots of a sharded call: present, device memory, reachable from the current GPU.
static int check_peers(int n_peers, void *const *peer_C, uint32_t *sync_local, uint32_t *const *sync_slots) {
    if (n_peers < 0 || n_peers > T81B200_MAX_PEERS)
        return fail(T81B200_ELIMIT, "gemm_trit_peers: %d peers, at most %d are supported", n_peers, T81B200_MAX_PEERS);
    if (int rc = check_device()) return rc;
    int cur = 0;
    T81_CUDA_TRY(cudaGetDevice(&cur));
    for (int i = 0; i < n_peers; ++i) {
        if (!peer_C || !peer_C[i]) return fail(T81B200_EINVAL, "gemm_trit_peers: null peer pointer");
        if (sync_local && (!sync_slots || !sync_slots[i])) return fail(T81B200_EINVAL, "gemm_trit_peers: null flag slot");
        // the kernels store to these addresses: they must be device memory this GPU can reach
        cudaPointerAttributes attr;
        T81_CUDA_TRY(cudaPointerGetAttributes(&attr, peer_C[i]));
        if (attr.type != cudaMemoryTypeDevice)
            return fail(T81B200_EINVAL, "gemm_trit_peers: peer result %d is not device memory", i);
        if (attr.device != cur) {
            int can = 0;
            T81_CUDA_TRY(cudaDeviceCanAccessPeer(&can, cur, attr.device));
            if (!can) return fail(T81B200_EINVAL, "gemm_trit_peers: GPU %d cannot reach GPU %d", cur, attr.device);
            const cudaError_t e = cudaDeviceEnablePeerAccess(attr.device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
            else if (e != cudaSuccess) return fail(T81B200_ECUDA, "gemm_trit_peers: enabling peer access to GPU %d: %s", attr.device, cudaGetErrorString(e));
        }
    }
    return T81B200_OK;
}

extern "C" int t81b200_gemm_trit_peers(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                                       int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                                       int64_t N, int64_t K, float alpha, float beta, void *workspace,
                                       size_t workspace_bytes, int n_peers, void *const *peer_C, uint32_t *sync_local,
                                       uint32_t *const *sync_slots, void *stream) {
    if (int rc = check_peers(n_peers, peer_C, sync_local, sync_slots)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PeerCtx ctx;
    ctx.n_peers = n_peers; ctx.peer_C = peer_C; ctx.sync_local = sync_local; ctx.sync_slots = sync_slots;
    if (M == 0 || N == 0) return T81B200_OK;
    if (int rc = gemm_trit_local(A, row_scale, B, b_dtype, layout, ldb, bias, C, c_dtype, ldc, M, N, K, alpha, beta,
                                 workspace, workspace_bytes, stream, &ctx))
        return rc;
    if (!ctx.peers_done && n_peers > 0) {
        // a kernel without peer stores produced C: push the block with the copy engines instead
        const int64_t esz = (int64_t)dtype_size(c_dtype);
        const int64_t rows = layout == T81B200_LAYOUT_NK ? N : M, width = (layout == T81B200_LAYOUT_NK ? M : N) * esz;
        for (int i = 0; i < n_peers; ++i)
            if (int rc = t81b200_copy_columns(peer_C[i], ldc * esz, C, ldc * esz, width, rows, stream)) return rc;
    }
    if (sync_local && !ctx.sync_fused) return exchange_signal_launch(sync_local, sync_slots, n_peers, st);
    return T81B200_OK;
}

namespace t81b200 { extern thread_local int g_hint_independent; }

extern "C" void t81b200_hint_independent(int on) { t81b200::g_hint_independent = on ? 1 : 0; }

extern "C" int t81b200_exchange_signal(uint32_t *sync_local, uint32_t *const *sync_slots, int n_peers, void *stream) {
    if (int rc = check_device()) return rc;
    if (!sync_local || !sync_slots || n_peers < 0 || n_peers > T81B200_MAX_PEERS) return fail(T81B200_EINVAL, "exchange_signal: bad arguments");
    for (int i = 0; i < n_peers; ++i)
        if (!sync_slots[i]) return fail(T81B200_EINVAL, "exchange_signal: null flag slot");
    return exchange_signal_launch(sync_local, sync_slots, n_peers, static_cast<cudaStream_t>(stream));
}

extern "C" int t81b200_exchange_wait(uint32_t *sync_local, int n_peers, void *stream) {
    if (int rc = check_device()) return rc;
    if (!sync_local || n_peers < 0 || n_peers > T81B200_MAX_PEERS) return fail(T81B200_EINVAL, "exchange_wait: bad arguments");
    return exchange_wait_launch(sync_local, n_peers, static_cast<cudaStream_t>(stream));
}

// 17 .. T81B200_T2_MAX_ROWS rows of B: slices of the streaming kernel, or tensor-core tiles?  Estimates fitted to
// measurements on the Llama- and Phi-shaped layers: a slice of 16 rows on the decode-stream layout costs about
// 1.5 us plus its weight bytes at 1.35 TB/s (overlapping slices included), 1.4 times that on the limbs; the
// tensor-core kernel runs its 128 x 256 tiles in waves of one per SM at about 8.5 ns per contraction step, whatever
// part of a tile the rows of B fill.
static bool streaming_wins(int64_t M, int64_t N, int64_t K, double layout_factor) {
    if (N <= 16) return true;
    if (N > T81B200_T2_MAX_ROWS || M <= 0 || K <= 0) return false;
    const double slices = (double)((N + 15) / 16);
    const double stream_us = layout_factor * slices * (1.5 + (double)M * (double)K * 0.25 / 1.35e6);
    const int64_t tiles = ((M + 127) / 128) * ((N + 255) / 256);
    const double waves = (double)((tiles + sm_count() - 1) / sm_count());
    return stream_us < 5.0 + waves * (double)K * 8.5e-3;
}

extern "C" int t81b200_prefers_streaming(int64_t M, int64_t N, int64_t K) { return streaming_wins(M, N, K, 1.0) ? 1 : 0; }

static int gemm_trit_local(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                           int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                           int64_t N, int64_t K, float alpha, float beta, void *workspace,
                           size_t workspace_bytes, void *stream, PeerCtx *ctx) {
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

    if (a_aligned && layout == T81B200_LAYOUT_NK && N <= 16 && K > 0)
        return gemv_trit_launch(A, row_scale, B, b_dtype, ldb, bias, C, c_dtype, ldc, M, (int)N, K, alpha, beta, st, ctx);
    // 17 to 128 rows of B: one launch of the streaming kernel per 16 rows often beats tensor-core tiles that would be
    // mostly empty (4096 x 4096 x 32: 10 us instead of 42); streaming_wins decides.  A later slice reads and writes nothing an earlier one
    // touches and is released by it only once its own input is complete: the slices are flagged independent and
    // overlap.  Not with peers: the exchange protocol counts calls, not slices.
    if (a_aligned && layout == T81B200_LAYOUT_NK && K > 0 && !ctx && streaming_wins(M, N, K, 1.4)) {
        const int64_t esz_b = (int64_t)dtype_size(b_dtype), esz_c = (int64_t)dtype_size(c_dtype);
        const int hint = t81b200::g_hint_independent;
        int rc = T81B200_OK;
        for (int64_t n0 = 0; n0 < N && rc == T81B200_OK; n0 += 16) {
            if (n0 > 0) t81b200::g_hint_independent = 1;
            rc = gemv_trit_launch(A, row_scale, static_cast<const char *>(B) + n0 * ldb * esz_b, b_dtype, ldb, bias,
                                  static_cast<char *>(C) + n0 * ldc * esz_c, c_dtype, ldc, M, (int)(N - n0 < 16 ? N - n0 : 16), K, alpha,
                                  beta, st, nullptr);
        }
        t81b200::g_hint_independent = hint;
        return rc;
    }

    // the other kernels do not carry the exchange protocol: wait for the peers' stores before they read
    if (ctx && ctx->sync_local && !ctx->waited) {
        if (int rc = exchange_wait_launch(ctx->sync_local, ctx->n_peers, st)) return rc;
        ctx->waited = true;
    }

    if (a_aligned && gemm_trit_tc_eligible(b_dtype, layout, c_dtype, M, N, K)) {
        const size_t need = gemm_trit_tc_workspace(b_dtype, layout, c_dtype, M, N, K);
        if (need > 0 && (!workspace || workspace_bytes < need))
            return fail(T81B200_EWORKSPACE, "gemm_trit: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        const int rc = gemm_trit_tc_launch(A, row_scale, B, b_dtype, layout, ldb, bias, C, c_dtype, ldc, M, N, K,
                                           alpha, beta, workspace, workspace_bytes, st, ctx ? ctx->n_peers : 0,
                                           ctx ? ctx->peer_C : nullptr);
        if (rc != T81B200_EALIGN) {  // unaligned activations: the general kernel takes them
            if (ctx) ctx->peers_done = rc == T81B200_OK;
            return rc;
        }
    }
    return gemm_trit_simt_launch(A, row_scale, B, b_dtype, layout, ldb, bias, C, c_dtype, ldc, M, N, K, alpha, beta, st);
}

extern "C" int t81b200_gemm_trit_t2(int n_group, const uint8_t *const *t2, const float *const *row_scale,
                                    const float *const *bias, void *const *C, const int64_t *M, const void *B, int b_dtype,
                                    int64_t ldb, int c_dtype, int64_t ldc, int64_t N, int64_t K, float alpha, float beta,
                                    void *stream) {
    if (n_group < 1 || n_group > T81B200_MAX_GROUP)
        return fail(T81B200_ELIMIT, "gemm_trit_t2: %d matrices, between 1 and %d are supported", n_group, T81B200_MAX_GROUP);
    if (!t2 || !C || !M) return fail(T81B200_EINVAL, "gemm_trit_t2: null pointer");
    if (N < 0 || K < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (N > T81B200_T2_MAX_ROWS)
        return fail(T81B200_ELIMIT, "gemm_trit_t2: %lld rows of B; the decode-stream layout serves 1 to %d", (long long)N, T81B200_T2_MAX_ROWS);
    if (!valid_dtype(b_dtype) || !valid_dtype(c_dtype)) return fail(T81B200_EINVAL, "gemm_trit: unknown dtype");
    if (ldb < K) return fail(T81B200_EINVAL, "gemm_trit: ldb (%lld) below the row length (%lld)", (long long)ldb, (long long)K);
    for (int i = 0; i < n_group; ++i) {
        if (M[i] <= 0 || K <= 0) return fail(T81B200_EINVAL, "gemm_trit_t2: dimensions must be positive");
        if (ldc < M[i]) return fail(T81B200_EINVAL, "gemm_trit: ldc (%lld) below the row length (%lld)", (long long)ldc, (long long)M[i]);
        if (N > 0 && (!C[i] || !t2[i] || !B)) return fail(T81B200_EINVAL, "gemm_trit: null pointer");
        if (reinterpret_cast<uintptr_t>(t2[i]) % 16 != 0) return fail(T81B200_EALIGN, "gemm_trit_t2: matrices must be 16-byte aligned");
    }
    if (int rc = check_device()) return rc;
    if (N == 0) return T81B200_OK;
    // The kernel takes 16 rows of B at a time; more rows run as one launch per 16.  A later slice reads and writes
    // nothing an earlier one touches, and an earlier slice releases it only once its own input is complete, so the
    // slices are flagged independent of their predecessor and overlap.
    const int64_t esz_b = (int64_t)dtype_size(b_dtype), esz_c = (int64_t)dtype_size(c_dtype);
    const int hint = t81b200::g_hint_independent;
    int rc = T81B200_OK;
    for (int64_t n0 = 0; n0 < N && rc == T81B200_OK; n0 += 16) {
        void *Cs[T81B200_MAX_GROUP];
        for (int i = 0; i < n_group; ++i) Cs[i] = static_cast<char *>(C[i]) + n0 * ldc * esz_c;
        if (n0 > 0) t81b200::g_hint_independent = 1;
        rc = gemv_trit_lut_launch(1, n_group, t2, row_scale, bias, Cs, M, static_cast<const char *>(B) + n0 * ldb * esz_b, b_dtype, ldb,
                                  c_dtype, ldc, (int)(N - n0 < 16 ? N - n0 : 16), K, alpha, beta, static_cast<cudaStream_t>(stream), nullptr);
    }
    t81b200::g_hint_independent = hint;
    if (rc == T81B200_EALIGN) return fail(T81B200_ELIMIT, "gemm_trit_t2: K = %lld does not fit the kernel's shared memory", (long long)K);
    return rc;
}

extern "C" int t81b200_gemm_trit_t2_peers(const uint8_t *t2, const float *row_scale, const float *bias, void *C, int64_t M,
                                          const void *B, int b_dtype, int64_t ldb, int c_dtype, int64_t ldc, int64_t N,
                                          int64_t K, float alpha, float beta, int n_peers, void *const *peer_C,
                                          uint32_t *sync_local, uint32_t *const *sync_slots, void *stream) {
    if (M <= 0 || K <= 0 || N < 0) return fail(T81B200_EINVAL, "gemm_trit_t2_peers: dimensions must be positive");
    if (N > 16) return fail(T81B200_ELIMIT, "gemm_trit_t2_peers: %lld rows of B; the decode-stream layout serves 1 to 16", (long long)N);
    if (!valid_dtype(b_dtype) || !valid_dtype(c_dtype)) return fail(T81B200_EINVAL, "gemm_trit: unknown dtype");
    if (ldb < K || ldc < M) return fail(T81B200_EINVAL, "gemm_trit: leading dimension below the row length");
    if (N > 0 && (!t2 || !B || !C)) return fail(T81B200_EINVAL, "gemm_trit: null pointer");
    if (reinterpret_cast<uintptr_t>(t2) % 16 != 0) return fail(T81B200_EALIGN, "gemm_trit_t2: matrices must be 16-byte aligned");
    if (int rc = check_peers(n_peers, peer_C, sync_local, sync_slots)) return rc;
    if (N == 0) return T81B200_OK;
    PeerCtx ctx;
    ctx.n_peers = n_peers; ctx.peer_C = peer_C; ctx.sync_local = sync_local; ctx.sync_slots = sync_slots;
    const int rc = gemv_trit_lut_launch(1, 1, &t2, &row_scale, &bias, &C, &M, B, b_dtype, ldb, c_dtype, ldc, (int)N, K, alpha, beta,
                                        static_cast<cudaStream_t>(stream), &ctx);
    if (rc == T81B200_EALIGN) return fail(T81B200_ELIMIT, "gemm_trit_t2: K = %lld does not fit the kernel's shared memory", (long long)K);
    return rc;
}

extern "C" int t81b200_gemm_trit_grouped(int n_group, const uint8_t *const *A, const float *const *row_scale,
                                         const float *const *bias, void *const *C, const int64_t *M, const void *B,
                                         int b_dtype, int64_t ldb, int c_dtype, int64_t ldc, int64_t N, int64_t K,
                                         float alpha, float beta, void *stream) {
    if (n_group < 1 || n_group > T81B200_MAX_GROUP)
        return fail(T81B200_ELIMIT, "gemm_trit_grouped: %d matrices, between 1 and %d are supported", n_group, T81B200_MAX_GROUP);
    if (!A || !C || !M) return fail(T81B200_EINVAL, "gemm_trit_grouped: null pointer");
    if (N < 0 || K < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (!valid_dtype(b_dtype) || !valid_dtype(c_dtype)) return fail(T81B200_EINVAL, "gemm_trit: unknown dtype");
    if (ldb < K) return fail(T81B200_EINVAL, "gemm_trit: ldb (%lld) below the row length (%lld)", (long long)ldb, (long long)K);
    bool streaming = N >= 1 && N <= 16 && K > 0;
    for (int i = 0; i < n_group; ++i) {
        if (M[i] < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
        if (ldc < M[i]) return fail(T81B200_EINVAL, "gemm_trit: ldc (%lld) below the row length (%lld)", (long long)ldc, (long long)M[i]);
        if (M[i] > 0 && N > 0 && (!C[i] || (K > 0 && (!A[i] || !B)))) return fail(T81B200_EINVAL, "gemm_trit: null pointer");
        streaming = streaming && M[i] > 0 && reinterpret_cast<uintptr_t>(A[i]) % 16 == 0;
    }
    if (int rc = check_device()) return rc;
    if (N == 0) return T81B200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (streaming) {
        const int rc = gemv_trit_lut_launch(0, n_group, A, row_scale, bias, C, M, B, b_dtype, ldb, c_dtype, ldc, (int)N, K, alpha,
                                            beta, st, nullptr);
        if (rc != T81B200_EALIGN) return rc;
    }
    // anything else: one call per matrix
    for (int i = 0; i < n_group; ++i)
        if (int rc = gemm_trit_local(A[i], row_scale ? row_scale[i] : nullptr, B, b_dtype, T81B200_LAYOUT_NK, ldb,
                                     bias ? bias[i] : nullptr, C[i], c_dtype, ldc, M[i], N, K, alpha, beta, nullptr, 0, stream,
                                     nullptr))
            return rc;
    return T81B200_OK;
}
