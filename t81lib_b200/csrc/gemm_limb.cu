// LIMB mode: the literal semantics of t81::linalg::gemm_ternary — every 16-byte
// limb is one scalar, the 48-trit balanced integer it encodes, and the GEMM runs
// over those scalars in fp64.
//
// A 16x16 output tile per CTA.  For each limb index k the CTA decodes 16 limbs of
// A and 16 of B to doubles once (32 threads, one limb each), so a decode is
// shared by 16 outputs instead of being redone per output element.
#include "common.cuh"

#include <mutex>

namespace t81b200 {

namespace {

constexpr int kTile = 16;
constexpr int kChunk = 8;  // limb indices decoded per barrier

// value = sum_pos (byte[pos] - 13) * 27^pos, summed in ascending position like
// limb_to_double (include/t81/linalg/gemm.hpp:48-57).
__device__ __forceinline__ double limb_value(const uint8_t *p) {
    double weight = 1.0, v = 0.0;
#pragma unroll
    for (int pos = 0; pos < 16; ++pos) {
        uint32_t b = p[pos];
        b = b > 26u ? 13u : b;
        v += (double)((int)b - 13) * weight;
        weight *= 27.0;
    }
    return v;
}

__global__ void __launch_bounds__(kTile *kTile)
gemm_limb_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, float *__restrict__ C,
                 int64_t M, int64_t N, int64_t KL, float alpha, float beta) {
    __shared__ double a_s[kChunk][kTile];
    __shared__ double b_s[kChunk][kTile];
    const int tx = threadIdx.x % kTile, ty = threadIdx.x / kTile;
    const int64_t i0 = (int64_t)blockIdx.y * kTile, j0 = (int64_t)blockIdx.x * kTile;
    const int64_t i = i0 + ty, j = j0 + tx;
    const bool live = i < M && j < N;
    double acc = live ? (double)C[i * N + j] * (double)beta : 0.0;
    const double a64 = (double)alpha;

    for (int64_t kb = 0; kb < KL; kb += kChunk) {
        // 2 * kChunk * kTile = 256 decodes, one per thread
        {
            const int t = threadIdx.x;
            const int which = t / (kChunk * kTile);      // 0: A, 1: B
            const int kk = (t % (kChunk * kTile)) / kTile;
            const int e = t % kTile;
            const int64_t k = kb + kk;
            double v = 0.0;
            if (k < KL) {
                if (which == 0) {
                    if (i0 + e < M) v = limb_value(A + ((i0 + e) * KL + k) * 16);
                } else {
                    if (j0 + e < N) v = limb_value(B + (k * N + (j0 + e)) * 16);
                }
            }
            if (which == 0) a_s[kk][e] = v; else b_s[kk][e] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kChunk; ++kk) acc += a_s[kk][ty] * b_s[kk][tx] * a64;
        __syncthreads();
    }
    if (live) C[i * N + j] = (float)acc;
}

// Staging buffers of the entry points that take host pointers: one set per device, kept for
// the life of the process and grown on demand.
struct HostStaging {
    std::mutex mu;
    void *a = nullptr, *b = nullptr, *c = nullptr, *ws = nullptr;
    size_t a_cap = 0, b_cap = 0, c_cap = 0, ws_cap = 0;
};
constexpr int kMaxDevices = 64;
HostStaging g_staging[kMaxDevices];

int staging_for_current_device(HostStaging **out) {
    int dev = 0;
    T81_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(T81B200_ELIMIT, "device index %d not supported", dev);
    *out = &g_staging[dev];
    return T81B200_OK;
}

int grow(void **p, size_t *cap, size_t need) {
    if (need <= *cap) return T81B200_OK;
    if (*p) cudaFree(*p);
    *p = nullptr; *cap = 0;
    T81_CUDA_TRY(cudaMalloc(p, need));
    *cap = need;
    return T81B200_OK;
}

}  // namespace

// 1: memory a kernel of the current device can dereference (device or managed memory);
// 0: host memory (pageable or pinned).  Null pointers count as "either".
void release_elementwise_staging();  // elementwise.cu

int pointer_is_device(const void *p, int *is_device) {
    *is_device = 0;
    if (!p) return T81B200_OK;
    cudaPointerAttributes attr;
    const cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();  // older runtimes report plain host memory as an error
        return T81B200_OK;
    }
    *is_device = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    return T81B200_OK;
}

}  // namespace t81b200

using namespace t81b200;

extern "C" int t81b200_release_staging(void) {
    if (int rc = check_device()) return rc;
    int cur = 0, count = 0;
    T81_CUDA_TRY(cudaGetDevice(&cur));
    T81_CUDA_TRY(cudaGetDeviceCount(&count));
    for (int d = 0; d < count && d < kMaxDevices; ++d) {
        HostStaging &s = g_staging[d];
        std::lock_guard<std::mutex> lock(s.mu);
        if (!s.a && !s.b && !s.c && !s.ws) continue;
        T81_CUDA_TRY(cudaSetDevice(d));
        void **bufs[4] = {&s.a, &s.b, &s.c, &s.ws};
        for (void **b : bufs) { if (*b) cudaFree(*b); *b = nullptr; }
        s.a_cap = s.b_cap = s.c_cap = s.ws_cap = 0;
    }
    T81_CUDA_TRY(cudaSetDevice(cur));
    release_elementwise_staging();
    T81_CUDA_TRY(cudaSetDevice(cur));
    return T81B200_OK;
}

extern "C" int t81b200_gemm_limb(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                                 int64_t k_limbs, float alpha, float beta, void *stream) {
    if (M < 0 || N < 0 || k_limbs < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (int rc = check_device()) return rc;
    if (M == 0 || N == 0) return T81B200_OK;
    if (!C || (k_limbs > 0 && (!A || !B))) return fail(T81B200_EINVAL, "gemm_limb: null pointer");
    dim3 grid((unsigned)((N + kTile - 1) / kTile), (unsigned)((M + kTile - 1) / kTile));
    if ((M + kTile - 1) / kTile > 65535) return fail(T81B200_ELIMIT, "gemm_limb: M too large");
    gemm_limb_kernel<<<grid, kTile * kTile, 0, static_cast<cudaStream_t>(stream)>>>(A, B, C, M, N, k_limbs, alpha, beta);
    T81_LAUNCH_CHECK("gemm_limb_kernel");
    return T81B200_OK;
}

extern "C" int t81b200_gemm_limb_host(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                                      int64_t k_limbs, float alpha, float beta) {
    if (M < 0 || N < 0 || k_limbs < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (int rc = check_device()) return rc;
    if (M == 0 || N == 0) return T81B200_OK;
    if (!C || (k_limbs > 0 && (!A || !B))) return fail(T81B200_EINVAL, "gemm_limb_host: null pointer");
    HostStaging *stg = nullptr;
    if (int rc = staging_for_current_device(&stg)) return rc;
    std::lock_guard<std::mutex> lock(stg->mu);
    const size_t a_bytes = (size_t)M * k_limbs * 16, b_bytes = (size_t)k_limbs * N * 16, c_bytes = (size_t)M * N * 4;
    if (int rc = grow(&stg->a, &stg->a_cap, a_bytes ? a_bytes : 16)) return rc;
    if (int rc = grow(&stg->b, &stg->b_cap, b_bytes ? b_bytes : 16)) return rc;
    if (int rc = grow(&stg->c, &stg->c_cap, c_bytes)) return rc;
    if (a_bytes) T81_CUDA_TRY(cudaMemcpyAsync(stg->a, A, a_bytes, cudaMemcpyHostToDevice, 0));
    if (b_bytes) T81_CUDA_TRY(cudaMemcpyAsync(stg->b, B, b_bytes, cudaMemcpyHostToDevice, 0));
    T81_CUDA_TRY(cudaMemcpyAsync(stg->c, C, c_bytes, cudaMemcpyHostToDevice, 0));
    if (int rc = t81b200_gemm_limb((const uint8_t *)stg->a, (const uint8_t *)stg->b, (float *)stg->c,
                                   M, N, k_limbs, alpha, beta, nullptr))
        return rc;
    T81_CUDA_TRY(cudaMemcpyAsync(C, stg->c, c_bytes, cudaMemcpyDeviceToHost, 0));
    T81_CUDA_TRY(cudaStreamSynchronize(0));
    return T81B200_OK;
}

extern "C" int t81b200_gemm_limb_auto(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                                      int64_t k_limbs, float alpha, float beta) {
    if (M < 0 || N < 0 || k_limbs < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (int rc = check_device()) return rc;
    if (M == 0 || N == 0) return T81B200_OK;
    int da = 0, db = 0, dc = 0;
    pointer_is_device(A, &da); pointer_is_device(B, &db); pointer_is_device(C, &dc);
    if (k_limbs == 0) da = db = dc;
    if (da != dc || db != dc)
        return fail(T81B200_EINVAL, "gemm_ternary: A, B and C must all be host memory or all be device memory");
    if (!dc) return t81b200_gemm_limb_host(A, B, C, M, N, k_limbs, alpha, beta);
    // device-resident operands (TensorMetadata with device_type CUDA and requires_sync): run in place on
    // the legacy default stream and return when the result is complete
    if (int rc = t81b200_gemm_limb(A, B, C, M, N, k_limbs, alpha, beta, nullptr)) return rc;
    T81_CUDA_TRY(cudaStreamSynchronize(0));
    return T81B200_OK;
}

static int gemm_trit_host_impl(const uint8_t *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                               float alpha, float beta) {
    HostStaging *stg = nullptr;
    if (int rc = staging_for_current_device(&stg)) return rc;
    std::lock_guard<std::mutex> lock(stg->mu);
    const int64_t kl = (K + 47) / 48;
    const size_t a_bytes = (size_t)M * kl * 16, b_bytes = (size_t)K * N * 4, c_bytes = (size_t)M * N * 4;
    const size_t ws_bytes = t81b200_gemm_trit_workspace_bytes(T81B200_F32, T81B200_LAYOUT_KN, T81B200_F32, M, N, K);
    if (int rc = grow(&stg->a, &stg->a_cap, a_bytes ? a_bytes : 16)) return rc;
    if (int rc = grow(&stg->b, &stg->b_cap, b_bytes ? b_bytes : 16)) return rc;
    if (int rc = grow(&stg->c, &stg->c_cap, c_bytes)) return rc;
    if (ws_bytes) if (int rc = grow(&stg->ws, &stg->ws_cap, ws_bytes)) return rc;
    if (a_bytes) T81_CUDA_TRY(cudaMemcpyAsync(stg->a, A, a_bytes, cudaMemcpyHostToDevice, 0));
    if (b_bytes) T81_CUDA_TRY(cudaMemcpyAsync(stg->b, B, b_bytes, cudaMemcpyHostToDevice, 0));
    if (beta != 0.0f) T81_CUDA_TRY(cudaMemcpyAsync(stg->c, C, c_bytes, cudaMemcpyHostToDevice, 0));
    if (int rc = t81b200_gemm_trit((const uint8_t *)stg->a, nullptr, stg->b, T81B200_F32, T81B200_LAYOUT_KN, N,
                                   nullptr, stg->c, T81B200_F32, N, M, N, K, alpha, beta, stg->ws, stg->ws_cap, nullptr))
        return rc;
    T81_CUDA_TRY(cudaMemcpyAsync(C, stg->c, c_bytes, cudaMemcpyDeviceToHost, 0));
    T81_CUDA_TRY(cudaStreamSynchronize(0));
    return T81B200_OK;
}

extern "C" int t81b200_gemm_trit_host(const uint8_t *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                                      float alpha, float beta) {
    if (M < 0 || N < 0 || K < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (int rc = check_device()) return rc;
    if (M == 0 || N == 0) return T81B200_OK;
    if (!C || (K > 0 && (!A || !B))) return fail(T81B200_EINVAL, "gemm_trit_host: null pointer");
    return gemm_trit_host_impl(A, B, C, M, N, K, alpha, beta);
}

extern "C" int t81b200_gemm_trit_auto(const uint8_t *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                                      float alpha, float beta) {
    if (M < 0 || N < 0 || K < 0) return fail(T81B200_EINVAL, "gemm_ternary dimensions must be non-negative");
    if (int rc = check_device()) return rc;
    if (M == 0 || N == 0) return T81B200_OK;
    if (!C || (K > 0 && (!A || !B))) return fail(T81B200_EINVAL, "gemm_trit: null pointer");
    int da = 0, db = 0, dc = 0;
    pointer_is_device(A, &da); pointer_is_device(B, &db); pointer_is_device(C, &dc);
    if (K == 0) da = db = dc;
    if (da != dc || db != dc)
        return fail(T81B200_EINVAL, "gemm_ternary: A, B and C must all be host memory or all be device memory");
    if (!dc) return gemm_trit_host_impl(A, B, C, M, N, K, alpha, beta);
    HostStaging *stg = nullptr;
    if (int rc = staging_for_current_device(&stg)) return rc;
    std::lock_guard<std::mutex> lock(stg->mu);
    const size_t ws_bytes = t81b200_gemm_trit_workspace_bytes(T81B200_F32, T81B200_LAYOUT_KN, T81B200_F32, M, N, K);
    if (ws_bytes) if (int rc = grow(&stg->ws, &stg->ws_cap, ws_bytes)) return rc;
    if (int rc = t81b200_gemm_trit(A, nullptr, B, T81B200_F32, T81B200_LAYOUT_KN, N, nullptr, C, T81B200_F32, N, M, N, K,
                                   alpha, beta, stg->ws, stg->ws_cap, nullptr))
        return rc;
    T81_CUDA_TRY(cudaStreamSynchronize(0));
    return T81B200_OK;
}
