// The four elementwise helpers the reference's CUDA backend slot declares next to its GEMM
// (cuda_where / cuda_clamp / cuda_lerp / cuda_addcmul, include/t81/linalg/gemm_gpu.hpp:75-78,217-231;
// kernels at src/linalg/gemm_cuda.cu:165-283).  Plain fp32 streaming kernels: 128-bit loads and
// stores when every pointer allows it, a grid of a few CTAs per SM striding over the array.
// Each expression is evaluated as the reference's CPU code writes it (src/linalg/gemm_dispatch.cpp:147-222),
// one IEEE operation per source operator, nothing fused, so results are bit-identical to that code
// compiled without contraction.
#include "common.cuh"

#include <mutex>

namespace t81b200 {

namespace {

template <int OP>
__device__ __forceinline__ float ew_apply(float a, float b, float c, float s0, float s1) {
    if constexpr (OP == T81B200_EW_WHERE) return a != 0.0f ? b : c;                       // condition, x, y
    if constexpr (OP == T81B200_EW_CLAMP) return a < s0 ? s0 : (a > s1 ? s1 : a);         // input; min, max
    if constexpr (OP == T81B200_EW_LERP) return __fadd_rn(a, __fmul_rn(c, __fsub_rn(b, a)));  // start, end, weight
    return __fadd_rn(a, __fmul_rn(__fmul_rn(s0, b), c));                                  // input + value * t1 * t2
}

template <int OP, bool VEC>
__global__ void __launch_bounds__(256) elementwise_kernel(const float *a, const float *b,
                                                          const float *c, float *out,
                                                          size_t n, float s0, float s1) {
    constexpr bool kTwo = OP != T81B200_EW_CLAMP;  // clamp reads one array
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if constexpr (VEC) {
        const size_t n4 = n / 4;
        for (; i < n4; i += stride) {
            const float4 va = reinterpret_cast<const float4 *>(a)[i];
            float4 vb = va, vc = va;
            if constexpr (kTwo) { vb = reinterpret_cast<const float4 *>(b)[i]; vc = reinterpret_cast<const float4 *>(c)[i]; }
            float4 r;
            r.x = ew_apply<OP>(va.x, vb.x, vc.x, s0, s1);
            r.y = ew_apply<OP>(va.y, vb.y, vc.y, s0, s1);
            r.z = ew_apply<OP>(va.z, vb.z, vc.z, s0, s1);
            r.w = ew_apply<OP>(va.w, vb.w, vc.w, s0, s1);
            reinterpret_cast<float4 *>(out)[i] = r;
        }
        // the last n % 4 elements
        const size_t t = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (t < n) out[t] = ew_apply<OP>(a[t], kTwo ? b[t] : 0.0f, kTwo ? c[t] : 0.0f, s0, s1);
    } else {
        for (; i < n; i += stride) out[i] = ew_apply<OP>(a[i], kTwo ? b[i] : 0.0f, kTwo ? c[i] : 0.0f, s0, s1);
    }
}

template <int OP>
int launch_ew(const float *a, const float *b, const float *c, float *out, size_t n, float s0, float s1, cudaStream_t st) {
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out) |
                           (OP != T81B200_EW_CLAMP ? reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) : 0);
    const bool vec = bits % 16 == 0;
    const size_t items = vec ? (n + 3) / 4 : n;
    size_t blocks = (items + 255) / 256;
    const size_t cap = (size_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    if (vec) elementwise_kernel<OP, true><<<(unsigned)blocks, 256, 0, st>>>(a, b, c, out, n, s0, s1);
    else elementwise_kernel<OP, false><<<(unsigned)blocks, 256, 0, st>>>(a, b, c, out, n, s0, s1);
    T81_LAUNCH_CHECK("elementwise_kernel");
    return T81B200_OK;
}

struct EwStaging {
    std::mutex mu;
    void *buf[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t cap[4] = {0, 0, 0, 0};
};
EwStaging g_ew_staging[64];

}  // namespace
}  // namespace t81b200

using namespace t81b200;

extern "C" int t81b200_elementwise(int op, const float *a, const float *b, const float *c, float *out, int64_t n,
                                   float s0, float s1, void *stream) {
    if (n < 0) return fail(T81B200_EINVAL, "elementwise: negative length");
    if (op < T81B200_EW_WHERE || op > T81B200_EW_ADDCMUL) return fail(T81B200_EINVAL, "elementwise: unknown operation %d", op);
    if (int rc = check_device()) return rc;
    if (n == 0) return T81B200_OK;
    if (!a || !out || (op != T81B200_EW_CLAMP && (!b || !c))) return fail(T81B200_EINVAL, "elementwise: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (op) {
        case T81B200_EW_WHERE: return launch_ew<T81B200_EW_WHERE>(a, b, c, out, (size_t)n, s0, s1, st);
        case T81B200_EW_CLAMP: return launch_ew<T81B200_EW_CLAMP>(a, b, c, out, (size_t)n, s0, s1, st);
        case T81B200_EW_LERP: return launch_ew<T81B200_EW_LERP>(a, b, c, out, (size_t)n, s0, s1, st);
        default: return launch_ew<T81B200_EW_ADDCMUL>(a, b, c, out, (size_t)n, s0, s1, st);
    }
}

namespace t81b200 {
void release_elementwise_staging() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) return;
    for (int d = 0; d < count && d < 64; ++d) {
        EwStaging &stg = g_ew_staging[d];
        std::lock_guard<std::mutex> lock(stg.mu);
        bool any = false;
        for (int i = 0; i < 4; ++i) any = any || stg.buf[i];
        if (!any || cudaSetDevice(d) != cudaSuccess) continue;
        for (int i = 0; i < 4; ++i) { if (stg.buf[i]) cudaFree(stg.buf[i]); stg.buf[i] = nullptr; stg.cap[i] = 0; }
    }
}
}  // namespace t81b200

extern "C" int t81b200_elementwise_auto(int op, const float *a, const float *b, const float *c, float *out, int64_t n,
                                        float s0, float s1) {
    if (n < 0) return fail(T81B200_EINVAL, "elementwise: negative length");
    if (op < T81B200_EW_WHERE || op > T81B200_EW_ADDCMUL) return fail(T81B200_EINVAL, "elementwise: unknown operation %d", op);
    if (int rc = check_device()) return rc;
    if (n == 0) return T81B200_OK;
    if (!a || !out || (op != T81B200_EW_CLAMP && (!b || !c))) return fail(T81B200_EINVAL, "elementwise: null pointer");
    const void *src[4] = {a, op == T81B200_EW_CLAMP ? nullptr : b, op == T81B200_EW_CLAMP ? nullptr : c, out};
    int on_dev[4] = {0, 0, 0, 0};
    bool any_host = false;
    for (int i = 0; i < 4; ++i)
        if (src[i]) { pointer_is_device(src[i], &on_dev[i]); any_host = any_host || !on_dev[i]; }
    if (!any_host) {
        if (int rc = t81b200_elementwise(op, a, b, c, out, n, s0, s1, nullptr)) return rc;
        T81_CUDA_TRY(cudaStreamSynchronize(0));
        return T81B200_OK;
    }
    int dev = 0;
    T81_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(T81B200_ELIMIT, "device index %d not supported", dev);
    EwStaging &stg = g_ew_staging[dev];
    std::lock_guard<std::mutex> lock(stg.mu);
    const size_t bytes = (size_t)n * sizeof(float);
    const void *use[4];
    for (int i = 0; i < 4; ++i) {
        use[i] = src[i];
        if (!src[i] || on_dev[i]) continue;
        if (stg.cap[i] < bytes) {
            if (stg.buf[i]) cudaFree(stg.buf[i]);
            stg.buf[i] = nullptr; stg.cap[i] = 0;
            T81_CUDA_TRY(cudaMalloc(&stg.buf[i], bytes));
            stg.cap[i] = bytes;
        }
        if (i < 3) T81_CUDA_TRY(cudaMemcpyAsync(stg.buf[i], src[i], bytes, cudaMemcpyHostToDevice, 0));
        use[i] = stg.buf[i];
    }
    if (int rc = t81b200_elementwise(op, (const float *)use[0], (const float *)use[1], (const float *)use[2],
                                     (float *)const_cast<void *>(use[3]), n, s0, s1, nullptr))
        return rc;
    if (!on_dev[3]) T81_CUDA_TRY(cudaMemcpyAsync(out, use[3], bytes, cudaMemcpyDeviceToHost, 0));
    T81_CUDA_TRY(cudaStreamSynchronize(0));
    return T81B200_OK;
}
