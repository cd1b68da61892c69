// General-purpose TRIT-mode kernel on CUDA cores: any operand layout, dtype and
// alignment, fp32 FMA accumulation in ascending k.  It exists so that every call
// the ABI accepts has a device path (odd strides, unaligned limbs, tiny shapes);
// the streaming and tensor-core kernels take the shapes that matter for speed.
#include "common.cuh"

namespace t81b200 {

namespace {

struct SimtParams {
    const uint8_t *A;
    const void *B;
    void *C;
    const float *row_scale, *bias;
    int64_t M, N, K, kl;
    int64_t sbk, sbn;  // element strides of B along k and n
    int64_t scm, scn;  // element strides of C along m and n
    float alpha, beta;
};

template <typename BT, typename CT>
__global__ void __launch_bounds__(256) gemm_trit_simt_kernel(const SimtParams p) {
    const int64_t n = (int64_t)blockIdx.x * 32 + threadIdx.x;
    const int64_t m = (int64_t)blockIdx.y * 8 + threadIdx.y;
    if (m >= p.M || n >= p.N) return;
    const BT *B = static_cast<const BT *>(p.B) + n * p.sbn;
    const uint8_t *a = p.A + m * p.kl * 16;
    float acc = 0.0f;
    for (int64_t byte = 0; byte * 3 < p.K; ++byte) {
        int d0, d1, d2;
        tryte_digits(a[byte], d0, d1, d2);
        const int64_t k = byte * 3;
        acc += (float)(d0 - 1) * to_float<BT>(B[k * p.sbk]);
        if (k + 1 < p.K) acc += (float)(d1 - 1) * to_float<BT>(B[(k + 1) * p.sbk]);
        if (k + 2 < p.K) acc += (float)(d2 - 1) * to_float<BT>(B[(k + 2) * p.sbk]);
    }
    float v = acc * p.alpha;
    if (p.row_scale) v *= p.row_scale[m];
    if (p.bias) v += p.bias[m];
    CT *c = static_cast<CT *>(p.C) + m * p.scm + n * p.scn;
    if (p.beta != 0.0f) v += p.beta * to_float<CT>(*c);
    *c = from_float<CT>(v);
}

template <typename BT>
int launch_ct(const SimtParams &p, int c_dtype, cudaStream_t st) {
    dim3 block(32, 8), grid((unsigned)((p.N + 31) / 32), (unsigned)((p.M + 7) / 8));
    if (grid.y > 65535u) return fail(T81B200_ELIMIT, "gemm_trit: M too large for the general kernel");
    switch (c_dtype) {
        case T81B200_F32: gemm_trit_simt_kernel<BT, float><<<grid, block, 0, st>>>(p); break;
        case T81B200_BF16: gemm_trit_simt_kernel<BT, __nv_bfloat16><<<grid, block, 0, st>>>(p); break;
        case T81B200_F16: gemm_trit_simt_kernel<BT, __half><<<grid, block, 0, st>>>(p); break;
        default: return fail(T81B200_EINVAL, "gemm_trit: unknown output dtype %d", c_dtype);
    }
    T81_LAUNCH_CHECK("gemm_trit_simt_kernel");
    return T81B200_OK;
}

}  // namespace

int gemm_trit_simt_launch(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                          int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                          int64_t N, int64_t K, float alpha, float beta, cudaStream_t st) {
    SimtParams p;
    p.A = A; p.B = B; p.C = C; p.row_scale = row_scale; p.bias = bias;
    p.M = M; p.N = N; p.K = K; p.kl = (K + 47) / 48;
    if (layout == T81B200_LAYOUT_KN) { p.sbk = ldb; p.sbn = 1; p.scm = ldc; p.scn = 1; }
    else { p.sbk = 1; p.sbn = ldb; p.scm = 1; p.scn = ldc; }
    p.alpha = alpha; p.beta = beta;
    switch (b_dtype) {
        case T81B200_F32: return launch_ct<float>(p, c_dtype, st);
        case T81B200_BF16: return launch_ct<__nv_bfloat16>(p, c_dtype, st);
        case T81B200_F16: return launch_ct<__half>(p, c_dtype, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown activation dtype %d", b_dtype);
}

}  // namespace t81b200
