// Quantisation-aware-training forward of the ternary Linear (t81/nn/linear.py:72-99 with t81/qat.py:12-57 of the
// reference), the two steps that touch every weight fused into two streaming kernels:
//   1. the running scale: candidate = max |w| over the whole weight, clamped to >= 1e-6, blended into the stored
//      scale with momentum 0.99 (_update_training_scale) — one reduction kernel, the blend done by the last CTA;
//   2. quantise + pack: trit = Q(w / scale, threshold) with the reference's rule (clamp to [-1, 1], |.| >= threshold
//      keeps the sign), written straight into the packed-limb layout, and the scale broadcast into a per-row
//      vector — so the forward product runs on the packed-trit matmul kernels with that vector as row scale and
//      no fp32 copy of the quantised weight is ever materialised (the reference builds quantized * scale in full).
// Both read the weight once (4 bytes per weight for fp32) and write 1/3 byte per weight: HBM-bound streams.
#include "common.cuh"

namespace t81b200 {

namespace {

// state[0]: the running scale (in/out)   state[1]: max |w| of this call as float bits (scratch, zero between calls)
// state[2]: CTAs that have contributed (scratch, zero between calls)   state[3]: 1 once state[0] holds a scale
template <typename T>
__global__ void __launch_bounds__(256) absmax_ema_kernel(const T *__restrict__ w, int64_t rows, int64_t cols, int64_t ld,
                                                         float momentum, float one_minus, float *__restrict__ state) {
    __shared__ float warp_max[8];
    float m = 0.0f;
    const int64_t n = rows * cols, stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t r = i / cols, c = i - r * cols;
        const float a = fabsf(to_float<T>(w[r * ld + c]));
        m = a > m ? a : m;  // a NaN compares false and never becomes the maximum
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const float o = __shfl_down_sync(0xffffffffu, m, off);
        m = o > m ? o : m;
    }
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int j = 1; j < 8; ++j) m = warp_max[j] > m ? warp_max[j] : m;
        unsigned int *bits = reinterpret_cast<unsigned int *>(state + 1);
        unsigned int *ticket = reinterpret_cast<unsigned int *>(state + 2);
        atomicMax(bits, __float_as_uint(m));  // non-negative floats order like their bit patterns
        __threadfence();
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
            // the last CTA blends and resets the scratch words for the next call
            __threadfence();
            float candidate = __uint_as_float(atomicExch(bits, 0u));
            candidate = candidate < 1e-6f ? 1e-6f : candidate;
            float scale = candidate;
            if (state[3] != 0.0f) {
                scale = __fadd_rn(__fmul_rn(state[0], momentum), __fmul_rn(candidate, one_minus));
                scale = scale < 1e-6f ? 1e-6f : scale;
            }
            state[0] = scale;
            state[3] = 1.0f;
            *ticket = 0u;
        }
    }
}

// One thread per output word: 12 weights -> 4 tryte bytes.
template <typename T>
__global__ void __launch_bounds__(256) qat_quantize_pack_kernel(const T *__restrict__ w, int64_t rows, int64_t cols, int64_t ld,
                                                                float thr, const float *__restrict__ scale_ptr,
                                                                uint8_t *__restrict__ packed, float *__restrict__ row_scale) {
    const float scale = *scale_ptr;
    const int64_t kl = (cols + 47) / 48, words_per_row = kl * 4, total = rows * words_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / words_per_row, q = i - r * words_per_row;
        const T *row = w + r * ld;
        uint32_t word = 0;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            uint32_t tryte = 0, weight = 1;
#pragma unroll
            for (int d = 0; d < 3; ++d, weight *= 3) {
                const int64_t c = 12 * q + 3 * t + d;
                uint32_t digit = 1;
                if (c < cols) {
                    const float x = __fdiv_rn(to_float<T>(row[c]), scale);  // weight / scale, as the reference divides
                    // |clamp(x)| >= thr keeps sign(x): the clamp changes neither compare (thr <= 1), a zero stays zero
                    digit = (x >= thr && x > 0.0f) ? 2u : ((x <= -thr && x < 0.0f) ? 0u : 1u);
                }
                tryte += digit * weight;
            }
            word |= tryte << (8 * t);
        }
        reinterpret_cast<uint32_t *>(packed)[i] = word;
        if (row_scale && q == 0) row_scale[r] = scale;
    }
}

}  // namespace
}  // namespace t81b200

using namespace t81b200;

extern "C" int t81b200_qat_update_scale(const void *w, int w_dtype, int64_t rows, int64_t cols, int64_t ld, float momentum,
                                        float *state, void *stream) {
    if (rows < 0 || cols < 0 || ld < cols) return fail(T81B200_EINVAL, "qat_update_scale: bad dimensions");
    if (!(momentum >= 0.0f && momentum <= 1.0f)) return fail(T81B200_EINVAL, "qat_update_scale: momentum must be in [0, 1]");
    if (int rc = check_device()) return rc;
    if (!state || ((rows > 0 && cols > 0) && !w)) return fail(T81B200_EINVAL, "qat_update_scale: null pointer");
    const int64_t n = rows * cols;
    int64_t blocks = (n + 256 * 8 - 1) / (256 * 8);
    const int64_t cap = (int64_t)sm_count() * 8;
    blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
    const float one_minus = (float)(1.0 - (double)momentum);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (w_dtype) {
        case T81B200_F32: absmax_ema_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const float *>(w), rows, cols, ld, momentum, one_minus, state); break;
        case T81B200_BF16: absmax_ema_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(w), rows, cols, ld, momentum, one_minus, state); break;
        case T81B200_F16: absmax_ema_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half *>(w), rows, cols, ld, momentum, one_minus, state); break;
        default: return fail(T81B200_EINVAL, "qat_update_scale: unknown dtype %d", w_dtype);
    }
    T81_LAUNCH_CHECK("absmax_ema_kernel");
    return T81B200_OK;
}

extern "C" int t81b200_qat_quantize_pack(const void *w, int w_dtype, int64_t rows, int64_t cols, int64_t ld, float threshold,
                                         const float *scale, uint8_t *packed, float *row_scale, void *stream) {
    if (rows < 0 || cols < 0 || ld < cols) return fail(T81B200_EINVAL, "qat_quantize_pack: bad dimensions");
    if (!(threshold >= 0.0f && threshold <= 1.0f)) return fail(T81B200_EINVAL, "threshold must be between 0 and 1");
    if (int rc = check_device()) return rc;
    if (rows == 0 || cols == 0) return T81B200_OK;
    if (!w || !scale || !packed) return fail(T81B200_EINVAL, "qat_quantize_pack: null pointer");
    if (reinterpret_cast<uintptr_t>(packed) % 4 != 0) return fail(T81B200_EALIGN, "qat_quantize_pack: packed must be 4-byte aligned");
    const int64_t total = rows * ((cols + 47) / 48) * 4;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    blocks = blocks > cap ? cap : blocks;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (w_dtype) {
        case T81B200_F32: qat_quantize_pack_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const float *>(w), rows, cols, ld, threshold, scale, packed, row_scale); break;
        case T81B200_BF16: qat_quantize_pack_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(w), rows, cols, ld, threshold, scale, packed, row_scale); break;
        case T81B200_F16: qat_quantize_pack_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __half *>(w), rows, cols, ld, threshold, scale, packed, row_scale); break;
        default: return fail(T81B200_EINVAL, "qat_quantize_pack: unknown dtype %d", w_dtype);
    }
    T81_LAUNCH_CHECK("qat_quantize_pack_kernel");
    return T81B200_OK;
}
