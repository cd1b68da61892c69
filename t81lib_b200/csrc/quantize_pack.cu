// Fused threshold-quantise + trit-pack kernel, and its inverse.
//
// One CTA of 256 threads owns one matrix row at a time.
//   ABSMEAN pass: every thread sums |w| of the float4 groups it owns in fp64,
//   in a fixed element order (group 4*(lane + 256*i), i ascending), then the 256
//   partials are folded by a fixed halving tree (inside each warp, then across
//   the 8 warps), so the row scale — and with it every trit — is reproducible
//   bit for bit.
//   Quantise pass: the same float4 groups (kept in registers when the row has at
//   most 4096 columns, re-read through L1/L2 otherwise) become digits d = t+1 in
//   a byte array in shared memory; then each thread turns 12 digits (3 words)
//   into 4 tryte bytes and stores one 32-bit word, so the packed row leaves in
//   fully coalesced stores.  HBM traffic is the algorithmic minimum: each weight
//   is read from DRAM once, each packed byte written once.
#include "common.cuh"

namespace t81b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kRegGroups = 4;  // float4 groups per thread cached in registers

// Reference rule: clamp to [-1,1], inclusive compares, NaN -> 0.  Returns t+1.
__device__ __forceinline__ uint32_t quantize_digit(float v, float thr) {
    const float c = fminf(fmaxf(v, -1.0f), 1.0f);  // NaN: fmaxf(NaN,-1) = -1; handled below
    uint32_t d = 1u;
    if (c >= thr) d = 2u;
    if (c <= -thr) d = 0u;
    if (v != v) d = 1u;  // std::clamp leaves NaN, and both compares are false
    return d;
}

template <typename T> struct Group4 {
    float v[4];
};

template <typename T>
__device__ __forceinline__ void load_group(const T *row, int64_t base, int64_t cols, bool vec,
                                           float (&v)[4]) {
    if (vec && base + 4 <= cols) {
        if constexpr (sizeof(T) == 4) {
            const float4 f = __ldg(reinterpret_cast<const float4 *>(row + base));
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            const uint2 u = __ldg(reinterpret_cast<const uint2 *>(row + base));
            const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
            for (int c = 0; c < 4; ++c) v[c] = to_float<T>(e[c]);
        }
    } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] = base + c < cols ? to_float<T>(row[base + c]) : 0.0f;
    }
}

template <typename T, bool ABSMEAN>
__global__ void __launch_bounds__(kThreads)
quantize_pack_kernel(const T *__restrict__ w, int64_t rows, int64_t cols, int64_t ld, float thr,
                     uint8_t *__restrict__ packed, float *__restrict__ row_scale, bool vec) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *digits = reinterpret_cast<uint32_t *>(smem);  // one byte per trit, kl*48 bytes
    __shared__ double warp_sum[kThreads / 32];
    __shared__ float inv_shared;

    const int tid = threadIdx.x;
    const int64_t kl = (cols + 47) / 48;
    const int64_t groups = (cols + 3) / 4;       // float4 groups holding data
    const int64_t digit_words = kl * 12;         // 48 digits = 12 words per limb
    const bool cached = groups <= (int64_t)kThreads * kRegGroups;

    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T *row = w + r * ld;
        float reg[kRegGroups][4];
        if (cached) {
#pragma unroll
            for (int i = 0; i < kRegGroups; ++i) {
                const int64_t g = tid + (int64_t)kThreads * i;
                if (g < groups) load_group<T>(row, 4 * g, cols, vec, reg[i]);
                else { reg[i][0] = reg[i][1] = reg[i][2] = reg[i][3] = 0.0f; }
            }
        }

        float inv = 1.0f;
        if constexpr (ABSMEAN) {
            double s = 0.0;
            if (cached) {
#pragma unroll
                for (int i = 0; i < kRegGroups; ++i) {
                    const int64_t g = tid + (int64_t)kThreads * i;
                    if (g < groups) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (4 * g + c < cols) s += (double)fabsf(reg[i][c]);
                    }
                }
            } else {
                for (int64_t g = tid; g < groups; g += kThreads) {
                    float v[4];
                    load_group<T>(row, 4 * g, cols, vec, v);
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (4 * g + c < cols) s += (double)fabsf(v[c]);
                }
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
            if ((tid & 31) == 0) warp_sum[tid >> 5] = s;
            __syncthreads();
            if (tid == 0) {
                double g8[kThreads / 32];
#pragma unroll
                for (int j = 0; j < kThreads / 32; ++j) g8[j] = warp_sum[j];
#pragma unroll
                for (int off = kThreads / 64; off >= 1; off >>= 1)
#pragma unroll
                    for (int j = 0; j < off; ++j) g8[j] += g8[j + off];
                const float sr = (float)(g8[0] / (double)cols);
                inv_shared = sr > 0.0f ? __fdiv_rn(1.0f, sr) : 0.0f;
                row_scale[r] = sr;
            }
            __syncthreads();
            inv = inv_shared;
        }

        // digits into shared memory, one 32-bit word (4 digits) per float4 group
        if (cached) {
#pragma unroll
            for (int i = 0; i < kRegGroups; ++i) {
                const int64_t g = tid + (int64_t)kThreads * i;
                if (g < digit_words) {
                    uint32_t word = 0x01010101u;
                    if (g < groups) {
                        word = 0;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float x = ABSMEAN ? __fmul_rn(reg[i][c], inv) : reg[i][c];
                            const uint32_t d = 4 * g + c < cols ? quantize_digit(x, thr) : 1u;
                            word |= d << (8 * c);
                        }
                    }
                    digits[g] = word;
                }
            }
            // the zero tail of the last limb can reach past the register-cached groups
            for (int64_t g = tid + (int64_t)kThreads * kRegGroups; g < digit_words; g += kThreads)
                digits[g] = 0x01010101u;
        } else {
            for (int64_t g = tid; g < digit_words; g += kThreads) {
                uint32_t word = 0x01010101u;
                if (g < groups) {
                    float v[4];
                    load_group<T>(row, 4 * g, cols, vec, v);
                    word = 0;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float x = ABSMEAN ? __fmul_rn(v[c], inv) : v[c];
                        const uint32_t d = 4 * g + c < cols ? quantize_digit(x, thr) : 1u;
                        word |= d << (8 * c);
                    }
                }
                digits[g] = word;
            }
        }
        __syncthreads();

        // 12 digits (3 words) -> 4 tryte bytes (1 word); word index q covers trytes 4q..4q+3
        uint32_t *out = reinterpret_cast<uint32_t *>(packed + r * kl * 16);
        for (int64_t q = tid; q < kl * 4; q += kThreads) {
            const uint32_t a = digits[3 * q], b = digits[3 * q + 1], c = digits[3 * q + 2];
            // digit bytes: a = d0 d1 d2 d3, b = d4 d5 d6 d7, c = d8 d9 d10 d11
            const uint32_t y0 = (a & 0xff) + 3u * ((a >> 8) & 0xff) + 9u * ((a >> 16) & 0xff);
            const uint32_t y1 = (a >> 24) + 3u * (b & 0xff) + 9u * ((b >> 8) & 0xff);
            const uint32_t y2 = ((b >> 16) & 0xff) + 3u * (b >> 24) + 9u * (c & 0xff);
            const uint32_t y3 = ((c >> 8) & 0xff) + 3u * ((c >> 16) & 0xff) + 9u * (c >> 24);
            out[q] = y0 | (y1 << 8) | (y2 << 16) | (y3 << 24);
        }
        __syncthreads();  // digits[] is reused by the next row
    }
}

__global__ void quantize_trits_kernel(const float *__restrict__ src, int64_t n, float thr,
                                      int8_t *__restrict__ dst) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = (int8_t)((int)quantize_digit(src[i], thr) - 1);
}

// One thread per tryte byte.
__global__ void unpack_kernel(const uint8_t *__restrict__ packed, int64_t rows, int64_t kl,
                              int64_t cols, int8_t *__restrict__ trits, int *bad_bytes) {
    const int64_t total = rows * kl * 16;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const uint32_t b = packed[i];
        if (b > 26u && bad_bytes) atomicAdd(bad_bytes, 1);
        int d0, d1, d2;
        tryte_digits(b, d0, d1, d2);
        const int64_t r = i / (kl * 16);
        const int64_t c = (i - r * kl * 16) * 3;
        int8_t *o = trits + r * cols + c;
        if (c < cols) o[0] = (int8_t)(d0 - 1);
        if (c + 1 < cols) o[1] = (int8_t)(d1 - 1);
        if (c + 2 < cols) o[2] = (int8_t)(d2 - 1);
    }
}

template <typename T>
int launch_quantize_pack(const void *w, int64_t rows, int64_t cols, int64_t ld, float thr, int rule,
                         uint8_t *packed, float *row_scale, cudaStream_t st) {
    const int64_t kl = (cols + 47) / 48;
    const size_t smem = (size_t)kl * 48;
    if (smem > 200 * 1024) return fail(T81B200_ELIMIT, "quantize_pack: cols=%lld exceeds %d", (long long)cols, 200 * 1024);
    const bool vec = (reinterpret_cast<uintptr_t>(w) % (4 * sizeof(T)) == 0) && (ld % 4 == 0);
    const int grid = (int)(rows < (int64_t)sm_count() * 16 ? rows : (int64_t)sm_count() * 16);
    auto kern = rule == T81B200_RULE_ABSMEAN ? quantize_pack_kernel<T, true> : quantize_pack_kernel<T, false>;
    if (smem > 48 * 1024)
        T81_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, st>>>(static_cast<const T *>(w), rows, cols, ld, thr, packed, row_scale, vec);
    T81_LAUNCH_CHECK("quantize_pack_kernel");
    return T81B200_OK;
}

}  // namespace

}  // namespace t81b200

using namespace t81b200;

extern "C" int t81b200_quantize_pack(const void *w, int w_dtype, int64_t rows, int64_t cols, int64_t ld,
                                     float threshold, int rule, uint8_t *packed, float *row_scale,
                                     void *stream) {
    if (rows < 0 || cols < 0) return fail(T81B200_EINVAL, "quantize_pack: rows and cols must be non-negative");
    if (!(threshold >= 0.0f && threshold <= 1.0f))
        return fail(T81B200_EINVAL, "threshold must be between 0 and 1");
    if (rule != T81B200_RULE_FIXED && rule != T81B200_RULE_ABSMEAN)
        return fail(T81B200_EINVAL, "quantize_pack: unknown rule %d", rule);
    if (ld < cols) return fail(T81B200_EINVAL, "quantize_pack: ld (%lld) < cols (%lld)", (long long)ld, (long long)cols);
    if (int rc = check_device()) return rc;
    if (rows == 0 || cols == 0) return T81B200_OK;
    if (!w || !packed) return fail(T81B200_EINVAL, "quantize_pack: null pointer");
    if (rule == T81B200_RULE_ABSMEAN && !row_scale)
        return fail(T81B200_EINVAL, "quantize_pack: the absmean rule needs row_scale");
    if (reinterpret_cast<uintptr_t>(packed) % 4 != 0)
        return fail(T81B200_EALIGN, "quantize_pack: packed must be 4-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (w_dtype) {
        case T81B200_F32: return launch_quantize_pack<float>(w, rows, cols, ld, threshold, rule, packed, row_scale, st);
        case T81B200_BF16: return launch_quantize_pack<__nv_bfloat16>(w, rows, cols, ld, threshold, rule, packed, row_scale, st);
        case T81B200_F16: return launch_quantize_pack<__half>(w, rows, cols, ld, threshold, rule, packed, row_scale, st);
    }
    return fail(T81B200_EINVAL, "quantize_pack: unknown dtype %d", w_dtype);
}

extern "C" int t81b200_quantize_trits(const float *src, int64_t n, float threshold, int8_t *dst, void *stream) {
    if (n < 0) return fail(T81B200_EINVAL, "quantize_trits: n must be non-negative");
    if (!(threshold >= 0.0f && threshold <= 1.0f))
        return fail(T81B200_EINVAL, "threshold must be between 0 and 1");
    if (int rc = check_device()) return rc;
    if (n == 0) return T81B200_OK;
    if (!src || !dst) return fail(T81B200_EINVAL, "quantize_trits: null pointer");
    const int64_t blocks = (n + 255) / 256;
    const int grid = (int)(blocks < (int64_t)sm_count() * 32 ? blocks : (int64_t)sm_count() * 32);
    quantize_trits_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, n, threshold, dst);
    T81_LAUNCH_CHECK("quantize_trits_kernel");
    return T81B200_OK;
}

extern "C" int t81b200_unpack(const uint8_t *packed, int64_t rows, int64_t k_limbs, int64_t cols,
                              int8_t *trits, int *bad_bytes, void *stream) {
    if (rows < 0 || cols < 0 || k_limbs < 0) return fail(T81B200_EINVAL, "rows and cols must be non-negative");
    if (cols > k_limbs * 48) return fail(T81B200_EINVAL, "cols exceeds packed trit capacity");
    if (int rc = check_device()) return rc;
    if (rows == 0 || cols == 0) return T81B200_OK;
    if (!packed || !trits) return fail(T81B200_EINVAL, "unpack: null pointer");
    const int64_t total = rows * k_limbs * 16;
    const int64_t blocks = (total + 255) / 256;
    const int grid = (int)(blocks < (int64_t)sm_count() * 32 ? blocks : (int64_t)sm_count() * 32);
    unpack_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(packed, rows, k_limbs, cols, trits, bad_bytes);
    T81_LAUNCH_CHECK("unpack_kernel");
    return T81B200_OK;
}
