// Fused threshold-quantise + trit-pack kernel, and its inverse.
//
// One warp owns one matrix row at a time; nothing synchronises wider than a warp.
//   ABSMEAN pass: |w| is summed in fp64 in a fixed order — 256 partials, partial l taking
//   the float4 groups l, l+256, ... — which a warp reproduces with 8 accumulators per lane;
//   the partials are folded by a fixed halving tree (32 consecutive partials = the 32 lanes
//   of one accumulator slot, then the 8 slot sums).  The row scale, and with it every trit,
//   is therefore reproducible bit for bit and independent of the launch shape.
//   Quantise pass: 768 weights (16 limbs) per step: six coalesced float4 loads per lane
//   become digits d = t+1 in a 768-byte per-warp array in shared memory, then every lane
//   turns 12 digits into 4 tryte bytes and the warp stores 2 x 128 contiguous bytes.
//   With the absmean rule the row is read twice; the second read is served by L1/L2 (a row
//   is 16 KB), so DRAM sees each weight once and each packed byte once.
#include "common.cuh"

namespace t81b200 {

namespace {

constexpr int kThreads = 256;

// Reference rule (clamp to [-1,1], then c >= thr -> +1, c <= -thr -> -1, else 0), returned
// as t+1.  With thr <= 1 the clamp cannot change either comparison, and NaN fails both, so
// two compares on the raw value are equivalent.  The negative test is applied last: at
// thr == 0 a zero becomes -1, like the reference's Python quantiser (t81/torch/__init__.py:44-50).
__device__ __forceinline__ uint32_t quantize_digit(float v, float thr) {
    return v <= -thr ? 0u : (v >= thr ? 2u : 1u);
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

constexpr int kWarpsPerCta = kThreads / 32;
constexpr int kChunkGroups = 192;  // float4 groups per warp step: 768 weights = 16 limbs

// One warp owns one row at a time; there is no block-wide barrier anywhere.
template <typename T, bool ABSMEAN>
__global__ void __launch_bounds__(kThreads, 2)
quantize_pack_kernel(const T *__restrict__ w, int64_t rows, int64_t cols, int64_t ld, float thr,
                     uint8_t *__restrict__ packed, float *__restrict__ row_scale, bool vec) {
    __shared__ uint32_t digit_smem[kWarpsPerCta][kChunkGroups];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t *digits = digit_smem[warp];
    const int64_t kl = (cols + 47) / 48;
    const int64_t groups = (cols + 3) / 4;  // float4 groups holding data
    const int64_t out_words = kl * 4;       // 32-bit words of the packed row
    const int64_t warp_global = (int64_t)blockIdx.x * kWarpsPerCta + warp;
    const int64_t warp_stride = (int64_t)gridDim.x * kWarpsPerCta;

    for (int64_t r = warp_global; r < rows; r += warp_stride) {
        const T *row = w + r * ld;
        float inv = 1.0f;
        if constexpr (ABSMEAN) {
            // Partial l = g % 256 of the reference order lives in lane l % 32, slot l / 32:
            // this lane's m-th group (g = lane + 32 m) belongs to slot m % 8.
            double part[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) part[j] = 0.0;
            // batches of 8 groups per lane (4 KB per warp), the next batch in flight while this one is summed
            auto load_batch = [&](int64_t g0, float (&v)[8][4]) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int64_t g = g0 + 32 * j;
                    if (g < groups) load_group<T>(row, 4 * g, cols, vec, v[j]);
                    else { v[j][0] = v[j][1] = v[j][2] = v[j][3] = 0.0f; }
                }
            };
            auto sum_batch = [&](int64_t g0, const float (&v)[8][4]) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int64_t g = g0 + 32 * j;
                    if (g < groups) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (4 * g + c < cols) part[j] += (double)fabsf(v[j][c]);
                    }
                }
            };
            {
                float va[8][4], vb[8][4];
                load_batch(lane, va);
                for (int64_t g0 = lane; g0 < groups; g0 += 512) {
                    if (g0 + 256 < groups) load_batch(g0 + 256, vb);
                    sum_batch(g0, va);
                    if (g0 + 256 < groups) {
                        if (g0 + 512 < groups) load_batch(g0 + 512, va);
                        sum_batch(g0 + 256, vb);
                    }
                }
            }
            // halving tree inside each group of 32 consecutive partials (= the 32 lanes of slot j)
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) part[j] += __shfl_down_sync(0xffffffffu, part[j], off);
            // then over the 8 group sums (offsets 4, 2, 1); only lane 0 holds valid sums
#pragma unroll
            for (int off = 4; off >= 1; off >>= 1)
#pragma unroll
                for (int j = 0; j < off; ++j) part[j] += part[j + off];
            float sr = (float)(part[0] / (double)cols);
            sr = __shfl_sync(0xffffffffu, sr, 0);
            inv = sr > 0.0f ? __fdiv_rn(1.0f, sr) : 0.0f;
            if (lane == 0) row_scale[r] = sr;
        }

        uint32_t *out = reinterpret_cast<uint32_t *>(packed + r * kl * 16);
        auto load_chunk = [&](int64_t gbase, float (&v)[6][4]) {
#pragma unroll
            for (int q = 0; q < 6; ++q) {
                const int64_t g = gbase + lane + 32 * q;
                if (g < groups) load_group<T>(row, 4 * g, cols, vec, v[q]);
                else { v[q][0] = v[q][1] = v[q][2] = v[q][3] = 0.0f; }
            }
        };
        float v[6][4], vnext[6][4];
        load_chunk(0, v);
        for (int64_t gbase = 0; gbase < kl * 12; gbase += kChunkGroups) {
            const bool more = gbase + kChunkGroups < kl * 12;
            if (more) load_chunk(gbase + kChunkGroups, vnext);  // in flight while this step is packed
#pragma unroll
            for (int q = 0; q < 6; ++q) {
                const int64_t g = gbase + lane + 32 * q;
                uint32_t word = 0x01010101u;  // zero trits: the tail of the last limb
                if (g < groups) {
                    word = 0;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float x = ABSMEAN ? __fmul_rn(v[q][c], inv) : v[q][c];
                        const uint32_t d = 4 * g + c < cols ? quantize_digit(x, thr) : 1u;
                        word |= d << (8 * c);
                    }
                }
                digits[lane + 32 * q] = word;
            }
            __syncwarp();
            // 12 digits (3 words) -> 4 tryte bytes (1 word); 64 output words per step
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int o = lane + 32 * h;
                const int64_t q = gbase / 3 + o;
                if (q < out_words) {
                    const uint32_t a = digits[3 * o], b = digits[3 * o + 1], c = digits[3 * o + 2];
                    const uint32_t y0 = (a & 0xff) + 3u * ((a >> 8) & 0xff) + 9u * ((a >> 16) & 0xff);
                    const uint32_t y1 = (a >> 24) + 3u * (b & 0xff) + 9u * ((b >> 8) & 0xff);
                    const uint32_t y2 = ((b >> 16) & 0xff) + 3u * (b >> 24) + 9u * (c & 0xff);
                    const uint32_t y3 = ((c >> 8) & 0xff) + 3u * ((c >> 16) & 0xff) + 9u * (c >> 24);
                    out[q] = y0 | (y1 << 8) | (y2 << 16) | (y3 << 24);
                }
            }
            __syncwarp();  // digits[] is reused by the next step
            if (more) {
#pragma unroll
                for (int q = 0; q < 6; ++q)
#pragma unroll
                    for (int c = 0; c < 4; ++c) v[q][c] = vnext[q][c];
            }
        }
    }
}

// Row-in-shared-memory variant: a small CTA (128 threads) owns one row at a time, keeps it as
// floats in shared memory between the absmean pass and the quantise pass (each weight is read
// from global memory exactly once), and many such CTAs share an SM (about 20 KB each for a
// 4096-column row), so the three block barriers per row overlap across CTAs.  The summation
// order is the same fixed one: thread tau owns partials tau and tau+128.
constexpr int kRowThreads = 128;

template <typename T, bool ABSMEAN>
__global__ void __launch_bounds__(kRowThreads, 8)
quantize_pack_row_kernel(const T *__restrict__ w, int64_t rows, int64_t cols, int64_t ld, float thr,
                         uint8_t *__restrict__ packed, float *__restrict__ row_scale, bool vec) {
    extern __shared__ __align__(16) uint8_t row_smem[];
    const int64_t kl = (cols + 47) / 48;
    const int64_t groups = (cols + 3) / 4;
    float4 *rowf = reinterpret_cast<float4 *>(row_smem);                         // groups float4
    __shared__ double group_sum[8];
    __shared__ float inv_shared;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T *row = w + r * ld;
        double part[2] = {0.0, 0.0};
        // m-th group of this thread: g = tid + 128 m; it belongs to partial g % 256 = tid + 128 (m % 2)
        const int ng = (int)groups;
        for (int g0 = tid; g0 < ng; g0 += 8 * kRowThreads) {
            float v[8][4];  // eight loads in flight per thread before any is used
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int g = g0 + kRowThreads * j;
                if (g < ng) load_group<T>(row, 4 * (int64_t)g, cols, vec, v[j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int g = g0 + kRowThreads * j;
                if (g < ng) {
                    rowf[g] = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
                    if constexpr (ABSMEAN) {
                        // columns past the end were loaded as 0: adding |0| leaves a non-negative fp64 sum unchanged
#pragma unroll
                        for (int c = 0; c < 4; ++c) part[j & 1] += (double)fabsf(v[j][c]);
                    }
                }
            }
        }
        float inv = 1.0f;
        if constexpr (ABSMEAN) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) part[j] += __shfl_down_sync(0xffffffffu, part[j], off);
                if (lane == 0) group_sum[warp + 4 * j] = part[j];  // partials 32*(warp+4j) .. +31
            }
            __syncthreads();
            if (tid == 0) {
                double g8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) g8[j] = group_sum[j];
#pragma unroll
                for (int off = 4; off >= 1; off >>= 1)
#pragma unroll
                    for (int j = 0; j < off; ++j) g8[j] += g8[j + off];
                const float sr = (float)(g8[0] / (double)cols);
                inv_shared = sr > 0.0f ? __fdiv_rn(1.0f, sr) : 0.0f;
                row_scale[r] = sr;
            }
            __syncthreads();
            inv = inv_shared;
        }
        if constexpr (!ABSMEAN) __syncthreads();  // the pack pass reads groups other threads loaded
        // pack: one thread per output word = 4 trytes = 12 weights = groups 3q .. 3q+2 of the cached row.
        // Digits are formed as floats (two compares each), a tryte is d0 + 3 d1 + 9 d2 (exact in fp32).
        uint32_t *out = reinterpret_cast<uint32_t *>(packed + r * kl * 16);
        const int nwords = (int)kl * 4;
        const int ngroups = (int)groups, ncols = (int)cols;
        for (int q = tid; q < nwords; q += kRowThreads) {
            float d[12];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int g = 3 * q + j;
                if (g < ngroups) {
                    const float4 f = rowf[g];
                    const float v[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float x = ABSMEAN ? __fmul_rn(v[c], inv) : v[c];
                        d[4 * j + c] = x <= -thr ? 0.0f : (x >= thr ? 2.0f : 1.0f);
                    }
                    if (4 * g + 4 > ncols) {  // the row's last, partial group: columns past the end are zero trits
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (4 * g + c >= ncols) d[4 * j + c] = 1.0f;
                    }
                } else {
                    d[4 * j] = d[4 * j + 1] = d[4 * j + 2] = d[4 * j + 3] = 1.0f;  // padding up to the limb: zero trits
                }
            }
            float y[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) y[t] = fmaf(9.0f, d[3 * t + 2], fmaf(3.0f, d[3 * t + 1], d[3 * t]));
            const float low = fmaf(65536.0f, y[2], fmaf(256.0f, y[1], y[0]));  // < 2^24: exact
            out[q] = (uint32_t)low + ((uint32_t)y[3] << 24);
        }
        __syncthreads();  // the cached row is reused by the next row
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
    const bool vec = (reinterpret_cast<uintptr_t>(w) % (4 * sizeof(T)) == 0) && (ld % 4 == 0);
    // rows that fit shared memory several times per SM: the row-in-shared-memory kernel
    const size_t row_bytes = (size_t)((cols + 3) / 4) * 16;  // the row as fp32, whatever the input type
    if (row_bytes <= 100 * 1024) {  // up to 25 600 columns: at least two rows resident per SM
        auto rk = rule == T81B200_RULE_ABSMEAN ? quantize_pack_row_kernel<T, true> : quantize_pack_row_kernel<T, false>;
        if (row_bytes > 48 * 1024)
            T81_CUDA_TRY(cudaFuncSetAttribute(rk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_bytes));
        const int64_t cap = (int64_t)sm_count() * 16;
        const int g = (int)(rows < cap ? rows : cap);
        rk<<<g, kRowThreads, row_bytes, st>>>(static_cast<const T *>(w), rows, cols, ld, thr, packed, row_scale, vec);
        T81_LAUNCH_CHECK("quantize_pack_row_kernel");
        return T81B200_OK;
    }
    const int64_t ctas = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
    const int grid = (int)(ctas < (int64_t)sm_count() * 8 ? ctas : (int64_t)sm_count() * 8);
    auto kern = rule == T81B200_RULE_ABSMEAN ? quantize_pack_kernel<T, true> : quantize_pack_kernel<T, false>;
    kern<<<grid, kThreads, 0, st>>>(static_cast<const T *>(w), rows, cols, ld, thr, packed, row_scale, vec);
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
