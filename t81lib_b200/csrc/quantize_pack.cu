// Fused threshold-quantise + trit-pack kernel, and its inverse.
//
// quantize_pack_row_kernel: a CTA of 128 threads owns one row at a time.  Thread tau owns the 32-bit words
// q = tau, tau + 128, ... of the packed row, i.e. the 12 weights (three float4 groups, 48 contiguous bytes of
// fp32) behind each of them.  Rows of up to 6144 columns are read from global memory ONCE, into registers;
// longer rows are read a second time for the pack pass (from L2).  With the absmean rule the row scale is
// the mean of |w| summed in a fixed order — fp32 inside a float4 group, fp64 across the groups of a thread in
// word order, then a halving tree over the 128 threads — that the CPU checker reproduces bit for bit,
// whatever the launch shape.  One block barrier per row (the four warp sums, double-buffered by row parity).
// Then every thread turns its 12 weights into 12 digits (two compares each), the digits into 4 tryte bytes
// d0 + 3 d1 + 9 d2 (exact in fp32), and stores one coalesced 32-bit word.
//
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

constexpr int kRowThreads = 128;
constexpr int kRegWords = 4;  // words (12 weights each) a thread keeps in registers: rows of up to 128 * 4 * 12 columns

// Three float4 groups (one output word) of a row: loads, and with ABSMEAN the group sums into the thread's partial.
template <typename T, bool ABSMEAN>
__device__ __forceinline__ void load_word(const T *row, int64_t q, int64_t groups, int64_t cols, bool vec, float (&v)[3][4],
                                          double &part) {
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const int64_t g = 3 * q + j;
        if (g < groups) load_group<T>(row, 4 * g, cols, vec, v[j]);  // columns past the end load as 0
        else { v[j][0] = v[j][1] = v[j][2] = v[j][3] = 0.0f; }
    }
    if constexpr (ABSMEAN) {
#pragma unroll
        for (int j = 0; j < 3; ++j)
            if (3 * q + j < groups)  // fp32 inside the group, fp64 across groups, in word order
                part += (double)__fadd_rn(__fadd_rn(fabsf(v[j][0]), fabsf(v[j][1])), __fadd_rn(fabsf(v[j][2]), fabsf(v[j][3])));
    }
}

template <bool ABSMEAN>
__device__ __forceinline__ uint32_t pack_word(const float (&v)[3][4], int64_t q, int64_t cols, float inv, float thr) {
    float d[12];
#pragma unroll
    for (int j = 0; j < 3; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float x = ABSMEAN ? __fmul_rn(v[j][c], inv) : v[j][c];
            d[4 * j + c] = x <= -thr ? 0.0f : (x >= thr ? 2.0f : 1.0f);
        }
    if (12 * q + 12 > cols) {  // the row's last words: columns past the end are zero trits
#pragma unroll
        for (int i = 0; i < 12; ++i)
            if (12 * q + i >= cols) d[i] = 1.0f;
    }
    float y[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) y[t] = fmaf(9.0f, d[3 * t + 2], fmaf(3.0f, d[3 * t + 1], d[3 * t]));
    const float low = fmaf(65536.0f, y[2], fmaf(256.0f, y[1], y[0]));  // < 2^24: exact
    return (uint32_t)low + ((uint32_t)y[3] << 24);
}

// IN_REGS: the row's words per thread fit kRegWords and stay in registers between the two passes.
template <typename T, bool ABSMEAN, bool IN_REGS>
__global__ void __launch_bounds__(kRowThreads, IN_REGS ? 6 : 12)
quantize_pack_row_kernel(const T *__restrict__ w, int64_t rows, int64_t cols, int64_t ld, float thr,
                         uint8_t *__restrict__ packed, float *__restrict__ row_scale, bool vec) {
    __shared__ double warp_sum[2][4];
    const int64_t kl = (cols + 47) / 48;
    const int64_t groups = (cols + 3) / 4;
    const int64_t nwords = kl * 4;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int parity = 0;

    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, parity ^= 1) {
        const T *row = w + r * ld;
        uint32_t *out = reinterpret_cast<uint32_t *>(packed + r * kl * 16);
        float keep[IN_REGS ? kRegWords : 1][3][4];
        double part = 0.0;
        if constexpr (IN_REGS) {
#pragma unroll
            for (int m = 0; m < kRegWords; ++m) {
                const int64_t q = tid + (int64_t)kRowThreads * m;
                if (q < nwords) load_word<T, ABSMEAN>(row, q, groups, cols, vec, keep[m], part);
            }
        } else if constexpr (ABSMEAN) {
            for (int64_t q = tid; q < nwords; q += kRowThreads) {
                float v[3][4];
                load_word<T, true>(row, q, groups, cols, vec, v, part);
            }
        }
        float inv = 1.0f;
        if constexpr (ABSMEAN) {
            // halving tree over the 128 partials: inside each warp, then over the four warp sums
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) part += __shfl_down_sync(0xffffffffu, part, off);
            if (lane == 0) warp_sum[parity][warp] = part;
            __syncthreads();  // the only block barrier of a row; the other parity's sums are free to be rewritten
            const double total = (warp_sum[parity][0] + warp_sum[parity][2]) + (warp_sum[parity][1] + warp_sum[parity][3]);
            const float sr = (float)(total / (double)cols);
            inv = sr > 0.0f ? __fdiv_rn(1.0f, sr) : 0.0f;
            if (tid == 0) row_scale[r] = sr;
        }
        if constexpr (IN_REGS) {
#pragma unroll
            for (int m = 0; m < kRegWords; ++m) {
                const int64_t q = tid + (int64_t)kRowThreads * m;
                if (q < nwords) out[q] = pack_word<ABSMEAN>(keep[m], q, cols, inv, thr);
            }
        } else {
            for (int64_t q = tid; q < nwords; q += kRowThreads) {
                float v[3][4];
                double unused = 0.0;
                load_word<T, false>(row, q, groups, cols, vec, v, unused);  // second read of the row: L2
                out[q] = pack_word<ABSMEAN>(v, q, cols, inv, thr);
            }
        }
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

template <typename T, bool IN_REGS>
int launch_row_kernel(const void *w, int64_t rows, int64_t cols, int64_t ld, float thr, int rule, uint8_t *packed,
                      float *row_scale, bool vec, cudaStream_t st) {
    const int64_t cap = (int64_t)sm_count() * 16;
    const int g = (int)(rows < cap ? rows : cap);
    if (rule == T81B200_RULE_ABSMEAN)
        quantize_pack_row_kernel<T, true, IN_REGS><<<g, kRowThreads, 0, st>>>(static_cast<const T *>(w), rows, cols, ld, thr, packed, row_scale, vec);
    else
        quantize_pack_row_kernel<T, false, IN_REGS><<<g, kRowThreads, 0, st>>>(static_cast<const T *>(w), rows, cols, ld, thr, packed, row_scale, vec);
    T81_LAUNCH_CHECK("quantize_pack_row_kernel");
    return T81B200_OK;
}

template <typename T>
int launch_quantize_pack(const void *w, int64_t rows, int64_t cols, int64_t ld, float thr, int rule,
                         uint8_t *packed, float *row_scale, cudaStream_t st) {
    const bool vec = (reinterpret_cast<uintptr_t>(w) % (4 * sizeof(T)) == 0) && (ld % 4 == 0);
    const int64_t nwords = (cols + 47) / 48 * 4;
    if (nwords <= (int64_t)kRowThreads * kRegWords)
        return launch_row_kernel<T, true>(w, rows, cols, ld, thr, rule, packed, row_scale, vec, st);
    return launch_row_kernel<T, false>(w, rows, cols, ld, thr, rule, packed, row_scale, vec, st);
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
