// Transcoders between the packed-limb layout and the GGUF ternary block formats TQ1_0 and TQ2_0, on the device:
// the on-disk formats either side of the matmul path (t81/gguf.py:518-662 of the reference, which quantises from
// and dequantises to float arrays on the CPU).  Here the trits never leave their integer form: export reads packed
// limbs (+ the per-row scale) and writes blocks, import reads blocks and writes packed limbs (+ the blocks' scales).
//
// A block holds 256 consecutive weights of one row:
//   TQ2_0 (66 bytes): 64 bytes of 2-bit digits q = trit + 1 — byte j of each 32-byte half holds elements
//          j, 32 + j, 64 + j, 96 + j of that half's 128 elements at bits 0, 2, 4, 6 — then the fp16 scale d.
//   TQ1_0 (54 bytes): 32 bytes for elements 0..159 (byte j: elements j, 32 + j, ..., 128 + j as base-3 digits,
//          first element most significant), 16 bytes for elements 160..239 (byte j: 160 + j, 176 + j, ...),
//          4 bytes for elements 240..255 (byte j: 240 + j, 244 + j, 248 + j, 252 + j, then a zero digit), each
//          value v in 0..242 stored as ceil(v * 256 / 243); then the fp16 scale d.
// A weight's value is d * (q - 1).  Rows are padded with zero trits to a whole number of blocks.
//
// In the limb layout a row is a flat stream of tryte bytes, byte = t0 + 3 t1 + 9 t2 + 13: element e of a row sits
// in byte e / 3 as digit e % 3, whatever the limb boundaries (48 trits = 16 bytes).
#include "common.cuh"

namespace t81b200 {

namespace {

constexpr int kBlock = 256;

__host__ __device__ constexpr int block_bytes(int format) { return format == T81B200_TQ2_0 ? 66 : 54; }

// One CTA per (block, row): 256 threads decode the block's 256 digits into shared memory, then pack them.
__global__ void __launch_bounds__(kBlock) packed_to_tq_kernel(const uint8_t *__restrict__ packed, const float *__restrict__ row_scale,
                                                              int64_t cols, int64_t row_bytes, int format,
                                                              uint8_t *__restrict__ blocks, int64_t blocks_per_row) {
    __shared__ uint8_t q[kBlock];
    __shared__ int nonzero;
    const int64_t row = blockIdx.x, blk = blockIdx.y;
    const int i = threadIdx.x;
    if (i == 0) nonzero = 0;
    __syncthreads();
    const int64_t e = blk * kBlock + i;
    int digit = 1;  // zero trit
    if (e < cols) {
        int d0, d1, d2;
        tryte_digits(packed[row * row_bytes + e / 3], d0, d1, d2);
        const int m = (int)(e % 3);
        digit = m == 0 ? d0 : (m == 1 ? d1 : d2);
    }
    q[i] = (uint8_t)digit;
    if (digit != 1) nonzero = 1;  // benign race: every writer stores 1
    __syncthreads();
    uint8_t *out = blocks + (row * blocks_per_row + blk) * block_bytes(format);
    if (format == T81B200_TQ2_0) {
        if (i < 64) {
            const int half = i >> 5, j = i & 31;
            const uint8_t *h = q + half * 128;
            out[i] = (uint8_t)(h[j] | (h[32 + j] << 2) | (h[64 + j] << 4) | (h[96 + j] << 6));
        }
    } else {
        if (i < 52) {
            int v;
            if (i < 32) v = ((((q[i] * 3 + q[32 + i]) * 3 + q[64 + i]) * 3 + q[96 + i]) * 3 + q[128 + i]);
            else if (i < 48) { const int j = i - 32; v = ((((q[160 + j] * 3 + q[176 + j]) * 3 + q[192 + j]) * 3 + q[208 + j]) * 3 + q[224 + j]); }
            else { const int j = i - 48; v = (((q[240 + j] * 3 + q[244 + j]) * 3 + q[248 + j]) * 3 + q[252 + j]) * 3; }
            out[i] = (uint8_t)((v * 256 + 242) / 243);
        }
    }
    if (i >= kBlock - 2) {
        // the scale of a block with no non-zero trit is 0, like the absmax of an all-zero block; the last two
        // threads store its fp16 bits, low byte first
        const float d = nonzero ? (row_scale ? row_scale[row] : 1.0f) : 0.0f;
        const unsigned int bits = __half_as_ushort(__float2half_rn(d));
        const int which = i - (kBlock - 2);
        out[block_bytes(format) - 2 + which] = (uint8_t)((bits >> (8 * which)) & 0xFFu);
    }
}

// Digit q (0, 1, 2; 3 reads as 2) of element i of a block.
__device__ __forceinline__ int tq_digit(const uint8_t *blk, int i, int format) {
    if (format == T81B200_TQ2_0) {
        const int half = i >> 7, r = i & 127;
        const int q = (blk[half * 32 + (r & 31)] >> (2 * (r >> 5))) & 3;
        return q > 2 ? 2 : q;
    }
    int byte, m;
    if (i < 160) { byte = blk[i & 31]; m = i >> 5; }
    else if (i < 240) { byte = blk[32 + ((i - 160) & 15)]; m = (i - 160) >> 4; }
    else { byte = blk[48 + ((i - 240) & 3)]; m = (i - 240) >> 2; }
    // the multiply wraps to 8 bits on purpose: it shifts digit m to the top (t81/gguf.py:629-637)
    const int pow3[5] = {1, 3, 9, 27, 81};
    const int shifted = (byte * pow3[m]) & 0xFF;
    return (shifted * 3) >> 8;
}

// One thread per tryte byte of the packed row (three consecutive elements, possibly from two blocks).
__global__ void __launch_bounds__(256) tq_to_packed_kernel(const uint8_t *__restrict__ blocks, int64_t cols, int64_t row_bytes,
                                                           int format, uint8_t *__restrict__ packed,
                                                           float *__restrict__ block_scale, int64_t blocks_per_row) {
    const int64_t row = blockIdx.x;
    const int64_t n = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;  // tryte index in the row
    const int bb = block_bytes(format);
    const uint8_t *rblocks = blocks + row * blocks_per_row * bb;
    if (n < row_bytes) {
        int v = 13;
        int w = 1;
        for (int m = 0; m < 3; ++m, w *= 3) {
            const int64_t e = 3 * n + m;
            if (e < cols) v += (tq_digit(rblocks + (e / kBlock) * bb, (int)(e % kBlock), format) - 1) * w;
        }
        packed[row * row_bytes + n] = (uint8_t)v;
    }
    if (block_scale && n < blocks_per_row) {
        const uint8_t *b = rblocks + n * bb + bb - 2;
        const uint16_t bits = (uint16_t)(b[0] | (b[1] << 8));
        block_scale[row * blocks_per_row + n] = __half2float(__ushort_as_half(bits));
    }
}

}  // namespace
}  // namespace t81b200

using namespace t81b200;

extern "C" int64_t t81b200_tq_bytes(int format, int64_t rows, int64_t cols) {
    if ((format != T81B200_TQ1_0 && format != T81B200_TQ2_0) || rows < 0 || cols < 0) return -1;
    return rows * ((cols + kBlock - 1) / kBlock) * block_bytes(format);
}

extern "C" int t81b200_packed_to_tq(const uint8_t *packed, const float *row_scale, int64_t rows, int64_t cols, int format,
                                    uint8_t *blocks, void *stream) {
    if (format != T81B200_TQ1_0 && format != T81B200_TQ2_0) return fail(T81B200_EINVAL, "tq: unknown block format %d", format);
    if (rows < 0 || cols < 0) return fail(T81B200_EINVAL, "tq: negative dimension");
    if (int rc = check_device()) return rc;
    if (rows == 0 || cols == 0) return T81B200_OK;
    if (!packed || !blocks) return fail(T81B200_EINVAL, "tq: null pointer");
    const int64_t bpr = (cols + kBlock - 1) / kBlock, row_bytes = (cols + 47) / 48 * 16;
    if (bpr > 65535 || rows >= (1ll << 31)) return fail(T81B200_ELIMIT, "tq: matrix too large for one call");
    packed_to_tq_kernel<<<dim3((unsigned)rows, (unsigned)bpr), kBlock, 0, static_cast<cudaStream_t>(stream)>>>(
        packed, row_scale, cols, row_bytes, format, blocks, bpr);
    T81_LAUNCH_CHECK("packed_to_tq_kernel");
    return T81B200_OK;
}

extern "C" int t81b200_tq_to_packed(const uint8_t *blocks, int64_t rows, int64_t cols, int format, uint8_t *packed,
                                    float *block_scale, void *stream) {
    if (format != T81B200_TQ1_0 && format != T81B200_TQ2_0) return fail(T81B200_EINVAL, "tq: unknown block format %d", format);
    if (rows < 0 || cols < 0) return fail(T81B200_EINVAL, "tq: negative dimension");
    if (int rc = check_device()) return rc;
    if (rows == 0 || cols == 0) return T81B200_OK;
    if (!packed || !blocks) return fail(T81B200_EINVAL, "tq: null pointer");
    const int64_t bpr = (cols + kBlock - 1) / kBlock, row_bytes = (cols + 47) / 48 * 16;
    if (bpr > 65535 || rows >= (1ll << 31)) return fail(T81B200_ELIMIT, "tq: matrix too large for one call");
    const int64_t work = row_bytes > bpr ? row_bytes : bpr;
    tq_to_packed_kernel<<<dim3((unsigned)rows, (unsigned)((work + 255) / 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        blocks, cols, row_bytes, format, packed, block_scale, bpr);
    T81_LAUNCH_CHECK("tq_to_packed_kernel");
    return T81B200_OK;
}
