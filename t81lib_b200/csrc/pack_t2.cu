// Packed limbs -> the decode-stream layout ("T2") that the streaming matmul kernel reads: two bits per trit, in
// the order of the mma.sync m16n8k16 A fragments, cut into blocks of 32 rows x 192 columns.  Made once per weight
// matrix; the trits are not changed, only re-arranged (the reference keeps a packed copy per module in the same
// way, t81/nn/linear.py:84-99).
//
//   block (chunk c = column / 192, row tile T = row / 32) at byte (c * tiles32 + T) * 1536, tiles32 = ceil(rows / 32);
//   inside it lane l = 4 g + t owns the twelve 32-bit words at l * 48; word 6 gr + m / 2 (gr = 0, 1; m = 0..11)
//   holds eight registers of two trits: register r = 0..3 of multiply m at j = 4 (m % 2) + r, its first trit's code in
//   bits 15 - 2j, 14 - 2j, its second trit's code in bits 31 - 2j, 30 - 2j;
//   register r, trit h  <->  row 32 T + 16 gr + g + 8 (r % 2),  column 192 c + 48 t + 4 m + 2 (r / 2) + h;
//   code 01 = +1, 11 = -1, 00 = 0; rows and columns past the matrix are 0.
#include "common.cuh"

namespace t81b200 {

namespace {

// One thread per output word; its 16 trits come from 16 different tryte bytes (two rows x eight columns), read
// through L1: the kernel runs once per matrix and is bound by the scattered reads, not by HBM.
__global__ void __launch_bounds__(256) pack_t2_kernel(const uint8_t *__restrict__ packed, int64_t rows, int64_t cols, int64_t row_bytes,
                                                      int64_t tiles32, int64_t total_words, uint32_t *__restrict__ out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_words; i += stride) {
        const int wi = (int)(i % 12);
        const int lane = (int)((i / 12) % 32);
        const int64_t block = i / (12 * 32);
        const int64_t T = block % tiles32, c = block / tiles32;
        const int g = lane >> 2, t = lane & 3, gr = wi / 6, mpair = wi % 6;
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = 2 * mpair + (j >> 2), r = j & 3;
            const int64_t row = 32 * T + 16 * gr + g + 8 * (r & 1);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t col = 192 * c + 48 * t + 4 * m + 2 * (r >> 1) + h;
                uint32_t code = 0;
                if (row < rows && col < cols) {
                    int d0, d1, d2;
                    tryte_digits(packed[row * row_bytes + col / 3], d0, d1, d2);
                    const int which = (int)(col % 3);
                    const int d = which == 0 ? d0 : (which == 1 ? d1 : d2);  // trit + 1
                    code = d == 2 ? 1u : (d == 0 ? 3u : 0u);
                }
                word |= code << ((h ? 30 : 14) - 2 * j);
            }
        }
        out[i] = word;
    }
}

}  // namespace
}  // namespace t81b200

using namespace t81b200;

extern "C" int64_t t81b200_t2_bytes(int64_t rows, int64_t cols) {
    if (rows < 0 || cols < 0) return -1;
    return ((rows + 31) / 32) * ((cols + 191) / 192) * 1536;
}

extern "C" int t81b200_pack_t2(const uint8_t *packed, int64_t rows, int64_t cols, uint8_t *t2, void *stream) {
    if (rows < 0 || cols < 0) return fail(T81B200_EINVAL, "pack_t2: rows and cols must be non-negative");
    if (int rc = check_device()) return rc;
    if (rows == 0 || cols == 0) return T81B200_OK;
    if (!packed || !t2) return fail(T81B200_EINVAL, "pack_t2: null pointer");
    if (reinterpret_cast<uintptr_t>(t2) % 16 != 0) return fail(T81B200_EALIGN, "pack_t2: the output must be 16-byte aligned");
    const int64_t tiles32 = (rows + 31) / 32, chunks = (cols + 191) / 192, words = tiles32 * chunks * 384;
    int64_t blocks = (words + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    blocks = blocks > cap ? cap : blocks;
    pack_t2_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(packed, rows, cols, (cols + 47) / 48 * 16, tiles32, words,
                                                                                   reinterpret_cast<uint32_t *>(t2));
    T81_LAUNCH_CHECK("pack_t2_kernel");
    return T81B200_OK;
}
