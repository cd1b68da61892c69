// Decode-shaped TRIT-mode kernel, table-decode form: packed ternary weights (M rows) times up to 16
// activation rows (tokens), HBM-bound by design.
//
// Pipeline of one CTA (up to 16 consumer warps + 1 producer warp):
//   * the producer thread streams the CTA's weight rows through a shared-memory ring with TMA
//     (stages of 32*RW rows x 64 bytes = one 4-limb chunk per row); nothing in that stream depends
//     on the previous kernel of the stream, so it starts before the programmatic-dependent-launch wait;
//   * the activations arrive by bulk copies (cp.async.bulk, one per token and piece of the contraction range, no
//     per-thread round trips) after that wait, in their natural order, each piece behind its own barrier so
//     that the first chunks are multiplied while the rest is still on its way from L2;
//   * consumer warp (rw, kw) takes chunks kw, kw + KW, ... of rows 32*rw .. 32*rw+31: lane (g, t) reads
//     limb t of rows g, g+8, g+16, g+24 with 128-bit shared loads and expands every tryte byte with ONE
//     shared-memory table look-up into exact bf16 {-1,0,+1}: the byte is dropped into bits 8..15 of the
//     look-up address by a single PRMT; the table holds, per byte value, a copy for each of 16 lanes
//     (256 bytes per value), so the 64-bit loads of a warp never meet on a bank whatever the bytes are.
//     Two tables (bytes at even / odd positions) place the three trits so that one OR per byte pair
//     gives registers holding adjacent trits: the A fragments of mma.sync m16n8k16 in natural
//     contraction order, which is why the activations need no re-ordering.  The same activation
//     fragments serve both 16-row groups of the warp.
//   * fp32 accumulation in registers; the K-slices of a CTA meet in shared memory, the K-slices of a
//     cluster (shapes with few rows) through distributed shared memory in rank order: deterministic,
//     no global scratch, no atomics.  Row scales and biases are fetched into shared memory at the start.
//
// Up to three weight matrices that share their activations (q/k/v, gate/up) can be served by one launch:
// row tiles are numbered through the segments.
//
// Bytes above 26 are not valid trytes (the packer never writes them; limb::from_bytes of the reference
// rejects them, include/t81/core/limb.hpp:160-169).  Every weight word is masked to five bits per byte before
// it is used as a table index and the table has 32 entries per position, the last five all zero: bytes 27..31
// decode as the zero tryte and larger ones as some valid tryte; no look-up can leave the table.
//
// Second weight format, FMT == 1 ("T2", the decode-stream layout made once per weight matrix by t81b200_pack_t2):
// two bits per trit, already in the order the mma.sync A fragments want them.  The matrix is cut into blocks of
// 32 rows x 192 columns (one warp's rows, one chunk); block (chunk c, row tile T) lies at byte
// (c * tiles32 + T) * 1536 and holds, for lane l = 4 g + t, twelve 32-bit words at l * 48: word 6 gr + m / 2 serves
// the 16-row group gr and the multiply m = 0..11 of the chunk; register r = 0..3 of that multiply sits at
// j = 4 (m % 2) + r: its low-half code in bits 15-2j, 14-2j and its high-half code in bits 31-2j, 30-2j, where
//   register r, half h  <->  row 32 T + 16 gr + g + 8 (r % 2),  column 192 c + 48 t + 4 m + 2 (r / 2) + h,
// and a code is 01 for +1, 11 for -1, 00 for 0: shifted to the top of a 16-bit half it IS the bf16 number
// +2, -2 or 0.  Decoding a register is one shift and one AND — no table, no shared-memory traffic beyond the
// 48 bytes per lane and chunk — and the factor 2 is taken out with alpha.  A stage of the ring (all RW row
// tiles of a chunk) is contiguous in memory: one bulk copy, no tensor map.  A quarter fewer bytes than the
// limb layout cross HBM.
#include "common.cuh"
#include "tma.cuh"
#include "exchange.cuh"

#include <cooperative_groups.h>

#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace cg = cooperative_groups;

namespace t81b200 {

namespace {

constexpr int kMaxSeg = T81B200_MAX_GROUP;
constexpr int kMaxConsumerWarps = 16;
constexpr int kThreads = (kMaxConsumerWarps + 1) * 32;
constexpr int kMaxStages = 48;
constexpr int kXPieces = 4;       // barriers the activations arrive behind
// The tables sit at this absolute shared-memory address: its bits 8..15 are zero, so a look-up address is
// this constant with the byte value dropped into byte 1 and the lane offset into byte 0.
constexpr uint32_t kLutAbs = 0x10000u;
constexpr int kLutBytes = 32 * 256;
// Dynamic shared memory starts a little above address 0; [kWindowLo, kWindowHi) of the dynamic allocation is
// kept free for the tables for any start below kMaxBase.
constexpr uint32_t kMaxBase = 4096u;
constexpr int kWindowLo = (int)(kLutAbs - kMaxBase);          // 61440
constexpr int kWindowHi = (int)kLutAbs + kLutBytes + 256;     // 73984
constexpr int kSmemBudget = 224 * 1024;

enum { LUT_STATUS_OK = 0, LUT_STATUS_TIMEOUT_PRODUCER = 5, LUT_STATUS_TIMEOUT_CONSUMER = 6, LUT_STATUS_TIMEOUT_EXCHANGE = 7,
       LUT_STATUS_LAYOUT = 8 };
__device__ int g_lut_status = 0;

#ifdef T81B200_GEMV_TRACE
// Instrumented build only (never the shipped library): %globaltimer stamps of up to kTraceCtas CTAs of the last
// kTraceLaunches launches, read back through t81b200_debug_trace.
constexpr int kTraceLaunches = 64, kTraceCtas = 512, kTraceStamps = 8;
__device__ unsigned long long g_trace[kTraceLaunches * kTraceCtas * kTraceStamps];
__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRACE_STAMP(i)                                                                                         \
    do {                                                                                                       \
        const int cta__ = blockIdx.y * gridDim.x + blockIdx.x;                                                 \
        if (threadIdx.x == 0 && cta__ < kTraceCtas)                                                            \
            g_trace[((size_t)(p.trace_slot % kTraceLaunches) * kTraceCtas + cta__) * kTraceStamps + (i)] = globaltimer(); \
    } while (0)
#else
#define TRACE_STAMP(i) do {} while (0)
#endif

struct LutSeg {
    const float *row_scale;  // M or null
    const float *bias;       // M or null
    void *C;                 // (ntok, M) row-major, ldc elements
    int64_t M;
    int tile_begin;          // first row tile (blockIdx.x) of this segment
    const uint8_t *t2;       // FMT 1: the matrix in the decode-stream layout
    int tiles32;             // FMT 1: 32-row tiles of the matrix
};

struct GemvLutParams {
    LutSeg seg[kMaxSeg];
    int n_seg;
    const void *X;           // (ntok, K) row-major, ldx elements
    int64_t K, kl, ldx, ldc;
    int ntok;
    float alpha, beta;
    int row_warps;           // RW: 32-row groups side by side in a CTA
    int k_warps;             // KW: slices of the CTA's contraction range
    int limbs_per_slice;     // limbs per CTA of a cluster, multiple of 4
    int stages, stage_bytes;
    int ring0_stages;        // ring slots [0, ring0_stages) lie at offset 0, the others at ring1_offset
    int ring1_offset, xs_offset, part_offset, sb_offset, bar_offset;
    int bulk_x;              // 1: bf16 activations, 16-byte aligned rows, K % 8 == 0: fetched by bulk copies
    int independent;         // 1: reads nothing the previous kernel of the stream wrote
    int n_peers;             // other GPUs whose result receives every output element too (one segment only)
    void *peer_C[T81B200_MAX_PEERS];
    uint32_t *sync_local;
    uint32_t *sync_peer[T81B200_MAX_PEERS];
    int trace_slot;          // instrumented builds: which trace record this launch writes
    uint32_t shl[8];         // FMT 1: 4^j.  Multiplying by a launch-time constant instead of shifting by a literal puts
                             // the shifts of the decode on the multiply-add pipe, beside the masks on the logic pipe
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16_pair(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

template <typename CT> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) { return pack_bf16_pair(lo, hi); }
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t pack_pair<float>(float lo, float) { return __float_as_uint(lo); }  // unused

// The decode tables as they lie in shared memory: [byte value 0..31][even / odd position][16 lane copies] of
// 64-bit entries, 8 KB, built at compile time and copied into every CTA by one bulk copy.
//   even position: {(t0, t1), (t2, 0)}     odd position: {(0, t0), (t1, t2)}      bf16 pairs, low half first
// Values 27..31 are not trytes: their entries are zero.
struct LutImage {
    uint32_t w[32 * 2 * 16 * 2];
};
constexpr uint32_t trit_bits(int d) { return d == 0 ? 0xBF80u : (d == 2 ? 0x3F80u : 0u); }  // digit d = trit + 1
constexpr LutImage make_lut_image() {
    LutImage im{};
    for (int b = 0; b < 32; ++b) {
        const uint32_t t0 = b < 27 ? trit_bits(b % 3) : 0u, t1 = b < 27 ? trit_bits((b / 3) % 3) : 0u, t2 = b < 27 ? trit_bits(b / 9) : 0u;
        for (int l = 0; l < 16; ++l) {
            im.w[((b * 2 + 0) * 16 + l) * 2 + 0] = t0 | (t1 << 16);
            im.w[((b * 2 + 0) * 16 + l) * 2 + 1] = t2;
            im.w[((b * 2 + 1) * 16 + l) * 2 + 0] = t0 << 16;
            im.w[((b * 2 + 1) * 16 + l) * 2 + 1] = t1 | (t2 << 16);
        }
    }
    return im;
}
__device__ __align__(128) const LutImage g_lut_image = make_lut_image();

// One 32-bit word of a limb (4 trytes = 12 trits) -> 6 registers of adjacent trit pairs.
// lane_key = the CTA's shared-memory window (top byte) | kLutAbs | (lane % 16) * 8.
__device__ __forceinline__ void lut_decode_word(uint32_t w, uint32_t lane_key, uint32_t (&o)[6]) {
    uint32_t a0, a1, a2, a3;
    asm("prmt.b32 %0, %1, %2, 0x7604;" : "=r"(a0) : "r"(w), "r"(lane_key));
    asm("prmt.b32 %0, %1, %2, 0x7614;" : "=r"(a1) : "r"(w), "r"(lane_key));
    asm("prmt.b32 %0, %1, %2, 0x7624;" : "=r"(a2) : "r"(w), "r"(lane_key));
    asm("prmt.b32 %0, %1, %2, 0x7634;" : "=r"(a3) : "r"(w), "r"(lane_key));
    uint32_t e0x, e0y, o0x, o0y, e1x, e1y, o1x, o1y;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e0x), "=r"(e0y) : "r"(a0));
    asm("ld.shared.v2.u32 {%0, %1}, [%2+128];" : "=r"(o0x), "=r"(o0y) : "r"(a1));
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(e1x), "=r"(e1y) : "r"(a2));
    asm("ld.shared.v2.u32 {%0, %1}, [%2+128];" : "=r"(o1x), "=r"(o1y) : "r"(a3));
    o[0] = e0x; o[1] = e0y | o0x; o[2] = o0y;
    o[3] = e1x; o[4] = e1y | o1x; o[5] = o1y;
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <typename XT> struct LutPlanes { static constexpr int value = 2; };
template <> struct LutPlanes<__nv_bfloat16> { static constexpr int value = 1; };

// Activations of the CTA's limbs [0, nl) (limb 0 = limb L0 of the row) for every token, element by element
// (fp32 / fp16 values, unaligned rows), in natural order, zero beyond K.  Plane 0 holds bf16(x); plane 1
// (PLANES == 2) holds bf16(x - plane 0), so that plane 0 + plane 1 carries 16 mantissa bits of an fp32 / fp16 input.
template <typename XT, int PLANES>
__device__ __forceinline__ void stage_elements(const GemvLutParams &p, int L0, int nl, uint32_t *xs, int tok_stride,
                                               int plane_stride, int tid, int nthreads) {
    const XT *X = static_cast<const XT *>(p.X);
    const int per_tok = nl * 24;
    for (int item = tid; item < p.ntok * per_tok; item += nthreads) {
        const int tok = item / per_tok, r = item - tok * per_tok;
        const int64_t k = (int64_t)L0 * 48 + 2 * r;
        const float e0 = k < p.K ? to_float<XT>(X[(int64_t)tok * p.ldx + k]) : 0.0f;
        const float e1 = k + 1 < p.K ? to_float<XT>(X[(int64_t)tok * p.ldx + k + 1]) : 0.0f;
        const uint32_t hi = pack_bf16_pair(e0, e1);
        uint32_t *dst = xs + tok * tok_stride + r;
        *dst = hi;
        if constexpr (PLANES == 2) {
            const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162 *>(&hi);
            dst[plane_stride] = pack_bf16_pair(e0 - __low2float(hv), e1 - __high2float(hv));
        }
    }
}

template <typename XT, typename CT, int TOKB, int FMT>
__global__ void __launch_bounds__(kThreads, 1)
gemv_trit_lut_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                     const __grid_constant__ CUtensorMap map2, const GemvLutParams p) {
    constexpr int PLANES = LutPlanes<XT>::value;
    constexpr int kTokPad = 8 * TOKB;
    extern __shared__ __align__(128) uint8_t smem[];
    TRACE_STAMP(0);
    // Shared-memory addresses of a CTA in a cluster carry the CTA's rank in their top byte (measured on sm_100a:
    // rank r sees its dynamic shared memory at r * 0x1000000 + 0x400); the low 24 bits are the offset in its window.
    const uint32_t base = smem_u32(smem);
    const uint32_t window = base & 0xFF000000u, base_off = base & 0x00FFFFFFu;
    // The table window was laid out for dynamic shared memory starting below kMaxBase.  Should it start higher,
    // the CTA still walks through every barrier (its cluster peers read its shared memory) but streams nothing,
    // and the launch reports LUT_STATUS_LAYOUT.
    const bool layout_ok = FMT == 1 || base_off < kMaxBase;  // the T2 format uses no table
    if (!layout_ok && threadIdx.x == 0) atomicCAS(&g_lut_status, LUT_STATUS_OK, LUT_STATUS_LAYOUT);
    uint8_t *lut = smem + (layout_ok ? kLutAbs - base_off : (uint32_t)kWindowLo);
    const int consumer_warps = p.row_warps * p.k_warps;
    const int consumer_threads = consumer_warps * 32;
    const int all_threads = consumer_threads + 32;
    uint32_t *xs = reinterpret_cast<uint32_t *>(smem + p.xs_offset);
    float *part = reinterpret_cast<float *>(smem + p.part_offset);
    float *sb = reinterpret_cast<float *>(smem + p.sb_offset);
    const uint32_t bars = smem_u32(smem + p.bar_offset);
    auto full_bar = [&](int st) { return bars + 8u * st; };
    auto empty_bar = [&](int st) { return bars + 8u * (p.stages + st); };
    const uint32_t x_bar = bars + 8u * (2 * p.stages);
    const uint32_t pro_bar = x_bar + 8u * kXPieces;  // decode tables, row scales and biases have landed
    auto ring_offset = [&](int st) { return st < p.ring0_stages ? st * p.stage_bytes : p.ring1_offset + (st - p.ring0_stages) * p.stage_bytes; };

    cg::cluster_group cluster = cg::this_cluster();
    const int slices = (int)cluster.num_blocks();
    const int slice = (int)cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    // which weight matrix this row tile belongs to
    int sg = 0;
    while (sg + 1 < p.n_seg && (int)blockIdx.x >= p.seg[sg + 1].tile_begin) ++sg;
    const LutSeg &S = p.seg[sg];
    const CUtensorMap *map_w = sg == 0 ? &map0 : (sg == 1 ? &map1 : &map2);
    const int rows_per_cta = p.row_warps * 32;
    const int prow = rows_per_cta + 4;  // row pitch of the partial sums, in floats
    const int64_t cta_row0 = (int64_t)((int)blockIdx.x - S.tile_begin) * rows_per_cta;

    const bool whole_tile = cta_row0 + rows_per_cta <= S.M;
    const bool scale_by_copy = layout_ok && S.row_scale && whole_tile && reinterpret_cast<uintptr_t>(S.row_scale) % 16 == 0;
    const bool bias_by_copy = layout_ok && S.bias && whole_tile && reinterpret_cast<uintptr_t>(S.bias) % 16 == 0;

    const int kl4 = (int)((p.kl + 3) & ~(int64_t)3);
    const int L0 = slice * p.limbs_per_slice;
    int nl = kl4 - L0;
    nl = nl < 0 ? 0 : (nl > p.limbs_per_slice ? p.limbs_per_slice : nl);
    const int chunks_cta = layout_ok ? nl >> 2 : 0;
    const int tok_stride = p.limbs_per_slice * 24 + 4;  // +16 bytes: conflict-free 128-bit reads across tokens
    const int plane_stride = p.ntok * tok_stride;

    // x arrives in up to kXPieces pieces of x_group chunks each, every piece behind its own barrier: the first
    // chunks can be multiplied while the rest of the activations is still on its way from L2
    const int x_group = (chunks_cta + kXPieces - 1) / kXPieces > 0 ? (chunks_cta + kXPieces - 1) / kXPieces : 1;
    if (threadIdx.x < p.stages) { mbar_init(full_bar(threadIdx.x), 1); mbar_init(empty_bar(threadIdx.x), p.row_warps); }
    if (threadIdx.x >= kMaxStages && threadIdx.x < kMaxStages + kXPieces) mbar_init(x_bar + 8u * (threadIdx.x - kMaxStages), 1);
    if (threadIdx.x == kMaxStages + kXPieces) mbar_init(pro_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    TRACE_STAMP(1);
    // Programmatic dependent launch: a kernel that depends on its predecessor lets its own successor start once
    // its input is complete (after its wait below); one that does not depend on it lets the successor start at
    // once and waits for the predecessor at its very end instead, so that "this grid has completed" still implies
    // "everything before it has".
    if (p.independent) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Activations by bulk copy (bf16, 16-byte aligned rows, K a multiple of 8): the copies bring exactly the
    // elements below K, one copy per token and piece; piece j holds the elements of chunks
    // [j * x_group, (j + 1) * x_group) that exist.  Issuing a copy costs its warp tens of nanoseconds, so the
    // consumer warps share them out (lane 0 of each), in piece order: no warp starts its chunks late.
    int64_t valid = p.K - (int64_t)L0 * 48;  // elements of this CTA's range that exist
    valid = valid < 0 ? 0 : (valid > (int64_t)nl * 48 ? (int64_t)nl * 48 : valid);
    auto x_piece = [&](int j, int &e0, int &e1) {
        const int64_t a = (int64_t)192 * x_group * j, b = (int64_t)192 * x_group * (j + 1);
        e0 = (int)(a < valid ? a : valid);
        e1 = (int)(b < valid ? b : valid);
    };
    auto expect_x = [&]() {  // one thread, before any copy is issued
        for (int j = 0; j < kXPieces; ++j) {
            int e0, e1;
            x_piece(j, e0, e1);
            if (e1 > e0) mbar_arrive_expect_tx(x_bar + 8u * j, (uint32_t)(e1 - e0) * 2u * (uint32_t)p.ntok);
            else mbar_arrive(x_bar + 8u * j);
        }
    };
    auto issue_x = [&](int who, int n_who) {  // copies who, who + n_who, ... in piece order
        const __nv_bfloat16 *X = static_cast<const __nv_bfloat16 *>(p.X);
        for (int i = who; i < kXPieces * p.ntok; i += n_who) {
            const int j = i / p.ntok, tok = i - j * p.ntok;
            int e0, e1;
            x_piece(j, e0, e1);
            if (e1 > e0)
                bulk_load(smem_u32(xs + tok * tok_stride + e0 / 2), X + (int64_t)tok * p.ldx + (int64_t)L0 * 48 + e0,
                          (uint32_t)(e1 - e0) * 2u, x_bar + 8u * j);
        }
    };

    constexpr int NACC = 2;
    float acc[2][NACC][TOKB][4];
#pragma unroll
    for (int gr = 0; gr < 2; ++gr)
#pragma unroll
        for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int b = 0; b < TOKB; ++b) acc[gr][a][b][0] = acc[gr][a][b][1] = acc[gr][a][b][2] = acc[gr][a][b][3] = 0.0f;
    int rw = 0, kw = 0;

    if (warp == consumer_warps) {
        // ---------------- producer: the weight stream ----------------
        if (lane == 0) {
            bool ok = true;
            auto load_weights = [&](int c) {
                const int st = c % p.stages;
                const uint32_t phase = (uint32_t)(c / p.stages) & 1u;
                if (!mbar_wait(empty_bar(st), phase ^ 1u)) return false;
                if constexpr (FMT == 1) {
                    // the chunk's blocks of this CTA's row tiles are contiguous; the matrix's last tiles may be fewer
                    const int tile0 = ((int)blockIdx.x - S.tile_begin) * p.row_warps;
                    const int ntile = S.tiles32 - tile0 < p.row_warps ? S.tiles32 - tile0 : p.row_warps;
                    mbar_arrive_expect_tx(full_bar(st), (uint32_t)ntile * 1536u);
                    bulk_load(base + (uint32_t)ring_offset(st), S.t2 + ((int64_t)(L0 / 4 + c) * S.tiles32 + tile0) * 1536,
                              (uint32_t)ntile * 1536u, full_bar(st));
                } else {
                    mbar_arrive_expect_tx(full_bar(st), (uint32_t)p.stage_bytes);
                    tma_load_2d(base + (uint32_t)ring_offset(st), map_w, (L0 + 4 * c) * 16, (int)cta_row0, full_bar(st));
                }
                return true;
            };
            // decode tables (a compile-time image in global memory), row scales and biases: bulk copies, none of
            // them the previous kernel's output.  Scales and biases that a copy cannot take (unaligned, or a tile
            // that reaches past the last row) are fetched by the consumer threads instead.
            if (layout_ok) {
                uint32_t bytes = FMT == 1 ? 0u : (uint32_t)kLutBytes;
                if (scale_by_copy) bytes += (uint32_t)rows_per_cta * 4u;
                if (bias_by_copy) bytes += (uint32_t)rows_per_cta * 4u;
                if (bytes) mbar_arrive_expect_tx(pro_bar, bytes);
                else mbar_arrive(pro_bar);
                if constexpr (FMT == 0) bulk_load(smem_u32(lut), &g_lut_image, (uint32_t)kLutBytes, pro_bar);
                if (scale_by_copy) bulk_load(smem_u32(sb), S.row_scale + cta_row0, (uint32_t)rows_per_cta * 4u, pro_bar);
                if (bias_by_copy) bulk_load(smem_u32(sb + rows_per_cta), S.bias + cta_row0, (uint32_t)rows_per_cta * 4u, pro_bar);
            }
            // the ring's first pass needs nothing but the weights: start it before the wait
            const int first = chunks_cta < p.stages ? chunks_cta : p.stages;
            for (int c = 0; c < first && ok; ++c) ok = load_weights(c);
            for (int c = first; c < chunks_cta && ok; ++c) ok = load_weights(c);
            if (!ok) atomicCAS(&g_lut_status, LUT_STATUS_OK, LUT_STATUS_TIMEOUT_PRODUCER);
        }
        if (!p.independent) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // before this warp's share of the output stores
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
    } else {
        // ---------------- consumers ----------------
        rw = warp % p.row_warps;
        kw = warp / p.row_warps;
        // row scales and biases the producer's bulk copies do not bring (see there); absent ones are 1 and 0
        if (!scale_by_copy)
            for (int r = threadIdx.x; r < rows_per_cta; r += consumer_threads)
                sb[r] = cta_row0 + r < S.M && S.row_scale ? S.row_scale[cta_row0 + r] : 1.0f;
        if (!bias_by_copy)
            for (int r = threadIdx.x; r < rows_per_cta; r += consumer_threads)
                sb[rows_per_cta + r] = cta_row0 + r < S.M && S.bias ? S.bias[cta_row0 + r] : 0.0f;
        // what lies between K and the end of the CTA's padded range is zero and is written now, before the wait
        if (p.bulk_x) {
            const int zero_words = nl * 24 - (int)(valid / 2);
            for (int item = threadIdx.x; item < p.ntok * zero_words; item += consumer_threads) {
                const int tok = item / zero_words;
                xs[tok * tok_stride + (int)(valid / 2) + (item - tok * zero_words)] = 0u;
            }
        }
        if (p.bulk_x && threadIdx.x == 0) expect_x();
        asm volatile("bar.sync 1, %0;" ::"r"(consumer_threads) : "memory");  // thread-written scales, zero padding, expected bytes
        if (!p.independent) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations may be the previous kernel's output
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
        TRACE_STAMP(2);
        if (p.sync_local) {
            // ... or what the peers stored into this GPU's memory: wait until all of them have published
            if (threadIdx.x == 0 && !exchange_wait(p.sync_local, p.n_peers))
                atomicCAS(&g_lut_status, LUT_STATUS_OK, LUT_STATUS_TIMEOUT_EXCHANGE);
            asm volatile("bar.sync 1, %0;" ::"r"(consumer_threads) : "memory");
        }
        bool ok = true;
        if (p.bulk_x) {
            issue_x(warp + lane * consumer_warps, 32 * consumer_warps);  // one copy per lane at most: one instruction per warp
        } else {
            stage_elements<XT, PLANES>(p, L0, nl, xs, tok_stride, plane_stride, threadIdx.x, consumer_threads);
            asm volatile("bar.sync 1, %0;" ::"r"(consumer_threads) : "memory");
        }
        TRACE_STAMP(3);

        int tok_off[TOKB];
#pragma unroll
        for (int b = 0; b < TOKB; ++b) tok_off[b] = (8 * b + g < p.ntok ? 8 * b + g : 0) * tok_stride + t * 24;
        const uint32_t lane_off = (uint32_t)((rw * 32 + g) * 64 + t * 16);
        const uint32_t lane_key = window | kLutAbs | (uint32_t)((lane & 15) << 3);
        if (layout_ok) ok = __all_sync(0xffffffffu, mbar_wait(pro_bar, 0));
        // ring slot, its phase and the activation piece of chunk c, carried along instead of divided out
        // (the ring has at least k_warps slots)
        int st = kw % p.stages, xg = 0, xc = kw;
        uint32_t phase = (uint32_t)(kw / p.stages) & 1u;
        for (int c = kw; c < chunks_cta && ok; c += p.k_warps, st += p.k_warps, xc += p.k_warps) {
            if (st >= p.stages) { st -= p.stages; phase ^= 1u; }
            while (xc >= x_group) { xc -= x_group; ++xg; }
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(st), phase) && (!p.bulk_x || mbar_wait(x_bar + 8u * xg, 0)));
            if (!ok) break;
            if constexpr (FMT == 1) {
                const uint8_t *tile = smem + ring_offset(st) + rw * 1536 + lane * 48;
                uint32_t wd[12];
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const uint4 q = *reinterpret_cast<const uint4 *>(tile + 16 * j);
                    wd[4 * j] = q.x; wd[4 * j + 1] = q.y; wd[4 * j + 2] = q.z; wd[4 * j + 3] = q.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(st));  // the codes are in registers: the slot can be refilled
                uint4 xr[TOKB][PLANES][6];
#pragma unroll
                for (int b = 0; b < TOKB; ++b)
#pragma unroll
                    for (int pl = 0; pl < PLANES; ++pl) {
                        const uint4 *xv = reinterpret_cast<const uint4 *>(xs + pl * plane_stride + tok_off[b] + c * 96);
#pragma unroll
                        for (int q = 0; q < 6; ++q) xr[b][pl][q] = xv[q];
                    }
#pragma unroll
                for (int m = 0; m < 12; ++m) {
#pragma unroll
                    for (int gr = 0; gr < 2; ++gr) {
                        const uint32_t w = wd[6 * gr + (m >> 1)];
                        const int j0 = 4 * (m & 1);
                        const uint32_t a0 = (j0 ? w * p.shl[j0] : w) & 0xC000C000u, a1 = (w * p.shl[j0 + 1]) & 0xC000C000u;
                        const uint32_t a2 = (w * p.shl[j0 + 2]) & 0xC000C000u, a3 = (w * p.shl[j0 + 3]) & 0xC000C000u;
#pragma unroll
                        for (int b = 0; b < TOKB; ++b)
#pragma unroll
                            for (int pl = 0; pl < PLANES; ++pl) {
                                const uint32_t *xw = reinterpret_cast<const uint32_t *>(&xr[b][pl][0]) + 2 * m;
                                mma_bf16_16816(acc[gr][m % NACC][b], a0, a1, a2, a3, xw[0], xw[1]);
                            }
                    }
                }
                continue;
            }
            const uint8_t *tile = smem + ring_offset(st) + lane_off;
            uint4 limb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // rows g + 8j; five bits per byte: no table index can leave the table
                limb[j] = *reinterpret_cast<const uint4 *>(tile + j * 8 * 64);
                limb[j].x &= 0x1F1F1F1Fu; limb[j].y &= 0x1F1F1F1Fu; limb[j].z &= 0x1F1F1F1Fu; limb[j].w &= 0x1F1F1F1Fu;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(st));  // the limbs are in registers: the slot can be refilled
            uint4 xr[TOKB][PLANES][6];
#pragma unroll
            for (int b = 0; b < TOKB; ++b)
#pragma unroll
                for (int pl = 0; pl < PLANES; ++pl) {
                    const uint4 *xv = reinterpret_cast<const uint4 *>(xs + pl * plane_stride + tok_off[b] + c * 96);
#pragma unroll
                    for (int q = 0; q < 6; ++q) xr[b][pl][q] = xv[q];
                }
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
                for (int gr = 0; gr < 2; ++gr) {
                    const uint4 &la = limb[2 * gr], &lb = limb[2 * gr + 1];
                    const uint32_t wa = w == 0 ? la.x : (w == 1 ? la.y : (w == 2 ? la.z : la.w));
                    const uint32_t wb = w == 0 ? lb.x : (w == 1 ? lb.y : (w == 2 ? lb.z : lb.w));
                    uint32_t oa[6], ob[6];
                    lut_decode_word(wa, lane_key, oa);
                    lut_decode_word(wb, lane_key, ob);
#pragma unroll
                    for (int b = 0; b < TOKB; ++b)
#pragma unroll
                        for (int pl = 0; pl < PLANES; ++pl) {
                            // registers 6w .. 6w+5 of the limb <-> activation registers 6w .. 6w+5
                            const uint32_t *xw = reinterpret_cast<const uint32_t *>(&xr[b][pl][0]) + 6 * w;
                            mma_bf16_16816(acc[gr][(3 * w) % NACC][b], oa[0], ob[0], oa[1], ob[1], xw[0], xw[1]);
                            mma_bf16_16816(acc[gr][(3 * w + 1) % NACC][b], oa[2], ob[2], oa[3], ob[3], xw[2], xw[3]);
                            mma_bf16_16816(acc[gr][(3 * w + 2) % NACC][b], oa[4], ob[4], oa[5], ob[5], xw[4], xw[5]);
                        }
                }
            }
        }
        if (!ok && lane == 0) atomicCAS(&g_lut_status, LUT_STATUS_OK, LUT_STATUS_TIMEOUT_CONSUMER);
        TRACE_STAMP(4);

        // acc[..][b][0]: (row g, token 8b+2t), [1]: (row g, 8b+2t+1), [2]: (row g+8, 8b+2t), [3]: (row g+8, 8b+2t+1)
        // partials are kept token-major, part[kw][token][row] with rows padded by 4: the eight rows a finishing
        // thread reads are contiguous, and the four tokens a quad writes fall on different banks
        float *pw = part + (size_t)kw * kTokPad * prow;
#pragma unroll
        for (int gr = 0; gr < 2; ++gr) {
            const int lr = rw * 32 + gr * 16 + g;
#pragma unroll
            for (int b = 0; b < TOKB; ++b) {
                float r[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) r[i] = acc[gr][0][b][i] + acc[gr][1][b][i];
                pw[(8 * b + 2 * t) * prow + lr] = r[0];
                pw[(8 * b + 2 * t + 1) * prow + lr] = r[1];
                pw[(8 * b + 2 * t) * prow + lr + 8] = r[2];
                pw[(8 * b + 2 * t + 1) * prow + lr + 8] = r[3];
            }
        }
    }
    __syncthreads();
    TRACE_STAMP(5);

    // Fold the K-slices' partials in a fixed order (deterministic), then, with more than one CTA per cluster, the
    // ranks' partials through distributed shared memory (also in a fixed order).  A finishing thread owns eight consecutive rows of one
    // token: two 128-bit reads per partial, one 128-bit (16-bit outputs) or two (fp32) stores.
    const int plane = kTokPad * prow;        // floats per K-slice
    const int blocks_per_tok = rows_per_cta / 8;
    bool vec_store = p.beta == 0.0f && reinterpret_cast<uintptr_t>(S.C) % 16 == 0 && (p.ldc * (int64_t)sizeof(CT)) % 16 == 0;
    for (int pj = 0; pj < p.n_peers; ++pj) vec_store = vec_store && reinterpret_cast<uintptr_t>(p.peer_C[pj]) % 16 == 0;
    auto finish = [&](int tok, int r0, const float (&v)[8]) {  // rows r0 .. r0+7 of the tile, one token
        if (tok >= p.ntok) return;
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = v[i] * p.alpha * sb[r0 + i] + sb[rows_per_cta + r0 + i];  // FMT 1: alpha arrives halved
        const int64_t row = cta_row0 + r0;
        CT *c = static_cast<CT *>(S.C) + (int64_t)tok * p.ldc + row;
        if (vec_store && row + 8 <= S.M) {
            // the same 128-bit stores go into every peer's result (column-sharded Linear), over NVLink
            const int64_t off = (int64_t)tok * p.ldc + row;
            if constexpr (sizeof(CT) == 4) {
                const float4 lo4 = make_float4(y[0], y[1], y[2], y[3]), hi4 = make_float4(y[4], y[5], y[6], y[7]);
                reinterpret_cast<float4 *>(c)[0] = lo4;
                reinterpret_cast<float4 *>(c)[1] = hi4;
                for (int pj = 0; pj < p.n_peers; ++pj) {
                    float4 *pc = reinterpret_cast<float4 *>(static_cast<CT *>(p.peer_C[pj]) + off);
                    pc[0] = lo4; pc[1] = hi4;
                }
            } else {
                const uint4 v16 = make_uint4(pack_pair<CT>(y[0], y[1]), pack_pair<CT>(y[2], y[3]),
                                             pack_pair<CT>(y[4], y[5]), pack_pair<CT>(y[6], y[7]));
                *reinterpret_cast<uint4 *>(c) = v16;
                for (int pj = 0; pj < p.n_peers; ++pj) *reinterpret_cast<uint4 *>(static_cast<CT *>(p.peer_C[pj]) + off) = v16;
            }
            return;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (row + i >= S.M) continue;
            float out = y[i];
            if (p.beta != 0.0f) out += p.beta * to_float<CT>(c[i]);
            const CT o = from_float<CT>(out);
            c[i] = o;
            for (int pj = 0; pj < p.n_peers; ++pj) static_cast<CT *>(p.peer_C[pj])[(int64_t)tok * p.ldc + row + i] = o;
        }
    };
    if (slices == 1) {
        for (int item = threadIdx.x; item < kTokPad * blocks_per_tok; item += all_threads) {
            const int tok = item / blocks_per_tok, r0 = (item - tok * blocks_per_tok) * 8;
            float v[8];
            const float4 *src = reinterpret_cast<const float4 *>(part + tok * prow + r0);
            float4 lo = src[0], hi = src[1];
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
            for (int w = 1; w < p.k_warps; ++w) {
                src = reinterpret_cast<const float4 *>(part + (size_t)w * plane + tok * prow + r0);
                lo = src[0]; hi = src[1];
                v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w; v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
            }
            finish(tok, r0, v);
        }
    } else {
        // Push: every CTA sums its K-slices and writes each block of rows into the receive buffer of the CTA that
        // finishes those rows (slot = the sender's rank), one cluster barrier orders the writes before the reads,
        // and the finisher adds the slots in rank order.  After the barrier no CTA touches another's memory, so
        // none has to outlive the others.
        const int span = rows_per_cta / slices;  // a multiple of 8: 32*RW rows; 2, 4 or (RW even) 8 slices
        const int spitch = span + 4;
        const int slot = kTokPad * spitch;       // floats per sender
        float *recv = part + (size_t)p.k_warps * plane;
        for (int item = threadIdx.x; item < kTokPad * blocks_per_tok; item += all_threads) {
            const int tok = item / blocks_per_tok, r0 = (item - tok * blocks_per_tok) * 8;
            const float4 *src = reinterpret_cast<const float4 *>(part + tok * prow + r0);
            float4 lo = src[0], hi = src[1];
            for (int w = 1; w < p.k_warps; ++w) {
                src = reinterpret_cast<const float4 *>(part + (size_t)w * plane + tok * prow + r0);
                const float4 a = src[0], b = src[1];
                lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w; hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
            }
            const int dst = r0 / span;
            float4 *out = reinterpret_cast<float4 *>(cluster.map_shared_rank(recv, dst) + (size_t)slice * slot + tok * spitch + (r0 - dst * span));
            out[0] = lo;
            out[1] = hi;
        }
        cluster.sync();
        const int span_blocks = span / 8;
        for (int item = threadIdx.x; item < kTokPad * span_blocks; item += all_threads) {
            const int tok = item / span_blocks, r0 = (item - tok * span_blocks) * 8;
            float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            for (int rk = 0; rk < slices; ++rk) {
                const float4 *src = reinterpret_cast<const float4 *>(recv + (size_t)rk * slot + tok * spitch + r0);
                const float4 lo = src[0], hi = src[1];
                v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w; v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
            }
            finish(tok, slice * span + r0, v);
        }
    }
    TRACE_STAMP(6);
    if (p.independent) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (p.sync_local) {
        // one system fence per CTA, by the signalling thread after the barrier: the barrier orders the CTA's stores before it
        __syncthreads();
        if (threadIdx.x == 0) exchange_signal(p.sync_local, p.sync_peer, p.n_peers, gridDim.x * gridDim.y);
    }
}

// ---------------------------------------------------------------------------------------------------------- host

// Debugging switches, read once per process:
//   T81B200_GEMV_CFG="row_warps,k_warps,slices"  forces the launch shape (sweeps)
//   T81B200_NO_PDL=1                              launches without programmatic dependent launch
//   T81B200_GEMV_CFG_LIVE=1                       re-reads T81B200_GEMV_CFG on every call and plans afresh (sweeps
//                                                 that try many shapes in one process)
struct Switches {
    int rw = 0, kw = 0, s = 0;
    bool pdl = true, live = false;
    void read_cfg() {
        rw = kw = s = 0;
        if (const char *env = getenv("T81B200_GEMV_CFG")) sscanf(env, "%d,%d,%d", &rw, &kw, &s);
    }
    Switches() {
        read_cfg();
        pdl = getenv("T81B200_NO_PDL") == nullptr;
        live = getenv("T81B200_GEMV_CFG_LIVE") != nullptr;
    }
};
Switches &switches() {
    static Switches sw;
    if (sw.live) sw.read_cfg();
    return sw;
}

// Everything about a launch that depends only on the weight matrices, the shapes and the dtypes: computed on
// the first call with that combination and reused afterwards (tensor maps, launch shape, shared-memory layout).
struct PlanKey {
    const void *A[kMaxSeg];
    int64_t M[kMaxSeg];
    int64_t K;
    int n_seg, ntok, x_dtype, c_dtype, device, fmt;
    bool operator==(const PlanKey &o) const { return memcmp(this, &o, sizeof *this) == 0; }
};
struct PlanKeyHash {
    size_t operator()(const PlanKey &k) const {
        const unsigned char *b = reinterpret_cast<const unsigned char *>(&k);
        uint64_t h = 1469598103934665603ull;
        for (size_t i = 0; i < sizeof k; ++i) { h ^= b[i]; h *= 1099511628211ull; }
        return (size_t)h;
    }
};
struct Plan {
    bool valid = false;
    CUtensorMap map[kMaxSeg];
    int tile_begin[kMaxSeg];
    int tiles = 0, slices = 1;
    int row_warps = 0, k_warps = 0, limbs_per_slice = 0, stages = 0, stage_bytes = 0;
    int ring0_stages = 0, ring1_offset = 0, xs_offset = 0, part_offset = 0, sb_offset = 0, bar_offset = 0;
    size_t smem = 0;
};
std::mutex g_plan_mu;
std::unordered_map<PlanKey, Plan, PlanKeyHash> g_plans;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Shared-memory layout for a launch shape; false when it does not fit.
bool lay_out(Plan &pl, int fmt, int planes, int ntok, int tokpad, int rwv, int kwv, int s, int lps, int chunks, int budget) {
    const int rows = 32 * rwv;
    const size_t stage_bytes = (size_t)rows * (fmt == 1 ? 48 : 64);
    const size_t xs_bytes = align_up((size_t)planes * ntok * (lps * 24 + 4) * 4, 128);
    // partial sums of the K-slices, and behind them the receive slots of the cluster fold (one per rank)
    const size_t part_bytes = align_up((size_t)kwv * tokpad * (rows + 4) * 4 + (s > 1 ? (size_t)tokpad * (rows + 4 * s) * 4 : 0), 128);
    const size_t sb_bytes = align_up((size_t)2 * rows * 4, 128);
    const size_t bar_bytes = 1024;  // 2 * 48 + 1 barriers
    size_t off = fmt == 1 ? 0 : kWindowHi;  // no table, no window to keep free
    pl.xs_offset = (int)off; off += xs_bytes;
    pl.part_offset = (int)off; off += part_bytes;
    pl.sb_offset = (int)off; off += sb_bytes;
    pl.bar_offset = (int)off; off += bar_bytes;
    if (off > (size_t)budget) return false;
    int stages0 = fmt == 1 ? 0 : (int)(kWindowLo / stage_bytes);
    int stages1 = (int)(((size_t)budget - off) / stage_bytes);
    int stages = stages0 + stages1;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > chunks) stages = chunks;
    if (stages < 2 * kwv && stages < chunks) return false;
    if (stages0 > stages) stages0 = stages;
    pl.stages = stages;
    pl.stage_bytes = (int)stage_bytes;
    pl.ring0_stages = stages0;
    pl.ring1_offset = (int)off;
    off += (size_t)(stages - stages0) * stage_bytes;
    pl.smem = off;
    return true;
}

int make_plan(Plan &pl, const PlanKey &key) {
    const int planes = key.x_dtype == T81B200_BF16 ? 1 : 2;
    const int tokpad = key.ntok > 8 ? 16 : 8;
    const int64_t kl = (key.K + 47) / 48;
    const int kl4 = (int)((kl + 3) & ~(int64_t)3);
    const int sms = sm_count();
    const Switches sw = switches();
    double best_t = 1e30;
    Plan best;
    for (int rwv = 1; rwv <= 8; ++rwv)
        for (int kwv = 1; rwv * kwv <= kMaxConsumerWarps; ++kwv)
            for (int s = 1; s <= 8; s *= 2) {
                if (s == 8 && rwv % 2) continue;  // the fold hands every rank a multiple of 8 rows
                if (sw.rw && (rwv != sw.rw || kwv != sw.kw || s != (sw.s ? sw.s : 1))) continue;
                int lps = (kl4 / 4 + s - 1) / s * 4;
                if (lps < 4) lps = 4;
                if (!sw.rw && kwv != 2 && kwv != 4 && kwv != 8 && !(kwv == 1 && lps == 4)) continue;  // one warp for a single chunk
                if (s > 1 && (int64_t)(s - 1) * lps >= kl4) continue;  // an empty slice
                const int chunks = lps / 4;
                if (kwv > chunks) continue;                            // a warp without work
                Plan cand;
                if (!lay_out(cand, key.fmt, planes, key.ntok, tokpad, rwv, kwv, s, lps, chunks, kSmemBudget)) continue;
                const int rows = 32 * rwv;
                int64_t row_tiles = 0;
                for (int i = 0; i < key.n_seg; ++i) row_tiles += (key.M[i] + rows - 1) / rows;
                // Cost model, fitted to a sweep of every launch shape over the Llama- and Phi-shaped layers (mean
                // regret 3 %): a warp needs about 0.6 us per chunk of 32 rows whatever shares its scheduler, up to
                // three warps per scheduler; every CTA pulls its own copy of its slice of the activations out of
                // L2, which delivers about 5 TB/s when all CTAs ask for the same lines at once; the longer of the
                // two bounds the CTA and a fifth of the shorter is not hidden; a launch costs 1.5 us, a cluster's
                // fold 0.5 to 0.7 us more.  Clusters must fit inside a GPC: fewer CTAs are co-resident than SMs.
                const double wave_ctas = s == 1 ? sms : (s == 2 ? sms - 8 : (s == 4 ? sms - 20 : sms - 36));
                const double waves = ceil((double)row_tiles * s / wave_ctas);
                const double warps_per_sched = rwv * kwv / 4.0;
                // The decode-stream layout has its own fit (mean regret 6 % over the same sweep plus the per-rank
                // shapes of 2, 4 and 8 GPUs): two warps per scheduler already saturate it, the activation fetch
                // weighs more (2 TB/s), half of the shorter bound is not hidden, the cluster fold is cheap, and
                // whole chunks per warp count for more.
                const bool t2 = key.fmt == 1;
                const double whole = t2 ? 0.6 : 0.3;
                const double chunks_per_warp = whole * ceil((double)chunks / kwv) + (1.0 - whole) * (double)chunks / kwv;
                const double per_chunk = 0.6e-6, sched_cap = t2 ? 2.0 : 3.0;
                const double work = chunks_per_warp * per_chunk * (1.0 + 0.4 * (planes * (tokpad / 8) - 1)) *
                                    (warps_per_sched > sched_cap ? warps_per_sched / sched_cap : 1.0);
                const double x_fetch = (double)row_tiles * s * planes * key.ntok * lps * 96.0 / (t2 ? 2.0e12 : 5.0e12);
                const double fold = t2 ? (s == 8 ? 0.3e-6 : 0.0)
                                       : (s == 2 ? 0.7e-6 : (s == 4 ? 0.5e-6 : (s == 8 ? 0.8e-6 : 0.0)));
                const double hidden = t2 ? 0.5 : 0.2;
                const double t = waves * (1.5e-6 + fold + (work > x_fetch ? work + hidden * x_fetch : x_fetch + hidden * work));
                if (t < best_t) {
                    best_t = t;
                    best = cand;
                    best.row_warps = rwv; best.k_warps = kwv; best.slices = s; best.limbs_per_slice = lps;
                    best.tiles = (int)row_tiles;
                }
            }
    if (best_t >= 1e30) return T81B200_EALIGN;  // nothing fits: the caller uses the register-prefetch kernel
    const int rows = 32 * best.row_warps;
    int tile = 0;
    for (int i = 0; i < key.n_seg; ++i) {
        best.tile_begin[i] = tile;
        tile += (int)((key.M[i] + rows - 1) / rows);
        if (key.fmt == 1) continue;  // contiguous stages: bulk copies, no tensor map
        if (int rc = make_map_2d(&best.map[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, key.A[i], (uint64_t)kl * 16, (uint64_t)key.M[i],
                                 (uint64_t)kl * 16, 64, (uint32_t)rows, CU_TENSOR_MAP_SWIZZLE_NONE))
            return rc;
    }
    if (key.fmt == 1) memset(best.map, 0, sizeof best.map);
    for (int i = key.n_seg; i < kMaxSeg; ++i) { best.tile_begin[i] = tile; best.map[i] = best.map[0]; }
    best.valid = true;
    pl = best;
    return T81B200_OK;
}

template <typename XT, typename CT, int TOKB, int FMT>
int launch_lut(const Plan &pl, const GemvLutParams &p, cudaStream_t st) {
    auto kern = gemv_trit_lut_kernel<XT, CT, TOKB, FMT>;
    // the shared-memory limit is a per-device attribute of the function: raised once per device
    static std::atomic<bool> configured[64];
    int dev = 0;
    T81_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        T81_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.tiles, (unsigned)pl.slices, 1);
    cfg.blockDim = dim3((unsigned)((pl.row_warps * pl.k_warps + 1) * 32), 1, 1);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)pl.slices;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = switches().pdl ? 2 : 1;
    T81_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, pl.map[0], pl.map[1], pl.map[2], p));
    return T81B200_OK;
}

template <typename XT, int FMT>
int launch_lut_ct(const Plan &pl, const GemvLutParams &p, int c_dtype, cudaStream_t st) {
    const bool wide = p.ntok > 8;
    switch (c_dtype) {
        case T81B200_F32: return wide ? launch_lut<XT, float, 2, FMT>(pl, p, st) : launch_lut<XT, float, 1, FMT>(pl, p, st);
        case T81B200_BF16: return wide ? launch_lut<XT, __nv_bfloat16, 2, FMT>(pl, p, st) : launch_lut<XT, __nv_bfloat16, 1, FMT>(pl, p, st);
        case T81B200_F16: return wide ? launch_lut<XT, __half, 2, FMT>(pl, p, st) : launch_lut<XT, __half, 1, FMT>(pl, p, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown output dtype %d", c_dtype);
}

template <int FMT>
int launch_lut_xt(const Plan &pl, const GemvLutParams &p, int x_dtype, int c_dtype, cudaStream_t st) {
    switch (x_dtype) {
        case T81B200_BF16: return launch_lut_ct<__nv_bfloat16, FMT>(pl, p, c_dtype, st);
        case T81B200_F32: return launch_lut_ct<float, FMT>(pl, p, c_dtype, st);
        case T81B200_F16: return launch_lut_ct<__half, FMT>(pl, p, c_dtype, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown activation dtype %d", x_dtype);
}

}  // namespace

extern thread_local int g_hint_independent;

// Launch of the streaming kernel over n_seg weight matrices that share X.  NK layout, ntok in 1..16, every A
// 16-byte aligned; fmt 0: A in the packed-limb layout (table decode), fmt 1: A in the decode-stream layout.
// Returns T81B200_EALIGN when no launch shape fits (K too long for shared memory).
int gemv_trit_lut_launch(int fmt, int n_seg, const uint8_t *const *A, const float *const *row_scale, const float *const *bias,
                         void *const *C, const int64_t *M, const void *X, int x_dtype, int64_t ldx, int c_dtype,
                         int64_t ldc, int ntok, int64_t K, float alpha, float beta, cudaStream_t st, const PeerCtx *ctx) {
    PlanKey key;
    memset(&key, 0, sizeof key);
    for (int i = 0; i < n_seg; ++i) { key.A[i] = A[i]; key.M[i] = M[i]; }
    key.K = K; key.n_seg = n_seg; key.ntok = ntok; key.x_dtype = x_dtype; key.c_dtype = c_dtype; key.fmt = fmt;
    T81_CUDA_TRY(cudaGetDevice(&key.device));
    Plan pl;
    {
        std::lock_guard<std::mutex> lock(g_plan_mu);
        auto it = g_plans.find(key);
        if (it != g_plans.end() && switches().live) { g_plans.erase(it); it = g_plans.end(); }
        if (it == g_plans.end()) {
            Plan fresh;
            if (int rc = make_plan(fresh, key)) return rc;
            if (g_plans.size() >= 8192) g_plans.clear();  // a bound, not a policy: plans are cheap to rebuild
            it = g_plans.emplace(key, fresh).first;
        }
        pl = it->second;
    }
    GemvLutParams p;
    memset(&p, 0, sizeof p);
    for (int i = 0; i < kMaxSeg; ++i) {
        const int j = i < n_seg ? i : 0;
        p.seg[i].row_scale = row_scale ? row_scale[j] : nullptr;
        p.seg[i].bias = bias ? bias[j] : nullptr;
        p.seg[i].C = C[j];
        p.seg[i].M = M[j];
        p.seg[i].tile_begin = pl.tile_begin[i];
        p.seg[i].t2 = A[j];
        p.seg[i].tiles32 = (int)((M[j] + 31) / 32);
    }
    p.n_seg = n_seg;
    p.X = X; p.K = K; p.kl = (K + 47) / 48; p.ldx = ldx; p.ldc = ldc; p.ntok = ntok; p.alpha = fmt == 1 ? 0.5f * alpha : alpha; p.beta = beta;
    p.row_warps = pl.row_warps; p.k_warps = pl.k_warps; p.limbs_per_slice = pl.limbs_per_slice;
    p.stages = pl.stages; p.stage_bytes = pl.stage_bytes; p.ring0_stages = pl.ring0_stages; p.ring1_offset = pl.ring1_offset;
    p.xs_offset = pl.xs_offset; p.part_offset = pl.part_offset; p.sb_offset = pl.sb_offset; p.bar_offset = pl.bar_offset;
    p.bulk_x = x_dtype == T81B200_BF16 && reinterpret_cast<uintptr_t>(X) % 16 == 0 && (ldx * 2) % 16 == 0 && K % 8 == 0 ? 1 : 0;
    p.n_peers = ctx ? ctx->n_peers : 0;
    for (int i = 0; i < T81B200_MAX_PEERS; ++i) p.peer_C[i] = i < p.n_peers ? ctx->peer_C[i] : nullptr;
    p.sync_local = ctx ? ctx->sync_local : nullptr;
    for (int i = 0; i < T81B200_MAX_PEERS; ++i) p.sync_peer[i] = p.sync_local && i < ctx->n_peers ? ctx->sync_slots[i] : nullptr;
    p.independent = (g_hint_independent && !p.sync_local) ? 1 : 0;
    for (int j = 0; j < 8; ++j) p.shl[j] = 1u << (2 * j);
#ifdef T81B200_GEMV_TRACE
    static std::atomic<int> trace_counter{0};
    p.trace_slot = trace_counter.fetch_add(1);
#endif
    return fmt == 1 ? launch_lut_xt<1>(pl, p, x_dtype, c_dtype, st) : launch_lut_xt<0>(pl, p, x_dtype, c_dtype, st);
}

#ifdef T81B200_GEMV_TRACE
extern "C" __attribute__((visibility("default"))) int t81b200_debug_trace(unsigned long long *out, int words) {
    const size_t total = (size_t)kTraceLaunches * kTraceCtas * kTraceStamps;
    if ((size_t)words > total) words = (int)total;
    return cudaMemcpyFromSymbol(out, g_trace, (size_t)words * 8) == cudaSuccess ? 0 : -1;
}
#endif

int gemv_trit_lut_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_lut_status, sizeof v) != cudaSuccess) return T81B200_ECUDA;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_lut_status, &zero, sizeof zero) != cudaSuccess) return T81B200_ECUDA;
    }
    return v;
}

}  // namespace t81b200
