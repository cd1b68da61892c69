// Prefill-shaped TRIT-mode kernel on the 5th-generation tensor cores (tcgen05).
//
//   D[o][t] = sum_k T[o][k] * x[t][k]       o: output feature (UMMA M = 128 per CTA tile)
//                                            t: token          (UMMA N = 256 per CTA tile)
// Operand A is produced on the fly: the packed limbs of 128 weight rows arrive by TMA as
// raw bytes, converter warps expand them to exact bf16 {-1,0,+1} (packed bf16 FMAs, see
// common.cuh) and write them in the K-major, 128-byte-swizzled layout UMMA expects.
// Operand B is the activations, brought by TMA (SWIZZLE_128B) straight from (tokens, K)
// bf16 memory.  Accumulators live in TMEM (2 x 256 fp32 columns, double-buffered across
// tiles) and are read back with tcgen05.ld for a fused scale/bias/beta epilogue.
//
// One persistent CTA per SM, 14 warps:
//   warp 0      TMA producer (raw weight bytes + activation tiles)
//   warp 1      MMA issuer (one elected lane), owns the TMEM allocation
//   warps 2-5   epilogue (TMEM lanes 32*(warp%4) ...)
//   warps 6-13  converters (256 threads; 2 limbs per thread per 192-trit super-block)
// The contraction runs in k-atoms of 64 (one 128-byte swizzle row); 48-trit limbs do not
// divide 64, so converters work in super-blocks of 4 limbs = 192 trits = 3 atoms.
//
// Every mbarrier wait is bounded; on expiry the role records a status code and all roles
// fall through to the common teardown (TMEM is always released).
#include "common.cuh"
#include "tma.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace t81b200 {

namespace {

constexpr int BM = 128;          // output features per tile (UMMA M)
constexpr int BN_MAX = 256;      // tokens per tile (UMMA N) with one activation plane; 128 with two
constexpr int BK = 64;           // k-atom: 64 bf16 = 128 bytes
constexpr int A_STAGES = 6;      // two super-blocks of expanded weights
constexpr int B_STAGES = 3;
constexpr int RAW_STAGES = 2;
constexpr int A_STAGE_BYTES = BM * BK * 2;    // 16 KB
constexpr int B_STAGE_BYTES = BN_MAX * BK * 2;  // 32 KB: one 256-token plane or two 128-token planes
#ifndef T81B200_TC_CONVERTER_WARPS
#define T81B200_TC_CONVERTER_WARPS 8
#endif
constexpr int CONVERTER_WARPS_ = T81B200_TC_CONVERTER_WARPS;
constexpr int RAW_STAGE_BYTES = BM * 64;      // 4 limbs per row: 8 KB
constexpr int NUM_THREADS = (6 + CONVERTER_WARPS_) * 32;
constexpr int CONVERTER_WARP0 = 6;
constexpr int CONVERTER_WARPS = CONVERTER_WARPS_;
constexpr int CONVERTER_THREADS = CONVERTER_WARPS * 32;
constexpr int LIMBS_PER_CONVERTER = BM * 4 / CONVERTER_THREADS;  // limbs of a 4-limb super-block per thread
constexpr int OUT_TOKENS = 32;                      // tokens per staged output block (one tcgen05.ld of 32 columns)
constexpr int OUT_STAGE_BYTES = OUT_TOKENS * BM * 2;  // [token][feature] block of a 16-bit output type: 8 KB
constexpr int OUT_STAGES = 2;
constexpr int SMEM_DATA_BYTES = A_STAGES * A_STAGE_BYTES + B_STAGES * B_STAGE_BYTES + RAW_STAGES * RAW_STAGE_BYTES +
                                OUT_STAGES * OUT_STAGE_BYTES;
constexpr int SMEM_BYTES = SMEM_DATA_BYTES + 256 /*barriers*/ + 1024 /*alignment slack*/;
constexpr uint32_t TMEM_COLS = 512;

// kind::f16 instruction descriptor: D fp32, A and B bf16, both K-major, N tokens, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

enum { STATUS_OK = 0, STATUS_TIMEOUT_PRODUCER = 1, STATUS_TIMEOUT_MMA = 2, STATUS_TIMEOUT_EPILOGUE = 3, STATUS_TIMEOUT_CONVERTER = 4 };

__device__ int g_tc_status = 0;

struct TcParams {
    const float *row_scale, *bias;
    void *C;
    int64_t c_row_stride, c_tok_stride;  // element strides of C along output features and tokens
    int64_t M, N, K, kl;
    int m_tiles, n_tiles, n_atoms;
    int plane_rows;  // row distance between the activation planes in the tensor map
    float alpha, beta;
    int n_out_maps;      // > 0: the epilogue stages output blocks in shared memory and stores them by TMA through
                         // this many tensor maps (the local C first, then the peers'); 0: per-element stores
    int n_peers;         // other GPUs that receive a copy of every output element
    void *peer_C[T81B200_MAX_PEERS];  // their C, same strides as the local one
    int c_vec;           // 1: tokens are contiguous in C (the (M, N) argument order) and 16-byte aligned per 32-token block:
                         // a thread's 32 tokens of one feature are one run of memory, moved with 128-bit accesses
};

// Tensor maps of the result, for the TMA-store epilogue: [0] the local C, then one per peer.
struct TcOutMaps {
    CUtensorMap m[1 + T81B200_MAX_PEERS];
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y)
                 : "memory");
}

// K-major, SWIZZLE_128B shared-memory descriptor: rows are 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset
    d |= (uint64_t)1 << 46;                       // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}


// AND of a predicate over the 128 epilogue threads (named barrier 2); every one of them must call it.
__device__ __forceinline__ bool epilogue_all(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "barrier.cta.red.and.pred p, 2, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}

// PLANES = 1: bf16 activations as they are.  PLANES = 2: activations split into a bf16 "hi"
// plane and a bf16 "lo" plane (x = hi + lo to 16 mantissa bits); both are multiplied with the
// same expanded weights into the same accumulator, on a 128-token tile.
// NSPLIT = 2 (one plane only): 128-token tiles, for launches whose 256-token tiles would leave most CTAs idle in
// the last wave; the weight expansion is then done twice as often per flop, so it is only used where it pays.
template <typename CT, int PLANES, int NSPLIT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_trit_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ TcOutMaps omaps, const TcParams p) {
    constexpr int BN = BN_MAX / PLANES / NSPLIT;
    constexpr int PLANE_BYTES = BN * BK * 2;
    constexpr uint32_t kInstrDesc = instr_desc(BN);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t a_smem = base;
    const uint32_t b_smem = a_smem + A_STAGES * A_STAGE_BYTES;
    const uint32_t raw_smem = b_smem + B_STAGES * B_STAGE_BYTES;
    const uint32_t out_smem = raw_smem + RAW_STAGES * RAW_STAGE_BYTES;
    const uint32_t bars = out_smem + OUT_STAGES * OUT_STAGE_BYTES;
    uint8_t *gen_base = smem_raw + (base - smem_u32(smem_raw));
    // barrier slots (8 bytes each)
    auto a_full = [&](int s) { return bars + 8u * s; };
    auto a_empty = [&](int s) { return bars + 8u * (A_STAGES + s); };
    auto b_full = [&](int s) { return bars + 8u * (2 * A_STAGES + s); };
    auto b_empty = [&](int s) { return bars + 8u * (2 * A_STAGES + B_STAGES + s); };
    auto raw_full = [&](int s) { return bars + 8u * (2 * A_STAGES + 2 * B_STAGES + s); };
    auto raw_empty = [&](int s) { return bars + 8u * (2 * A_STAGES + 2 * B_STAGES + RAW_STAGES + s); };
    auto acc_full = [&](int s) { return bars + 8u * (2 * A_STAGES + 2 * B_STAGES + 2 * RAW_STAGES + s); };
    auto acc_empty = [&](int s) { return bars + 8u * (2 * A_STAGES + 2 * B_STAGES + 2 * RAW_STAGES + 2 + s); };
    const uint32_t tmem_slot = bars + 8u * (2 * A_STAGES + 2 * B_STAGES + 2 * RAW_STAGES + 4);
    volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(
        gen_base + SMEM_DATA_BYTES + 8 * (2 * A_STAGES + 2 * B_STAGES + 2 * RAW_STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; ++s) { mbar_init(a_full(s), CONVERTER_WARPS); mbar_init(a_empty(s), 1); }
        for (int s = 0; s < B_STAGES; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
        for (int s = 0; s < RAW_STAGES; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), CONVERTER_WARPS); }
        for (int s = 0; s < 2; ++s) { mbar_init(acc_full(s), 1); mbar_init(acc_empty(s), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot_gen;

    const int total_tiles = p.m_tiles * p.n_tiles;
    const int n_super = (p.n_atoms + 2) / 3;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            Ring raw, b;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * BM, n0 = (tile / p.m_tiles) * BN;
                for (int s = 0; s < n_super && ok; ++s) {
                    ok = mbar_wait(raw_empty(raw.stage), raw.phase ^ 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(raw_full(raw.stage), RAW_STAGE_BYTES);
                    tma_load_2d(raw_smem + raw.stage * RAW_STAGE_BYTES, &map_w, s * 64, m0, raw_full(raw.stage));
                    raw.advance(RAW_STAGES);
                    for (int a = 3 * s; a < 3 * s + 3 && a < p.n_atoms; ++a) {
                        ok = mbar_wait(b_empty(b.stage), b.phase ^ 1);
                        if (!ok) break;
                        mbar_arrive_expect_tx(b_full(b.stage), PLANES * PLANE_BYTES);
#pragma unroll
                        for (int pl = 0; pl < PLANES; ++pl)
                            tma_load_2d(b_smem + b.stage * B_STAGE_BYTES + pl * PLANE_BYTES, &map_x, a * BK,
                                        pl * p.plane_rows + n0, b_full(b.stage));
                        b.advance(B_STAGES);
                    }
                }
            }
            if (!ok) atomicCAS(&g_tc_status, STATUS_OK, STATUS_TIMEOUT_PRODUCER);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            Ring a, b;
            bool ok = true;
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                ok = mbar_wait(acc_empty(buf), acc_phase ^ 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN_MAX;
                for (int at = 0; at < p.n_atoms; ++at) {
                    ok = mbar_wait(a_full(a.stage), a.phase) && mbar_wait(b_full(b.stage), b.phase);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ad = umma_desc(a_smem + a.stage * A_STAGE_BYTES);
#pragma unroll
                    for (int pl = 0; pl < PLANES; ++pl) {
                        const uint64_t bd = umma_desc(b_smem + b.stage * B_STAGE_BYTES + pl * PLANE_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_bf16(d_tmem, ad + (uint64_t)(2 * k), bd + (uint64_t)(2 * k), kInstrDesc,
                                      (at | k | pl) != 0 ? 1u : 0u);
                    }
                    umma_commit(a_empty(a.stage));
                    umma_commit(b_empty(b.stage));
                    a.advance(A_STAGES);
                    b.advance(B_STAGES);
                }
                if (!ok) break;
                umma_commit(acc_full(buf));
            }
            if (!ok) atomicCAS(&g_tc_status, STATUS_OK, STATUS_TIMEOUT_MMA);
        }
    } else if (warp < CONVERTER_WARP0) {
        // ---------------- epilogue ----------------
        const int lane_group = warp & 3;  // TMEM lanes 32*lane_group .. +31 are this warp's
        bool ok = true;
        int it = 0;
        int out_count = 0;  // staged output blocks so far (picks the staging buffer)
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int m0 = (tile % p.m_tiles) * BM, n0 = (tile / p.m_tiles) * BN;
            const int buf = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            // One decision for all four epilogue warps (tcgen05.ld is .aligned, and the staging path below
            // meets at named barriers): every thread's bounded wait returns, then the 128 threads agree.
            ok = epilogue_all(mbar_wait(acc_full(buf), acc_phase));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int64_t row = (int64_t)m0 + lane_group * 32 + lane;
            const bool row_ok = row < p.M;
            const float scale = (row_ok && p.row_scale ? p.row_scale[row] : 1.0f) * p.alpha;
            const float bias = row_ok && p.bias ? p.bias[row] : 0.0f;
            CT *crow = static_cast<CT *>(p.C) + row * p.c_row_stride;
            if (p.n_out_maps > 0) {
                // 16-bit output, token-major C: stage [32 tokens][128 features] blocks in shared memory and let
                // TMA write them (whole 256-byte rows; the tensor map clips rows and tokens past the end)
                const int epi_tid = threadIdx.x - 2 * 32;  // 0..127
                uint8_t *stage0 = gen_base + (out_smem - base);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c, ++out_count) {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * BN_MAX + c * 32), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int sb = out_count & 1;
                    // the stores issued from this buffer two blocks ago must have read it
                    if (epi_tid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    CT *dst = reinterpret_cast<CT *>(stage0 + sb * OUT_STAGE_BYTES) + lane_group * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 32; ++i) dst[i * BM] = from_float<CT>(__uint_as_float(v[i]) * scale + bias);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (epi_tid == 0) {
                        for (int j = 0; j < p.n_out_maps; ++j)
                            tma_store_2d(&omaps.m[j], out_smem + (uint32_t)sb * OUT_STAGE_BYTES, m0, n0 + c * 32);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            } else
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * BN_MAX + c * 32), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row_ok && p.c_vec && (int64_t)n0 + c * 32 + 32 <= p.N) {
                    // (M, N) argument order: the thread's 32 tokens are contiguous — whole 16-byte pieces, and with
                    // beta the old values are all fetched before the first store
                    constexpr int PER = 16 / (int)sizeof(CT);  // elements per 128-bit access
                    uint4 *dst = reinterpret_cast<uint4 *>(crow + (int64_t)n0 + c * 32);
                    uint4 old[32 / PER];
                    if (p.beta != 0.0f) {
#pragma unroll
                        for (int q = 0; q < 32 / PER; ++q) old[q] = dst[q];
                    }
#pragma unroll
                    for (int q = 0; q < 32 / PER; ++q) {
                        CT out[PER];
                        const CT *was = reinterpret_cast<const CT *>(&old[q]);
#pragma unroll
                        for (int e = 0; e < PER; ++e) {
                            float y = __uint_as_float(v[q * PER + e]) * scale + bias;
                            if (p.beta != 0.0f) y += p.beta * to_float<CT>(was[e]);
                            out[e] = from_float<CT>(y);
                        }
                        dst[q] = *reinterpret_cast<const uint4 *>(out);
                    }
                } else if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int64_t tok = (int64_t)n0 + c * 32 + i;
                        if (tok < p.N) {
                            float y = __uint_as_float(v[i]) * scale + bias;
                            CT *dst = crow + tok * p.c_tok_stride;
                            if (p.beta != 0.0f) y += p.beta * to_float<CT>(*dst);
                            *dst = from_float<CT>(y);
                        }
                    }
                    // column-sharded Linear: the same elements go into every peer's result over NVLink
                    for (int pj = 0; pj < p.n_peers; ++pj) {
                        CT *prow = static_cast<CT *>(p.peer_C[pj]) + row * p.c_row_stride;
#pragma unroll 1  // a rare path: unrolled it costs the whole kernel 40 registers
                        for (int i = 0; i < 32; ++i) {
                            const int64_t tok = (int64_t)n0 + c * 32 + i;
                            if (tok < p.N) prow[tok * p.c_tok_stride] = crow[tok * p.c_tok_stride];
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));
        }
        // every TMA store of this CTA has completed before the kernel ends
        if (threadIdx.x == 2 * 32) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (!ok && lane == 0) atomicCAS(&g_tc_status, STATUS_OK, STATUS_TIMEOUT_EPILOGUE);
    } else {
        // ---------------- converters ----------------
        const int cthread = threadIdx.x - CONVERTER_WARP0 * 32;  // 0..255
        Ring raw, a;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            for (int s = 0; s < n_super && ok; ++s) {
                ok = __all_sync(0xffffffffu, mbar_wait(raw_full(raw.stage), raw.phase));
                if (!ok) break;
                uint4 limb[LIMBS_PER_CONVERTER];
#pragma unroll
                for (int h = 0; h < LIMBS_PER_CONVERTER; ++h) {
                    const int item = cthread + CONVERTER_THREADS * h;  // row = item / 4, limb = item % 4
                    limb[h] = *reinterpret_cast<const uint4 *>(gen_base + A_STAGES * A_STAGE_BYTES + B_STAGES * B_STAGE_BYTES +
                                                               raw.stage * RAW_STAGE_BYTES + item * 16);
                    if ((int64_t)4 * s + (item & 3) >= p.kl)  // past the row's last limb: zero trits
                        limb[h] = make_uint4(kZeroTryteWord, kZeroTryteWord, kZeroTryteWord, kZeroTryteWord);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(raw_empty(raw.stage));
                raw.advance(RAW_STAGES);

                // the (up to) three atoms of this super-block
                const int atoms_here = p.n_atoms - 3 * s < 3 ? p.n_atoms - 3 * s : 3;
                Ring aw = a;
                for (int j = 0; j < atoms_here && ok; ++j) {
                    ok = mbar_wait(a_empty(aw.stage), aw.phase ^ 1);
                    aw.advance(A_STAGES);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
#pragma unroll
                for (int h = 0; h < LIMBS_PER_CONVERTER; ++h) {
                    const int item = cthread + CONVERTER_THREADS * h;
                    const int r = item >> 2, j = item & 3;
                    uint32_t o[24];
                    decode_limb(limb[h], o);
                    // decode order -> natural order: pairs (trit 2m, trit 2m+1)
                    uint32_t nat[24];
#pragma unroll
                    for (int pr = 0; pr < 8; ++pr) {
                        nat[3 * pr + 0] = __byte_perm(o[3 * pr], o[3 * pr + 1], 0x5410);
                        nat[3 * pr + 1] = __byte_perm(o[3 * pr + 2], o[3 * pr], 0x7610);
                        nat[3 * pr + 2] = __byte_perm(o[3 * pr + 1], o[3 * pr + 2], 0x7632);
                    }
                    const uint32_t row_off = (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
#pragma unroll
                    for (int q = 0; q < 6; ++q) {
                        const int chunk = 6 * j + q;         // 16-byte chunk inside the 384-byte super-block row
                        const int atom = chunk >> 3, cc = chunk & 7;
                        if (atom < atoms_here) {
                            int st = a.stage + atom;
                            st = st >= A_STAGES ? st - A_STAGES : st;
                            const uint32_t off = (uint32_t)st * A_STAGE_BYTES + row_off + (uint32_t)((cc ^ (r & 7)) << 4);
                            *reinterpret_cast<uint4 *>(gen_base + off) = make_uint4(nat[4 * q], nat[4 * q + 1], nat[4 * q + 2], nat[4 * q + 3]);
                        }
                    }
                }
                // generic-proxy writes must be visible to the tensor core's async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0)
                    for (int j = 0; j < atoms_here; ++j) {
                        int st = a.stage + j;
                        st = st >= A_STAGES ? st - A_STAGES : st;
                        mbar_arrive(a_full(st));
                    }
                a = aw;
            }
        }
        if (!ok && lane == 0) atomicCAS(&g_tc_status, STATUS_OK, STATUS_TIMEOUT_CONVERTER);
    }

    // ---------------- teardown ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <typename CT, int PLANES, int NSPLIT>
int launch_tc(const CUtensorMap &mw, const CUtensorMap &mx, const TcOutMaps &om, const TcParams &p, cudaStream_t st) {
    auto kern = gemm_trit_tc_kernel<CT, PLANES, NSPLIT>;
    // the shared-memory limit is a per-device attribute of the function: set it once on every device
    static std::atomic<bool> configured[64];
    int dev = 0;
    T81_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        T81_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    const int tiles = p.m_tiles * p.n_tiles;
    const int sms = sm_count();
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, NUM_THREADS, SMEM_BYTES, st>>>(mw, mx, om, p);
    T81_LAUNCH_CHECK("gemm_trit_tc_kernel");
    return T81B200_OK;
}

template <int PLANES, int NSPLIT>
int launch_tc_ct(int c_dtype, const CUtensorMap &mw, const CUtensorMap &mx, const TcOutMaps &om, const TcParams &p, cudaStream_t st) {
    switch (c_dtype) {
        case T81B200_F32: return launch_tc<float, PLANES, NSPLIT>(mw, mx, om, p, st);
        case T81B200_BF16: return launch_tc<__nv_bfloat16, PLANES, NSPLIT>(mw, mx, om, p, st);
        case T81B200_F16: return launch_tc<__half, PLANES, NSPLIT>(mw, mx, om, p, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown output dtype %d", c_dtype);
}

// Pre-pass for activations the TMA path cannot read directly (fp32 / fp16 values, the
// (K, N) layout, unaligned rows): writes token-major bf16 planes into scratch memory,
//   plane 0 = bf16(x), plane 1 = bf16(x - plane 0)      (PLANES == 2)
// as scratch[plane][token][k], row length kpad.  32 x 32 tiles through shared memory so
// that both the read (along n for KN, along k for NK) and the write (along k) coalesce.
template <typename BT, int PLANES>
__global__ void __launch_bounds__(256) stage_planes_kernel(const BT *__restrict__ B, int64_t sbk, int64_t sbn, int64_t N,
                                                           int64_t K, __nv_bfloat16 *__restrict__ out, int64_t kpad,
                                                           int64_t plane_elems) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const int64_t n0 = (int64_t)blockIdx.x * 32, k0 = (int64_t)blockIdx.y * 32;
    const bool k_fast = sbk == 1;  // NK layout: k is the contiguous index of the source
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int a = ty + 8 * i;
        const int64_t n = k_fast ? n0 + a : n0 + tx, k = k_fast ? k0 + tx : k0 + a;
        float v = 0.0f;
        if (n < N && k < K) v = to_float<BT>(B[k * sbk + n * sbn]);
        if (k_fast) tile[a][tx] = v; else tile[tx][a] = v;  // tile[n][k]
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int a = ty + 8 * i;
        const int64_t n = n0 + a, k = k0 + tx;
        if (n < N && k < kpad) {
            const float v = tile[a][tx];
            const __nv_bfloat16 hi = __float2bfloat16_rn(v);
            out[n * kpad + k] = hi;
            if (PLANES == 2) out[plane_elems + n * kpad + k] = __float2bfloat16_rn(v - __bfloat162float(hi));
        }
    }
}

template <typename BT>
int launch_stage(const void *B, int layout, int64_t ldb, int64_t N, int64_t K, int planes, __nv_bfloat16 *out,
                 int64_t kpad, int64_t plane_elems, cudaStream_t st) {
    const int64_t sbk = layout == T81B200_LAYOUT_KN ? ldb : 1, sbn = layout == T81B200_LAYOUT_KN ? 1 : ldb;
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)((kpad + 31) / 32));
    if (grid.y > 65535u) return fail(T81B200_ELIMIT, "gemm_trit: K too large");
    if (planes == 2)
        stage_planes_kernel<BT, 2><<<grid, 256, 0, st>>>(static_cast<const BT *>(B), sbk, sbn, N, K, out, kpad, plane_elems);
    else
        stage_planes_kernel<BT, 1><<<grid, 256, 0, st>>>(static_cast<const BT *>(B), sbk, sbn, N, K, out, kpad, plane_elems);
    T81_LAUNCH_CHECK("stage_planes_kernel");
    return T81B200_OK;
}

// How the dense operand reaches the tensor-core kernel.
struct TcPlan {
    bool direct;       // bf16, token-major: TMA reads the caller's buffer
    int planes;        // 1 or 2
    int bn;            // tokens per tile
    int64_t kpad;      // scratch row length (elements)
    int64_t rows_pad;  // scratch rows per plane (a whole number of tiles)
    size_t scratch_bytes;
};

TcPlan make_plan(int b_dtype, int layout, int64_t M, int64_t N, int64_t K) {
    TcPlan pl;
    pl.direct = b_dtype == T81B200_BF16 && layout == T81B200_LAYOUT_NK;
    pl.planes = b_dtype == T81B200_BF16 ? 1 : 2;
    pl.bn = BN_MAX / pl.planes;
    if (pl.planes == 1 && M > 0) {
        // 128-token tiles only when 256-token tiles would leave more than half of the SMs without any tile: every
        // tile expands its own 128 x K block of weights, and at 128 tokens the eight converter warps cannot keep
        // up with the MMAs (measured: 612 instead of 1128 TFLOP/s on 4096 x 4096 x 16384, 470 instead of 627 on
        // 3072 x 3072 x 2048), so the smaller tile pays only where the extra expansions run on idle SMs
        // (1024 x 4096 x 1024: 39.5 instead of 42.6 us).  T81B200_TC_TILE_TOKENS=128|256 (read once) forces one.
        static const int forced = [] { const char *e = getenv("T81B200_TC_TILE_TOKENS"); return e ? atoi(e) : 0; }();
        const int64_t sms = sm_count(), tiles256 = ((M + BM - 1) / BM) * ((N + 255) / 256);
        if (forced == 128 || (forced == 0 && tiles256 * 2 <= sms && N > 128)) pl.bn = 128;
    }
    pl.kpad = (K + 7) & ~(int64_t)7;
    pl.rows_pad = (N + pl.bn - 1) / pl.bn * pl.bn;
    pl.scratch_bytes = pl.direct ? 0 : (size_t)pl.planes * pl.rows_pad * pl.kpad * 2;
    return pl;
}

}  // namespace

// The tensor-core path reads bf16 token-major activations in place; other dtypes and the
// (K, N) layout go through the staging pre-pass into scratch memory first.  Small problems
// stay on the general kernel (they are launch-bound either way).
bool gemm_trit_tc_eligible(int b_dtype, int layout, int c_dtype, int64_t M, int64_t N, int64_t K) {
    (void)c_dtype;
    if (M < 1 || N < 1 || K < 1 || M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return false;
    const bool direct = b_dtype == T81B200_BF16 && layout == T81B200_LAYOUT_NK;
    if (direct) return N >= 1;  // the dispatcher sends N <= 16 to the streaming kernel first
    return (double)M * (double)N * (double)K >= 1.6e7 && N >= 8;
}

size_t gemm_trit_tc_workspace(int b_dtype, int layout, int c_dtype, int64_t M, int64_t N, int64_t K) {
    (void)c_dtype; (void)M;
    return make_plan(b_dtype, layout, 0, N, K).scratch_bytes;
}

int gemm_trit_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof v) != cudaSuccess) return T81B200_ECUDA;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_tc_status, &zero, sizeof zero) != cudaSuccess) return T81B200_ECUDA;
    }
    return v;
}

int gemm_trit_tc_launch(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                        int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M, int64_t N,
                        int64_t K, float alpha, float beta, void *workspace, size_t workspace_bytes, cudaStream_t st,
                        int n_peers, void *const *peer_C) {
    const TcPlan plan = make_plan(b_dtype, layout, M, N, K);
    const void *x_ptr = B;
    int64_t x_ld = ldb, x_rows = N;
    if (plan.direct) {
        if (reinterpret_cast<uintptr_t>(B) % 16 != 0 || (ldb * 2) % 16 != 0)
            return T81B200_EALIGN;  // caller falls back to the general kernel
    } else {
        if (!workspace || workspace_bytes < plan.scratch_bytes || reinterpret_cast<uintptr_t>(workspace) % 16 != 0)
            return fail(T81B200_EWORKSPACE, "gemm_trit: %zu bytes of 16-byte aligned workspace needed, %zu given",
                        plan.scratch_bytes, workspace_bytes);
        __nv_bfloat16 *scratch = static_cast<__nv_bfloat16 *>(workspace);
        const int64_t plane_elems = plan.rows_pad * plan.kpad;
        int rc = T81B200_EINVAL;
        switch (b_dtype) {
            case T81B200_F32: rc = launch_stage<float>(B, layout, ldb, N, K, plan.planes, scratch, plan.kpad, plane_elems, st); break;
            case T81B200_BF16: rc = launch_stage<__nv_bfloat16>(B, layout, ldb, N, K, plan.planes, scratch, plan.kpad, plane_elems, st); break;
            case T81B200_F16: rc = launch_stage<__half>(B, layout, ldb, N, K, plan.planes, scratch, plan.kpad, plane_elems, st); break;
        }
        if (rc) return rc;
        x_ptr = scratch; x_ld = plan.kpad; x_rows = (int64_t)plan.planes * plan.rows_pad;
    }
    const int64_t kl = (K + 47) / 48;
    CUtensorMap mw, mx;
    if (int rc = make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)kl * 16, (uint64_t)M, (uint64_t)kl * 16, 64, BM,
                             CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
    if (int rc = make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x_ptr, (uint64_t)K, (uint64_t)x_rows, (uint64_t)x_ld * 2, BK,
                             (uint32_t)plan.bn, CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;
    TcParams p;
    p.row_scale = row_scale; p.bias = bias; p.C = C; p.M = M; p.N = N; p.K = K; p.kl = kl;
    if (layout == T81B200_LAYOUT_NK) { p.c_row_stride = 1; p.c_tok_stride = ldc; }
    else { p.c_row_stride = ldc; p.c_tok_stride = 1; }
    p.m_tiles = (int)((M + BM - 1) / BM);
    p.n_tiles = (int)((N + plan.bn - 1) / plan.bn);
    p.n_atoms = (int)((K + BK - 1) / BK);
    p.plane_rows = (int)plan.rows_pad;
    p.alpha = alpha; p.beta = beta;
    p.n_peers = n_peers;
    for (int i = 0; i < T81B200_MAX_PEERS; ++i) p.peer_C[i] = i < n_peers ? peer_C[i] : nullptr;
    p.c_vec = layout == T81B200_LAYOUT_KN && n_peers == 0 && reinterpret_cast<uintptr_t>(C) % 16 == 0 &&
                      (ldc * (int64_t)dtype_size(c_dtype)) % 16 == 0 ? 1 : 0;
    // TMA-store epilogue: 16-bit output, token-major C (features contiguous), no read-modify-write, and every
    // result 16-byte aligned with a 16-byte multiple as its row pitch
    TcOutMaps om;
    memset(&om, 0, sizeof om);
    p.n_out_maps = 0;
    const size_t esz = dtype_size(c_dtype);
    bool tma_out = esz == 2 && layout == T81B200_LAYOUT_NK && beta == 0.0f && (ldc * 2) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(C) % 16 == 0;
    for (int i = 0; i < n_peers; ++i) tma_out = tma_out && reinterpret_cast<uintptr_t>(peer_C[i]) % 16 == 0;
    if (tma_out) {
        const CUtensorMapDataType dt = c_dtype == T81B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        for (int i = 0; i <= n_peers; ++i) {
            void *dst = i == 0 ? C : peer_C[i - 1];
            if (int rc = make_map_2d(&om.m[i], dt, 2, dst, (uint64_t)M, (uint64_t)N, (uint64_t)ldc * 2, BM, OUT_TOKENS,
                                     CU_TENSOR_MAP_SWIZZLE_NONE))
                return rc;
        }
        p.n_out_maps = 1 + n_peers;
    }
    if (plan.planes == 2) return launch_tc_ct<2, 1>(c_dtype, mw, mx, om, p, st);
    return plan.bn == 128 ? launch_tc_ct<1, 2>(c_dtype, mw, mx, om, p, st) : launch_tc_ct<1, 1>(c_dtype, mw, mx, om, p, st);
}

}  // namespace t81b200

// ---- entry point that allocates nothing -------------------------------------------------

namespace {

// Scratch for the staging pre-pass of t81b200_gemm_trit_static.  It is part of the loaded
// module: every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[T81B200_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address;
// the address the kernels need is looked up once per device, with that device current.
void *g_static_scratch_ptr[64] = {nullptr};
std::mutex g_static_scratch_mu;

int static_scratch_address(void **out) {
    int dev = 0;
    T81_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return t81b200::fail(T81B200_ELIMIT, "gemm_trit_static: device index %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (!g_static_scratch_ptr[dev]) {
        void *ptr = nullptr;
        T81_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return T81B200_OK;
}

}  // namespace

extern "C" int t81b200_gemm_trit_static(const uint8_t *A, const float *row_scale, const void *B, int b_dtype, int layout,
                                        int64_t ldb, const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M,
                                        int64_t N, int64_t K, float alpha, float beta, void *stream) {
    if (int rc = t81b200::check_device()) return rc;
    const size_t need = t81b200_gemm_trit_workspace_bytes(b_dtype, layout, c_dtype, M, N, K);
    if (need > (size_t)T81B200_STATIC_SCRATCH_BYTES)
        return t81b200::fail(T81B200_ELIMIT,
                             "gemm_trit_static: this call needs %zu bytes of scratch, the built-in buffer holds %zu; "
                             "use t81b200_gemm_trit with a caller-provided workspace",
                             need, (size_t)T81B200_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    return t81b200_gemm_trit(A, row_scale, B, b_dtype, layout, ldb, bias, C, c_dtype, ldc, M, N, K, alpha, beta, scratch,
                             (size_t)T81B200_STATIC_SCRATCH_BYTES, stream);
}

