// Decode-shaped TRIT-mode kernel on tcgen05 with the weight operand in tensor memory.
//
// The legacy mma.sync path (gemv_trit.cu) pays ~14 issue-blocking cycles per m16n8k16 on
// sm_100a on top of the tryte decode.  Here the decoded weights never meet a warp-level MMA:
//   * one producer thread streams the packed weights of 128 rows through a shared-memory ring
//     with TMA (one 4-limb chunk = 128 rows x 64 bytes per slot);
//   * 16 converter warps decode: thread = (row, limb of the chunk); the 24 packed bf16
//     registers of a limb go straight into TENSOR MEMORY with tcgen05.st (lane = row,
//     24 columns per limb), so the expanded weights cost no shared-memory bandwidth at all;
//   * one thread issues tcgen05.mma (M = 128 rows, N = 16 token slots, K = 16) with A read
//     from tensor memory and B = the activations, staged once per CTA in shared memory in
//     the canonical K-major layout and in the same permuted k order the decode produces;
//   * the fp32 accumulator (128 lanes x 16 columns of tensor memory) is read back once at
//     the end for the scale / bias / beta epilogue.
// The contraction can be split over the CTAs of a cluster (partials meet through distributed
// shared memory in rank order).  Every wait is bounded and reports through a status word.
#include "common.cuh"
#include "tma.cuh"

#include <cooperative_groups.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>

namespace cg = cooperative_groups;

namespace t81b200 {

namespace {

constexpr int UM_ROWS = 128;                // rows per CTA (UMMA M)
constexpr int UM_TOK = 16;                  // token slots (UMMA N)
constexpr int UM_CONVERTER_WARPS = 16;
constexpr int UM_THREADS = (UM_CONVERTER_WARPS + 2) * 32;  // + producer warp + MMA warp
constexpr int UM_STAGE_LIMBS = 8;                          // limbs per row in one ring stage (128-byte rows)
constexpr int UM_STAGE_BYTES = UM_ROWS * UM_STAGE_LIMBS * 16;
constexpr int UM_A_SLOTS = 4;                              // half stages (4 limbs) of decoded weights resident in TMEM
constexpr int UM_A_COLS = 96;                              // 4 limbs x 24 columns
constexpr int UM_ACCS = 4;                                 // independent accumulators, summed in the epilogue
constexpr int UM_A_COL0 = UM_ACCS * 16;                    // accumulators occupy the columns below
constexpr uint32_t UM_TMEM_COLS = 512;
constexpr int UM_MAX_STAGES = 12;

// kind::f16: D fp32, A and B bf16, K-major, N = 16, M = 128
constexpr uint32_t kUmInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(UM_TOK >> 3) << 17) | ((uint32_t)(UM_ROWS >> 4) << 24);

enum { UM_STATUS_OK = 0, UM_TIMEOUT_PRODUCER = 7, UM_TIMEOUT_CONVERTER = 8, UM_TIMEOUT_MMA = 9, UM_TIMEOUT_EPILOGUE = 10 };
__device__ int g_umma_status = 0;
__device__ long long g_umma_trace[64];
#define UM_TRACE(i) do { if (trace) g_umma_trace[i] = clock64(); } while (0)

struct UmParams {
    const void *X;            // (ntok, K) bf16, ldx elements
    const float *row_scale, *bias;
    void *C;                  // (ntok, M) row-major, ldc elements
    int64_t M, K, kl, ldx, ldc;
    int ntok;
    int limbs_per_slice;      // multiple of 8
    int stages;               // weight ring depth
    int ring_offset, part_offset, bar_offset;  // bytes from the 1024-aligned base of dynamic smem
    float alpha, beta;
    int debug;
};

// Activations in the canonical K-major no-swizzle layout: 8x8 core matrices of 128 bytes;
// along K the two token groups of a core column are adjacent (SBO = 128), successive
// k-groups of 8 follow at LBO = 256 bytes.
__device__ __forceinline__ uint64_t um_b_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(256 >> 4) << 16;  // leading byte offset: next k-group
    d |= (uint64_t)(128 >> 4) << 32;  // stride byte offset: next 8 tokens
    d |= (uint64_t)1 << 46;           // descriptor version
    return d;                         // layout type 0: no swizzle
}

__device__ __forceinline__ void um_mma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(kUmInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void um_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void um_st8(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void um_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

template <typename CT>
__device__ __forceinline__ void um_store_out(const UmParams &p, int64_t row, int tok, float acc) {
    if (row >= p.M || tok >= p.ntok) return;
    float v = acc * p.alpha;
    if (p.row_scale) v *= p.row_scale[row];
    if (p.bias) v += p.bias[row];
    CT *c = static_cast<CT *>(p.C) + (int64_t)tok * p.ldc + row;
    if (p.beta != 0.0f) v += p.beta * to_float<CT>(*c);
    *c = from_float<CT>(v);
}


template <typename CT>
__global__ void __launch_bounds__(UM_THREADS, 1)
gemv_trit_umma_kernel(const __grid_constant__ CUtensorMap map_w, const UmParams p) {
    extern __shared__ uint8_t um_smem_raw[];
    const uint32_t base = (smem_u32(um_smem_raw) + 1023u) & ~1023u;
    uint8_t *gbase = um_smem_raw + (base - smem_u32(um_smem_raw));
    // [activations: limbs_per_slice * 6 k-groups * 256 B][ring][partials][barriers]
    const uint32_t xs_addr = base;
    const uint32_t ring = base + p.ring_offset;
    float *part = reinterpret_cast<float *>(gbase + p.part_offset);
    const uint32_t bars = base + p.bar_offset;
    auto ring_full = [&](int s) { return bars + 8u * s; };
    auto ring_empty = [&](int s) { return bars + 8u * (p.stages + s); };
    auto a_full = [&](int s) { return bars + 8u * (2 * p.stages + s); };
    auto a_free = [&](int s) { return bars + 8u * (2 * p.stages + UM_A_SLOTS + s); };
    const uint32_t d_full = bars + 8u * (2 * p.stages + 2 * UM_A_SLOTS);
    const uint32_t tmem_slot = bars + 8u * (2 * p.stages + 2 * UM_A_SLOTS + 1);
    volatile uint32_t *tmem_slot_gen = reinterpret_cast<volatile uint32_t *>(gbase + p.bar_offset + 8 * (2 * p.stages + 2 * UM_A_SLOTS + 1));

    cg::cluster_group cluster = cg::this_cluster();
    const int slices = (int)cluster.num_blocks();
    const int slice = (int)cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kl8 = (int)((p.kl + 7) & ~(int64_t)7);
    const int L0 = slice * p.limbs_per_slice;
    int nl = kl8 - L0;
    nl = nl < 0 ? 0 : (nl > p.limbs_per_slice ? p.limbs_per_slice : nl);
    const int nstages = nl / UM_STAGE_LIMBS;  // ring stages this CTA walks; two half stages of 4 limbs each
    const int64_t row0 = (int64_t)blockIdx.x * UM_ROWS;

    const bool trace = (p.debug & 16) && blockIdx.x == 0 && blockIdx.y == 0;
    if (threadIdx.x == 0) UM_TRACE(0);
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(ring_full(s), 1); mbar_init(ring_empty(s), UM_CONVERTER_WARPS); }
        for (int s = 0; s < UM_A_SLOTS; ++s) { mbar_init(a_full(s), UM_CONVERTER_WARPS); mbar_init(a_free(s), 1); }
        mbar_init(d_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == UM_CONVERTER_WARPS + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(UM_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot_gen;
    if (threadIdx.x == 0) UM_TRACE(1);
    // the next kernel of the stream may start; the weight stream below depends on no earlier kernel
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == UM_CONVERTER_WARPS) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool ok = true;
            for (int c = 0; c < nstages && ok; ++c) {
                const int st = c % p.stages;
                const uint32_t phase = (uint32_t)(c / p.stages) & 1u;
                ok = mbar_wait(ring_empty(st), phase ^ 1u);
                if (!ok) break;
                mbar_arrive_expect_tx(ring_full(st), UM_STAGE_BYTES);
                tma_load_2d(ring + (uint32_t)st * UM_STAGE_BYTES, &map_w, (L0 + UM_STAGE_LIMBS * c) * 16, (int)row0, ring_full(st));
                if (c == 0) UM_TRACE(3);
            }
            if (!ok) atomicCAS(&g_umma_status, UM_STATUS_OK, UM_TIMEOUT_PRODUCER);
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
    } else if (warp == UM_CONVERTER_WARPS + 1) {
        // ---------------- MMA issuer ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"n"((UM_CONVERTER_WARPS + 1) * 32) : "memory");  // activations are staged
        if (lane == 0) {
            bool ok = true;
            const int accs = (p.debug & 32) ? 1 : UM_ACCS;
            for (int hc = 0; hc < 2 * nstages && ok; ++hc) {  // half stages of 4 limbs
                const int slot = hc % UM_A_SLOTS;
                const uint32_t phase = (uint32_t)(hc / UM_A_SLOTS) & 1u;
                ok = mbar_wait(a_full(slot), phase);
                if (!ok) break;
                if (hc < 24) UM_TRACE(5 + hc);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (!(p.debug & 1)) {
#pragma unroll
                    for (int m = 0; m < 12; ++m) {  // 12 k-steps of 16 per half stage, rotating over the accumulators
                        const int acc = m % accs;
                        um_mma(tmem_base + (uint32_t)(16 * acc), tmem_base + (uint32_t)(UM_A_COL0 + slot * UM_A_COLS + m * 8),
                               um_b_desc(xs_addr + (uint32_t)(hc * 12 + m) * 512u), (hc != 0 || m >= accs) ? 1u : 0u);
                    }
                }
                um_commit(a_free(slot));
            }
            UM_TRACE(30);
            if (ok) um_commit(d_full);
            else atomicCAS(&g_umma_status, UM_STATUS_OK, UM_TIMEOUT_MMA);
        }
    } else {
        // ---------------- converters ----------------
        asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations may be the previous kernel's output
        // stage the activations: item = (token slot, limb); 24 permuted registers -> 6 pieces of 16 bytes
        {
            const __nv_bfloat16 *X = static_cast<const __nv_bfloat16 *>(p.X);
            const bool vec_ok = (reinterpret_cast<uintptr_t>(X) % 16 == 0) && (p.ldx % 8 == 0);
            for (int item = threadIdx.x; item < UM_TOK * nl; item += UM_CONVERTER_WARPS * 32) {
                const int tok = item % UM_TOK, l = item / UM_TOK;
                const int64_t k0 = (int64_t)(L0 + l) * 48;
                uint32_t o[24];
                if (tok >= p.ntok || k0 >= p.K) {
#pragma unroll
                    for (int r = 0; r < 24; ++r) o[r] = 0u;
                } else if (vec_ok && k0 + 48 <= p.K) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(X + (int64_t)tok * p.ldx + k0);
                    uint32_t n[24];
#pragma unroll
                    for (int q = 0; q < 6; ++q) {
                        const uint4 v = __ldg(src + q);
                        n[4 * q] = v.x; n[4 * q + 1] = v.y; n[4 * q + 2] = v.z; n[4 * q + 3] = v.w;
                    }
#pragma unroll
                    for (int pr = 0; pr < 8; ++pr) {
                        o[3 * pr + 0] = __byte_perm(n[3 * pr], n[3 * pr + 1], 0x7610);
                        o[3 * pr + 1] = __byte_perm(n[3 * pr], n[3 * pr + 2], 0x5432);
                        o[3 * pr + 2] = __byte_perm(n[3 * pr + 1], n[3 * pr + 2], 0x7610);
                    }
                } else {
                    for (int r = 0; r < 24; ++r) {
                        float e[2];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int64_t k = k0 + decoded_trit_index(r, h);
                            e[h] = k < p.K ? __bfloat162float(X[(int64_t)tok * p.ldx + k]) : 0.0f;
                        }
                        const __nv_bfloat162 v = __floats2bfloat162_rn(e[0], e[1]);
                        o[r] = *reinterpret_cast<const uint32_t *>(&v);
                    }
                }
                uint8_t *dst = gbase + (size_t)l * 6 * 256 + (tok >> 3) * 128 + (tok & 7) * 16;
#pragma unroll
                for (int q = 0; q < 6; ++q)
                    *reinterpret_cast<uint4 *>(dst + q * 256) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads them through the async proxy
            asm volatile("bar.sync 1, %0;" ::"n"((UM_CONVERTER_WARPS + 1) * 32) : "memory");
        }
        if (threadIdx.x == 0) UM_TRACE(2);

        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
        const int j = warp >> 2;       // limb j of each half stage
        const int row_local = quarter * 32 + lane;
        const uint32_t lane_field = (uint32_t)(quarter * 32) << 16;
        // 128-byte swizzle of the tensor map: 16-byte piece q of row r sits at piece q ^ (r & 7),
        // which spreads the 32 rows a warp reads over all banks
        const uint8_t *my_row = gbase + p.ring_offset + row_local * 128;
        const int piece0 = (j ^ (row_local & 7)) << 4, piece1 = ((j + 4) ^ (row_local & 7)) << 4;
        const uint4 zero_limb = make_uint4(kZeroTryteWord, kZeroTryteWord, kZeroTryteWord, kZeroTryteWord);
        bool ok = true;
        for (int c = 0; c < nstages; ++c) {
            const int st = c % p.stages;
            ok = __all_sync(0xffffffffu, mbar_wait(ring_full(st), (uint32_t)(c / p.stages) & 1u));
            if (!ok) break;
            if (threadIdx.x == 0 && c == 0) UM_TRACE(4);
            uint4 limb0 = *reinterpret_cast<const uint4 *>(my_row + st * UM_STAGE_BYTES + piece0);
            uint4 limb1 = *reinterpret_cast<const uint4 *>(my_row + st * UM_STAGE_BYTES + piece1);
            __syncwarp();
            if (lane == 0) mbar_arrive(ring_empty(st));
            const int64_t l_abs = (int64_t)L0 + UM_STAGE_LIMBS * c + j;
            if (l_abs >= p.kl) limb0 = zero_limb;  // past the row's last limb
            if (l_abs + 4 >= p.kl) limb1 = zero_limb;
            uint32_t w0[24], w1[24];
            if (p.debug & 2) {
#pragma unroll
                for (int r = 0; r < 24; ++r) { w0[r] = (&limb0.x)[r & 3]; w1[r] = (&limb1.x)[r & 3]; }
            } else {
                decode_limb(limb0, w0);
                decode_limb(limb1, w1);
            }
            const int slot0 = (2 * c) % UM_A_SLOTS, slot1 = slot0 + 1;
            const uint32_t free_parity = ((uint32_t)((2 * c) / UM_A_SLOTS) & 1u) ^ 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(a_free(slot0), free_parity) && mbar_wait(a_free(slot1), free_parity));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t0 = tmem_base + lane_field + (uint32_t)(UM_A_COL0 + slot0 * UM_A_COLS + j * 24);
            const uint32_t t1 = t0 + UM_A_COLS;
            if (!(p.debug & 4)) {
                um_st8(t0, w0);
                um_st8(t0 + 8, w0 + 8);
                um_st8(t0 + 16, w0 + 16);
                um_st8(t1, w1);
                um_st8(t1 + 8, w1 + 8);
                um_st8(t1 + 16, w1 + 16);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            } else if (w0[0] + w0[7] + w1[13] + w1[23] == 0x12345) {
                part[0] = 1.0f;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) { mbar_arrive(a_full(slot0)); mbar_arrive(a_full(slot1)); }
        }
        if (!ok && lane == 0) atomicCAS(&g_umma_status, UM_STATUS_OK, UM_TIMEOUT_CONVERTER);

        // ---------------- epilogue (warps 0..3, one TMEM lane quarter each) ----------------
        if (warp < 4) {
            bool eok = ok && (nstages == 0 || __all_sync(0xffffffffu, mbar_wait(d_full, 0)));
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
            if (eok && nstages > 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int accs = (p.debug & 32) ? 1 : UM_ACCS;
                for (int a = 0; a < accs; ++a) {
                    uint32_t v[16];
                    um_ld16(tmem_base + lane_field + (uint32_t)(16 * a), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[i] += __uint_as_float(v[i]);
                }
            } else if (!eok && lane == 0) {
                atomicCAS(&g_umma_status, UM_STATUS_OK, UM_TIMEOUT_EPILOGUE);
            }
            if (slices == 1) {
#pragma unroll
                for (int i = 0; i < 16; ++i) um_store_out<CT>(p, row0 + row_local, i, acc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) part[row_local * UM_TOK + i] = acc[i];
            }
        }
    }

    if (threadIdx.x == 0) UM_TRACE(31);
    if (slices > 1) {
        cluster.sync();
        const int span = (UM_ROWS + slices - 1) / slices;
        const int lo = slice * span;
        const int hi = lo + span < UM_ROWS ? lo + span : UM_ROWS;
        for (int idx = lo * UM_TOK + threadIdx.x; idx < hi * UM_TOK; idx += UM_THREADS) {
            float s = 0.0f;
            for (int rk = 0; rk < slices; ++rk) s += cluster.map_shared_rank(part, rk)[idx];
            um_store_out<CT>(p, row0 + idx / UM_TOK, idx % UM_TOK, s);
        }
        cluster.sync();
    }
    // ---------------- teardown ----------------
    if (threadIdx.x == 0) UM_TRACE(32);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == UM_CONVERTER_WARPS + 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(UM_TMEM_COLS) : "memory");
    }
}

}  // namespace

namespace {

template <typename CT>
int um_launch(const CUtensorMap &map, const UmParams &p, int slices, size_t smem_bytes, cudaStream_t st) {
    auto kern = gemv_trit_umma_kernel<CT>;
    T81_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    if (slices > 8) T81_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((p.M + UM_ROWS - 1) / UM_ROWS), (unsigned)slices, 1);
    cfg.blockDim = dim3(UM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)slices;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    static const bool pdl = !(getenv("T81B200_NO_PDL"));
    cfg.numAttrs = pdl ? 2 : 1;
    T81_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, map, p));
    return T81B200_OK;
}

}  // namespace

// bf16 activations, token-major, 1..16 tokens, 16-byte aligned weights.  Returns T81B200_EALIGN when
// the shape does not fit this kernel (the caller then takes the mma.sync kernel).
int gemv_trit_umma_launch(const uint8_t *A, const float *row_scale, const void *X, int64_t ldx, const float *bias,
                          void *C, int c_dtype, int64_t ldc, int64_t M, int ntok, int64_t K, float alpha, float beta,
                          cudaStream_t st) {
    if (ntok < 1 || ntok > UM_TOK || M < 1 || K < 1) return T81B200_EALIGN;
    if (reinterpret_cast<uintptr_t>(A) % 16 != 0) return T81B200_EALIGN;
    UmParams p;
    p.X = X; p.row_scale = row_scale; p.bias = bias; p.C = C;
    p.M = M; p.K = K; p.kl = (K + 47) / 48; p.ldx = ldx; p.ldc = ldc; p.ntok = ntok;
    p.alpha = alpha; p.beta = beta;
    p.debug = getenv("T81B200_UMMA_DEBUG") ? atoi(getenv("T81B200_UMMA_DEBUG")) : 0;
    const int kl8 = (int)((p.kl + 7) & ~(int64_t)7);
    const int sms = sm_count();
    const size_t budget = 227 * 1024 - 1024;  // dynamic shared memory minus the alignment slack
    const int64_t row_blocks = (M + UM_ROWS - 1) / UM_ROWS;
    int forced_s = 0;  // T81B200_GEMV_UMMA_CFG="slices" (sweeps)
    if (const char *env = getenv("T81B200_GEMV_UMMA_CFG")) sscanf(env, "%d", &forced_s);
    int best_s = 0, best_lps = 0, best_stages = 0;
    double best_t = 1e30;
    for (int s = 1; s <= 8; s *= 2) {
        if (forced_s && s != forced_s) continue;
        const int lps = (kl8 / UM_STAGE_LIMBS + s - 1) / s * UM_STAGE_LIMBS;
        if (s > 1 && (int64_t)(s - 1) * lps >= kl8) continue;  // an empty slice
        const int nst = lps / UM_STAGE_LIMBS;
        const size_t xs_bytes = ((size_t)lps * 6 * 256 + 1023) & ~(size_t)1023;
        const size_t fixed_bytes = xs_bytes + (size_t)UM_ROWS * UM_TOK * 4 + 8 * (2 * UM_MAX_STAGES + 2 * UM_A_SLOTS + 2);
        if (fixed_bytes + 2 * (size_t)UM_STAGE_BYTES > budget) continue;
        int stages = (int)((budget - fixed_bytes) / UM_STAGE_BYTES);
        if (stages > UM_MAX_STAGES) stages = UM_MAX_STAGES;
        if (stages > nst) stages = nst;
        // one CTA per SM; clusters must fit inside a GPC, so fewer CTAs are co-resident than there are SMs
        const double wave_ctas = s == 1 ? sms : (s == 2 ? sms - 8 : (s == 4 ? sms - 20 : sms - 36));
        const double waves = ceil((double)row_blocks * s / wave_ctas);
        const double work = nst * 1200.0 / 1.9e9;               // converter time per 16 KB stage
        const double staging = (double)UM_TOK * lps * 96 / 1.0e11;
        const double t = waves * (2.5e-6 + (s > 1 ? 0.7e-6 : 0.0) + staging + work);
        if (t < best_t) { best_t = t; best_s = s; best_lps = lps; best_stages = stages; }
    }
    if (!best_s) return T81B200_EALIGN;
    p.limbs_per_slice = best_lps;
    p.stages = best_stages;
    const size_t xs_bytes = ((size_t)best_lps * 6 * 256 + 1023) & ~(size_t)1023;
    p.ring_offset = (int)xs_bytes;
    p.part_offset = (int)(xs_bytes + (size_t)best_stages * UM_STAGE_BYTES);
    p.bar_offset = p.part_offset + UM_ROWS * UM_TOK * 4;
    const size_t smem = (size_t)p.bar_offset + 8 * (2 * (size_t)best_stages + 2 * UM_A_SLOTS + 2) + 1024;
    CUtensorMap map;
    if (int rc = make_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)p.kl * 16, (uint64_t)M,
                             (uint64_t)p.kl * 16, UM_STAGE_LIMBS * 16, UM_ROWS, CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;
    switch (c_dtype) {
        case T81B200_F32: return um_launch<float>(map, p, best_s, smem, st);
        case T81B200_BF16: return um_launch<__nv_bfloat16>(map, p, best_s, smem, st);
        case T81B200_F16: return um_launch<__half>(map, p, best_s, smem, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown output dtype %d", c_dtype);
}

int gemv_trit_umma_status(int reset) {
    int v = 0;
    if (getenv("T81B200_UMMA_TRACE")) {
        long long t[64];
        if (cudaMemcpyFromSymbol(t, g_umma_trace, sizeof t) == cudaSuccess) {
            fprintf(stderr, "umma trace (cycles from entry):");
            for (int i = 1; i < 33; ++i) fprintf(stderr, " %d:%lld", i, t[i] ? t[i] - t[0] : -1);
            fprintf(stderr, "\n");
        }
    }
    if (cudaMemcpyFromSymbol(&v, g_umma_status, sizeof v) != cudaSuccess) return T81B200_ECUDA;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_umma_status, &zero, sizeof zero) != cudaSuccess) return T81B200_ECUDA;
    }
    return v;
}

}  // namespace t81b200
