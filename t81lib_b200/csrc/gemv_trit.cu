// Decode-shaped TRIT-mode kernel: packed ternary weights (M rows) times up to 16
// activation rows (tokens).  The weight stream is the only large operand, so the
// kernel is HBM-bound by design: each lane pulls whole 16-byte limbs with 128-bit
// loads, expands them to exact bf16 {-1,0,+1} in registers with packed bf16 FMAs
// (common.cuh), and feeds them straight into mma.sync m16n8k16 as the A fragment —
// the expanded weights never touch shared or global memory.
//
// Work split
//   CTA    : W = 8 or 16 warps arranged as RW row groups (16 rows each) x W/RW slices of
//            the contraction; the slices' partial sums meet in shared memory.
//   grid.x : row tiles of 16*RW*RG rows (RG groups walked in sequence)
//   grid.y : S more slices of the contraction, S = cluster size (1..8), for shapes with
//            too few rows to fill the GPU.  The S CTAs of a cluster combine their partial
//            sums through distributed shared memory in rank order (deterministic): no
//            global scratch and no atomics are involved.
//   lane (g = lane/4, t = lane%4) of a warp loads, for each chunk of 4 limbs,
//   limb 4c+t of rows g and g+8.  The order of the contraction index inside an
//   MMA is free as long as both operands agree, so the activations are staged in
//   shared memory already permuted into the register order decode_limb produces.
#include "common.cuh"
#include "tma.cuh"
#include "exchange.cuh"

#include <cooperative_groups.h>

#include <cmath>
#include <cstdlib>

namespace cg = cooperative_groups;

namespace t81b200 {

namespace {


struct GemvParams {
    const uint8_t *A;       // (M, kl, 16)
    const void *X;          // (ntok, K) row-major, ldx elements
    const float *row_scale; // M or null
    const float *bias;      // M or null
    void *C;                // (ntok, M) row-major, ldc elements
    int64_t M, K, kl, ldx, ldc;
    int ntok;
    int limbs_per_slice;    // multiple of 4
    int row_groups;         // RG: 16-row groups each row-warp walks in sequence
    int row_warps;          // RW: warps side by side along the rows; W/RW warps split the contraction
    float alpha, beta;
    int n_peers;            // other GPUs whose result receives every output element too
    void *peer_C[T81B200_MAX_PEERS];
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// Stage the activations of limbs [L0, L0+nl) for `ntok` tokens into shared memory in
// decode_limb register order.  Plane 0 holds bf16(x); plane 1 (PLANES == 2) holds
// bf16(x - plane0), so that plane0 + plane1 carries 16 mantissa bits of an fp32 input.
template <typename XT, int PLANES>
__device__ __forceinline__ void stage_activations(const GemvParams &p, int L0, int nl, uint32_t *xs,
                                                  int tok_stride, int plane_stride, int THREADS) {
    const XT *X = static_cast<const XT *>(p.X);
    const bool vec_ok = sizeof(XT) == 2 && (reinterpret_cast<uintptr_t>(X) % 16 == 0) && (p.ldx % 8 == 0);
    for (int item = threadIdx.x; item < p.ntok * nl; item += THREADS) {
        const int tok = item / nl, l = item - tok * nl;
        const int64_t k0 = (int64_t)(L0 + l) * 48;
        uint32_t *dst = xs + tok * tok_stride + l * 24;
        if constexpr (PLANES == 1) {
            if (vec_ok && k0 + 48 <= p.K) {
                const uint4 *src = reinterpret_cast<const uint4 *>(X + (int64_t)tok * p.ldx + k0);
                uint32_t n[24];
#pragma unroll
                for (int q = 0; q < 6; ++q) {
                    const uint4 v = __ldg(src + q);
                    n[4 * q] = v.x; n[4 * q + 1] = v.y; n[4 * q + 2] = v.z; n[4 * q + 3] = v.w;
                }
                uint32_t o[24];
#pragma unroll
                for (int pr = 0; pr < 8; ++pr) {
                    o[3 * pr + 0] = __byte_perm(n[3 * pr], n[3 * pr + 1], 0x7610);
                    o[3 * pr + 1] = __byte_perm(n[3 * pr], n[3 * pr + 2], 0x5432);
                    o[3 * pr + 2] = __byte_perm(n[3 * pr + 1], n[3 * pr + 2], 0x7610);
                }
#pragma unroll
                for (int q = 0; q < 6; ++q)
                    reinterpret_cast<uint4 *>(dst)[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
                continue;
            }
        }
        for (int r = 0; r < 24; ++r) {
            float e[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t k = k0 + decoded_trit_index(r, h);
                e[h] = k < p.K ? to_float<XT>(X[(int64_t)tok * p.ldx + k]) : 0.0f;
            }
            const uint32_t hi = pack_bf16(e[0], e[1]);
            dst[r] = hi;
            if constexpr (PLANES == 2) {
                const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162 *>(&hi);
                dst[plane_stride + r] = pack_bf16(e[0] - __low2float(hv), e[1] - __high2float(hv));
            }
        }
    }
}

template <typename CT>
__device__ __forceinline__ void store_out(const GemvParams &p, int64_t row, int tok, float acc) {
    if (row >= p.M || tok >= p.ntok) return;
    float v = acc * p.alpha;
    if (p.row_scale) v *= p.row_scale[row];
    if (p.bias) v += p.bias[row];
    CT *c = static_cast<CT *>(p.C) + (int64_t)tok * p.ldc + row;
    if (p.beta != 0.0f) v += p.beta * to_float<CT>(*c);
    const CT out = from_float<CT>(v);
    *c = out;
    for (int pj = 0; pj < p.n_peers; ++pj) static_cast<CT *>(p.peer_C[pj])[(int64_t)tok * p.ldc + row] = out;
}

template <typename XT> struct Planes { static constexpr int value = 2; };
template <> struct Planes<__nv_bfloat16> { static constexpr int value = 1; };

// VAR 0: whole limbs decoded at once, 4 chunks in flight, one CTA per SM (up to 128 registers).
// VAR 1: half limbs at a time, 2 chunks in flight, two CTAs per SM (64 registers): twice the
//        resident warps to hide the latency of the dependent decode chains.
template <typename XT, typename CT, int TOKB, int WARPS, int VAR>
__global__ void __launch_bounds__(WARPS * 32, VAR == 1 ? (WARPS == 8 ? 4 : 2) : 1) gemv_trit_kernel(const GemvParams p) {
    constexpr int kPrefetch = VAR == 1 ? 2 : 4;  // chunks of 4 limbs in flight per lane
    constexpr int PLANES = Planes<XT>::value;
    constexpr int THREADS = WARPS * 32;
    constexpr int kTokPad = 8 * TOKB;
    extern __shared__ __align__(16) uint32_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int slices = (int)cluster.num_blocks();
    const int slice = (int)cluster.block_rank();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rw = warp % p.row_warps;   // which 16-row group of the tile
    const int kw = warp / p.row_warps;   // which slice of the CTA's contraction range
    const int k_warps = WARPS / p.row_warps;
    const int kl4 = (int)((p.kl + 3) & ~(int64_t)3);
    const int L0 = slice * p.limbs_per_slice;
    int nl = kl4 - L0;
    nl = nl < 0 ? 0 : (nl > p.limbs_per_slice ? p.limbs_per_slice : nl);

    // shared memory: [activations: PLANES x ntok x tok_stride] [partials: k_warps x rows x kTokPad floats]
    const int tok_stride = p.limbs_per_slice * 24 + 4;  // +16 bytes: conflict-free 128-bit reads
    const int plane_stride = p.ntok * tok_stride;
    uint32_t *xs = smem;
    float *part = reinterpret_cast<float *>(smem + PLANES * plane_stride);
    const int rows_per_cta = p.row_warps * 16 * p.row_groups;
    const int64_t cta_row0 = (int64_t)blockIdx.x * rows_per_cta;

    // chunk range (4 limbs per chunk) of this warp inside the CTA's range
    const int chunks_cta = nl >> 2;
    const int cpw = (chunks_cta + k_warps - 1) / k_warps;
    const int c_begin = kw * cpw < chunks_cta ? kw * cpw : chunks_cta;
    const int c_end = c_begin + cpw < chunks_cta ? c_begin + cpw : chunks_cta;
    const int last_limb = (int)p.kl - 1;

    // Row pointers of row group `rg` for this lane (clamped: rows >= M are never stored).
    const uint4 *pa, *pb;
    auto set_rows = [&](int rg) {
        const int64_t r0 = cta_row0 + (int64_t)(rg * p.row_warps + rw) * 16;
        int64_t ra = r0 + g, rb = r0 + g + 8;
        ra = ra < p.M ? ra : p.M - 1;
        rb = rb < p.M ? rb : p.M - 1;
        pa = reinterpret_cast<const uint4 *>(p.A) + ra * p.kl;
        pb = reinterpret_cast<const uint4 *>(p.A) + rb * p.kl;
    };
    // Limb index of chunk c for this lane.  Past the row's last limb the last limb is read
    // again: the activations staged for those positions are zero, so it contributes nothing.
    auto limb_of = [&](int c) {
        const int l = L0 + 4 * c + t;
        return l < last_limb ? l : last_limb;
    };
    uint4 qa[kPrefetch], qb[kPrefetch];
    auto prefetch_head = [&]() {
#pragma unroll
        for (int s = 0; s < kPrefetch; ++s) {
            const int l = limb_of(c_begin + s < c_end ? c_begin + s : c_begin);
            qa[s] = ldg_stream(pa + l);
            qb[s] = ldg_stream(pb + l);
        }
    };

    // The weight stream does not depend on shared memory: get its first loads in flight
    // before the activations are staged.
    set_rows(0);
    if (c_begin < c_end) prefetch_head();
    stage_activations<XT, PLANES>(p, L0, nl, xs, tok_stride, plane_stride, THREADS);
    __syncthreads();

    // lanes whose token does not exist read token 0; their results are never stored
    int tok_off[TOKB];
#pragma unroll
    for (int b = 0; b < TOKB; ++b) tok_off[b] = (8 * b + g < p.ntok ? 8 * b + g : 0) * tok_stride + t * 24;

    for (int rg = 0; rg < p.row_groups; ++rg) {
        float acc[TOKB][4];
#pragma unroll
        for (int b = 0; b < TOKB; ++b) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f;

        for (int c0 = c_begin; c0 < c_end; c0 += kPrefetch) {
#pragma unroll
            for (int s = 0; s < kPrefetch; ++s) {
                const int c = c0 + s;
                if (c < c_end) {
                    const uint4 la = qa[s], lb = qb[s];
                    const int cn = c + kPrefetch;
                    if (cn < c_end) {
                        const int l = limb_of(cn);
                        qa[s] = ldg_stream(pa + l);
                        qb[s] = ldg_stream(pb + l);
                    }
                    if constexpr (VAR == 0) {
                        uint32_t wa[24], wb[24];
                        decode_limb(la, wa);
                        decode_limb(lb, wb);
#pragma unroll
                        for (int b = 0; b < TOKB; ++b) {
#pragma unroll
                            for (int pl = 0; pl < PLANES; ++pl) {
                                const uint4 *xv = reinterpret_cast<const uint4 *>(xs + pl * plane_stride + tok_off[b] + c * 96);
#pragma unroll
                                for (int q = 0; q < 6; ++q) {
                                    const uint4 x = xv[q];
                                    mma_bf16_16816(acc[b], wa[4 * q], wb[4 * q], wa[4 * q + 1], wb[4 * q + 1], x.x, x.y);
                                    mma_bf16_16816(acc[b], wa[4 * q + 2], wb[4 * q + 2], wa[4 * q + 3], wb[4 * q + 3], x.z, x.w);
                                }
                            }
                        }
                    } else {
                        const uint32_t aw[4] = {la.x, la.y, la.z, la.w}, bw[4] = {lb.x, lb.y, lb.z, lb.w};
#pragma unroll
                        for (int h = 0; h < 2; ++h) {  // words 2h, 2h+1 -> decode registers 12h .. 12h+11
                            uint32_t wa[12], wb[12];
                            decode_words(aw[2 * h], aw[2 * h + 1], wa);
                            decode_words(bw[2 * h], bw[2 * h + 1], wb);
#pragma unroll
                            for (int b = 0; b < TOKB; ++b) {
#pragma unroll
                                for (int pl = 0; pl < PLANES; ++pl) {
                                    const uint4 *xv = reinterpret_cast<const uint4 *>(xs + pl * plane_stride + tok_off[b] + c * 96 + 12 * h);
#pragma unroll
                                    for (int q = 0; q < 3; ++q) {
                                        const uint4 x = xv[q];
                                        mma_bf16_16816(acc[b], wa[4 * q], wb[4 * q], wa[4 * q + 1], wb[4 * q + 1], x.x, x.y);
                                        mma_bf16_16816(acc[b], wa[4 * q + 2], wb[4 * q + 2], wa[4 * q + 3], wb[4 * q + 3], x.z, x.w);
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }

        if (rg + 1 < p.row_groups) {  // next group's first loads overlap this group's stores
            set_rows(rg + 1);
            if (c_begin < c_end) prefetch_head();
        }

        // acc[b][0]: (row g, token 8b+2t), [1]: (row g, 8b+2t+1), [2]: (row g+8, 8b+2t), [3]: (row g+8, 8b+2t+1)
        const int lr = (rg * p.row_warps + rw) * 16;  // local row of this warp's group
        float *pw = part + (size_t)kw * rows_per_cta * kTokPad;
#pragma unroll
        for (int b = 0; b < TOKB; ++b) {
            *reinterpret_cast<float2 *>(pw + (lr + g) * kTokPad + 8 * b + 2 * t) = make_float2(acc[b][0], acc[b][1]);
            *reinterpret_cast<float2 *>(pw + (lr + g + 8) * kTokPad + 8 * b + 2 * t) = make_float2(acc[b][2], acc[b][3]);
        }
    }
    __syncthreads();

    // Fold the k-warps' partials in a fixed order (deterministic), then, with more than one
    // CTA per cluster, the ranks' partials through distributed shared memory.
    const int outs = rows_per_cta * kTokPad;
    if (slices == 1) {
        for (int o = threadIdx.x; o < outs; o += THREADS) {
            // with peers: rows fastest, so that a warp stores runs of consecutive rows of one token over NVLink
            const int r = p.n_peers > 0 ? o % rows_per_cta : o / kTokPad, tk = p.n_peers > 0 ? o / rows_per_cta : o % kTokPad;
            const int idx = r * kTokPad + tk;
            float s = part[idx];
            for (int w = 1; w < k_warps; ++w) s += part[(size_t)w * outs + idx];
            store_out<CT>(p, cta_row0 + r, tk, s);
        }
    } else {
        for (int idx = threadIdx.x; idx < outs; idx += THREADS) {
            float s = part[idx];
            for (int w = 1; w < k_warps; ++w) s += part[(size_t)w * outs + idx];
            part[idx] = s;
        }
        cluster.sync();
        // CTA `slice` finishes rows [slice*span, (slice+1)*span) of the tile, summing ranks 0..S-1 in order.
        const int span = (rows_per_cta + slices - 1) / slices;
        const int lo = slice * span;
        const int hi = lo + span < rows_per_cta ? lo + span : rows_per_cta;
        for (int o = threadIdx.x; o < (hi - lo) * kTokPad; o += THREADS) {
            const int r = lo + (p.n_peers > 0 ? o % (hi - lo) : o / kTokPad), tk = p.n_peers > 0 ? o / (hi - lo) : o % kTokPad;
            const int idx = r * kTokPad + tk;
            float s = 0.0f;
            for (int rk = 0; rk < slices; ++rk) s += cluster.map_shared_rank(part, rk)[idx];
            store_out<CT>(p, cta_row0 + r, tk, s);
        }
        cluster.sync();  // peers may still be reading this CTA's partials
    }
}

template <typename XT, typename CT, int TOKB, int WARPS, int VAR>
int launch(const GemvParams &p, int slices, size_t smem_bytes, cudaStream_t st) {
    auto kern = gemv_trit_kernel<XT, CT, TOKB, WARPS, VAR>;
    if (smem_bytes > 48 * 1024)
        T81_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    const int rows_per_cta = p.row_warps * 16 * p.row_groups;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((p.M + rows_per_cta - 1) / rows_per_cta), (unsigned)slices, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)slices;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    T81_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    return T81B200_OK;
}

template <typename XT, typename CT, int VAR>
int launch_tokb(const GemvParams &p, int warps, int slices, size_t smem_bytes, cudaStream_t st) {
    if (p.ntok > 8)
        return warps == 8 ? launch<XT, CT, 2, 8, VAR>(p, slices, smem_bytes, st) : launch<XT, CT, 2, 16, VAR>(p, slices, smem_bytes, st);
    return warps == 8 ? launch<XT, CT, 1, 8, VAR>(p, slices, smem_bytes, st) : launch<XT, CT, 1, 16, VAR>(p, slices, smem_bytes, st);
}

template <typename XT>
int launch_ct(const GemvParams &p, int c_dtype, int warps, int slices, size_t smem_bytes, int variant, cudaStream_t st) {
    // the two-CTAs-per-SM variant is built for the bf16 -> bf16 case only (the decode hot path)
    if constexpr (Planes<XT>::value == 1)
        if (variant == 1 && c_dtype == T81B200_BF16)
            return launch_tokb<XT, __nv_bfloat16, 1>(p, warps, slices, smem_bytes, st);
    switch (c_dtype) {
        case T81B200_F32: return launch_tokb<XT, float, 0>(p, warps, slices, smem_bytes, st);
        case T81B200_BF16: return launch_tokb<XT, __nv_bfloat16, 0>(p, warps, slices, smem_bytes, st);
        case T81B200_F16: return launch_tokb<XT, __half, 0>(p, warps, slices, smem_bytes, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown output dtype %d", c_dtype);
}

// ---------------------------------------------------------------------------------------------
// TMA-fed variant.  The register-prefetch kernel above keeps at most a few KB per warp in
// flight, and measured throughput follows bytes-in-flight / latency, far below HBM speed.
// Here one producer thread streams the weight tile (16*RW rows x 64 bytes = one 4-limb chunk
// per row) through a deep shared-memory ring with cp.async.bulk.tensor, so the bytes in flight
// per SM are set by the ring size (tens of KB), not by registers.  16 consumer warps
// (RW row groups x KW interleaved K slices: warp (rw, kw) takes chunks kw, kw+KW, ...) read
// their two limbs per chunk with conflict-free 128-bit shared loads, release the slot at once,
// and decode / multiply exactly as above.
// ---------------------------------------------------------------------------------------------

constexpr int kTmaMaxConsumerWarps = 16;
constexpr int kTmaMaxThreads = (kTmaMaxConsumerWarps + 1) * 32;
constexpr int kTmaMaxStages = 48;

enum { GEMV_STATUS_OK = 0, GEMV_STATUS_TIMEOUT_PRODUCER = 5, GEMV_STATUS_TIMEOUT_CONSUMER = 6, GEMV_STATUS_TIMEOUT_EXCHANGE = 7 };
__device__ int g_gemv_status = 0;

struct GemvTmaParams {
    GemvParams g;
    int consumer_warps;  // RW * KW <= 16; one more warp produces
    int stages;        // ring depth
    int stage_bytes;   // 16*RW*64
    int ring_offset;   // bytes from the start of dynamic shared memory (128-byte aligned)
    int part_offset;   // bytes: partial sums, KW x rows x tokpad floats
    int bar_offset;    // bytes: full[stages], empty[stages]
    int independent;   // 1: reads nothing the previous kernel of the stream wrote (see t81b200_hint_independent)
    uint32_t *sync_local;                     // exchange flags (null: no exchange protocol in this launch)
    uint32_t *sync_peer[T81B200_MAX_PEERS];   // this rank's slot in each peer's flags
};

template <typename XT, typename CT, int TOKB>
__global__ void __launch_bounds__(kTmaMaxThreads, 1)
gemv_trit_tma_kernel(const __grid_constant__ CUtensorMap map_w, const GemvTmaParams tp) {
    constexpr int PLANES = Planes<XT>::value;
    constexpr int kTokPad = 8 * TOKB;
    const int consumer_threads = tp.consumer_warps * 32;
    const int all_threads = consumer_threads + 32;
    const GemvParams &p = tp.g;
    extern __shared__ __align__(128) uint8_t smem_bytes_tma[];
    uint32_t *xs = reinterpret_cast<uint32_t *>(smem_bytes_tma);
    float *part = reinterpret_cast<float *>(smem_bytes_tma + tp.part_offset);
    const uint32_t ring = smem_u32(smem_bytes_tma + tp.ring_offset);
    const uint32_t bars = smem_u32(smem_bytes_tma + tp.bar_offset);
    auto full_bar = [&](int st) { return bars + 8u * st; };
    auto empty_bar = [&](int st) { return bars + 8u * (tp.stages + st); };

    cg::cluster_group cluster = cg::this_cluster();
    const int slices = (int)cluster.num_blocks();
    const int slice = (int)cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int k_warps = tp.consumer_warps / p.row_warps;
    const int kl4 = (int)((p.kl + 3) & ~(int64_t)3);
    const int L0 = slice * p.limbs_per_slice;
    int nl = kl4 - L0;
    nl = nl < 0 ? 0 : (nl > p.limbs_per_slice ? p.limbs_per_slice : nl);
    const int chunks_cta = nl >> 2;
    const int tok_stride = p.limbs_per_slice * 24 + 4;
    const int plane_stride = p.ntok * tok_stride;
    const int rows_per_cta = p.row_warps * 16;
    const int64_t cta_row0 = (int64_t)blockIdx.x * rows_per_cta;

    if (threadIdx.x == 0) {
        for (int st = 0; st < tp.stages; ++st) { mbar_init(full_bar(st), 1); mbar_init(empty_bar(st), p.row_warps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // Programmatic dependent launch: the next kernel in the stream may start now (it will wait
    // for this one where it needs to).  The weight stream below depends on no earlier kernel,
    // so it starts before the wait; activations, C and every store come after it.
    // A kernel that depends on its predecessor lets its own successor start only once its input is
    // complete (after its wait below); one that does not depend on it has nothing to wait for here:
    // it lets the successor start at once and waits for the predecessor at its very end instead, so
    // that "this grid has completed" still implies "everything before it has".
    if (tp.independent) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Several accumulator sets: consecutive MMAs of a chunk do not wait for one another.
    constexpr int NACC = 4;
    float acc[NACC][TOKB][4];
#pragma unroll
    for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int b = 0; b < TOKB; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.0f;
    int rw = 0, kw = 0;

    if (warp == tp.consumer_warps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            bool ok = true;
            for (int c = 0; c < chunks_cta && ok; ++c) {
                const int st = c % tp.stages;
                const uint32_t phase = (uint32_t)(c / tp.stages) & 1u;
                ok = mbar_wait(empty_bar(st), phase ^ 1u);
                if (!ok) break;
                mbar_arrive_expect_tx(full_bar(st), (uint32_t)tp.stage_bytes);
                tma_load_2d(ring + (uint32_t)st * tp.stage_bytes, &map_w, (L0 + 4 * c) * 16, (int)cta_row0, full_bar(st));
            }
            if (!ok) atomicCAS(&g_gemv_status, GEMV_STATUS_OK, GEMV_STATUS_TIMEOUT_PRODUCER);
        }
        if (!tp.independent) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // before this warp's share of the output stores
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
    } else {
        // ---------------- consumers ----------------
        rw = warp % p.row_warps;
        kw = warp / p.row_warps;
        if (!tp.independent) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations may be the previous kernel's output
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        }
        if (tp.sync_local) {
            // ... or what the peers stored into this GPU's memory: wait until all of them have published
            if (threadIdx.x == 0 && !exchange_wait(tp.sync_local, p.n_peers))
                atomicCAS(&g_gemv_status, GEMV_STATUS_OK, GEMV_STATUS_TIMEOUT_EXCHANGE);
            asm volatile("bar.sync 1, %0;" ::"r"(consumer_threads) : "memory");
        }
        stage_activations<XT, PLANES>(p, L0, nl, xs, tok_stride, plane_stride, consumer_threads);
        asm volatile("bar.sync 1, %0;" ::"r"(consumer_threads) : "memory");  // consumers only; the producer is already streaming

        int tok_off[TOKB];
#pragma unroll
        for (int b = 0; b < TOKB; ++b) tok_off[b] = (8 * b + g < p.ntok ? 8 * b + g : 0) * tok_stride + t * 24;
        const uint32_t lane_off = (uint32_t)((rw * 16 + g) * 64 + t * 16);
        bool ok = true;
        for (int c = kw; c < chunks_cta; c += k_warps) {
            const int st = c % tp.stages;
            const uint32_t phase = (uint32_t)(c / tp.stages) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(st), phase));
            if (!ok) break;
            const uint8_t *tile = smem_bytes_tma + tp.ring_offset + st * tp.stage_bytes + lane_off;
            const uint4 la = *reinterpret_cast<const uint4 *>(tile);
            const uint4 lb = *reinterpret_cast<const uint4 *>(tile + 8 * 64);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(st));  // the limbs are in registers: the slot can be refilled
            // activations of this chunk first (their latency hides behind the first decode), then,
            // word by word: decode 4 + 4 trytes, issue the 3 MMAs that consume them.
            uint4 xr[TOKB][PLANES][6];
#pragma unroll
            for (int b = 0; b < TOKB; ++b)
#pragma unroll
                for (int pl = 0; pl < PLANES; ++pl) {
                    const uint4 *xv = reinterpret_cast<const uint4 *>(xs + pl * plane_stride + tok_off[b] + c * 96);
#pragma unroll
                    for (int q = 0; q < 6; ++q) xr[b][pl][q] = xv[q];
                }
            const uint32_t aw[4] = {la.x, la.y, la.z, la.w}, bw[4] = {lb.x, lb.y, lb.z, lb.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                uint32_t oa[6], ob[6];
                decode_word_pair(aw[w], bw[w], oa, ob);
#pragma unroll
                for (int b = 0; b < TOKB; ++b)
#pragma unroll
                    for (int pl = 0; pl < PLANES; ++pl) {
                        // registers 6w .. 6w+5 of the limb <-> activation registers 6w .. 6w+5
                        const uint32_t *xw = reinterpret_cast<const uint32_t *>(&xr[b][pl][0]) + 6 * w;
                        mma_bf16_16816(acc[(3 * w) % NACC][b], oa[0], ob[0], oa[1], ob[1], xw[0], xw[1]);
                        mma_bf16_16816(acc[(3 * w + 1) % NACC][b], oa[2], ob[2], oa[3], ob[3], xw[2], xw[3]);
                        mma_bf16_16816(acc[(3 * w + 2) % NACC][b], oa[4], ob[4], oa[5], ob[5], xw[4], xw[5]);
                    }
            }
        }
        if (!ok && lane == 0) atomicCAS(&g_gemv_status, GEMV_STATUS_OK, GEMV_STATUS_TIMEOUT_CONSUMER);

        float *pw = part + (size_t)kw * rows_per_cta * kTokPad;
        const int lr = rw * 16;
#pragma unroll
        for (int b = 0; b < TOKB; ++b) {
            float r[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) r[i] = (acc[0][b][i] + acc[1][b][i]) + (acc[2][b][i] + acc[3][b][i]);
            *reinterpret_cast<float2 *>(pw + (lr + g) * kTokPad + 8 * b + 2 * t) = make_float2(r[0], r[1]);
            *reinterpret_cast<float2 *>(pw + (lr + g + 8) * kTokPad + 8 * b + 2 * t) = make_float2(r[2], r[3]);
        }
    }
    __syncthreads();

    const int outs = rows_per_cta * kTokPad;
    if (slices == 1) {
        for (int o = threadIdx.x; o < outs; o += all_threads) {
            // with peers: rows fastest, so that a warp stores runs of consecutive rows of one token over NVLink
            const int r = p.n_peers > 0 ? o % rows_per_cta : o / kTokPad, tk = p.n_peers > 0 ? o / rows_per_cta : o % kTokPad;
            const int idx = r * kTokPad + tk;
            float s = part[idx];
            for (int w = 1; w < k_warps; ++w) s += part[(size_t)w * outs + idx];
            store_out<CT>(p, cta_row0 + r, tk, s);
        }
    } else {
        for (int idx = threadIdx.x; idx < outs; idx += all_threads) {
            float s = part[idx];
            for (int w = 1; w < k_warps; ++w) s += part[(size_t)w * outs + idx];
            part[idx] = s;
        }
        cluster.sync();
        const int span = (rows_per_cta + slices - 1) / slices;
        const int lo = slice * span;
        const int hi = lo + span < rows_per_cta ? lo + span : rows_per_cta;
        for (int o = threadIdx.x; o < (hi - lo) * kTokPad; o += all_threads) {
            const int r = lo + (p.n_peers > 0 ? o % (hi - lo) : o / kTokPad), tk = p.n_peers > 0 ? o / (hi - lo) : o % kTokPad;
            const int idx = r * kTokPad + tk;
            float s = 0.0f;
            for (int rk = 0; rk < slices; ++rk) s += cluster.map_shared_rank(part, rk)[idx];
            store_out<CT>(p, cta_row0 + r, tk, s);
        }
        cluster.sync();
    }
    if (tp.independent) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tp.sync_local) {
        // one system fence per CTA, by the signalling thread after the barrier (a fence in every
        // thread costs ten times the kernel): the barrier orders the CTA's stores before it
        __syncthreads();
        if (threadIdx.x == 0) exchange_signal(tp.sync_local, tp.sync_peer, p.n_peers, gridDim.x * gridDim.y);
    }
}

// The same protocol as separate launches, around kernels that do not carry it themselves.
__global__ void exchange_wait_kernel(uint32_t *sync_local, int n_peers) {
    if (threadIdx.x == 0 && !exchange_wait(sync_local, n_peers))
        atomicCAS(&g_gemv_status, GEMV_STATUS_OK, GEMV_STATUS_TIMEOUT_EXCHANGE);
}

struct SignalSlots {
    uint32_t *slot[T81B200_MAX_PEERS];
};
__global__ void exchange_signal_kernel(uint32_t *sync_local, SignalSlots slots, int n_peers) {
    if (threadIdx.x == 0) exchange_signal(sync_local, slots.slot, n_peers, 1u);
}

template <typename XT, typename CT, int TOKB>
int launch_tma(const CUtensorMap &map, const GemvTmaParams &tp, int slices, size_t smem_bytes, cudaStream_t st) {
    auto kern = gemv_trit_tma_kernel<XT, CT, TOKB>;
    T81_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    const int rows_per_cta = tp.g.row_warps * 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((tp.g.M + rows_per_cta - 1) / rows_per_cta), (unsigned)slices, 1);
    cfg.blockDim = dim3((tp.consumer_warps + 1) * 32, 1, 1);
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
    T81_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, map, tp));
    return T81B200_OK;
}

template <typename XT>
int launch_tma_ct(const CUtensorMap &map, const GemvTmaParams &tp, int c_dtype, int slices, size_t smem_bytes, cudaStream_t st) {
    const bool wide = tp.g.ntok > 8;
    switch (c_dtype) {
        case T81B200_F32:
            return wide ? launch_tma<XT, float, 2>(map, tp, slices, smem_bytes, st) : launch_tma<XT, float, 1>(map, tp, slices, smem_bytes, st);
        case T81B200_BF16:
            return wide ? launch_tma<XT, __nv_bfloat16, 2>(map, tp, slices, smem_bytes, st) : launch_tma<XT, __nv_bfloat16, 1>(map, tp, slices, smem_bytes, st);
        case T81B200_F16:
            return wide ? launch_tma<XT, __half, 2>(map, tp, slices, smem_bytes, st) : launch_tma<XT, __half, 1>(map, tp, slices, smem_bytes, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown output dtype %d", c_dtype);
}

size_t gemv_smem_bytes(int planes, int ntok, int tokpad, int lps, int warps, int row_warps, int rg) {
    return (size_t)planes * ntok * (lps * 24 + 4) * 4 + (size_t)(warps / row_warps) * row_warps * 16 * rg * tokpad * 4;
}

}  // namespace

// Shape choice and launch of the TMA-fed kernel.  Returns T81B200_EALIGN when no configuration
// fits (the caller then uses the register-prefetch kernel).
extern thread_local int g_hint_independent;

int gemv_trit_tma_launch(const GemvParams &base, int x_dtype, int c_dtype, cudaStream_t st, const PeerCtx *ctx) {
    GemvTmaParams tp;
    tp.g = base;
    tp.independent = (g_hint_independent && !(ctx && ctx->sync_local)) ? 1 : 0;
    tp.sync_local = ctx ? ctx->sync_local : nullptr;
    for (int i = 0; i < T81B200_MAX_PEERS; ++i) tp.sync_peer[i] = tp.sync_local && i < ctx->n_peers ? ctx->sync_slots[i] : nullptr;
    const int ntok = base.ntok;
    const int planes = x_dtype == T81B200_BF16 ? 1 : 2;
    const int tokpad = ntok > 8 ? 16 : 8;
    const int kl4 = (int)((base.kl + 3) & ~(int64_t)3);
    const int sms = sm_count();
    const size_t budget = 200 * 1024;
    int best_rw = 0, best_s = 1, best_lps = 4, best_stages = 0;
    double best_t = 1e30;
    const int forced_rw = 0, forced_s = 0, forced_kw = 0;
    int best_kw = 1;
    for (int rwv = 1; rwv <= kTmaMaxConsumerWarps; ++rwv)
        for (int kwv = 1; rwv * kwv <= kTmaMaxConsumerWarps; ++kwv)
            for (int s = 1; s <= 4; s *= 2) {  // clusters of 8 were slower in every measured case
                if (forced_rw && (rwv != forced_rw || s != forced_s || (forced_kw && kwv != forced_kw))) continue;
                if (!forced_rw && kwv != 2 && kwv != 4) continue;  // 1 couples all warps to one slot, 8 starves each slice
                int lps = (kl4 / 4 + s - 1) / s * 4;
                if (lps < 4) lps = 4;
                if (s > 1 && (int64_t)(s - 1) * lps >= kl4) continue;
                const int chunks = lps / 4;
                if (kwv > chunks) continue;
                const int rows = 16 * rwv;
                const size_t xs_bytes = ((size_t)planes * ntok * (lps * 24 + 4) * 4 + 127) & ~(size_t)127;
                const size_t part_bytes = ((size_t)kwv * rows * tokpad * 4 + 127) & ~(size_t)127;
                const size_t stage_bytes = (size_t)rows * 64;
                if (xs_bytes + part_bytes + 1024 + 2 * stage_bytes * kwv > budget) continue;
                int stages = (int)((budget - xs_bytes - part_bytes - 1024) / stage_bytes);
                if (stages > kTmaMaxStages) stages = kTmaMaxStages;
                if (stages > chunks) stages = chunks;
                if (stages < 2 * kwv && stages < chunks) continue;
                // Cost model fitted to a sweep over the Llama / Phi shapes (zero regret on it): a warp needs
                // about 1400 cycles per chunk whatever shares its scheduler, up to four warps per scheduler;
                // staging the activations runs at ~80 GB/s per CTA; a launch costs ~2.5 us, a cluster 0.7 more.
                const int64_t row_tiles = (base.M + rows - 1) / rows;
                // clusters must fit inside a GPC: fewer CTAs are co-resident than there are SMs
                // (148 CTAs in clusters of 4 measured twice as slow as 128)
                const double wave_ctas = s == 1 ? sms : (s == 2 ? sms - 8 : sms - 20);
                const double waves = ceil((double)row_tiles * s / wave_ctas);
                const double warps_per_sched = ceil(rwv * kwv / 4.0);
                const double chunks_per_warp = ceil((double)chunks / kwv);
                const double work = chunks_per_warp * 1400.0 * (warps_per_sched > 4.0 ? warps_per_sched / 4.0 : 1.0) *
                                    (1.0 + 0.25 * (planes * (tokpad / 8) - 1)) / 1.9e9;
                const double staging = (double)planes * ntok * lps * 96 / 8.0e10;
                const double t = waves * (2.5e-6 + (s > 1 ? 0.7e-6 : 0.0) + staging + work);
                if (t < best_t) { best_t = t; best_rw = rwv; best_kw = kwv; best_s = s; best_lps = lps; best_stages = stages; }
            }
    if (!best_rw) return T81B200_EALIGN;
    const int kwv = best_kw;
    const int rows = 16 * best_rw;
    tp.consumer_warps = best_rw * best_kw;
    tp.g.row_warps = best_rw;
    tp.g.row_groups = 1;
    tp.g.limbs_per_slice = best_lps;
    tp.stages = best_stages;
    tp.stage_bytes = rows * 64;
    const size_t xs_bytes = ((size_t)planes * ntok * (best_lps * 24 + 4) * 4 + 127) & ~(size_t)127;
    const size_t part_bytes = ((size_t)kwv * rows * tokpad * 4 + 127) & ~(size_t)127;
    tp.ring_offset = (int)xs_bytes;
    tp.part_offset = (int)(xs_bytes + (size_t)best_stages * tp.stage_bytes);
    tp.bar_offset = (int)(tp.part_offset + part_bytes);
    const size_t smem = (size_t)tp.bar_offset + 16 * (size_t)best_stages + 128;
    CUtensorMap map;
    if (int rc = make_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base.A, (uint64_t)base.kl * 16, (uint64_t)base.M,
                             (uint64_t)base.kl * 16, 64, (uint32_t)rows, CU_TENSOR_MAP_SWIZZLE_NONE))
        return rc;
    switch (x_dtype) {
        case T81B200_BF16: return launch_tma_ct<__nv_bfloat16>(map, tp, c_dtype, best_s, smem, st);
        case T81B200_F32: return launch_tma_ct<float>(map, tp, c_dtype, best_s, smem, st);
        case T81B200_F16: return launch_tma_ct<__half>(map, tp, c_dtype, best_s, smem, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown activation dtype %d", x_dtype);
}

thread_local int g_hint_independent = 0;

int exchange_wait_launch(uint32_t *sync_local, int n_peers, cudaStream_t st) {
    exchange_wait_kernel<<<1, 32, 0, st>>>(sync_local, n_peers);
    T81_LAUNCH_CHECK("exchange_wait_kernel");
    return T81B200_OK;
}

int exchange_signal_launch(uint32_t *sync_local, uint32_t *const *slots, int n_peers, cudaStream_t st) {
    SignalSlots sl;
    for (int i = 0; i < T81B200_MAX_PEERS; ++i) sl.slot[i] = i < n_peers ? slots[i] : nullptr;
    exchange_signal_kernel<<<1, 32, 0, st>>>(sync_local, sl, n_peers);
    T81_LAUNCH_CHECK("exchange_signal_kernel");
    return T81B200_OK;
}

int gemv_trit_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_status, sizeof v) != cudaSuccess) return T81B200_ECUDA;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof zero) != cudaSuccess) return T81B200_ECUDA;
    }
    return v;
}

namespace {
}  // namespace

int gemv_trit_lut_launch(int fmt, int n_seg, const uint8_t *const *A, const float *const *row_scale, const float *const *bias,
                         void *const *C, const int64_t *M, const void *X, int x_dtype, int64_t ldx, int c_dtype,
                         int64_t ldc, int ntok, int64_t K, float alpha, float beta, cudaStream_t st, const PeerCtx *ctx);

// Host entry used by the dispatcher in capi.cu.  NK layout, ntok in 1..16, A 16-byte aligned.
int gemv_trit_launch(const uint8_t *A, const float *row_scale, const void *X, int x_dtype, int64_t ldx,
                     const float *bias, void *C, int c_dtype, int64_t ldc, int64_t M, int ntok, int64_t K,
                     float alpha, float beta, cudaStream_t st, PeerCtx *ctx) {
    GemvParams p;
    p.A = A; p.X = X; p.row_scale = row_scale; p.bias = bias; p.C = C;
    p.M = M; p.K = K; p.kl = (K + 47) / 48; p.ldx = ldx; p.ldc = ldc; p.ntok = ntok;
    p.alpha = alpha; p.beta = beta;
    p.n_peers = ctx ? ctx->n_peers : 0;
    for (int i = 0; i < T81B200_MAX_PEERS; ++i) p.peer_C[i] = i < p.n_peers ? ctx->peer_C[i] : nullptr;
    if (ctx) ctx->peers_done = true;  // both streaming kernels store into the peers themselves
    const int planes = x_dtype == T81B200_BF16 ? 1 : 2;
    const int tokpad = ntok > 8 ? 16 : 8;
    const int kl4 = (int)((p.kl + 3) & ~(int64_t)3);

    // Default: the table-decode kernel.  T81B200_GEMV_PATH (read once per process; A/B runs) selects an older
    // kernel instead: "fma" the TMA-fed kernel with arithmetic decode, "ldg" the register-prefetch kernel.
    static const bool live = getenv("T81B200_GEMV_CFG_LIVE") != nullptr;
    static char path = [] { const char *e = getenv("T81B200_GEMV_PATH"); return e ? e[0] : '\0'; }();
    if (live) { const char *e = getenv("T81B200_GEMV_PATH"); path = e ? e[0] : '\0'; }
    if (path == '\0') {
        const float *rs = row_scale, *bs = bias;
        void *cc = C;
        const int rc = gemv_trit_lut_launch(0, 1, &A, &rs, &bs, &cc, &M, X, x_dtype, ldx, c_dtype, ldc, ntok, K, alpha, beta, st, ctx);
        if (rc != T81B200_EALIGN) {
            if (ctx && ctx->sync_local && rc == T81B200_OK) ctx->sync_fused = true;
            return rc;
        }
    } else if (path == 'f') {
        p.row_warps = 1; p.row_groups = 1; p.limbs_per_slice = 4;
        const int rc = gemv_trit_tma_launch(p, x_dtype, c_dtype, st, ctx);
        if (rc != T81B200_EALIGN) {
            if (ctx && ctx->sync_local && rc == T81B200_OK) ctx->sync_fused = true;
            return rc;
        }
    }
    if (ctx && ctx->sync_local) {  // the register-prefetch kernel does not carry the exchange protocol
        if (int rc = exchange_wait_launch(ctx->sync_local, ctx->n_peers, st)) return rc;
        ctx->waited = true;
    }

    // Pick the CTA shape with a small cost model.  A CTA has W warps arranged as RW row groups
    // (16 rows each) x W/RW slices of its contraction range; RG row groups are walked in
    // sequence; S CTAs of a cluster split the contraction further.  One CTA per SM per wave:
    //   time = waves * (fixed + staging + max(stream, issue))
    const int sms = sm_count();
    const double sm_bw = 6.5e12 / sms;   // HBM share of one SM, bytes/s
    const double l2_bw = 1.0e11;         // L2 -> one SM, bytes/s (staging of activations)
    const double chunk_rate = 4 * 1.8e9 / 450.0;  // 4-limb chunks per second one SM sustains (measured: ~450 clk each)
    int best_w = 16, best_rw = 4, best_rg = 1, best_s = 1, best_lps = 4, variant = 0;
    double best_t = 1e30;
    for (int w = 8; w <= 16; w += 8)
        for (int rwv = 1; rwv <= w; rwv *= 2)
            for (int rg = 1; rg <= 4; rg *= 2)
                for (int s = 1; s <= 8; s *= 2) {
                    const int rows_per_cta = rwv * 16 * rg;
                    int lps = (kl4 / 4 + s - 1) / s * 4;
                    if (lps < 4) lps = 4;
                    if (s > 1 && (int64_t)(s - 1) * lps >= kl4) continue;  // an empty slice
                    const int kwv = w / rwv;
                    if (kwv > lps / 4) continue;                           // a warp without work
                    const size_t smem = gemv_smem_bytes(planes, ntok, tokpad, lps, w, rwv, rg);
                    if (smem > 200 * 1024) continue;
                    const int64_t row_tiles = (M + rows_per_cta - 1) / rows_per_cta;
                    const double ctas = (double)row_tiles * s;
                    const double waves = ceil(ctas / sms);
                    const double stream = (double)rows_per_cta * lps * 16 / sm_bw;
                    const double chunks = (double)rwv * rg * (lps / 4.0);
                    const double work = chunks * (1.0 + 0.25 * (planes * (tokpad / 8) - 1)) / chunk_rate;
                    const double staging = (double)planes * ntok * lps * 96 / l2_bw;
                    const double fixed = 2.0e-6 + (s > 1 ? 1.0e-6 : 0.0) + (w == 16 ? 0.3e-6 : 0.0);
                    const double t = waves * (fixed + staging + (stream > work ? stream : work));
                    if (t < best_t) { best_t = t; best_w = w; best_rw = rwv; best_rg = rg; best_s = s; best_lps = lps; }
                }
    if (best_t >= 1e30)
        return fail(T81B200_ELIMIT, "gemm_trit: K=%lld too large for the streaming kernel", (long long)K);
    p.row_warps = best_rw;
    p.row_groups = best_rg;
    p.limbs_per_slice = best_lps;
    const size_t smem = gemv_smem_bytes(planes, ntok, tokpad, best_lps, best_w, best_rw, best_rg);
    switch (x_dtype) {
        case T81B200_BF16: return launch_ct<__nv_bfloat16>(p, c_dtype, best_w, best_s, smem, variant, st);
        case T81B200_F32: return launch_ct<float>(p, c_dtype, best_w, best_s, smem, variant, st);
        case T81B200_F16: return launch_ct<__half>(p, c_dtype, best_w, best_s, smem, variant, st);
    }
    return fail(T81B200_EINVAL, "gemm_trit: unknown activation dtype %d", x_dtype);
}

}  // namespace t81b200
