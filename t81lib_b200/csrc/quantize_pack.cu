// Fused threshold-quantise + trit-pack kernel, and its inverse.
//
// quantize_pack_row_kernel: a CTA of 128 threads owns one row at a time; each of its four warps owns chunks of
// 96 consecutive float4 groups (384 weights = 32 packed words), chunk c going to warp c % 4.  A lane reads the
// chunk's groups lane, 32 + lane and 64 + lane: three fully coalesced 512-byte warp loads.  Rows of up to 6144
// columns are read from global memory ONCE, into registers; longer rows are read a second time for the pack
// pass (from L2).  With the absmean rule the row scale is the mean of |w| summed in a fixed order — fp32 inside
// a float4 group, fp64 across the groups of a thread in column order, then a halving tree over the 128 threads —
// that the CPU checker reproduces bit for bit, whatever the launch shape.  One block barrier per row (the four
// warp sums, double-buffered by row parity).  The row's cut is threshold (fixed rule) or threshold * mean
// (absmean rule, one multiply per row): a weight becomes -1 at or below -cut, +1 at or above cut, else 0.
// Every lane turns each of its groups into that group's share of its packed word — three instructions per
// weight, see group_share — and nine warp shuffles hand lane w the three shares of word w, which it adds and
// stores: one coalesced 128-byte warp store per chunk.
//
#include "common.cuh"
#include "tma.cuh"

#include <atomic>
#include <type_traits>
#include <cstdlib>
#include <cstring>

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
constexpr int kChunkGroups = 96;  // float4 groups per warp chunk = 32 packed words

// What a lane needs to turn a float4 group into that group's share of its packed word.  A word is 12 digits =
// three consecutive groups; group g holds digits i = 4 (g % 3) .. + 3 of its word, digit i weighs 3^(i % 3) in
// byte i / 3.  Chunks start at a multiple of 3 groups, so for the lane's group k of a chunk g % 3 = (32 k + lane) % 3.
// A share spans at most two neighbouring bytes, i.e. 13 bits: sums of its weights are exact in fp32.
struct PackConsts {
    float mult[3][4];  // digit weights
    float base[3];     // share of a group of zero trits (every digit 1)
};

__device__ __forceinline__ void make_pack_consts(int lane, PackConsts &pc) {
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        pc.base[k] = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 4 * ((32 * k + lane) % 3) + e;
            pc.mult[k][e] = (float)((i % 3 == 0 ? 1u : (i % 3 == 1 ? 3u : 9u)) << (8 * (i / 3)));
            pc.base[k] += pc.mult[k][e];
        }
    }
}

// Share of one group.  trit = -1 where v <= -cut, else +1 where v >= cut, else 0.
// FAST (cut > 0): |v| >= cut decides whether the trit is non-zero and the sign bit of v which one — a compare, a
// bit operation and a multiply-add per weight; zeros loaded for columns past the end give zero trits by themselves.
// Otherwise (cut == 0: every value is +-1, a zero -1) the two compares are made as written and `valid` elements count.
template <bool FAST>
__device__ __forceinline__ float group_share(const float (&v)[4], float cut, const float (&mult)[4], float base, int valid) {
    float acc = base;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if constexpr (FAST) {
            const float nz = fabsf(v[e]) >= cut ? 1.0f : 0.0f;
            const float signed_weight = __uint_as_float(__float_as_uint(mult[e]) | (__float_as_uint(v[e]) & 0x80000000u));
            acc = fmaf(nz, signed_weight, acc);
        } else {
            if (e < valid) acc += v[e] <= -cut ? -mult[e] : (v[e] >= cut ? mult[e] : 0.0f);
        }
    }
    return acc;
}

// Words 32 c .. 32 c + 31 of the packed row from the chunk's three shares per lane: word w = groups 3 w, 3 w + 1,
// 3 w + 2 of the chunk, group G sits in share[G / 32] of lane G % 32.  Returns this lane's word.  Whole-warp.
__device__ __forceinline__ uint32_t gather_word(const float (&share)[3], int lane) {
    uint32_t s[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) s[k] = (uint32_t)share[k];  // exact: non-negative integers below 2^29
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        const int G = 3 * lane + j;
        const uint32_t s0 = __shfl_sync(0xffffffffu, s[0], G & 31);
        const uint32_t s1 = __shfl_sync(0xffffffffu, s[1], G & 31);
        const uint32_t s2 = __shfl_sync(0xffffffffu, s[2], G & 31);
        word += G < 32 ? s0 : (G < 64 ? s1 : s2);
    }
    return word;
}

template <bool FAST>
__device__ __forceinline__ uint32_t pack_chunk(const float (&v)[3][4], int c, int lane, int cols, float cut, const PackConsts &pc) {
    float share[3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int left = cols - 4 * (kChunkGroups * c + 32 * k + lane);  // columns of the row from this group on
        share[k] = group_share<FAST>(v[k], cut, pc.mult[k], pc.base[k], left);
    }
    return gather_word(share, lane);
}

__device__ __forceinline__ double group_abs_sum(const float (&v)[4]) {  // fp32 inside the group
    return (double)__fadd_rn(__fadd_rn(fabsf(v[0]), fabsf(v[1])), __fadd_rn(fabsf(v[2]), fabsf(v[3])));
}

// The cut of a row under the absmean rule: threshold * mean |w| (one fp32 multiply); a row whose mean is not a
// positive number (all zero, or NaN) gets +inf: zero trits.
__device__ __forceinline__ float absmean_cut(float mean, float thr) { return mean > 0.0f ? __fmul_rn(thr, mean) : __int_as_float(0x7f800000); }

// The three groups of chunk c that this lane owns, from global memory; columns past the end load as 0.
template <typename T, bool ABSMEAN>
__device__ __forceinline__ void load_chunk(const T *row, int c, int lane, int cols, bool vec, float (&v)[3][4], double &part) {
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int col = 4 * (kChunkGroups * c + 32 * k + lane);
        if (col < cols) load_group<T>(row, col, cols, vec, v[k]);
        else { v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.0f; }
    }
    if constexpr (ABSMEAN) {
#pragma unroll
        for (int k = 0; k < 3; ++k)  // fp64 across groups, in column order; groups past the end add +0: no change
            part += group_abs_sum(v[k]);
    }
}

// REG_CHUNKS > 0: a warp's chunks of the row number at most REG_CHUNKS and stay in registers between the two
// passes; 0: the row is read twice.
template <typename T, bool ABSMEAN, int REG_CHUNKS>
__global__ void __launch_bounds__(kRowThreads, REG_CHUNKS == 0 ? 10 : (REG_CHUNKS <= 3 ? 6 : 5))
quantize_pack_row_kernel(const T *__restrict__ w, int64_t rows, int cols, int64_t ld, float thr,
                         uint8_t *__restrict__ packed, float *__restrict__ row_scale, bool vec) {
    __shared__ double warp_sum[2][4];
    const int kl = (cols + 47) / 48, nwords = kl * 4, nchunks = (nwords + 31) / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int parity = 0;
    constexpr bool IN_REGS = REG_CHUNKS > 0;
    constexpr int kRegChunks = IN_REGS ? REG_CHUNKS : 1;
    PackConsts pc;
    make_pack_consts(lane, pc);

    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x, parity ^= 1) {
        const T *row = w + r * ld;
        uint32_t *out = reinterpret_cast<uint32_t *>(packed + r * (int64_t)kl * 16);
        float keep[kRegChunks][3][4];
        double part = 0.0;
        if constexpr (IN_REGS) {
#pragma unroll
            for (int m = 0; m < kRegChunks; ++m) {
                const int c = warp + 4 * m;
                if (c < nchunks) load_chunk<T, ABSMEAN>(row, c, lane, cols, vec, keep[m], part);
            }
        } else if constexpr (ABSMEAN) {
            for (int c = warp; c < nchunks; c += 4) {
                float v[3][4];
                load_chunk<T, true>(row, c, lane, cols, vec, v, part);
            }
        }
        float cut = thr;
        if constexpr (ABSMEAN) {
            // halving tree over the 128 partials: inside each warp, then over the four warp sums
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) part += __shfl_down_sync(0xffffffffu, part, off);
            if (lane == 0) warp_sum[parity][warp] = part;
            __syncthreads();  // the only block barrier of a row; the other parity's sums are free to be rewritten
            const double total = (warp_sum[parity][0] + warp_sum[parity][2]) + (warp_sum[parity][1] + warp_sum[parity][3]);
            const float mean = __fdiv_rn((float)total, (float)cols);
            cut = absmean_cut(mean, thr);
            if (tid == 0) row_scale[r] = mean;
        }
        // cut > 0 (the same in the whole CTA) takes the short form of the pack step; the branch stays outside the loops
        auto pack_row = [&](auto fast) {
            if constexpr (IN_REGS) {
#pragma unroll
                for (int m = 0; m < kRegChunks; ++m) {
                    const int c = warp + 4 * m;
                    if (c < nchunks) {  // the same for every lane of the warp: the shuffles inside are whole-warp
                        const uint32_t word = pack_chunk<decltype(fast)::value>(keep[m], c, lane, cols, cut, pc);
                        if (32 * c + lane < nwords) out[32 * c + lane] = word;
                    }
                }
            } else {
                for (int c = warp; c < nchunks; c += 4) {
                    float v[3][4];
                    double unused = 0.0;
                    load_chunk<T, false>(row, c, lane, cols, vec, v, unused);  // second read of the row: L2
                    const uint32_t word = pack_chunk<decltype(fast)::value>(v, c, lane, cols, cut, pc);
                    if (32 * c + lane < nwords) out[32 * c + lane] = word;
                }
            }
        };
        if (cut > 0.0f) pack_row(std::true_type{});
        else pack_row(std::false_type{});
    }
}

// ---- the streaming form: rows land in a shared-memory ring by bulk copies ----
//
// quantize_pack_ring_kernel: one persistent CTA per SM.  A producer thread keeps a ring of whole rows in flight
// (one bulk copy per row, up to 16 rows and ~220 KB per SM: the bytes in flight that HBM needs, which registers of
// resident CTAs cannot hold); TEAMS teams of four warps each take every TEAMS-th row of the CTA from the ring, with
// the chunk ownership, the summation order and the pack step of the row kernel above, reading the row from
// shared memory twice (sum, then pack) and handing the slot back after the second pass.
// Needs 16-byte aligned rows of a multiple of 16 bytes and TEAMS rows in 226 KB; the row kernel covers the rest.
constexpr int kMaxTeams = 7;
constexpr int kMaxSlots = 16;
constexpr int kRingBytes = 226 * 1024;  // rows; barriers and team sums are static shared memory

enum { QUANT_STATUS_TIMEOUT_PRODUCER = 9, QUANT_STATUS_TIMEOUT_CONSUMER = 10 };
__device__ int g_quant_status = 0;

template <typename T, bool ABSMEAN>
__device__ __forceinline__ void load_chunk_shared(const T *row, int c, int lane, int cols, float (&v)[3][4], double &part) {
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        const int col = 4 * (kChunkGroups * c + 32 * k + lane);
        if (col < cols) {  // whole groups: cols is a multiple of 4
            if constexpr (sizeof(T) == 4) {
                const float4 f = *reinterpret_cast<const float4 *>(row + col);
                v[k][0] = f.x; v[k][1] = f.y; v[k][2] = f.z; v[k][3] = f.w;
            } else {
                const uint2 u = *reinterpret_cast<const uint2 *>(row + col);
                const T *e = reinterpret_cast<const T *>(&u);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[k][i] = to_float<T>(e[i]);
            }
        } else { v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.0f; }
    }
    if constexpr (ABSMEAN) {
#pragma unroll
        for (int k = 0; k < 3; ++k) part += group_abs_sum(v[k]);
    }
}

__device__ __forceinline__ bool team_all(int team, bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "barrier.cta.red.and.pred q, %2, %3, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)ok), "r"(1 + team), "r"(kRowThreads)
        : "memory");
    return r != 0;
}

template <typename T, bool ABSMEAN, int TEAMS>
__global__ void __launch_bounds__(TEAMS * kRowThreads + 32, 1)
quantize_pack_ring_kernel(const T *__restrict__ w, int rows, int cols, int64_t ld, float thr, uint8_t *__restrict__ packed,
                          float *__restrict__ row_scale, int slots, int slot_bytes) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ __align__(8) uint64_t bars[2 * kMaxSlots];
    __shared__ double warp_sum[TEAMS][2][4];
    const int tid = threadIdx.x, lane = tid & 31, warp_in_cta = tid >> 5;
    const int kl = (cols + 47) / 48, nwords = kl * 4, nchunks = (nwords + 31) / 32;
    const uint32_t row_bytes = (uint32_t)cols * (uint32_t)sizeof(T);
    const int n_local = rows > (int)blockIdx.x ? (rows - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8u * kMaxSlots;
    if (tid < slots) { mbar_init(full0 + 8u * tid, 1); mbar_init(empty0 + 8u * tid, 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    // launched with programmatic stream serialization: everything above overlaps the tail of the kernel before
    // this one in the stream; nothing below reads or writes global memory before that kernel has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp_in_cta == TEAMS * 4) {
        // producer: row i of this CTA goes to slot i % slots as soon as the slot's previous row was handed back
        if (lane == 0) {
            for (int i = 0; i < n_local; ++i) {
                const int slot = i % slots, use = i / slots;
                if (use > 0 && !mbar_wait(empty0 + 8u * slot, (uint32_t)(use - 1) & 1u)) { atomicCAS(&g_quant_status, 0, QUANT_STATUS_TIMEOUT_PRODUCER); break; }
                const int64_t r = (int64_t)blockIdx.x + (int64_t)i * gridDim.x;
                mbar_arrive_expect_tx(full0 + 8u * slot, row_bytes);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(ring) + (uint32_t)slot * (uint32_t)slot_bytes), "l"(w + r * ld), "r"(row_bytes),
                               "r"(full0 + 8u * slot)
                             : "memory");
            }
        }
        return;
    }

    const int team = warp_in_cta >> 2, warp = warp_in_cta & 3;
    PackConsts pc;
    make_pack_consts(lane, pc);

    int parity = 0;
    for (int i = team; i < n_local; i += TEAMS, parity ^= 1) {
        // slots is a multiple of the team count: every use of a slot is consumed by the same team, in order
        const int slot = i % slots, use = i / slots;
        const int64_t r = (int64_t)blockIdx.x + (int64_t)i * gridDim.x;
        const T *row = reinterpret_cast<const T *>(ring + (size_t)slot * slot_bytes);
        uint32_t *out = reinterpret_cast<uint32_t *>(packed + r * (int64_t)kl * 16);
        bool ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8u * slot, (uint32_t)use & 1u));
        float cut = thr;
        if constexpr (ABSMEAN) {
            double part = 0.0;
            if (ok) {
                for (int c = warp; c < nchunks; c += 4) {
                    float v[3][4];
                    load_chunk_shared<T, true>(row, c, lane, cols, v, part);
                }
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) part += __shfl_down_sync(0xffffffffu, part, off);
            if (lane == 0) warp_sum[team][parity][warp] = part;
            ok = team_all(team, ok);  // the team's only barrier of a row; it also carries the verdict of the waits
            if (ok) {
                const double total = (warp_sum[team][parity][0] + warp_sum[team][parity][2]) + (warp_sum[team][parity][1] + warp_sum[team][parity][3]);
                const float mean = __fdiv_rn((float)total, (float)cols);
                cut = absmean_cut(mean, thr);
                if (warp == 0 && lane == 0) row_scale[r] = mean;
            }
        }
        if (!ok) {  // a wait ran out: the same verdict in the whole team (ABSMEAN) or warp; report and stop
            if (lane == 0) atomicCAS(&g_quant_status, 0, QUANT_STATUS_TIMEOUT_CONSUMER);
            break;
        }
        // cut > 0 (the same in the whole team) takes the short form of the pack step; the branch stays outside the loop
        auto pack_row = [&](auto fast) {
            for (int c = warp; c < nchunks; c += 4) {
                float v[3][4];
                double unused = 0.0;
                load_chunk_shared<T, false>(row, c, lane, cols, v, unused);
                const uint32_t word = pack_chunk<decltype(fast)::value>(v, c, lane, cols, cut, pc);
                if (32 * c + lane < nwords) out[32 * c + lane] = word;
            }
        };
        if (cut > 0.0f) pack_row(std::true_type{});
        else pack_row(std::false_type{});
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8u * slot);  // this warp has read the row for the last time
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

template <typename T, int REG_CHUNKS>
int launch_row_kernel(const void *w, int64_t rows, int64_t cols, int64_t ld, float thr, int rule, uint8_t *packed,
                      float *row_scale, bool vec, cudaStream_t st) {
    const int64_t cap = (int64_t)sm_count() * 16;
    const int g = (int)(rows < cap ? rows : cap);
    if (rule == T81B200_RULE_ABSMEAN)
        quantize_pack_row_kernel<T, true, REG_CHUNKS><<<g, kRowThreads, 0, st>>>(static_cast<const T *>(w), rows, (int)cols, ld, thr, packed, row_scale, vec);
    else
        quantize_pack_row_kernel<T, false, REG_CHUNKS><<<g, kRowThreads, 0, st>>>(static_cast<const T *>(w), rows, (int)cols, ld, thr, packed, row_scale, vec);
    T81_LAUNCH_CHECK("quantize_pack_row_kernel");
    return T81B200_OK;
}

template <typename T, bool ABSMEAN, int TEAMS>
int launch_ring_kernel(const T *w, int64_t rows, int64_t cols, int64_t ld, float thr, uint8_t *packed, float *row_scale,
                       int slots, int slot_bytes, cudaStream_t st) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    T81_CUDA_TRY(cudaGetDevice(&dev));
    auto kernel = quantize_pack_ring_kernel<T, ABSMEAN, TEAMS>;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        T81_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes));
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    const int g = (int)(rows < sm_count() ? rows : sm_count());
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)g, 1, 1);
    cfg.blockDim = dim3(TEAMS * kRowThreads + 32, 1, 1);
    cfg.dynamicSmemBytes = (size_t)slots * slot_bytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    T81_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, w, (int)rows, (int)cols, ld, thr, packed, row_scale, slots, slot_bytes));
    return T81B200_OK;
}

template <typename T, int TEAMS>
int launch_ring(const T *w, int64_t rows, int64_t cols, int64_t ld, float thr, int rule, uint8_t *packed, float *row_scale,
                int64_t slot_bytes, cudaStream_t st) {
    int slots = (int)(kRingBytes / slot_bytes) / TEAMS * TEAMS;
    slots = slots > kMaxSlots / TEAMS * TEAMS ? kMaxSlots / TEAMS * TEAMS : slots;
    return rule == T81B200_RULE_ABSMEAN
               ? launch_ring_kernel<T, true, TEAMS>(w, rows, cols, ld, thr, packed, row_scale, slots, (int)slot_bytes, st)
               : launch_ring_kernel<T, false, TEAMS>(w, rows, cols, ld, thr, packed, row_scale, slots, (int)slot_bytes, st);
}

template <typename T>
int launch_quantize_pack(const void *w, int64_t rows, int64_t cols, int64_t ld, float thr, int rule,
                         uint8_t *packed, float *row_scale, cudaStream_t st) {
    const bool vec = (reinterpret_cast<uintptr_t>(w) % (4 * sizeof(T)) == 0) && (ld % 4 == 0);
    const int64_t nchunks = ((cols + 47) / 48 * 4 + 31) / 32;  // 384 columns each
    // the streaming form: rows that bulk copies can move (16-byte aligned, a multiple of 16 bytes), four or more
    // of which fit the ring, and enough of them to give every SM a few; T81B200_QUANT_PATH=row (read once) turns it off
    const int64_t row_bytes = cols * (int64_t)sizeof(T);
    const int64_t slot_bytes = (row_bytes + 127) / 128 * 128;
    const bool movable = reinterpret_cast<uintptr_t>(w) % 16 == 0 && (ld * (int64_t)sizeof(T)) % 16 == 0 && row_bytes % 16 == 0;
    static const bool ring_off = [] { const char *e = getenv("T81B200_QUANT_PATH"); return e && strcmp(e, "row") == 0; }();
    const T *wt = static_cast<const T *>(w);
    if (!ring_off && movable && rows >= 2 * (int64_t)sm_count() && rows < (1ll << 31)) {
        const int fit = (int)(kRingBytes / slot_bytes);  // rows the ring holds; a team needs one, and one more in flight
        if (fit >= 12) return launch_ring<T, 6>(wt, rows, cols, ld, thr, rule, packed, row_scale, slot_bytes, st);
        if (fit >= 4) return launch_ring<T, 4>(wt, rows, cols, ld, thr, rule, packed, row_scale, slot_bytes, st);
    }
    if (nchunks <= 4 * 3)  // up to 4608 columns
        return launch_row_kernel<T, 3>(w, rows, cols, ld, thr, rule, packed, row_scale, vec, st);
    if (nchunks <= 4 * 4)  // up to 6144 columns
        return launch_row_kernel<T, 4>(w, rows, cols, ld, thr, rule, packed, row_scale, vec, st);
    return launch_row_kernel<T, 0>(w, rows, cols, ld, thr, rule, packed, row_scale, vec, st);
}

}  // namespace

int quantize_pack_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_quant_status, sizeof v) != cudaSuccess) return T81B200_ECUDA;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_quant_status, &zero, sizeof zero) != cudaSuccess) return T81B200_ECUDA;
    }
    return v;
}

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
    if (cols > (1ll << 31) - 1024) return fail(T81B200_ELIMIT, "quantize_pack: rows of more than 2^31 - 1024 columns");
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
