// Shared device helpers and host-side error plumbing for libt81_b200.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/t81_b200.h"

namespace t81b200 {

// ---- host: error reporting ------------------------------------------------

void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);
int check_device();  // T81B200_OK or T81B200_ENODEVICE (cached per process)
// Column-sharded Linear: where the result also goes, and the flags that order the exchange.
struct PeerCtx {
    int n_peers = 0;
    void *const *peer_C = nullptr;           // the peers' results (same strides as the local C)
    uint32_t *sync_local = nullptr;          // this rank's exchange flags, or null
    uint32_t *const *sync_slots = nullptr;   // this rank's slot in each peer's flags
    bool peers_done = false;                 // set by a launcher whose kernel stored into the peers itself
    bool sync_fused = false;                 // ... and waited / signalled inside the kernel
    bool waited = false;                     // a stand-alone wait has been queued before the kernel
};
int exchange_wait_launch(uint32_t *sync_local, int n_peers, cudaStream_t st);
int exchange_signal_launch(uint32_t *sync_local, uint32_t *const *slots, int n_peers, cudaStream_t st);

int sm_count();      // multiprocessors of the current device (cached per device)
// *is_device = 1 when a kernel of the current device can dereference p (device or managed memory), 0 for host memory
int pointer_is_device(const void *p, int *is_device);

#define T81_CUDA_TRY(expr)                                                              \
    do {                                                                                \
        cudaError_t err__ = (expr);                                                     \
        if (err__ != cudaSuccess)                                                       \
            return ::t81b200::fail(T81B200_ECUDA, "%s failed: %s", #expr,               \
                                   cudaGetErrorString(err__));                          \
    } while (0)

#define T81_LAUNCH_CHECK(name)                                                          \
    do {                                                                                \
        cudaError_t err__ = cudaGetLastError();                                         \
        if (err__ != cudaSuccess)                                                       \
            return ::t81b200::fail(T81B200_ECUDA, "launch of %s failed: %s", name,      \
                                   cudaGetErrorString(err__));                          \
    } while (0)

// ---- device: tryte codec ---------------------------------------------------
// byte = t0 + 3*t1 + 9*t2 + 13  with t in {-1,0,+1}   (zero tryte = 13).

constexpr uint32_t kZeroTryteWord = 0x0D0D0D0Du;

// Scalar decode of one tryte byte into digits d = t + 1 in {0,1,2}.  Bytes above
// 26 are treated as the zero tryte.
__device__ __forceinline__ void tryte_digits(uint32_t b, int &d0, int &d1, int &d2) {
    b = b > 26u ? 13u : b;
    d2 = (int)((b * 57u) >> 9);  // b / 9 for b < 27
    const uint32_t r = b - 9u * (uint32_t)d2;
    d1 = (int)((r * 11u) >> 5);  // r / 3 for r < 9
    d0 = (int)(r - 3u * (uint32_t)d1);
}

// Packed decode: two tryte bytes -> their six trits as exact bf16 values.
//
// The two bytes are first placed in the mantissas of two bf16 lanes
// (0x4300 | b  ==  128 + b), then base-3 digits are peeled off with packed bf16
// FMAs whose single rounding does the floor():
//   v  = b - 13                      balanced value of the tryte, -13..13
//   Q  = RN(v * (57/512) + 130)      = 130 + t2          (ulp is 1 in [128,256))
//   t2 = Q - 130
//   r  = v - 9*t2                    -4..4
//   P  = RN(r * (171/512) + 130)     = 130 + t1
//   t1 = P - 130
//   t0 = r - 3*t1
// Every intermediate is an integer below 256 or lands on the magic grid, so each
// step is exact; the 27 byte values are checked exhaustively by the test suite.
struct TrytePairTrits {
    __nv_bfloat162 t0, t1, t2;  // .x from the first byte, .y from the second
};

__device__ __forceinline__ __nv_bfloat162 bf162_from_bits(uint32_t u) {
    __nv_bfloat162 r;
    *reinterpret_cast<uint32_t *>(&r) = u;
    return r;
}
__device__ __forceinline__ uint32_t bf162_bits(__nv_bfloat162 v) {
    return *reinterpret_cast<uint32_t *>(&v);
}

// d = a * b + c on two bf16 lanes, one rounding (HFMA2.BF16).  Additions are written as
// fma(a, 1, c): measured on sm_100a a packed bf16 add and a packed bf16 fma issue at the same
// rate (about 64 lanes per clock per SM, half the fp32 rate), so one instruction form serves all.
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ TrytePairTrits decode_tryte_pair(uint32_t x128) {
    // x128: lanes hold 128 + byte (bit pattern 0x4300 | byte).
    constexpr uint32_t kOne = 0x3F803F80u;    //  1
    constexpr uint32_t kM141 = 0xC30DC30Du;   // -141
    constexpr uint32_t kNinth = 0x3DE43DE4u;  //  57/512
    constexpr uint32_t kThird = 0x3EAB3EABu;  //  171/512
    constexpr uint32_t k130 = 0x43024302u;    //  130
    constexpr uint32_t kM130 = 0xC302C302u;   // -130
    constexpr uint32_t kM9 = 0xC110C110u;     // -9
    constexpr uint32_t kM3 = 0xC040C040u;     // -3
    const uint32_t v = fma_bf16x2(x128, kOne, kM141);
    const uint32_t q = fma_bf16x2(v, kNinth, k130);
    const uint32_t t2 = fma_bf16x2(q, kOne, kM130);
    const uint32_t r = fma_bf16x2(t2, kM9, v);
    const uint32_t p = fma_bf16x2(r, kThird, k130);
    const uint32_t t1 = fma_bf16x2(p, kOne, kM130);
    const uint32_t t0 = fma_bf16x2(t1, kM3, r);
    TrytePairTrits o;
    o.t0 = bf162_from_bits(t0);
    o.t1 = bf162_from_bits(t1);
    o.t2 = bf162_from_bits(t2);
    return o;
}

// Bytes (2p, 2p+1) of a 4-byte word as 128+byte bf16 lanes.
__device__ __forceinline__ uint32_t tryte_pair_lo(uint32_t w) {
    return __byte_perm(w, 0x43434343u, 0x4140);
}
__device__ __forceinline__ uint32_t tryte_pair_hi(uint32_t w) {
    return __byte_perm(w, 0x43434343u, 0x4342);
}

// Decode a whole limb (4 words = 16 trytes) into 24 packed registers.
// Register 3*p + i holds digit i of bytes 2p (low half) and 2p+1 (high half),
// i.e. trits 6p + i and 6p + 3 + i of the limb.
__device__ __forceinline__ void decode_limb(const uint4 &limb, uint32_t (&out)[24]) {
    const uint32_t w[4] = {limb.x, limb.y, limb.z, limb.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const TrytePairTrits a = decode_tryte_pair(tryte_pair_lo(w[i]));
        const TrytePairTrits b = decode_tryte_pair(tryte_pair_hi(w[i]));
        out[6 * i + 0] = bf162_bits(a.t0);
        out[6 * i + 1] = bf162_bits(a.t1);
        out[6 * i + 2] = bf162_bits(a.t2);
        out[6 * i + 3] = bf162_bits(b.t0);
        out[6 * i + 4] = bf162_bits(b.t1);
        out[6 * i + 5] = bf162_bits(b.t2);
    }
}

// Half a limb: two words (8 trytes) -> 12 packed registers, same order as decode_limb.
__device__ __forceinline__ void decode_words(uint32_t w0, uint32_t w1, uint32_t (&out)[12]) {
    const uint32_t w[2] = {w0, w1};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const TrytePairTrits a = decode_tryte_pair(tryte_pair_lo(w[i]));
        const TrytePairTrits b = decode_tryte_pair(tryte_pair_hi(w[i]));
        out[6 * i + 0] = bf162_bits(a.t0);
        out[6 * i + 1] = bf162_bits(a.t1);
        out[6 * i + 2] = bf162_bits(a.t2);
        out[6 * i + 3] = bf162_bits(b.t0);
        out[6 * i + 4] = bf162_bits(b.t1);
        out[6 * i + 5] = bf162_bits(b.t2);
    }
}

// One 32-bit word of each of two limbs (4 + 4 trytes) -> 6 + 6 packed registers, in the order
// of decode_limb (registers 6w .. 6w+5 of word w).  The four tryte-pair chains are written
// step by step side by side and kept in program order (volatile), so that an in-order warp
// always has four independent FMAs to issue and the MMAs that follow each word can run on
// the tensor pipe while the next word is being decoded.
__device__ __forceinline__ uint32_t fma_bf16x2_ordered(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm volatile("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ void decode_word_pair(uint32_t wa, uint32_t wb, uint32_t (&oa)[6], uint32_t (&ob)[6]) {
    constexpr uint32_t kOne = 0x3F803F80u, kM141 = 0xC30DC30Du, kNinth = 0x3DE43DE4u, kThird = 0x3EAB3EABu;
    constexpr uint32_t k130 = 0x43024302u, kM130 = 0xC302C302u, kM9 = 0xC110C110u, kM3 = 0xC040C040u;
    uint32_t x[4] = {tryte_pair_lo(wa), tryte_pair_hi(wa), tryte_pair_lo(wb), tryte_pair_hi(wb)};
    uint32_t v[4], q[4], t2[4], r[4], pp[4], t1[4], t0[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = fma_bf16x2_ordered(x[i], kOne, kM141);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = fma_bf16x2_ordered(v[i], kNinth, k130);
#pragma unroll
    for (int i = 0; i < 4; ++i) t2[i] = fma_bf16x2_ordered(q[i], kOne, kM130);
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = fma_bf16x2_ordered(t2[i], kM9, v[i]);
#pragma unroll
    for (int i = 0; i < 4; ++i) pp[i] = fma_bf16x2_ordered(r[i], kThird, k130);
#pragma unroll
    for (int i = 0; i < 4; ++i) t1[i] = fma_bf16x2_ordered(pp[i], kOne, kM130);
#pragma unroll
    for (int i = 0; i < 4; ++i) t0[i] = fma_bf16x2_ordered(t1[i], kM3, r[i]);
    oa[0] = t0[0]; oa[1] = t1[0]; oa[2] = t2[0]; oa[3] = t0[1]; oa[4] = t1[1]; oa[5] = t2[1];
    ob[0] = t0[2]; ob[1] = t1[2]; ob[2] = t2[2]; ob[3] = t0[3]; ob[4] = t1[3]; ob[5] = t2[3];
}

// Position inside a limb of the trit held by (register r, half h) of decode_limb.
__host__ __device__ __forceinline__ int decoded_trit_index(int r, int h) {
    return 6 * (r / 3) + 3 * h + (r % 3);
}

// ---- device: dtype loads/stores ---------------------------------------------

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_float<__half>(float v) {
    return __float2half_rn(v);
}

__host__ __device__ inline size_t dtype_size(int dtype) { return dtype == T81B200_F32 ? 4 : 2; }

}  // namespace t81b200
