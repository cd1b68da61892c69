// Device-side flag protocol that orders the exchanges of a column-sharded Linear between the GPUs
// of one node (no collective, no host): shared by the kernels that carry it.
#pragma once

#include "common.cuh"

namespace t81b200 {

// ---- exchange flags of the column-sharded Linear ----------------------------------------------
// sync_local (this GPU's memory, T81B200_SYNC_WORDS words, zero at start):
//   [0] CTAs of the running kernel that have finished storing   [1] exchanges this rank has completed
//   [2] non-zero once a wait has expired on this rank
//   [16 * (1 + j)] the sequence number peer j has published here
// A kernel that stores into the peers ends with exchange_signal (the last CTA publishes the new
// sequence number into each peer's slot); a kernel that reads what the peers stored starts with
// exchange_wait.  Every wait is bounded.
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ bool exchange_wait(uint32_t *sync_local, int n_peers) {
    const uint32_t expected = *reinterpret_cast<const volatile uint32_t *>(sync_local + 1);
    // [2]: a wait on this rank has expired before (a peer is gone or out of step).  Later waits give up at
    // once, so a lost peer costs one time limit (a few seconds), not one per call.
    if (*reinterpret_cast<const volatile uint32_t *>(sync_local + 2) != 0u) return false;
    for (int j = 0; j < n_peers; ++j) {
        const uint32_t *flag = sync_local + 16 * (1 + j);
        bool seen = false;
        for (uint32_t spin = 0; spin < (1u << 23); ++spin) {
            if ((int32_t)(ld_acquire_sys(flag) - expected) >= 0) { seen = true; break; }
            if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
        }
        if (!seen) {
            *reinterpret_cast<volatile uint32_t *>(sync_local + 2) = 1u;
            return false;
        }
    }
    return true;
}

// Called by one thread per CTA after the CTA's stores and a CTA barrier.
__device__ __forceinline__ void exchange_signal(uint32_t *sync_local, uint32_t *const *sync_peer, int n_peers,
                                                uint32_t total_ctas) {
    __threadfence_system();
    const uint32_t old = atomicAdd(sync_local, 1u);
    if (old == total_ctas - 1) {
        *reinterpret_cast<volatile uint32_t *>(sync_local) = 0u;
        const uint32_t seq = *reinterpret_cast<volatile uint32_t *>(sync_local + 1) + 1u;
        *reinterpret_cast<volatile uint32_t *>(sync_local + 1) = seq;
        __threadfence_system();
        for (int j = 0; j < n_peers; ++j) st_release_sys(sync_peer[j], seq);
    }
}

}  // namespace t81b200
