// Glue between the reference's C++ linalg API and libt81_b200.so.
//
// The reference's headers declare a CUDA backend — cuda_available(),
// cuda_gemm_ternary(), cuda_where/clamp/lerp/addcmul() in namespace
// t81::linalg::detail (include/t81/linalg/gemm_gpu.hpp:68-78,122-129) — that its
// dispatcher calls when built with T81LIB_USE_CUDA=1 (gemm_gpu.hpp:191-195,
// src/linalg/gemm_dispatch.cpp:222-227).  This file defines those symbols on top of
// the C ABI in t81_b200.h, so a maintainer compiles it into the reference (in place of
// src/linalg/gemm_cuda.cu) and links -lt81_b200; no reference header changes.
//
// It also offers the additive TRIT-mode overload gemm_ternary(A limbs, B floats, ...).
//
// Build (from the reference checkout):
//   g++ -std=c++20 -DT81LIB_USE_CUDA=1 -Iinclude -I<this repo>/include -c linalg_cuda_shim.cpp
#include <span>
#include <stdexcept>
#include <string>

#include <t81/linalg/gemm_gpu.hpp>

#include "t81_b200.h"

namespace t81::linalg {

namespace detail {

namespace {
[[noreturn]] void raise(int code) {
    const std::string message = t81b200_last_error();
    // argument problems are std::invalid_argument like the dispatcher's own checks
    // (gemm_gpu.hpp:171-186); device failures std::runtime_error (gemm_cuda.cu:22-27)
    if (code == T81B200_EINVAL || code == T81B200_EALIGN || code == T81B200_ELIMIT || code == T81B200_EWORKSPACE)
        throw std::invalid_argument(message);
    throw std::runtime_error(message);
}
}  // namespace

bool cuda_available() noexcept { return t81b200_device_available() != 0; }

// Backend selection of the reference build (declared gemm_gpu.hpp:61): prefer the device.
Backend get_current_backend() noexcept { return cuda_available() ? Backend::CUDA : Backend::CPU; }

// LIMB mode: host spans in, host span out, synchronous — the contract of the reference's
// cuda_gemm_ternary (src/linalg/gemm_cuda.cu:284-341).
void cuda_gemm_ternary(std::span<const core::limb> A, std::span<const core::limb> B, std::span<float> C, int M,
                       int N, int K, float alpha, float beta) {
    const int rc = t81b200_gemm_limb_host(reinterpret_cast<const std::uint8_t *>(A.data()),
                                          reinterpret_cast<const std::uint8_t *>(B.data()), C.data(), M, N,
                                          K / core::limb::TRITS, alpha, beta);
    if (rc != T81B200_OK) raise(rc);
}

// The four elementwise helpers are not part of the packed-matmul path and are not
// provided by libt81_b200; the reference's CPU implementations stay in charge of them.
void cuda_where(const TensorMetadata &, const TensorMetadata &, const TensorMetadata &, TensorMetadata &) {
    throw std::runtime_error("cuda_where is not provided by t81_b200; use Backend::CPU");
}
void cuda_clamp(const TensorMetadata &, TensorMetadata &, float, float) {
    throw std::runtime_error("cuda_clamp is not provided by t81_b200; use Backend::CPU");
}
void cuda_lerp(const TensorMetadata &, const TensorMetadata &, const TensorMetadata &, TensorMetadata &) {
    throw std::runtime_error("cuda_lerp is not provided by t81_b200; use Backend::CPU");
}
void cuda_addcmul(const TensorMetadata &, const TensorMetadata &, const TensorMetadata &, float, TensorMetadata &) {
    throw std::runtime_error("cuda_addcmul is not provided by t81_b200; use Backend::CPU");
}

}  // namespace detail

// TRIT mode (additive): A packed limbs (M, K/48), B dense floats (K, N), C (M, N):
// C = alpha * T(A) * B + beta * C with T(A) in {-1, 0, +1}.
void gemm_ternary(std::span<const core::limb> A, std::span<const float> B, std::span<float> C, int M, int N, int K,
                  float alpha, float beta) {
    if (M < 0 || N < 0 || K < 0) throw std::invalid_argument("gemm_ternary dimensions must be non-negative");
    if (K % core::limb::TRITS != 0) throw std::invalid_argument("gemm_ternary requires K divisible by 48");
    const std::size_t kl = static_cast<std::size_t>(K / core::limb::TRITS);
    if (static_cast<std::size_t>(M) * kl != A.size()) throw std::invalid_argument("A span size does not match (M, K / 48)");
    if (static_cast<std::size_t>(K) * static_cast<std::size_t>(N) != B.size())
        throw std::invalid_argument("B span size does not match (K, N)");
    if (static_cast<std::size_t>(M) * static_cast<std::size_t>(N) != C.size())
        throw std::invalid_argument("C span size does not match (M, N)");
    const int rc = t81b200_gemm_trit_host(reinterpret_cast<const std::uint8_t *>(A.data()), B.data(), C.data(), M, N, K,
                                          alpha, beta);
    if (rc != T81B200_OK) detail::raise(rc);
}

}  // namespace t81::linalg
