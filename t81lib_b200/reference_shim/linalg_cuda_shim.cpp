// Glue between the reference's C++ linalg API and libt81_b200.so.
//
// The reference's headers declare a CUDA backend — cuda_available(), cuda_gemm_ternary(),
// cuda_where / cuda_clamp / cuda_lerp / cuda_addcmul in namespace t81::linalg::detail
// (include/t81/linalg/gemm_gpu.hpp:68,75-78,122-129,217-231) — that its dispatcher calls when
// built with T81LIB_USE_CUDA=1 (gemm_gpu.hpp:191-195, src/linalg/gemm_dispatch.cpp:222-227,
// 252-324).  This file defines exactly those six symbols on top of the C ABI in t81_b200.h.  A
// maintainer compiles it into the reference in place of src/linalg/gemm_cuda.cu and links
// libt81_b200.so; no reference source changes.  get_current_backend() stays where the reference
// defines it (src/linalg/gemm_dispatch.cpp:220-237).
//
// Where the data lives.  The dispatcher hands over spans (gemm) or TensorMetadata (elementwise)
// whose pointers are host arrays for numpy / std::vector callers and device memory for torch
// CUDA tensors (python/bindings.cpp:297-326 sets device_type CUDA and requires_sync for those;
// detail::gemm_ternary(const TensorMetadata&...) turns them into spans over the same pointers,
// src/linalg/gemm_dispatch.cpp:325-344).  The *_auto entry points look at each pointer, use device
// memory in place and stage host arrays, and return when the result is complete, which covers the
// synchronise-on-requires_sync rule of the reference (src/linalg/gemm_cuda.cu:205-209).
//
// It also offers the additive TRIT-mode overload gemm_ternary(A limbs, B floats, ...) and a
// TensorMetadata form of it.
//
// Build (from the reference checkout):
//   g++ -std=c++20 -DT81LIB_USE_CUDA=1 -Iinclude -I<this repo>/include -c linalg_cuda_shim.cpp
#include <algorithm>
#include <cstdint>
#include <limits>
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

// The checks of read_ptr / write_ptr (src/linalg/gemm_cuda.cu:29-60), with their messages.
const float *float_ptr(const TensorMetadata &meta) {
    if (meta.data_ptr == nullptr) throw std::invalid_argument("tensor metadata lacks a data pointer");
    if (!meta.dtype_is_float32()) throw std::invalid_argument("CUDA kernels only support float32");
    if (!meta.is_contiguous()) throw std::invalid_argument("CUDA kernels require contiguous storage");
    const auto offset = static_cast<std::size_t>(std::max<int64_t>(meta.storage_offset, 0LL)) * sizeof(float);
    return reinterpret_cast<const float *>(reinterpret_cast<const std::uint8_t *>(meta.data_ptr) + offset);
}

void elementwise(int op, const TensorMetadata *a, const TensorMetadata *b, const TensorMetadata *c, TensorMetadata &out,
                 std::size_t total, float s0, float s1) {
    if (total == 0) return;
    for (const TensorMetadata *in : {a, b, c})
        if (in && in->numel() != total) throw std::invalid_argument("input shapes must match the output length");
    if (out.numel() != total) throw std::invalid_argument("input shapes must match the output length");
    const int rc = t81b200_elementwise_auto(op, float_ptr(*a), b ? float_ptr(*b) : nullptr, c ? float_ptr(*c) : nullptr,
                                            const_cast<float *>(float_ptr(out)), static_cast<int64_t>(total), s0, s1);
    if (rc != T81B200_OK) raise(rc);
}

}  // namespace

bool cuda_available() noexcept { return t81b200_device_available() != 0; }

// LIMB mode (src/linalg/gemm_cuda.cu:284-341): spans over host arrays or over device memory.
void cuda_gemm_ternary(std::span<const core::limb> A, std::span<const core::limb> B, std::span<float> C, int M,
                       int N, int K, float alpha, float beta) {
    const int rc = t81b200_gemm_limb_auto(reinterpret_cast<const std::uint8_t *>(A.data()),
                                          reinterpret_cast<const std::uint8_t *>(B.data()), C.data(), M, N,
                                          K / core::limb::TRITS, alpha, beta);
    if (rc != T81B200_OK) raise(rc);
}

// src/linalg/gemm_cuda.cu:211-283: the element count comes from the condition / input for where and
// clamp and from the output for lerp and addcmul.
void cuda_where(const TensorMetadata &condition, const TensorMetadata &x, const TensorMetadata &y, TensorMetadata &out) {
    elementwise(T81B200_EW_WHERE, &condition, &x, &y, out, condition.numel(), 0.0f, 0.0f);
}
void cuda_clamp(const TensorMetadata &input, TensorMetadata &out, float min_value, float max_value) {
    elementwise(T81B200_EW_CLAMP, &input, nullptr, nullptr, out, input.numel(), min_value, max_value);
}
void cuda_lerp(const TensorMetadata &start, const TensorMetadata &end, const TensorMetadata &weight, TensorMetadata &out) {
    elementwise(T81B200_EW_LERP, &start, &end, &weight, out, out.numel(), 0.0f, 0.0f);
}
void cuda_addcmul(const TensorMetadata &input, const TensorMetadata &tensor1, const TensorMetadata &tensor2, float value,
                  TensorMetadata &out) {
    elementwise(T81B200_EW_ADDCMUL, &input, &tensor1, &tensor2, out, out.numel(), value, 0.0f);
}

// TRIT mode on TensorMetadata (additive): A packed limbs (M, K/48), B float32 (K, N), C float32 (M, N),
// each on the host or on the device as its metadata says; the checks and messages follow
// detail::gemm_ternary (src/linalg/gemm_dispatch.cpp:39-122,325-344).
void gemm_ternary_dense(const TensorMetadata &A, const TensorMetadata &B, TensorMetadata &C, float alpha, float beta) {
    auto shape = [](const TensorMetadata &meta) {
        if (meta.sizes.size() != 2) throw std::invalid_argument("tensor metadata must describe a rank-2 matrix");
        for (const int64_t v : meta.sizes)
            if (v < 0 || v > std::numeric_limits<int>::max()) throw std::invalid_argument("tensor dimension exceeds supported range");
        return std::pair<int64_t, int64_t>{meta.sizes[0], meta.sizes[1]};
    };
    const auto [M, k_limbs] = shape(A);
    const auto [b_rows, N] = shape(B);
    const int64_t K = k_limbs * core::limb::TRITS;
    if (b_rows != K) throw std::invalid_argument("B shape must match the K dimension of A");
    const auto [c_rows, c_cols] = shape(C);
    if (c_rows != M || c_cols != N) throw std::invalid_argument("C shape must match the output dimensions");
    if (!A.dtype_is_ternary_limb()) throw std::invalid_argument("tensor metadata must describe ternary limbs");
    if (A.data_ptr == nullptr) throw std::invalid_argument("tensor metadata must provide a valid data pointer");
    if (!A.is_contiguous() || !B.is_contiguous() || !C.is_contiguous())
        throw std::invalid_argument("tensor metadata must describe contiguous storage");
    if (!B.dtype_is_float32() || !C.dtype_is_float32()) throw std::invalid_argument("tensor metadata must describe float32 data");
    if (B.data_ptr == nullptr || C.data_ptr == nullptr) throw std::invalid_argument("tensor metadata must provide a valid data pointer");
    const auto *a = reinterpret_cast<const std::uint8_t *>(A.data_ptr) +
                    static_cast<std::size_t>(std::max<int64_t>(A.storage_offset, 0LL)) * core::limb::BYTES;
    const int rc = t81b200_gemm_trit_auto(a, float_ptr(B), const_cast<float *>(float_ptr(C)), M, N, K, alpha, beta);
    if (rc != T81B200_OK) raise(rc);
}

}  // namespace detail

// TRIT mode (additive): A packed limbs (M, K/48), B dense floats (K, N), C (M, N):
// C = alpha * T(A) * B + beta * C with T(A) in {-1, 0, +1}.  Same validation as
// gemm_ternary_dispatch (gemm_gpu.hpp:171-190).
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
    if (M == 0 || N == 0) return;
    const int rc = t81b200_gemm_trit_auto(reinterpret_cast<const std::uint8_t *>(A.data()), B.data(), C.data(), M, N, K,
                                          alpha, beta);
    if (rc != T81B200_OK) detail::raise(rc);
}

}  // namespace t81::linalg
