// Declarations of what linalg_cuda_shim.cpp adds to the reference's t81::linalg API.  Everything
// else the shim defines is already declared by the reference's own include/t81/linalg/gemm_gpu.hpp.
#pragma once

#include <span>

#include <t81/core/limb.hpp>
#include <t81/tensor_metadata.hpp>

namespace t81::linalg {

// TRIT mode: C = alpha * T(A) * B + beta * C, A packed limbs (M, K/48) whose trits T(A) are
// -1/0/+1, B dense (K, N), C (M, N); host or device memory (all three alike).  The LIMB-mode
// overload with packed B stays the reference's (include/t81/linalg/gemm.hpp:68-77).
void gemm_ternary(std::span<const core::limb> A, std::span<const float> B, std::span<float> C, int M, int N, int K,
                  float alpha, float beta);

namespace detail {
// The same on TensorMetadata: A dtype TernaryLimb (M, K/48), B and C Float; device_type says where each lives.
void gemm_ternary_dense(const TensorMetadata &A, const TensorMetadata &B, TensorMetadata &C, float alpha, float beta);
}  // namespace detail

}  // namespace t81::linalg
