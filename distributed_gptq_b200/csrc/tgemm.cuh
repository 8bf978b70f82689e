// fp32-accurate matrix product on the sm_100a tensor cores (declaration).
//
//   C(m x n) = alpha * A(m x k) * B + beta * C        all fp32, row-major
//
// A is (m, k) with k contiguous.  B is given either as (n, k) with k contiguous
// ("NT": C = A * Bt^T) or as (k, n) with n contiguous ("NN").  Each fp32 operand is
// split in shared memory into a tf32-representable high part and a low remainder and
// three tcgen05 kind::tf32 products are accumulated (hi*hi, hi*lo, lo*hi), which keeps
// the relative error of a product near 2^-21.
//
// Optional structure, as in sgemm_view.cuh: per-tile clipping of the reduction range for
// triangular operands and a lower-triangle-only result.
#pragma once

#include <stdint.h>

#include <cuda_runtime.h>

namespace dgq {

struct TGemmArgs {
  const float* a; int64_t lda;      // (m, k)
  const float* b; int64_t ldb;      // NT: (n, k)   NN: (k, n)
  float* c; int64_t ldc;            // (m, n)
  int m, n, k;
  float alpha, beta;
  int b_is_kn;                      // 0 = NT, 1 = NN
  int lo_from_j, hi_from_j, hi_from_i, lower_only;
  int32_t* info;                    // device status words for bounded-wait timeouts, may be null
};

// Tile edge of the kernel: reduction clipping uses multiples of it.
constexpr int TGEMM_TILE = 128;

// True when the operands satisfy the kernel's alignment rules (16-byte aligned bases,
// leading dimensions that are multiples of 4 floats) and the problem is large enough to be
// worth a tensor-core launch.
bool tgemm_supported(const TGemmArgs& g);

// Enqueues the product on `st`.  Returns false if a tensor map could not be encoded or the
// launch was refused.
bool tgemm_launch(const TGemmArgs& g, cudaStream_t st);

}  // namespace dgq
