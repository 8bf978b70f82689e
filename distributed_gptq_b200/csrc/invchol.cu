// Damped-Hessian inverse factor: A (symmetric positive definite) -> U upper
// triangular with A^-1 = U^T U, in place, in fp32 on the CUDA cores.
//
// Identity used: let R be the upper-triangular factor with A = R R^T (a Cholesky
// factorisation that starts from the last row/column).  Then
// A^-1 = R^-T R^-1 = (R^-1)^T (R^-1), and R^-1 is upper triangular with a
// positive diagonal, so U = R^-1.  One Cholesky (K^3/3 flops) and one triangular
// inverse (K^3/3) replace the Cholesky -> full inverse -> Cholesky chain (4K^3/3).
//
// Both steps are written as ordinary *lower* algorithms on the index-reversed
// view V(i,j) = A[K-1-i][K-1-j] (a pointer to the last element with negative
// strides): V = L L^T, then L <- L^-1 in place.  The lower triangle of V is the
// upper triangle of A, which is exactly where U belongs.
//
//   phase 1, per 64-wide panel: factor the diagonal block in one CTA (also keeping
//            its explicit inverse), panel <- panel * inv(L11)^T, trailing SYRK.
//   phase 2, panels from last to first: ws <- -panel * inv(L11);
//            panel <- inv(L22) * ws (triangular matrix product), diagonal block <- inv(L11).
//
// The matrix products run on one strided-view SGEMM kernel (64x64 tile, 4x4 per
// thread).
#include <algorithm>

#include "common.cuh"
#include "sgemm_view.cuh"

namespace {

constexpr int NB = 64;  // panel width

struct View {
  float* p;      // element (0,0)
  int64_t rs;    // row stride (elements, may be negative)
  int64_t cs;    // column stride
  __host__ __device__ float* at(int64_t i, int64_t j) const { return p + i * rs + j * cs; }
  __host__ __device__ View sub(int64_t i, int64_t j) const { return View{p + i * rs + j * cs, rs, cs}; }
};

// ---- diagonal block: Cholesky + explicit inverse -------------------------------------
// One CTA.  D (nb x nb, lower part read) -> L in place (lower part written), and
// Dinv (dense nb x NB, row-major, zeros above the diagonal) <- L^-1.
__global__ void __launch_bounds__(256)
potf2_inv_kernel(View D, int nb, float* __restrict__ Dinv, int32_t* info, int pivot_base,
                 int pivot_sign) {
  __shared__ float S[NB][NB + 1];
  __shared__ float X[NB][NB + 1];
  const int tid = threadIdx.x;
  for (int idx = tid; idx < NB * NB; idx += blockDim.x) {
    int i = idx / NB, j = idx % NB;
    S[i][j] = (i < nb && j <= i) ? *D.at(i, j) : (i == j ? 1.f : 0.f);
  }
  __syncthreads();
  for (int k = 0; k < nb; ++k) {
    if (tid == 0) {
      float d = S[k][k];
      if (!(d > 0.f) || !isfinite(d)) {
        if (info && atomicCAS(info, DGQ_INFO_OK, DGQ_INFO_NOT_POSDEF) == DGQ_INFO_OK)
          info[1] = pivot_base + pivot_sign * k;
        d = 1.f;
      }
      S[k][k] = sqrtf(d);
    }
    __syncthreads();
    const float dk = S[k][k];
    if (tid > k && tid < nb) S[tid][k] = __fdiv_rn(S[tid][k], dk);
    __syncthreads();
    const int rem = nb - k - 1;
    for (int idx = tid; idx < rem * rem; idx += blockDim.x) {
      int i = k + 1 + idx / rem, j = k + 1 + idx % rem;
      if (j <= i) S[i][j] -= S[i][k] * S[j][k];
    }
    __syncthreads();
  }
  // inverse by forward substitution: thread j owns column j of X = L^-1
  if (tid < NB) {
    const int j = tid;
    for (int i = 0; i < NB; ++i) X[i][j] = 0.f;
    if (j < nb) {
      for (int i = j; i < nb; ++i) {
        float acc = (i == j) ? 1.f : 0.f;
        for (int k = j; k < i; ++k) acc -= S[i][k] * X[k][j];
        X[i][j] = __fdiv_rn(acc, S[i][i]);
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < NB * NB; idx += blockDim.x) {
    int i = idx / NB, j = idx % NB;
    if (i < nb && j <= i) *D.at(i, j) = S[i][j];
    Dinv[idx] = X[i][j];
  }
}

__global__ void __launch_bounds__(256)
copy_lower_block_kernel(View D, int nb, const float* __restrict__ Dinv) {
  for (int idx = threadIdx.x; idx < nb * nb; idx += blockDim.x) {
    int i = idx / nb, j = idx % nb;
    if (j <= i) *D.at(i, j) = Dinv[i * NB + j];
  }
}

__global__ void __launch_bounds__(256)
zero_strict_lower_kernel(float* A, int K, int64_t lda) {
  const int64_t total = (int64_t)K * K;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int i = (int)(idx / K), j = (int)(idx - (int64_t)i * K);
    if (j < i) A[(int64_t)i * lda + j] = 0.f;
  }
}

}  // namespace

DGQ_EXPORT int64_t dgq_inv_chol_workspace_bytes(int32_t K) {
  if (K <= 0) return DGQ_ERR_ARG;
  int64_t nblk = dgq_cdiv(K, NB);
  // explicit inverses of all diagonal blocks + one K x NB panel
  return (nblk * NB * NB + (int64_t)K * NB) * (int64_t)sizeof(float);
}

DGQ_EXPORT int32_t dgq_inv_chol_upper(float* A, int32_t K, int64_t lda, int32_t* info, void* ws,
                                      int64_t ws_bytes, void* stream) {
  DGQ_REQUIRE(A && ws && K > 0 && lda >= K, DGQ_ERR_ARG);
  DGQ_REQUIRE(ws_bytes >= dgq_inv_chol_workspace_bytes(K), DGQ_ERR_WORKSPACE);
  DGQ_REQUIRE(dgq_aligned(A, 16) && dgq_aligned(ws, 16), DGQ_ERR_ALIGN);
  cudaStream_t st = dgq_stream(stream);
  const int nblk = (int)dgq_cdiv(K, NB);
  float* dinv_all = reinterpret_cast<float*>(ws);
  float* panel = dinv_all + (int64_t)nblk * NB * NB;  // (K x NB) row-major scratch

  // index-reversed view: V(i,j) = A[K-1-i][K-1-j]
  const View V{A + (int64_t)(K - 1) * lda + (K - 1), -lda, -1};

  // ---- phase 1: V = L L^T (lower, in place)
  for (int b = 0; b < nblk; ++b) {
    const int k0 = b * NB;
    const int nb = std::min(NB, K - k0);
    const int m = K - k0 - nb;  // rows below the diagonal block
    float* dinv = dinv_all + (int64_t)b * NB * NB;
    potf2_inv_kernel<<<1, 256, 0, st>>>(V.sub(k0, k0), nb, dinv, info, K - 1 - k0, -1);
    if (m > 0) {
      View P = V.sub(k0 + nb, k0);
      // P <- P * inv(L11)^T : C[i][j] = sum_k P[i][k] * Dinv[j][k]; one tile column
      // wide, so a CTA reads all of its rows before it writes them (in place is safe)
      GemmArgs t{P.p, P.rs, P.cs, dinv, 1, NB, P.p, P.rs, P.cs, m, nb, nb, 1.f, 0.f};
      launch_gemm<0>(t, st);
      // trailing update, lower part only: V22 -= P P^T
      View C = V.sub(k0 + nb, k0 + nb);
      GemmArgs s{P.p, P.rs, P.cs, P.p, P.cs, P.rs, C.p, C.rs, C.cs, m, m, nb, -1.f, 1.f};
      launch_gemm<1>(s, st);
    }
  }
  // ---- phase 2: L <- L^-1 in place, block columns from last to first
  for (int b = nblk - 1; b >= 0; --b) {
    const int k0 = b * NB;
    const int nb = std::min(NB, K - k0);
    const int m = K - k0 - nb;
    float* dinv = dinv_all + (int64_t)b * NB * NB;
    if (m > 0) {
      View P = V.sub(k0 + nb, k0);
      // panel <- -P * inv(L11)   (m x nb, contiguous scratch with row stride NB)
      GemmArgs a{P.p, P.rs, P.cs, dinv, NB, 1, panel, NB, 1, m, nb, nb, -1.f, 0.f};
      launch_gemm<0>(a, st);
      // P <- inv(L22) * panel, inv(L22) lower triangular and already in place
      View T = V.sub(k0 + nb, k0 + nb);
      GemmArgs t{T.p, T.rs, T.cs, panel, NB, 1, P.p, P.rs, P.cs, m, nb, m, 1.f, 0.f};
      launch_gemm<2>(t, st);
    }
    copy_lower_block_kernel<<<1, 256, 0, st>>>(V.sub(k0, k0), nb, dinv);
  }
  zero_strict_lower_kernel<<<dgq_grid((int64_t)K * K, 256), 256, 0, st>>>(A, K, lda);
  return dgq_launch_status(2 * (int64_t)nblk + 1);  // + the matrix products counted as they go
}
