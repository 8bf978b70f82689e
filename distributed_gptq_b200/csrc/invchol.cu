// Damped-Hessian inverse factor: A (symmetric positive definite) -> U upper
// triangular with A^-1 = U^T U, in fp32.
//
// Identity used: let R be the upper-triangular factor with A = R R^T (a Cholesky
// factorisation that starts from the last row/column).  Then
// A^-1 = R^-T R^-1 = (R^-1)^T (R^-1), and R^-1 is upper triangular with a
// positive diagonal, so U = R^-1.  With J the index reversal, J A J = L L^T is an
// ordinary lower Cholesky factorisation and U = J L^-1 J.  One factorisation and
// one triangular inverse (2K^3/3 flops together) replace the
// Cholesky -> full inverse -> Cholesky chain (4K^3/3).
//
// The work is done on a reversed copy V = J A J (lower triangle, zeros above) by a
// recursion that produces L^-1 directly, without ever storing L:
//
//   inv_chol(V):  split V = [V11 . ; V21 V22] at a multiple of 64
//     X11 = inv_chol(V11)                      (recursion; X11 = L11^-1, lower)
//     T   = V21 * X11^T                        (= L21)
//     V22 -= T * T^T                           (Schur complement, lower part)
//     X22 = inv_chol(V22)                      (recursion)
//     V21 = -X22 * (T * X11)                   (block of the inverse)
//   leaves (<= 64 x 64) are factored and inverted by one small CTA in registers.
//
// All products are large, independent-tile matrix products (sgemm_view.cuh) whose
// reduction ranges are clipped to the non-zero part of the triangular operands.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "sgemm_view.cuh"

namespace {

constexpr int NB = 64;  // leaf size

// ---- reversal copies ---------------------------------------------------------------------
// V[i][j] = (j <= i) ? A[K-1-i][K-1-j] : 0     (reads the upper triangle of A)
__global__ void __launch_bounds__(256)
reverse_in_kernel(const float* __restrict__ A, int64_t lda, float* __restrict__ V, int64_t ldv,
                  int K) {
  const int64_t total = (int64_t)K * K;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx / K), j = (int)(idx - (int64_t)i * K);
    V[(int64_t)i * ldv + j] = (j <= i) ? A[(int64_t)(K - 1 - i) * lda + (K - 1 - j)] : 0.f;
  }
}
// A[i][j] = (j >= i) ? V[K-1-i][K-1-j] : 0
__global__ void __launch_bounds__(256)
reverse_out_kernel(const float* __restrict__ V, int64_t ldv, float* __restrict__ A, int64_t lda,
                   int K) {
  const int64_t total = (int64_t)K * K;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx / K), j = (int)(idx - (int64_t)i * K);
    A[(int64_t)i * lda + j] = (j >= i) ? V[(int64_t)(K - 1 - i) * ldv + (K - 1 - j)] : 0.f;
  }
}

// ---- leaf: Cholesky + inverse of one diagonal block ------------------------------------------
// 64 threads.  D (nb x nb, nb <= 64, lower part read) is replaced by inv(chol(D)) (lower;
// the part above the diagonal is written as zeros).  Thread i owns row i of the block
// in registers during the factorisation and column i of the inverse afterwards; all
// loops are fully unrolled so the register arrays are never indexed dynamically.
__global__ void __launch_bounds__(NB)
leaf_inv_chol_kernel(float* __restrict__ D, int64_t ldd, int nb, int32_t* info, int pivot_base) {
  __shared__ float S[NB][NB + 1];
  __shared__ float col[2][NB];
  __shared__ float piv;
  const int t = threadIdx.x;
  for (int idx = t; idx < NB * NB; idx += NB) {
    const int i = idx / NB, j = idx % NB;
    S[i][j] = (i < nb && j < nb) ? (j <= i ? D[(int64_t)i * ldd + j] : 0.f) : (i == j ? 1.f : 0.f);
  }
  __syncthreads();
  float a[NB];
#pragma unroll
  for (int j = 0; j < NB; ++j) a[j] = S[t][j];

#pragma unroll
  for (int k = 0; k < NB; ++k) {
    if (t == k) {
      float d = a[k];
      if (!(d > 0.f) || !isfinite(d)) {
        if (info && atomicCAS(info, DGQ_INFO_OK, DGQ_INFO_NOT_POSDEF) == DGQ_INFO_OK)
          info[1] = pivot_base - k;
        d = 1.f;
      }
      piv = sqrtf(d);
    }
    __syncthreads();
    const float d = piv;
    if (t == k) a[k] = d;
    if (t > k) a[k] = __fdiv_rn(a[k], d);
    col[k & 1][t] = (t > k) ? a[k] : 0.f;
    __syncthreads();
    const float lik = a[k];
#pragma unroll
    for (int j = k + 1; j < NB; ++j)
      if (j <= t) a[j] = fmaf(-lik, col[k & 1][j], a[j]);
  }
  // L back to shared memory (row t), zeros above the diagonal
  __syncthreads();
#pragma unroll
  for (int j = 0; j < NB; ++j) S[t][j] = (j <= t) ? a[j] : 0.f;
  __syncthreads();
  // column t of X = L^-1 by forward substitution; entries above the diagonal come out 0
  float x[NB];
#pragma unroll
  for (int i = 0; i < NB; ++i) {
    float acc = (i == t) ? 1.f : 0.f;
#pragma unroll
    for (int k = 0; k < i; ++k) acc = fmaf(-S[i][k], x[k], acc);
    x[i] = (i >= t) ? __fdiv_rn(acc, S[i][i]) : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < NB; ++i) S[i][t] = x[i];
  __syncthreads();
  for (int idx = t; idx < NB * NB; idx += NB) {
    const int i = idx / NB, j = idx % NB;
    if (i < nb && j < nb) D[(int64_t)i * ldd + j] = S[i][j];
  }
}

// ---- the recursion, unrolled on the host into a launch sequence --------------------------------
struct Plan {
  float* V; int64_t ldv; int K;
  float* T1[32];        // per recursion depth: the L21 block of the node being processed
  float* T2;            // transient product T * X11
  int32_t* info;
  cudaStream_t st;
  int64_t leaves;
};

int split_point(int n) {
  const int blocks = (n + NB - 1) / NB;
  return (blocks / 2) * NB;  // first half gets floor(blocks/2) leaves (>= 1 when n > NB)
}

void rec_workspace(int n, int depth, std::vector<int64_t>& need, int64_t& t2) {
  if (n <= NB) return;
  const int h = split_point(n), m2 = n - h;
  if ((int)need.size() <= depth) need.resize(depth + 1, 0);
  need[depth] = std::max<int64_t>(need[depth], (int64_t)m2 * h);
  t2 = std::max<int64_t>(t2, (int64_t)m2 * h);
  rec_workspace(h, depth + 1, need, t2);
  rec_workspace(m2, depth + 1, need, t2);
}

void rec(Plan& p, int o, int n, int depth) {
  float* V = p.V;
  const int64_t ld = p.ldv;
  if (n <= NB) {
    leaf_inv_chol_kernel<<<1, NB, 0, p.st>>>(V + (int64_t)o * ld + o, ld, n, p.info, p.K - 1 - o);
    ++p.leaves;
    return;
  }
  const int h = split_point(n), m2 = n - h;
  float* V11 = V + (int64_t)o * ld + o;
  float* V21 = V + (int64_t)(o + h) * ld + o;
  float* V22 = V + (int64_t)(o + h) * ld + (o + h);
  float* T1 = p.T1[depth];
  rec(p, o, h, depth + 1);
  {  // T1 = V21 * X11^T : B(k,j) = X11[j][k], non-zero for k <= j
    GemmArgs g = gemm_args(V21, ld, 1, V11, 1, ld, T1, h, 1, m2, h, h, 1.f, 0.f);
    g.hi_from_j = 1;
    launch_gemm(g, p.st);
  }
  {  // V22 -= T1 * T1^T, lower part
    GemmArgs g = gemm_args(T1, h, 1, T1, 1, h, V22, ld, 1, m2, m2, h, -1.f, 1.f);
    g.lower_only = 1;
    launch_gemm(g, p.st);
  }
  rec(p, o + h, m2, depth + 1);
  {  // T2 = T1 * X11 : B(k,j) = X11[k][j], non-zero for k >= j
    GemmArgs g = gemm_args(T1, h, 1, V11, ld, 1, p.T2, h, 1, m2, h, h, 1.f, 0.f);
    g.lo_from_j = 1;
    launch_gemm(g, p.st);
  }
  {  // V21 = -X22 * T2 : A = X22 lower triangular, non-zero for k <= i
    GemmArgs g = gemm_args(V22, ld, 1, p.T2, h, 1, V21, ld, 1, m2, h, m2, -1.f, 0.f);
    g.hi_from_i = 1;
    launch_gemm(g, p.st);
  }
}

int64_t round4(int64_t x) { return (x + 3) / 4 * 4; }

}  // namespace

DGQ_EXPORT int64_t dgq_inv_chol_workspace_bytes(int32_t K) {
  if (K <= 0) return DGQ_ERR_ARG;
  std::vector<int64_t> need;
  int64_t t2 = 0;
  rec_workspace(K, 0, need, t2);
  int64_t floats = (int64_t)K * round4(K) + round4(t2);
  for (int64_t v : need) floats += round4(v);
  return (floats + 4) * (int64_t)sizeof(float);
}

DGQ_EXPORT int32_t dgq_inv_chol_upper(float* A, int32_t K, int64_t lda, int32_t* info, void* ws,
                                      int64_t ws_bytes, void* stream) {
  DGQ_REQUIRE(A && ws && K > 0 && lda >= K, DGQ_ERR_ARG);
  DGQ_REQUIRE(ws_bytes >= dgq_inv_chol_workspace_bytes(K), DGQ_ERR_WORKSPACE);
  DGQ_REQUIRE(dgq_aligned(A, 16) && dgq_aligned(ws, 16), DGQ_ERR_ALIGN);
  Plan p;
  p.st = dgq_stream(stream);
  p.K = K;
  p.info = info;
  p.leaves = 0;
  p.ldv = round4(K);
  float* w = reinterpret_cast<float*>(ws);
  p.V = w;
  w += (int64_t)K * p.ldv;
  std::vector<int64_t> need;
  int64_t t2 = 0;
  rec_workspace(K, 0, need, t2);
  DGQ_REQUIRE(need.size() <= 32, DGQ_ERR_SIZE);
  p.T2 = w;
  w += round4(t2);
  for (size_t d = 0; d < need.size(); ++d) {
    p.T1[d] = w;
    w += round4(need[d]);
  }
  const unsigned grid = dgq_grid((int64_t)K * K, 256);
  reverse_in_kernel<<<grid, 256, 0, p.st>>>(A, lda, p.V, p.ldv, K);
  rec(p, 0, K, 0);
  reverse_out_kernel<<<grid, 256, 0, p.st>>>(p.V, p.ldv, A, lda, K);
  return dgq_launch_status(2 + p.leaves);  // matrix products are counted as they are launched
}
