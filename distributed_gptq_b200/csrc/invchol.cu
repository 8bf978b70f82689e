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
//   leaves (<= 64 x 64) are factored and inverted by one small CTA in shared memory.
//
// All products are independent-tile matrix products whose reduction ranges are clipped
// to the non-zero part of the triangular operands: on the tensor cores with the
// split-fp32 scheme of tgemm.cu when both output dimensions reach 128, on the CUDA
// cores (sgemm_view.cuh) below that.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "sgemm_view.cuh"
#include "tgemm.cuh"

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
// One CTA of 256 threads, the block lives in shared memory.  D (nb x nb, nb <= 64, lower
// part read) is replaced by inv(chol(D)) (lower; the part above the diagonal is written as
// zeros).  This kernel sits on the critical path K/64 times, so it is written for latency:
//  * all 256 threads move the block in and out of shared memory;
//  * factorisation, right-looking: row r = tid % 64 is shared by four threads that update
//    every fourth entry of it; the pivot's reciprocal square root comes from rsqrt plus one
//    Newton step (every thread computes it itself: no broadcast step), the column is
//    broadcast through a double-buffered array so one barrier per step is enough for it;
//  * inverse: thread t < 64 solves L x = e_t for column t by forward substitution, all
//    threads walking the same row of L (a broadcast read) against their own column of X.
// Loops are ordinary loops so that the code stays resident in the instruction cache.
constexpr int LEAF_THREADS = 256;

__global__ void __launch_bounds__(LEAF_THREADS)
leaf_inv_chol_kernel(float* __restrict__ D, int64_t ldd, int nb, int32_t* info, int pivot_base) {
  __shared__ float S[NB][NB + 1];
  __shared__ float X[NB][NB + 1];
  __shared__ float colk[2][NB];
  const int tid = threadIdx.x;
  const int r = tid & (NB - 1);   // row owned during the factorisation
  const int part = tid >> 6;      // which quarter of the row's entries
#pragma unroll 4
  for (int idx = tid; idx < NB * NB; idx += LEAF_THREADS) {
    const int i = idx / NB, j = idx % NB;
    S[i][j] = (i < nb && j < nb) ? (j <= i ? D[(int64_t)i * ldd + j] : 0.f) : (i == j ? 1.f : 0.f);
  }
  __syncthreads();
  for (int k = 0; k < NB; ++k) {
    float d = S[k][k];
    if (!(d > 0.f) || !isfinite(d)) {
      if (tid == k && info && atomicCAS(info, DGQ_INFO_OK, DGQ_INFO_NOT_POSDEF) == DGQ_INFO_OK)
        info[1] = pivot_base - k;
      d = 1.f;
    }
    float rs = rsqrtf(d);
    rs = rs * fmaf(-0.5f * d * rs, rs, 1.5f);   // one Newton step: 1/sqrt(d) to ~1 ulp
    const float lik = (r == k) ? d * rs : (r > k ? S[r][k] * rs : 0.f);
    float* ck = colk[k & 1];
    if (part == 0) ck[r] = lik;
    __syncthreads();
    if (r > k) {
      if (part == 0) S[r][k] = lik;
      // entries j = k+1+part, k+5+part, ... <= r of row r, eight at a time with all loads
      // of a batch issued before its stores
      int j = k + 1 + part;
      for (; j + 28 <= r; j += 32) {
        float c[8], v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) { c[u] = ck[j + 4 * u]; v[u] = S[r][j + 4 * u]; }
#pragma unroll
        for (int u = 0; u < 8; ++u) S[r][j + 4 * u] = fmaf(-lik, c[u], v[u]);
      }
      for (; j <= r; j += 4) S[r][j] = fmaf(-lik, ck[j], S[r][j]);
    } else if (r == k && part == 0) {
      S[r][k] = lik;
    }
    __syncthreads();  // the next pivot S[k+1][k+1] and the column buffer's reuse two steps on
  }
  // X = L^-1, column t; entries above the diagonal come out as exact zeros
  if (tid < NB) {
    const int t = tid;
    for (int i = 0; i < NB; ++i) {
      float a0 = (i == t) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      int k = 0;
      for (; k + 3 < i; k += 4) {
        a0 = fmaf(-S[i][k], X[k][t], a0);
        a1 = fmaf(-S[i][k + 1], X[k + 1][t], a1);
        a2 = fmaf(-S[i][k + 2], X[k + 2][t], a2);
        a3 = fmaf(-S[i][k + 3], X[k + 3][t], a3);
      }
      for (; k < i; ++k) a0 = fmaf(-S[i][k], X[k][t], a0);
      X[i][t] = (i >= t) ? __fdiv_rn((a0 + a1) + (a2 + a3), S[i][i]) : 0.f;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < NB * NB; idx += LEAF_THREADS) {
    const int i = idx / NB, j = idx % NB;
    if (i < nb && j < nb) D[(int64_t)i * ldd + j] = X[i][j];
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
  bool use_tensor;
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

// One product of the recursion.  B is (n, k) row-major when !b_is_kn, (k, n) when b_is_kn.
void mm(Plan& p, const float* a, int64_t lda, const float* b, int64_t ldb, bool b_is_kn, float* c,
        int64_t ldc, int m, int n, int k, float alpha, float beta, int lo_from_j, int hi_from_j,
        int hi_from_i, int lower_only) {
  if (p.use_tensor && m >= dgq::TGEMM_TILE && n >= dgq::TGEMM_TILE) {
    dgq::TGemmArgs t;
    t.a = a; t.lda = lda; t.b = b; t.ldb = ldb; t.c = c; t.ldc = ldc;
    t.m = m; t.n = n; t.k = k; t.alpha = alpha; t.beta = beta; t.b_is_kn = b_is_kn ? 1 : 0;
    t.lo_from_j = lo_from_j; t.hi_from_j = hi_from_j; t.hi_from_i = hi_from_i;
    t.lower_only = lower_only; t.info = p.info;
    if (dgq::tgemm_supported(t) && dgq::tgemm_launch(t, p.st)) return;
  }
  GemmArgs g = b_is_kn ? gemm_args(a, lda, 1, b, ldb, 1, c, ldc, 1, m, n, k, alpha, beta)
                       : gemm_args(a, lda, 1, b, 1, ldb, c, ldc, 1, m, n, k, alpha, beta);
  g.lo_from_j = lo_from_j; g.hi_from_j = hi_from_j; g.hi_from_i = hi_from_i;
  g.lower_only = lower_only;
  launch_gemm(g, p.st);
}

void rec(Plan& p, int o, int n, int depth) {
  float* V = p.V;
  const int64_t ld = p.ldv;
  if (n <= NB) {
    leaf_inv_chol_kernel<<<1, LEAF_THREADS, 0, p.st>>>(V + (int64_t)o * ld + o, ld, n, p.info, p.K - 1 - o);
    ++p.leaves;
    return;
  }
  const int h = split_point(n), m2 = n - h;
  float* V11 = V + (int64_t)o * ld + o;
  float* V21 = V + (int64_t)(o + h) * ld + o;
  float* V22 = V + (int64_t)(o + h) * ld + (o + h);
  float* T1 = p.T1[depth];
  rec(p, o, h, depth + 1);
  // T1 = V21 * X11^T : X11[j][k] is non-zero for k <= j
  mm(p, V21, ld, V11, ld, false, T1, h, m2, h, h, 1.f, 0.f, 0, 1, 0, 0);
  // V22 -= T1 * T1^T, lower part
  mm(p, T1, h, T1, h, false, V22, ld, m2, m2, h, -1.f, 1.f, 0, 0, 0, 1);
  rec(p, o + h, m2, depth + 1);
  // T2 = T1 * X11 : X11[k][j] is non-zero for k >= j
  mm(p, T1, h, V11, ld, true, p.T2, h, m2, h, h, 1.f, 0.f, 1, 0, 0, 0);
  // V21 = -X22 * T2 : X22[i][k] is non-zero for k <= i
  mm(p, V22, ld, p.T2, h, true, V21, ld, m2, h, m2, -1.f, 0.f, 0, 0, 1, 0);
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
  p.use_tensor = dgq_use_tensor_gemm();
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
