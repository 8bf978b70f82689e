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
//   inv_chol(V):  split V = [V11 . ; V21 V22] at a multiple of 128
//     X11 = inv_chol(V11)                      (recursion; X11 = L11^-1, lower)
//     T   = V21 * X11^T                        (= L21)
//     V22 -= T * T^T                           (Schur complement, lower part)
//     X22 = inv_chol(V22)                      (recursion)
//     V21 = -X22 * (T * X11)                   (block of the inverse)
//   leaves (<= 128 x 128) are factored and inverted by one CTA in shared memory.
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

constexpr int NB = 128;  // leaf size: blocks of at most NB x NB are handled by one CTA

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
// One CTA of 256 threads.  D (nb x nb, nb <= 128, lower part read) is replaced by
// inv(chol(D)) (lower; the part above the diagonal is written as zeros).  This kernel
// sits on the critical path K/128 times, so it is written for latency; the whole block
// lives in shared memory.  It applies the same recursion as the host code, twice:
//   128 = 2 x 64:  X11 = leaf64(A11); L21 = A21 X11^T; A22 -= L21 L21^T; X22 = leaf64(A22);
//                  X21 = -X22 (L21 X11)                      (products: all eight warps)
//   64  = 2 x 32:  the same with 32 x 32 tiles, whose factorisation and inverse are done by
//                  one warp each:
// chol32: lane i keeps row i of the tile in 32 registers, rotated so that the current
// column always sits in register 0 (the shift is folded into the update's destination
// register), pivots and column entries travel by warp shuffles - no barriers, no
// dynamically indexed registers, and a rolled loop that stays in the instruction cache.
// inv32: lane t keeps column t of the inverse the same way; the entries of L it needs are
// the same for all lanes and are read from shared memory as broadcasts.
constexpr int LEAF = 128;             // largest block the leaf kernel takes
constexpr int LEAF_THREADS = 256;
constexpr int HT = 32;                // tile edge
constexpr int LD = LEAF + 1;          // row stride of the shared-memory block (odd: no bank conflicts)
constexpr int LD64 = 64 + 1;

// Eight consecutive steps k0 .. k0+7 of the factorisation with W live columns to the right
// of the current one (W = 31 - k0: the rolled loop cannot shrink its body step by step, so
// it is cut into four phases of decreasing width).
template <int W>
__device__ __forceinline__ void chol32_phase(float* S, float* rdiag, float (&a)[HT], int r0,
                                             int k0, int lane, int32_t* info, int pivot_base) {
#pragma unroll 1
  for (int k = k0; k < k0 + 8; ++k) {
    float d = __shfl_sync(0xffffffffu, a[0], k);
    if (!(d > 0.f) || !isfinite(d)) {
      if (lane == k && info && atomicCAS(info, DGQ_INFO_OK, DGQ_INFO_NOT_POSDEF) == DGQ_INFO_OK)
        info[1] = pivot_base - k;
      d = 1.f;
    }
    float rs = rsqrtf(d);
    rs = rs * fmaf(-0.5f * d * rs, rs, 1.5f);   // one Newton step: 1/sqrt(d) to ~1 ulp
    const float l = (lane == k) ? d * rs : (lane > k ? a[0] * rs : 0.f);
    S[(r0 + lane) * LD + r0 + k] = l;
    if (lane == k) rdiag[r0 + k] = rs;   // 1 / L[k][k], reused by the inverse
    // all shuffles of the step are issued before the first dependent multiply-add, so
    // that their latencies overlap instead of adding up
    float lj[W + 1];
#pragma unroll
    for (int j = 1; j <= W; ++j) lj[j] = __shfl_sync(0xffffffffu, l, (k + j) & (HT - 1));
    // column k+j of the row moves from register j to register j-1 while it is updated
#pragma unroll
    for (int j = 1; j <= W; ++j) a[j - 1] = fmaf(-l, lj[j], a[j]);
    a[W] = 0.f;
  }
}

// L (lower, including the diagonal) of the 32 x 32 tile at S[r0.., r0..] replaces it; the
// entries above the diagonal are written as zeros.  One warp.
__device__ __forceinline__ void chol32(float* S, float* rdiag, int r0, int lane, int32_t* info,
                                       int pivot_base) {
  float a[HT];
#pragma unroll
  for (int j = 0; j < HT; ++j) a[j] = S[(r0 + lane) * LD + r0 + j];
  chol32_phase<31>(S, rdiag, a, r0, 0, lane, info, pivot_base);
  chol32_phase<23>(S, rdiag, a, r0, 8, lane, info, pivot_base);
  chol32_phase<15>(S, rdiag, a, r0, 16, lane, info, pivot_base);
  chol32_phase<7>(S, rdiag, a, r0, 24, lane, info, pivot_base);
}

template <int W>
__device__ __forceinline__ void inv32_phase(const float* S, float* X, const float* rdiag,
                                            float (&y)[HT], int r0, int k0, int lane) {
#pragma unroll 1
  for (int k = k0; k < k0 + 8; ++k) {
    // column k of L first (independent of y), then the dependent arithmetic
    float lk[W + 1];
#pragma unroll
    for (int i = 1; i <= W; ++i) lk[i] = S[(r0 + min(k + i, HT - 1)) * LD + r0 + k];  // past the tile: dead
    const float xk = y[0] * rdiag[r0 + k];                 // row k of X is final
    X[(r0 + k) * LD + r0 + lane] = xk;
#pragma unroll
    for (int i = 1; i <= W; ++i) y[i - 1] = fmaf(-lk[i], xk, y[i]);
    y[W] = 0.f;
  }
}

// X[r0.., r0..] = inverse of the lower-triangular tile L = S[r0.., r0..].  One warp.
__device__ __forceinline__ void inv32(const float* S, float* X, const float* rdiag, int r0,
                                      int lane) {
  float y[HT];
#pragma unroll
  for (int i = 0; i < HT; ++i) y[i] = (i == lane) ? 1.f : 0.f;
  inv32_phase<31>(S, X, rdiag, y, r0, 0, lane);
  inv32_phase<23>(S, X, rdiag, y, r0, 8, lane);
  inv32_phase<15>(S, X, rdiag, y, r0, 16, lane);
  inv32_phase<7>(S, X, rdiag, y, r0, 24, lane);
}

// C(E x E) = A * B on tiles in shared memory, E = 32 or 64; element accessors are passed as
// lambdas so that transposes and offsets cost nothing.  All 256 threads.
template <int E, typename FA, typename FB, typename FC>
__device__ __forceinline__ void mm_tile(int tid, FA a_at, FB b_at, FC store) {
  constexpr int RM = (E == 64) ? 4 : 1, RN = 4;          // outputs per thread
  const int i0 = (tid / (E / RN)) * RM, j0 = (tid % (E / RN)) * RN;
  float acc[RM][RN];
#pragma unroll
  for (int a = 0; a < RM; ++a)
#pragma unroll
    for (int b = 0; b < RN; ++b) acc[a][b] = 0.f;
#pragma unroll 4
  for (int k = 0; k < E; ++k) {
    float av[RM], bv[RN];
#pragma unroll
    for (int a = 0; a < RM; ++a) av[a] = a_at(i0 + a, k);
#pragma unroll
    for (int b = 0; b < RN; ++b) bv[b] = b_at(k, j0 + b);
#pragma unroll
    for (int a = 0; a < RM; ++a)
#pragma unroll
      for (int b = 0; b < RN; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
  }
#pragma unroll
  for (int a = 0; a < RM; ++a)
#pragma unroll
    for (int b = 0; b < RN; ++b) store(i0 + a, j0 + b, acc[a][b]);
}

// inv(chol()) of the 64 x 64 block at S[o.., o..] into X[o.., o..].  Whole CTA; T32a/T32b are
// two 32 x 33 scratch tiles.
__device__ __forceinline__ void leaf64(float* S, float* X, float* rdiag, float* T32a, float* T32b,
                                       int o, int tid, int32_t* info, int pivot_base) {
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int TL = HT + 1;
  if (warp == 0) {
    chol32(S, rdiag, o, lane, info, pivot_base);
    __syncwarp();
    inv32(S, X, rdiag, o, lane);
  }
  __syncthreads();
  // L21 = A21 * X11^T
  mm_tile<HT>(tid, [&](int i, int k) { return S[(o + HT + i) * LD + o + k]; },
              [&](int k, int j) { return X[(o + j) * LD + o + k]; },
              [&](int i, int j, float v) { T32a[i * TL + j] = v; });
  __syncthreads();
  // A22 -= L21 * L21^T
  mm_tile<HT>(tid, [&](int i, int k) { return T32a[i * TL + k]; },
              [&](int k, int j) { return T32a[j * TL + k]; },
              [&](int i, int j, float v) { S[(o + HT + i) * LD + o + HT + j] -= v; });
  __syncthreads();
  if (warp == 0) {
    chol32(S, rdiag, o + HT, lane, info, pivot_base - HT);
    __syncwarp();
    inv32(S, X, rdiag, o + HT, lane);
  }
  __syncthreads();
  // T = L21 * X11 ;  X21 = -X22 * T
  mm_tile<HT>(tid, [&](int i, int k) { return T32a[i * TL + k]; },
              [&](int k, int j) { return X[(o + k) * LD + o + j]; },
              [&](int i, int j, float v) { T32b[i * TL + j] = v; });
  __syncthreads();
  mm_tile<HT>(tid, [&](int i, int k) { return X[(o + HT + i) * LD + o + HT + k]; },
              [&](int k, int j) { return T32b[k * TL + j]; },
              [&](int i, int j, float v) { X[(o + HT + i) * LD + o + j] = -v; });
  __syncthreads();
}

constexpr size_t LEAF_SMEM_FLOATS = 2 * (size_t)LEAF * LD + 2 * 64 * LD64 + 2 * HT * (HT + 1) + LEAF;

__global__ void __launch_bounds__(LEAF_THREADS)
leaf_inv_chol_kernel(float* __restrict__ D, int64_t ldd, int nb, int32_t* info, int pivot_base) {
  extern __shared__ float leaf_smem[];
  float* S = leaf_smem;                      // [LEAF][LD]   the block, then its Cholesky factor
  float* X = S + LEAF * LD;                  // [LEAF][LD]   the inverse factor
  float* T1 = X + LEAF * LD;                 // [64][LD64]   L21 of the 128-level
  float* T2 = T1 + 64 * LD64;                // [64][LD64]
  float* T32a = T2 + 64 * LD64;              // [32][33]
  float* T32b = T32a + HT * (HT + 1);
  float* rdiag = T32b + HT * (HT + 1);       // [LEAF]
  const int tid = threadIdx.x;
  const int span = nb <= 64 ? 64 : LEAF;     // a block of at most 64 skips the 128-level
  for (int idx0 = tid; idx0 < span * span; idx0 += LEAF_THREADS * 8) {
    // a batch of global loads is issued before the first store to shared memory
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int idx = idx0 + e * LEAF_THREADS, i = idx / span, j = idx % span;
      v[e] = (idx < span * span && i < nb && j < nb) ? (j <= i ? D[(int64_t)i * ldd + j] : 0.f)
                                                      : (i == j ? 1.f : 0.f);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int idx = idx0 + e * LEAF_THREADS, i = idx / span, j = idx % span;
      if (idx < span * span) { S[i * LD + j] = v[e]; X[i * LD + j] = 0.f; }
    }
  }
  __syncthreads();
  leaf64(S, X, rdiag, T32a, T32b, 0, tid, info, pivot_base);
  if (span == LEAF) {
    // L21 = A21 * X11^T
    mm_tile<64>(tid, [&](int i, int k) { return S[(64 + i) * LD + k]; },
                [&](int k, int j) { return X[j * LD + k]; },
                [&](int i, int j, float v) { T1[i * LD64 + j] = v; });
    __syncthreads();
    // A22 -= L21 * L21^T
    mm_tile<64>(tid, [&](int i, int k) { return T1[i * LD64 + k]; },
                [&](int k, int j) { return T1[j * LD64 + k]; },
                [&](int i, int j, float v) { S[(64 + i) * LD + 64 + j] -= v; });
    __syncthreads();
    leaf64(S, X, rdiag, T32a, T32b, 64, tid, info, pivot_base - 64);
    // T2 = L21 * X11 ;  X21 = -X22 * T2
    mm_tile<64>(tid, [&](int i, int k) { return T1[i * LD64 + k]; },
                [&](int k, int j) { return X[k * LD + j]; },
                [&](int i, int j, float v) { T2[i * LD64 + j] = v; });
    __syncthreads();
    mm_tile<64>(tid, [&](int i, int k) { return X[(64 + i) * LD + 64 + k]; },
                [&](int k, int j) { return T2[k * LD64 + j]; },
                [&](int i, int j, float v) { X[(64 + i) * LD + j] = -v; });
    __syncthreads();
  }
  for (int idx = tid; idx < nb * nb; idx += LEAF_THREADS) {
    const int i = idx / nb, j = idx % nb;
    D[(int64_t)i * ldd + j] = X[i * LD + j];
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
    leaf_inv_chol_kernel<<<1, LEAF_THREADS, LEAF_SMEM_FLOATS * sizeof(float), p.st>>>(
        V + (int64_t)o * ld + o, ld, n, p.info, p.K - 1 - o);
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
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(leaf_inv_chol_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(LEAF_SMEM_FLOATS * sizeof(float))) != cudaSuccess)
      return DGQ_ERR_LAUNCH;
    attr_set = true;
  }
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
