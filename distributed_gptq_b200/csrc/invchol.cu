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
//     V21 = -X22 * (T * X11)                   (block of the inverse; T * X11 is formed on a
//                                               side stream beside the two steps before)
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
  dgq_chain_release();
  dgq_chain_wait();
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
  dgq_chain_release();
  dgq_chain_wait();
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
//                  one warp each (chol32, inv32 below).
constexpr int LEAF = 128;             // largest block the leaf kernel takes
constexpr int LEAF_THREADS = 256;
constexpr int HT = 32;                // tile edge
// Row strides (floats) of the shared-memory matrices: multiples of 4, so that rows start on
// 16-byte boundaries, and = 4 mod 32, so that 16-byte accesses to 8 consecutive rows at the
// same column fall into 8 different groups of 4 banks.
constexpr int LD = LEAF + 4;
constexpr int LD64 = 64 + 4;
constexpr int TL = HT + 4;

__device__ __forceinline__ float rsqrt_newton(float d) {
  float rs;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(rs) : "f"(d));
  return rs * fmaf(-0.5f * d * rs, rs, 1.5f);   // one Newton step: 1/sqrt(d) to ~1 ulp
}

// Cholesky factor of the 32 x 32 tile at S[r0.., r0..] (lower part read).  The factor is
// written transposed to LT (row k of LT = column k of L, contiguous, zeros in front of the
// diagonal), the reciprocals of its diagonal to rdiag; S is left as it was.  One warp; one
// copy of the code (not inlined) serves all four tiles of a 128-block.
//
// Lane i keeps row i of the tile in 32 registers.  Step k: every lane scales its entry of
// column k by 1/sqrt(pivot) and stores it to LT[k][lane]; all lanes then read the part of
// that row they need as 16-byte broadcast loads (at most 8 loads instead of 31 shuffles) and
// update their row.  The steps are fully unrolled, so that every register index is static
// and step k touches only the 31-k live columns.  The next pivot, A[k+1][k+1] - L[k+1][k]^2,
// needs nothing from other lanes: lane k+1 forms it as soon as it has its own entry of
// column k, and one shuffle hands it to the warp.  The chain from step to step is therefore
// multiply-add -> shuffle -> reciprocal square root -> multiply, and the round trip through
// shared memory is off it.
__device__ __noinline__ void chol32(const float* __restrict__ S, float* __restrict__ LT,
                                    float* __restrict__ rdiag, int r0, int lane, int32_t* info,
                                    int pivot_base) {
  float a[HT];
#pragma unroll
  for (int q = 0; q < HT / 4; ++q) {
    const float4 v = *reinterpret_cast<const float4*>(S + (r0 + lane) * LD + r0 + 4 * q);
    a[4 * q] = v.x; a[4 * q + 1] = v.y; a[4 * q + 2] = v.z; a[4 * q + 3] = v.w;
  }
  float d = __shfl_sync(0xffffffffu, a[0], 0);
  int first_bad = HT;   // first step whose pivot was not positive and finite
#pragma unroll
  for (int k = 0; k < HT; ++k) {
    // no branch inside the loop: the steps stay one basic block, so that the update of step k
    // is scheduled beside the reciprocal square root of step k+1
    const bool bad = !(d > 0.f) || !isfinite(d);
    first_bad = (bad && first_bad == HT) ? k : first_bad;
    d = bad ? 1.f : d;
    const float rs = rsqrt_newton(d);
    const float l = (lane == k) ? d * rs : (lane > k ? a[k] * rs : 0.f);
    LT[k * HT + lane] = l;
    if (lane == k) rdiag[r0 + k] = rs;   // 1 / L[k][k], reused by the inverse
    if (k + 1 < HT) {
      d = __shfl_sync(0xffffffffu, fmaf(-l, l, a[k + 1]), k + 1);
      __syncwarp();
      float lr[HT];
#pragma unroll
      for (int q = (k + 1) / 4; q < HT / 4; ++q) {
        const float4 v = *reinterpret_cast<const float4*>(LT + k * HT + 4 * q);
        lr[4 * q] = v.x; lr[4 * q + 1] = v.y; lr[4 * q + 2] = v.z; lr[4 * q + 3] = v.w;
      }
#pragma unroll
      for (int j = k + 1; j < HT; ++j) a[j] = fmaf(-l, lr[j], a[j]);
    }
  }
  if (first_bad < HT && lane == first_bad && info &&
      atomicCAS(info, DGQ_INFO_OK, DGQ_INFO_NOT_POSDEF) == DGQ_INFO_OK)
    info[1] = pivot_base - first_bad;
}

// X[r0.., r0..] = inverse of the lower-triangular tile whose transpose is in LT.  One warp:
// lane t keeps column t of the inverse in registers; the entries of L that step k needs are
// the same for all lanes and come from row k of LT as 16-byte broadcast loads, fetched one
// step ahead of their use.
__device__ __noinline__ void inv32(const float* __restrict__ LT, float* __restrict__ X,
                                   const float* __restrict__ rdiag, int r0, int lane) {
  float y[HT], rd[HT];
#pragma unroll
  for (int q = 0; q < HT / 4; ++q) {
    const float4 v = *reinterpret_cast<const float4*>(rdiag + r0 + 4 * q);
    rd[4 * q] = v.x; rd[4 * q + 1] = v.y; rd[4 * q + 2] = v.z; rd[4 * q + 3] = v.w;
  }
#pragma unroll
  for (int i = 0; i < HT; ++i) y[i] = (i == lane) ? 1.f : 0.f;
  float lr[HT], nx[HT];
#pragma unroll
  for (int q = 0; q < HT / 4; ++q) {
    const float4 v = *reinterpret_cast<const float4*>(LT + 4 * q);
    lr[4 * q] = v.x; lr[4 * q + 1] = v.y; lr[4 * q + 2] = v.z; lr[4 * q + 3] = v.w;
  }
#pragma unroll
  for (int k = 0; k < HT; ++k) {
    if (k + 2 < HT) {
#pragma unroll
      for (int q = (k + 2) / 4; q < HT / 4; ++q) {
        const float4 v = *reinterpret_cast<const float4*>(LT + (k + 1) * HT + 4 * q);
        nx[4 * q] = v.x; nx[4 * q + 1] = v.y; nx[4 * q + 2] = v.z; nx[4 * q + 3] = v.w;
      }
    }
    const float xk = y[k] * rd[k];                         // row k of X is final
    X[(r0 + k) * LD + r0 + lane] = xk;
#pragma unroll
    for (int i = k + 1; i < HT; ++i) y[i] = fmaf(-lr[i], xk, y[i]);
#pragma unroll
    for (int i = 0; i < HT; ++i) lr[i] = nx[i];
  }
}

// C (E x E) = A * B on tiles in shared memory, E = 32 or 64, all 256 threads.  A is given by
// rows (A[i * lda + k]); B by rows of its transpose when !B_KN (B[j * ldb + k]), or as it is
// when B_KN (B[k * ldb + j]).  Everything that is contiguous is read 16 bytes at a time: four
// reduction steps of A per load, and of B either four reduction steps of one column (!B_KN;
// the thread's columns are interleaved, g, g+E/4, .., so that the rows it reads with its
// neighbours fall into different banks) or one step of four adjacent columns (B_KN).
// All base addresses and strides must be multiples of 16 bytes.
template <int E, bool B_KN, typename FC>
__device__ __forceinline__ void mm_tile(int tid, const float* __restrict__ A, int lda,
                                        const float* __restrict__ B, int ldb, FC store) {
  constexpr int RM = (E == 64) ? 4 : 1, RN = 4;          // outputs per thread
  constexpr int G = E / RN;                              // column groups
  constexpr int RSTEP = LEAF_THREADS / G;                // distance between a thread's rows
  const int g = tid % G, r = tid / G;
  float acc[RM][RN];
#pragma unroll
  for (int a = 0; a < RM; ++a)
#pragma unroll
    for (int b = 0; b < RN; ++b) acc[a][b] = 0.f;
#pragma unroll 2
  for (int k = 0; k < E; k += 4) {
    float4 av[RM];
#pragma unroll
    for (int a = 0; a < RM; ++a)
      av[a] = *reinterpret_cast<const float4*>(A + (r + a * RSTEP) * lda + k);
    if (!B_KN) {
      float4 bv[RN];
#pragma unroll
      for (int b = 0; b < RN; ++b)
        bv[b] = *reinterpret_cast<const float4*>(B + (g + b * G) * ldb + k);
#pragma unroll
      for (int a = 0; a < RM; ++a)
#pragma unroll
        for (int b = 0; b < RN; ++b) {
          acc[a][b] = fmaf(av[a].x, bv[b].x, acc[a][b]);
          acc[a][b] = fmaf(av[a].y, bv[b].y, acc[a][b]);
          acc[a][b] = fmaf(av[a].z, bv[b].z, acc[a][b]);
          acc[a][b] = fmaf(av[a].w, bv[b].w, acc[a][b]);
        }
    } else {
      float4 bk[4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        bk[kk] = *reinterpret_cast<const float4*>(B + (k + kk) * ldb + 4 * g);
#pragma unroll
      for (int a = 0; a < RM; ++a) {
        const float ak[4] = {av[a].x, av[a].y, av[a].z, av[a].w};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          acc[a][0] = fmaf(ak[kk], bk[kk].x, acc[a][0]);
          acc[a][1] = fmaf(ak[kk], bk[kk].y, acc[a][1]);
          acc[a][2] = fmaf(ak[kk], bk[kk].z, acc[a][2]);
          acc[a][3] = fmaf(ak[kk], bk[kk].w, acc[a][3]);
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < RM; ++a)
#pragma unroll
    for (int b = 0; b < RN; ++b)
      store(r + a * RSTEP, B_KN ? 4 * g + b : g + b * G, acc[a][b]);
}

// inv(chol()) of the 64 x 64 block at S[o.., o..] into X[o.., o..].  Whole CTA; T32a/T32b are
// two 32 x TL scratch tiles, LT a 32 x 32 one.
__device__ __forceinline__ void leaf64(float* S, float* X, float* rdiag, float* T32a, float* T32b,
                                       float* LT, int o, int tid, int32_t* info, int pivot_base) {
  const int lane = tid & 31, warp = tid >> 5;
  float* S21 = S + (o + HT) * LD + o;
  float* S22 = S21 + HT;
  float* X11 = X + o * LD + o;
  float* X21 = X + (o + HT) * LD + o;
  float* X22 = X21 + HT;
  if (warp == 0) {
    chol32(S, LT, rdiag, o, lane, info, pivot_base);
    __syncwarp();
    inv32(LT, X, rdiag, o, lane);
  }
  __syncthreads();
  // L21 = A21 * X11^T
  mm_tile<HT, false>(tid, S21, LD, X11, LD, [&](int i, int j, float v) { T32a[i * TL + j] = v; });
  __syncthreads();
  // A22 -= L21 * L21^T
  mm_tile<HT, false>(tid, T32a, TL, T32a, TL, [&](int i, int j, float v) { S22[i * LD + j] -= v; });
  __syncthreads();
  if (warp == 0) {
    chol32(S, LT, rdiag, o + HT, lane, info, pivot_base - HT);
    __syncwarp();
    inv32(LT, X, rdiag, o + HT, lane);
  }
  __syncthreads();
  // T = L21 * X11 ;  X21 = -X22 * T
  mm_tile<HT, true>(tid, T32a, TL, X11, LD, [&](int i, int j, float v) { T32b[i * TL + j] = v; });
  __syncthreads();
  mm_tile<HT, true>(tid, X22, LD, T32b, TL, [&](int i, int j, float v) { X21[i * LD + j] = -v; });
  __syncthreads();
}

constexpr size_t LEAF_SMEM_FLOATS =
    2 * (size_t)LEAF * LD + 2 * 64 * LD64 + 2 * HT * TL + LEAF + HT * HT;

__global__ void __launch_bounds__(LEAF_THREADS)
leaf_inv_chol_kernel(float* __restrict__ D, int64_t ldd, int nb, int32_t* info, int pivot_base) {
  extern __shared__ __align__(16) float leaf_smem[];
  float* S = leaf_smem;                      // [LEAF][LD]   the block, updated as the levels proceed
  float* X = S + LEAF * LD;                  // [LEAF][LD]   the inverse factor
  float* T1 = X + LEAF * LD;                 // [64][LD64]   L21 of the 128-level
  float* T2 = T1 + 64 * LD64;                // [64][LD64]
  float* T32a = T2 + 64 * LD64;              // [32][TL]
  float* T32b = T32a + HT * TL;
  float* rdiag = T32b + HT * TL;             // [LEAF]
  float* LT = rdiag + LEAF;                  // [32][32]     transpose of the current 32 x 32 factor
  const int tid = threadIdx.x;
  dgq_chain_release();
  dgq_chain_wait();
  const int span = nb <= 64 ? 64 : LEAF;     // a block of at most 64 skips the 128-level
  const bool vec = nb == LEAF && (ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(D) & 15) == 0;
  if (vec) {
    // full block: every thread has all its sixteen 16-byte loads in flight at once
    constexpr int PER = LEAF * LEAF / 4 / LEAF_THREADS;
    float4 v[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = tid + e * LEAF_THREADS, i = idx / (LEAF / 4), c = (idx % (LEAF / 4)) * 4;
      v[e] = c <= i ? *reinterpret_cast<const float4*>(D + (int64_t)i * ldd + c)
                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = tid + e * LEAF_THREADS, i = idx / (LEAF / 4), c = (idx % (LEAF / 4)) * 4;
      float4 w = v[e];
      if (c + 1 > i) w.y = 0.f;
      if (c + 2 > i) w.z = 0.f;
      if (c + 3 > i) w.w = 0.f;
      *reinterpret_cast<float4*>(S + i * LD + c) = w;
      *reinterpret_cast<float4*>(X + i * LD + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  } else {
    for (int idx = tid; idx < span * span; idx += LEAF_THREADS) {
      const int i = idx / span, j = idx % span;
      S[i * LD + j] = (i < nb && j < nb) ? (j <= i ? D[(int64_t)i * ldd + j] : 0.f)
                                         : (i == j ? 1.f : 0.f);
      X[i * LD + j] = 0.f;
    }
  }
  __syncthreads();
  leaf64(S, X, rdiag, T32a, T32b, LT, 0, tid, info, pivot_base);
  if (span == LEAF) {
    float* S21 = S + 64 * LD;
    float* S22 = S21 + 64;
    float* X21 = X + 64 * LD;
    float* X22 = X21 + 64;
    // L21 = A21 * X11^T
    mm_tile<64, false>(tid, S21, LD, X, LD, [&](int i, int j, float v) { T1[i * LD64 + j] = v; });
    __syncthreads();
    // A22 -= L21 * L21^T
    mm_tile<64, false>(tid, T1, LD64, T1, LD64, [&](int i, int j, float v) { S22[i * LD + j] -= v; });
    __syncthreads();
    leaf64(S, X, rdiag, T32a, T32b, LT, 64, tid, info, pivot_base - 64);
    // T2 = L21 * X11 ;  X21 = -X22 * T2
    mm_tile<64, true>(tid, T1, LD64, X, LD, [&](int i, int j, float v) { T2[i * LD64 + j] = v; });
    __syncthreads();
    mm_tile<64, true>(tid, X22, LD, T2, LD64, [&](int i, int j, float v) { X21[i * LD + j] = -v; });
    __syncthreads();
  }
  if (vec) {
#pragma unroll 4
    for (int idx = tid; idx < LEAF * LEAF / 4; idx += LEAF_THREADS) {
      const int i = idx / (LEAF / 4), c = (idx % (LEAF / 4)) * 4;
      *reinterpret_cast<float4*>(D + (int64_t)i * ldd + c) =
          *reinterpret_cast<const float4*>(X + i * LD + c);
    }
  } else {
    for (int idx = tid; idx < nb * nb; idx += LEAF_THREADS) {
      const int i = idx / nb, j = idx % nb;
      D[(int64_t)i * ldd + j] = X[i * LD + j];
    }
  }
}

// ---- the recursion, unrolled on the host into a launch sequence --------------------------------
struct Plan {
  float* V; int64_t ldv; int K;
  float* T1[32];        // per recursion depth: the L21 block of the node being processed
  float* T2[32];        // per recursion depth: the product T1 * X11
  int32_t* info;
  cudaStream_t st;      // the caller's stream
  cudaStream_t* side;   // per depth: takes T2 = T1 * X11, which nothing needs before the node's
                        // last product
  cudaEvent_t* fork;    // per depth: T1 is ready (recorded on st)
  cudaEvent_t* join;    // per depth: T2 is ready (recorded on side)
  int64_t leaves;
  bool use_tensor;
};

// One side stream and one pair of events per recursion depth for every (device, caller
// stream) this host thread has used, created on first use and kept for the life of the
// thread: calls on different streams must not share a side stream, or they would wait for
// each other's products.  Depths do not share one either: the small product of a node deep
// in the second half of the recursion would queue behind its ancestor's large one, and the
// node's last product waits for it.  The table is small; when it is full an entry is taken
// over (see side_resources).
constexpr int SIDE_STREAMS = 10;
struct SideResources {
  int device = -1;
  cudaStream_t caller = nullptr;
  cudaStream_t stream[SIDE_STREAMS] = {};   // depth d uses stream[min(d, SIDE_STREAMS - 1)]
  cudaEvent_t fork[32] = {}, join[32] = {};
  bool ok = false;
};
// Creates the entry's streams and events on the current device (same priority as the
// caller's stream: the side products are on the chain's critical path).
bool side_create(SideResources* r, int dev, cudaStream_t caller) {
  int prio = 0;
  if (cudaStreamGetPriority(caller, &prio) != cudaSuccess) prio = 0;
  for (int d = 0; d < SIDE_STREAMS; ++d)
    if (cudaStreamCreateWithPriority(&r->stream[d], cudaStreamNonBlocking, prio) != cudaSuccess)
      return false;
  for (int d = 0; d < 32; ++d) {
    if (cudaEventCreateWithFlags(&r->fork[d], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&r->join[d], cudaEventDisableTiming) != cudaSuccess)
      return false;
  }
  r->device = dev;
  r->caller = caller;
  r->ok = true;
  return true;
}

// Releases an entry that belongs to another device (work already queued on its streams still
// completes: destroying a stream only releases it once it has drained).
void side_destroy(SideResources* r, int current_dev) {
  if (!r->ok) return;
  cudaSetDevice(r->device);
  for (int d = 0; d < SIDE_STREAMS; ++d) cudaStreamDestroy(r->stream[d]);
  for (int d = 0; d < 32; ++d) {
    cudaEventDestroy(r->fork[d]);
    cudaEventDestroy(r->join[d]);
  }
  cudaSetDevice(current_dev);
  (void)cudaGetLastError();
  *r = SideResources();
}

SideResources* side_resources(cudaStream_t caller) {
  constexpr int SLOTS = 32;
  thread_local SideResources table[SLOTS];
  thread_local int next_victim = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  for (int i = 0; i < SLOTS; ++i)
    if (table[i].ok && table[i].device == dev && table[i].caller == caller) return &table[i];
  for (int i = 0; i < SLOTS; ++i)
    if (!table[i].ok) return side_create(&table[i], dev, caller) ? &table[i] : nullptr;
  // The table is full: an entry is taken over.  One of the same device keeps its streams and
  // events (stream order keeps that correct, it only couples the two callers); one of another
  // device is released and made anew here.
  SideResources* r = &table[next_victim];
  next_victim = (next_victim + 1) % SLOTS;
  if (r->device == dev) {
    r->caller = caller;
    return r;
  }
  side_destroy(r, dev);
  return side_create(r, dev, caller) ? r : nullptr;
}

int split_point(int n) {
  const int blocks = (n + NB - 1) / NB;
  return (blocks / 2) * NB;  // first half gets floor(blocks/2) leaves (>= 1 when n > NB)
}

void rec_workspace(int n, int depth, std::vector<int64_t>& need) {
  if (n <= NB) return;
  const int h = split_point(n), m2 = n - h;
  if ((int)need.size() <= depth) need.resize(depth + 1, 0);
  need[depth] = std::max<int64_t>(need[depth], (int64_t)m2 * h);
  rec_workspace(h, depth + 1, need);
  rec_workspace(m2, depth + 1, need);
}

// One product of the recursion.  B is (n, k) row-major when !b_is_kn, (k, n) when b_is_kn.
void mm(Plan& p, cudaStream_t st, const float* a, int64_t lda, const float* b, int64_t ldb,
        bool b_is_kn, float* c, int64_t ldc, int m, int n, int k, float alpha, float beta,
        int lo_from_j, int hi_from_j, int hi_from_i, int lower_only) {
  if (p.use_tensor && m >= dgq::TGEMM_TILE && n >= dgq::TGEMM_TILE) {
    dgq::TGemmArgs t;
    t.a = a; t.lda = lda; t.b = b; t.ldb = ldb; t.c = c; t.ldc = ldc;
    t.m = m; t.n = n; t.k = k; t.alpha = alpha; t.beta = beta; t.b_is_kn = b_is_kn ? 1 : 0;
    t.lo_from_j = lo_from_j; t.hi_from_j = hi_from_j; t.hi_from_i = hi_from_i;
    t.lower_only = lower_only; t.info = p.info;
    if (dgq::tgemm_supported(t) && dgq::tgemm_launch(t, st)) return;
  }
  GemmArgs g = b_is_kn ? gemm_args(a, lda, 1, b, ldb, 1, c, ldc, 1, m, n, k, alpha, beta)
                       : gemm_args(a, lda, 1, b, 1, ldb, c, ldc, 1, m, n, k, alpha, beta);
  g.lo_from_j = lo_from_j; g.hi_from_j = hi_from_j; g.hi_from_i = hi_from_i;
  g.lower_only = lower_only;
  launch_gemm(g, st);
}

void rec(Plan& p, int o, int n, int depth) {
  float* V = p.V;
  const int64_t ld = p.ldv;
  if (n <= NB) {
    dgq_launch_chained(leaf_inv_chol_kernel, dim3(1), dim3(LEAF_THREADS),
                       LEAF_SMEM_FLOATS * sizeof(float), p.st, V + (int64_t)o * ld + o, ld, n,
                       p.info, p.K - 1 - o);
    ++p.leaves;
    return;
  }
  const int h = split_point(n), m2 = n - h;
  float* V11 = V + (int64_t)o * ld + o;
  float* V21 = V + (int64_t)(o + h) * ld + o;
  float* V22 = V + (int64_t)(o + h) * ld + (o + h);
  float* T1 = p.T1[depth];
  float* T2 = p.T2[depth];
  rec(p, o, h, depth + 1);
  // T1 = V21 * X11^T : X11[j][k] is non-zero for k <= j
  mm(p, p.st, V21, ld, V11, ld, false, T1, h, m2, h, h, 1.f, 0.f, 0, 1, 0, 0);
  // T2 = T1 * X11 (X11[k][j] is non-zero for k >= j) runs beside the Schur complement and
  // the whole second half of the recursion
  cudaStream_t side = p.side[std::min(depth, SIDE_STREAMS - 1)];
  cudaEventRecord(p.fork[depth], p.st);
  cudaStreamWaitEvent(side, p.fork[depth], 0);
  mm(p, side, T1, h, V11, ld, true, T2, h, m2, h, h, 1.f, 0.f, 1, 0, 0, 0);
  cudaEventRecord(p.join[depth], side);
  // V22 -= T1 * T1^T, lower part
  mm(p, p.st, T1, h, T1, h, false, V22, ld, m2, m2, h, -1.f, 1.f, 0, 0, 0, 1);
  rec(p, o + h, m2, depth + 1);
  // V21 = -X22 * T2 : X22[i][k] is non-zero for k <= i
  cudaStreamWaitEvent(p.st, p.join[depth], 0);
  mm(p, p.st, V22, ld, T2, h, true, V21, ld, m2, h, m2, -1.f, 0.f, 0, 0, 1, 0);
}

int64_t round4(int64_t x) { return (x + 3) / 4 * 4; }

}  // namespace

DGQ_EXPORT int64_t dgq_inv_chol_workspace_bytes(int32_t K) {
  if (K <= 0) return DGQ_ERR_ARG;
  std::vector<int64_t> need;
  rec_workspace(K, 0, need);
  int64_t floats = (int64_t)K * round4(K);
  for (int64_t v : need) floats += 2 * round4(v);
  return (floats + 4) * (int64_t)sizeof(float);
}

DGQ_EXPORT int32_t dgq_inv_chol_upper(float* A, int32_t K, int64_t lda, int32_t* info, void* ws,
                                      int64_t ws_bytes, void* stream) {
  DGQ_REQUIRE(A && ws && K > 0 && lda >= K, DGQ_ERR_ARG);
  DGQ_REQUIRE(ws_bytes >= dgq_inv_chol_workspace_bytes(K), DGQ_ERR_WORKSPACE);
  DGQ_REQUIRE(dgq_aligned(A, 16) && dgq_aligned(ws, 16), DGQ_ERR_ALIGN);
  static DgqDeviceOnce once;
  if (!once.run([] {
        return cudaFuncSetAttribute(leaf_inv_chol_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)(LEAF_SMEM_FLOATS * sizeof(float))) == cudaSuccess;
      }))
    return DGQ_ERR_LAUNCH;
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
  rec_workspace(K, 0, need);
  DGQ_REQUIRE(need.size() <= 32, DGQ_ERR_SIZE);
  for (size_t d = 0; d < need.size(); ++d) {
    p.T1[d] = w;
    w += round4(need[d]);
    p.T2[d] = w;
    w += round4(need[d]);
  }
  SideResources* side = side_resources(p.st);
  DGQ_REQUIRE(side != nullptr, DGQ_ERR_LAUNCH);
  p.side = side->stream;
  p.fork = side->fork;
  p.join = side->join;
  const unsigned grid = dgq_grid((int64_t)K * K, 256);
  dgq_launch_chained(reverse_in_kernel, dim3(grid), dim3(256), 0, p.st, A, lda, p.V, p.ldv, K);
  rec(p, 0, K, 0);
  dgq_launch_chained(reverse_out_kernel, dim3(grid), dim3(256), 0, p.st, p.V, p.ldv, A, lda, K);
  return dgq_launch_status(2 + p.leaves);  // matrix products are counted as they are launched
}
