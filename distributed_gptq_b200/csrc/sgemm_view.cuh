// fp32 matrix product on the CUDA cores with every operand addressed through signed
// strides (so transposed, reversed and sub-matrix views need no copies).
//
//   C(m x n) = alpha * A(m x k) * B(k x n) + beta * C
//
// Triangular structure is expressed as limits on the reduction range of an output
// tile (the skipped parts of the operands must read as zero where a tile straddles
// the boundary, which holds for matrices whose other triangle is stored as zeros)
// and as a write mask for symmetric-lower results.  Two tile shapes: 128 x 128 with
// 8 x 8 outputs per thread for large products, 64 x 64 with 4 x 4 for small ones.
#pragma once

#include "common.cuh"

namespace {

struct GemmArgs {
  const float* a; int64_t ars, acs;
  const float* b; int64_t brs, bcs;
  float* c; int64_t crs, ccs;
  int m, n, k;
  float alpha, beta;
  // reduction limits of the tile at rows [i0, i0+TM), columns [j0, j0+TN):
  //   k_lo = lo_from_j ? j0 : 0
  //   k_hi = min(k, hi_from_j ? j0 + TN : (hi_from_i ? i0 + TM : k))
  int lo_from_j, hi_from_j, hi_from_i;
  // lower_only: tiles strictly above the diagonal are skipped, entries with j > i not written
  int lower_only;
};

inline GemmArgs gemm_args(const float* a, int64_t ars, int64_t acs, const float* b, int64_t brs,
                          int64_t bcs, float* c, int64_t crs, int64_t ccs, int m, int n, int k,
                          float alpha, float beta) {
  GemmArgs g;
  g.a = a; g.ars = ars; g.acs = acs; g.b = b; g.brs = brs; g.bcs = bcs;
  g.c = c; g.crs = crs; g.ccs = ccs; g.m = m; g.n = n; g.k = k; g.alpha = alpha; g.beta = beta;
  g.lo_from_j = g.hi_from_j = g.hi_from_i = g.lower_only = 0;
  return g;
}

template <int TM, int TN, int RM, int RN>
__global__ void __launch_bounds__(256)
sgemm_view_kernel(const GemmArgs g) {
  constexpr int TK = 16;
  static_assert((TM / RM) * (TN / RN) == 256, "256 threads per tile");
  dgq_chain_release();
  dgq_chain_wait();
  const int i0 = blockIdx.y * TM, j0 = blockIdx.x * TN;
  if (g.lower_only && j0 > i0 + TM - 1) return;
  __shared__ __align__(16) float As[2][TK][TM + 4];
  __shared__ __align__(16) float Bs[2][TK][TN + 4];
  const int tid = threadIdx.x;
  const int ty = tid / (TN / RN), tx = tid % (TN / RN);
  float acc[RM][RN];
#pragma unroll
  for (int a = 0; a < RM; ++a)
#pragma unroll
    for (int b = 0; b < RN; ++b) acc[a][b] = 0.f;

  const int k_lo = g.lo_from_j ? (j0 / TK) * TK : 0;
  const int k_hi = min(g.k, g.hi_from_j ? j0 + TN : (g.hi_from_i ? i0 + TM : g.k));
  const bool a_kfast = (g.acs == 1 || g.acs == -1);
  const bool b_nfast = (g.bcs == 1 || g.bcs == -1);
  constexpr int A_PER = TM * TK / 256, B_PER = TN * TK / 256;
  float ra[A_PER], rb[B_PER];

  auto fetch = [&](int k0) {
#pragma unroll
    for (int e = 0; e < A_PER; ++e) {
      const int idx = tid + e * 256;
      int ii, kk;
      if (a_kfast) { ii = idx / TK; kk = idx % TK; } else { kk = idx / TM; ii = idx % TM; }
      const int gi = i0 + ii, gk = k0 + kk;
      ra[e] = (gi < g.m && gk < k_hi) ? g.a[gi * g.ars + gk * g.acs] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < B_PER; ++e) {
      const int idx = tid + e * 256;
      int jj, kk;
      if (b_nfast) { kk = idx / TN; jj = idx % TN; } else { jj = idx / TK; kk = idx % TK; }
      const int gj = j0 + jj, gk = k0 + kk;
      rb[e] = (gj < g.n && gk < k_hi) ? g.b[gk * g.brs + gj * g.bcs] : 0.f;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int e = 0; e < A_PER; ++e) {
      const int idx = tid + e * 256;
      int ii, kk;
      if (a_kfast) { ii = idx / TK; kk = idx % TK; } else { kk = idx / TM; ii = idx % TM; }
      As[buf][kk][ii] = ra[e];
    }
#pragma unroll
    for (int e = 0; e < B_PER; ++e) {
      const int idx = tid + e * 256;
      int jj, kk;
      if (b_nfast) { kk = idx / TN; jj = idx % TN; } else { jj = idx / TK; kk = idx % TK; }
      Bs[buf][kk][jj] = rb[e];
    }
  };

  if (k_lo < k_hi) {
    fetch(k_lo);
    stash(0);
  }
  __syncthreads();
  int buf = 0;
  for (int k0 = k_lo; k0 < k_hi; k0 += TK) {
    const bool more = k0 + TK < k_hi;
    if (more) fetch(k0 + TK);  // global loads of the next slice overlap this slice's math
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a4[RM], b4[RN];
#pragma unroll
      for (int v = 0; v < RM / 4; ++v) {
        // rows ty*4 + v*(TM/ (RM/4)) ... : interleave 4-wide groups to keep loads conflict free
        const float4 t = *reinterpret_cast<const float4*>(&As[buf][kk][v * (TM / (RM / 4)) + ty * 4]);
        a4[v * 4 + 0] = t.x; a4[v * 4 + 1] = t.y; a4[v * 4 + 2] = t.z; a4[v * 4 + 3] = t.w;
      }
#pragma unroll
      for (int v = 0; v < RN / 4; ++v) {
        const float4 t = *reinterpret_cast<const float4*>(&Bs[buf][kk][v * (TN / (RN / 4)) + tx * 4]);
        b4[v * 4 + 0] = t.x; b4[v * 4 + 1] = t.y; b4[v * 4 + 2] = t.z; b4[v * 4 + 3] = t.w;
      }
#pragma unroll
      for (int a = 0; a < RM; ++a)
#pragma unroll
        for (int b = 0; b < RN; ++b) acc[a][b] = fmaf(a4[a], b4[b], acc[a][b]);
    }
    if (more) stash(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
#pragma unroll
  for (int a = 0; a < RM; ++a) {
    const int gi = i0 + (a / 4) * (TM / (RM / 4)) + ty * 4 + (a % 4);
    if (gi >= g.m) continue;
#pragma unroll
    for (int b = 0; b < RN; ++b) {
      const int gj = j0 + (b / 4) * (TN / (RN / 4)) + tx * 4 + (b % 4);
      if (gj >= g.n) continue;
      if (g.lower_only && gj > gi) continue;
      float* cp = g.c + gi * g.crs + gj * g.ccs;
      float v = g.alpha * acc[a][b];
      if (g.beta != 0.f) v += g.beta * *cp;
      *cp = v;
    }
  }
}

inline void launch_gemm(const GemmArgs& g, cudaStream_t st) {
  if (g.m <= 0 || g.n <= 0) return;
  if (g.m > 64 && g.n > 64) {
    dim3 grid((unsigned)dgq_cdiv(g.n, 128), (unsigned)dgq_cdiv(g.m, 128));
    dgq_launch_chained(sgemm_view_kernel<128, 128, 8, 8>, grid, dim3(256), 0, st, g);
  } else {
    dim3 grid((unsigned)dgq_cdiv(g.n, 64), (unsigned)dgq_cdiv(g.m, 64));
    dgq_launch_chained(sgemm_view_kernel<64, 64, 4, 4>, grid, dim3(256), 0, st, g);
  }
  dgq_note_launches(1);
}

}  // namespace
