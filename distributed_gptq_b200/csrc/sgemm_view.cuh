// fp32 matrix product on the CUDA cores with every operand addressed through signed
// strides (so transposed, reversed and sub-matrix views need no copies), plus two
// triangular variants.  64 x 64 output tile per CTA, 4 x 4 outputs per thread.
#pragma once

#include "common.cuh"

namespace {

// C(m x n) = alpha * A(m x k) * B(k x n) + beta * C, every operand addressed through
// signed strides.  TRI selects a triangular variant:
//   0 plain
//   1 C is symmetric-lower: tiles strictly above the diagonal are skipped and
//     entries with j > i are not written (SYRK when B = A^T)
//   2 A is lower triangular (m == k): entries with k > i read as zero and the
//     reduction stops at the tile's last row (triangular matrix product)
struct GemmArgs {
  const float* a; int64_t ars, acs;
  const float* b; int64_t brs, bcs;
  float* c; int64_t crs, ccs;
  int m, n, k;
  float alpha, beta;
};

constexpr int TM = 64, TN = 64, TK = 16;

template <int TRI>
__global__ void __launch_bounds__(256)
sgemm_view_kernel(const GemmArgs g) {
  const int i0 = blockIdx.y * TM, j0 = blockIdx.x * TN;
  if (TRI == 1 && j0 > i0 + TM - 1) return;
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;

  const int kmax = (TRI == 2) ? min(g.k, i0 + TM) : g.k;
  // loader mapping: the fast thread index follows whichever stride is +-1
  const bool a_kfast = (g.acs == 1 || g.acs == -1);
  const bool b_nfast = (g.bcs == 1 || g.bcs == -1);
  for (int k0 = 0; k0 < kmax; k0 += TK) {
    // A tile: TM x TK = 1024 elements, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + e * 256;
      int ii, kk;
      if (a_kfast) { ii = idx / TK; kk = idx % TK; } else { kk = idx / TM; ii = idx % TM; }
      int gi = i0 + ii, gk = k0 + kk;
      float v = 0.f;
      if (gi < g.m && gk < g.k && !(TRI == 2 && gk > gi)) v = g.a[gi * g.ars + gk * g.acs];
      As[kk][ii] = v;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int idx = tid + e * 256;
      int jj, kk;
      if (b_nfast) { kk = idx / TN; jj = idx % TN; } else { jj = idx / TK; kk = idx % TK; }
      int gj = j0 + jj, gk = k0 + kk;
      float v = 0.f;
      if (gj < g.n && gk < g.k) v = g.b[gk * g.brs + gj * g.bcs];
      Bs[kk][jj] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a4[4] = {av.x, av.y, av.z, av.w};
      const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(a4[a], b4[b], acc[a][b]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    int gi = i0 + ty * 4 + a;
    if (gi >= g.m) continue;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      int gj = j0 + tx * 4 + b;
      if (gj >= g.n) continue;
      if (TRI == 1 && gj > gi) continue;
      float* cp = g.c + gi * g.crs + gj * g.ccs;
      float v = g.alpha * acc[a][b];
      if (g.beta != 0.f) v += g.beta * *cp;
      *cp = v;
    }
  }
}

template <int TRI>
void launch_gemm(const GemmArgs& g, cudaStream_t st) {
  if (g.m <= 0 || g.n <= 0) return;
  dim3 grid((unsigned)dgq_cdiv(g.n, TN), (unsigned)dgq_cdiv(g.m, TM));
  sgemm_view_kernel<TRI><<<grid, 256, 0, st>>>(g);
  dgq_note_launches(1);
}

}  // namespace
