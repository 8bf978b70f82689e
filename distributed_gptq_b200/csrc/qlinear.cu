// y = x * dequant(qweight)^T + bias for small batches (the operator behind
// torch.ops.gptq.linear).  Bound by the HBM traffic of the packed weights: every
// weight byte is read exactly once, activations are staged in shared memory per
// 512-column slice and shared by all warps of the CTA.
//
// qlinear_kernel (K a multiple of 8) is the main kernel; qlinear_generic_kernel covers
// ragged K.  Both accumulate up to 16 batch rows in fp32 and dequantize with the column's
// group scale/zero (through g_idx when given).
#include "common.cuh"

namespace {

constexpr int SLICE = 512;          // input columns staged per step
constexpr int WARPS = 8;
constexpr int ROWS_PER_WARP = 4;
constexpr int ROWS_PER_CTA = WARPS * ROWS_PER_WARP;

struct LinArgs {
  const void* x; void* y;
  const uint8_t* qw; int64_t row_bytes;
  const __half* scales; const __half* zeros; const int32_t* g_idx;
  const void* bias; int bias_dtype;
  int M, N_out, K, n_groups, group_size, bits;
  int vec16;   // rows of qweight start on 16-byte boundaries
};

template <typename XT>
__device__ __forceinline__ float load_bias(const void* b, int dt, int n) {
  if (dt == DGQ_F32) return reinterpret_cast<const float*>(b)[n];
  if (dt == DGQ_F16) return __half2float(reinterpret_cast<const __half*>(b)[n]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[n]);
}

template <typename XT, int MC, bool FOURBIT>
__global__ void __launch_bounds__(WARPS * 32)
qlinear_generic_kernel(const LinArgs a, int m0) {
  __shared__ __align__(16) float xs[MC][SLICE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * ROWS_PER_CTA + warp * ROWS_PER_WARP;
  const XT* x = reinterpret_cast<const XT*>(a.x) + (int64_t)m0 * a.K;
  const int mrows = min(MC, a.M - m0);
  const bool fast = (a.K % 8 == 0);

  float acc[ROWS_PER_WARP][MC];
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
    for (int m = 0; m < MC; ++m) acc[r][m] = 0.f;

  for (int k0 = 0; k0 < a.K; k0 += SLICE) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < MC * SLICE; idx += blockDim.x) {
      int m = idx / SLICE, c = idx % SLICE;
      xs[m][c] = (m < mrows && k0 + c < a.K) ? dgq_to_float<XT>(x[(int64_t)m * a.K + k0 + c]) : 0.f;
    }
    __syncthreads();
    const int kend = min(SLICE, a.K - k0);
#pragma unroll
    for (int r = 0; r < ROWS_PER_WARP; ++r) {
      const int n = n0 + r;
      if (n >= a.N_out) break;
      const uint8_t* wrow = a.qw + (int64_t)n * a.row_bytes;
      const __half* srow = a.scales + (int64_t)n * a.n_groups;
      const __half* zrow = a.zeros + (int64_t)n * a.n_groups;
      for (int cl = lane * 8; cl < kend; cl += 256) {
        const int c = k0 + cl;
        uint32_t cd[8];
        if (FOURBIT) {
          uint32_t wv = 0;
          if (fast) {
            wv = __ldg(reinterpret_cast<const uint32_t*>(wrow + (c >> 1)));
          } else {
            for (int b = 0; b < 4; ++b)
              if ((c >> 1) + b < a.row_bytes) wv |= (uint32_t)wrow[(c >> 1) + b] << (8 * b);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) cd[j] = (wv >> (4 * j)) & 0xF;  // low nibble = even column
        } else {
          if (fast) {
            uint2 wv = __ldg(reinterpret_cast<const uint2*>(wrow + c));
#pragma unroll
            for (int j = 0; j < 4; ++j) { cd[j] = (wv.x >> (8 * j)) & 0xFF; cd[4 + j] = (wv.y >> (8 * j)) & 0xFF; }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) cd[j] = (c + j < a.K) ? wrow[c + j] : 0;
          }
        }
        float wf[8];
        if (a.g_idx == nullptr && (a.n_groups == 1 || a.group_size % 8 == 0)) {
          const int g = a.n_groups == 1 ? 0 : c / a.group_size;
          const float s = __half2float(srow[g]), z = __half2float(zrow[g]);
#pragma unroll
          for (int j = 0; j < 8; ++j) wf[j] = dgq_dequant_level((float)cd[j], s, z);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int cc = min(c + j, a.K - 1);
            const int g = a.g_idx ? a.g_idx[cc] : (a.n_groups == 1 ? 0 : cc / a.group_size);
            wf[j] = dgq_dequant_level((float)cd[j], __half2float(srow[g]), __half2float(zrow[g]));
          }
        }
#pragma unroll
        for (int m = 0; m < MC; ++m) {
          const float4 x0 = *reinterpret_cast<const float4*>(&xs[m][cl]);
          const float4 x1 = *reinterpret_cast<const float4*>(&xs[m][cl + 4]);
          float s = acc[r][m];
          s = fmaf(wf[0], x0.x, s); s = fmaf(wf[1], x0.y, s);
          s = fmaf(wf[2], x0.z, s); s = fmaf(wf[3], x0.w, s);
          s = fmaf(wf[4], x1.x, s); s = fmaf(wf[5], x1.y, s);
          s = fmaf(wf[6], x1.z, s); s = fmaf(wf[7], x1.w, s);
          acc[r][m] = s;
        }
      }
    }
  }
  XT* y = reinterpret_cast<XT*>(a.y);
#pragma unroll
  for (int r = 0; r < ROWS_PER_WARP; ++r) {
    const int n = n0 + r;
#pragma unroll
    for (int m = 0; m < MC; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && n < a.N_out && m < mrows) {
        if (a.bias) v += load_bias<XT>(a.bias, a.bias_dtype, n);
        y[(int64_t)(m0 + m) * a.N_out + n] = dgq_from_float<XT>(v);
      }
    }
  }
}

// ---- main kernel: K a multiple of 8 -----------------------------------------------------------
// A CTA owns 8 warps x R consecutive output features and walks K in slices.  Per slice the
// activations are staged in shared memory as fp32, split per 8-column chunk into a low and
// a high float4, stored so that lane l reading 32-column quad (32 i + l) touches consecutive
// 16-byte words (no bank conflicts).  A lane takes the quads l, l+32, ... of R rows at once:
// one 16-byte load of nibble pairs per row (all R in flight together), the integer -> float
// conversion by the 2^23 trick, one fused multiply-add per code for (code - zero) * scale,
// and M multiply-adds per code against the staged activations, which are read once per
// quad for all R rows.
template <int MC>
struct FastCfg {
  static constexpr int R = (MC >= 8) ? 4 : 8;                       // rows per warp
  static constexpr int SLICE = (MC >= 16) ? 768 : (MC >= 8 ? 1536 : (MC >= 4 ? 3072 : 4096));
};

__device__ __forceinline__ float nibble_to_float(uint32_t w, int j) {
  return __uint_as_float(0x4B000000u | ((w >> (4 * j)) & 0xFu)) - 8388608.f;
}
__device__ __forceinline__ float byte_to_float(uint32_t w, int j) {
  return __uint_as_float(0x4B000000u | ((w >> (8 * j)) & 0xFFu)) - 8388608.f;
}

template <typename XT, int MC, bool FOURBIT>
__global__ void __launch_bounds__(WARPS * 32)
qlinear_kernel(const LinArgs a, int m0) {
  constexpr int R = FastCfg<MC>::R;
  constexpr int SLICE = FastCfg<MC>::SLICE;
  constexpr int SCH = SLICE / 8;                       // 8-column chunks per slice
  constexpr int SQ = SCH / 4;                          // 32-column quads per slice
  extern __shared__ float4 xs4[];                      // [MC][2 halves][4 sub-chunks][SQ]
  float* xs = reinterpret_cast<float*>(xs4);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = (blockIdx.x * WARPS + warp) * R;
  const XT* x = reinterpret_cast<const XT*>(a.x) + (int64_t)m0 * a.K;
  const int mrows = min(MC, a.M - m0);
  const bool grouped_fast = (a.g_idx == nullptr) && (a.n_groups == 1 || a.group_size % 8 == 0);

  float acc[R][MC];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < MC; ++m) acc[r][m] = 0.f;

  for (int k0 = 0; k0 < a.K; k0 += SLICE) {
    const int kcols = min(SLICE, a.K - k0);
    __syncthreads();
    // column c of the slice = quad (c >> 5), sub-chunk ((c >> 3) & 3), half ((c >> 2) & 1),
    // element (c & 3); quads are the fastest index so that lane l reading quad (32 i + l)
    // touches consecutive 16-byte words
    for (int idx = threadIdx.x; idx < MC * SLICE; idx += blockDim.x) {
      const int m = idx / SLICE, c = idx - m * SLICE;
      const float v = (m < mrows && c < kcols) ? dgq_to_float<XT>(x[(int64_t)m * a.K + k0 + c]) : 0.f;
      xs[((((m * 2 + ((c >> 2) & 1)) * 4 + ((c >> 3) & 3)) * SQ) + (c >> 5)) * 4 + (c & 3)] = v;
    }
    __syncthreads();
    const int nquads = (kcols + 31) >> 5;   // a ragged last quad reads zero-padded activations
    for (int qd = lane; qd < nquads; qd += 32) {
      // the R rows' loads of this quad are independent and in flight together:
      // 16 bytes of nibble pairs (32 codes) or 2 x 16 bytes of code bytes per row
      uint32_t w[R][FOURBIT ? 4 : 8];
      const bool whole = a.vec16 && (qd * 32 + 32 <= kcols);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int n = min(n0 + r, a.N_out - 1);   // rows past the end shadow the last row
        const uint8_t* wrow = a.qw + (int64_t)n * a.row_bytes + (FOURBIT ? (k0 >> 1) : k0);
        if (FOURBIT) {
          if (whole) {
            const uint4 t = __ldg(reinterpret_cast<const uint4*>(wrow) + qd);
            w[r][0] = t.x; w[r][1] = t.y; w[r][2] = t.z; w[r][3] = t.w;
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              w[r][q] = (qd * 32 + q * 8 < kcols)
                            ? __ldg(reinterpret_cast<const uint32_t*>(wrow) + qd * 4 + q) : 0u;
          }
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint2 t = make_uint2(0u, 0u);
            if (qd * 32 + q * 8 < kcols) t = __ldg(reinterpret_cast<const uint2*>(wrow) + qd * 4 + q);
            w[r][2 * q] = t.x; w[r][2 * q + 1] = t.y;
          }
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int c = k0 + qd * 32 + q * 8;
        if (c >= a.K) break;
        float wf[R][8];
        if (grouped_fast) {
          const int g = a.n_groups == 1 ? 0 : c / a.group_size;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const int n = min(n0 + r, a.N_out - 1);
            const float s = __half2float(a.scales[(int64_t)n * a.n_groups + g]);
            const float nzs = -__half2float(a.zeros[(int64_t)n * a.n_groups + g]) * s;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float cq = FOURBIT ? nibble_to_float(w[r][q], j)
                                       : byte_to_float(w[r][(FOURBIT ? 0 : 2 * q) + (j >> 2)], j & 3);
              wf[r][j] = fmaf(cq, s, nzs);
            }
          }
        } else {
          int gj[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) gj[j] = a.g_idx ? a.g_idx[c + j] : (c + j) / a.group_size;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const int n = min(n0 + r, a.N_out - 1);
            const __half* srow = a.scales + (int64_t)n * a.n_groups;
            const __half* zrow = a.zeros + (int64_t)n * a.n_groups;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float s = __half2float(srow[gj[j]]);
              const float cq = FOURBIT ? nibble_to_float(w[r][q], j)
                                       : byte_to_float(w[r][(FOURBIT ? 0 : 2 * q) + (j >> 2)], j & 3);
              wf[r][j] = fmaf(cq, s, -__half2float(zrow[gj[j]]) * s);
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MC; ++m) {
          const float4 lo = xs4[((m * 2 + 0) * 4 + q) * SQ + qd];
          const float4 hi = xs4[((m * 2 + 1) * 4 + q) * SQ + qd];
#pragma unroll
          for (int r = 0; r < R; ++r) {
            float t = acc[r][m];
            t = fmaf(wf[r][0], lo.x, t); t = fmaf(wf[r][1], lo.y, t);
            t = fmaf(wf[r][2], lo.z, t); t = fmaf(wf[r][3], lo.w, t);
            t = fmaf(wf[r][4], hi.x, t); t = fmaf(wf[r][5], hi.y, t);
            t = fmaf(wf[r][6], hi.z, t); t = fmaf(wf[r][7], hi.w, t);
            acc[r][m] = t;
          }
        }
      }
    }
  }
  XT* y = reinterpret_cast<XT*>(a.y);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int n = n0 + r;
#pragma unroll
    for (int m = 0; m < MC; ++m) {
      float v = acc[r][m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && n < a.N_out && m < mrows) {
        if (a.bias) v += load_bias<XT>(a.bias, a.bias_dtype, n);
        y[(int64_t)(m0 + m) * a.N_out + n] = dgq_from_float<XT>(v);
      }
    }
  }
}

template <typename XT, int MC>
void launch_fast(const LinArgs& a, int m0, cudaStream_t st) {
  constexpr int R = FastCfg<MC>::R;
  const unsigned grid = (unsigned)dgq_cdiv(a.N_out, WARPS * R);
  const size_t smem = (size_t)MC * FastCfg<MC>::SLICE * sizeof(float);
  if (a.bits == 4)
    qlinear_kernel<XT, MC, true><<<grid, WARPS * 32, smem, st>>>(a, m0);
  else
    qlinear_kernel<XT, MC, false><<<grid, WARPS * 32, smem, st>>>(a, m0);
}

template <typename XT, int MC>
void launch_mc(const LinArgs& a, int m0, cudaStream_t st) {
  if (a.K % 8 == 0) {
    launch_fast<XT, MC>(a, m0, st);
    return;
  }
  unsigned grid = (unsigned)dgq_cdiv(a.N_out, ROWS_PER_CTA);
  if (a.bits == 4)
    qlinear_generic_kernel<XT, MC, true><<<grid, WARPS * 32, 0, st>>>(a, m0);
  else
    qlinear_generic_kernel<XT, MC, false><<<grid, WARPS * 32, 0, st>>>(a, m0);
}

template <typename XT>
void launch_all(const LinArgs& a, cudaStream_t st) {
  for (int m0 = 0; m0 < a.M; m0 += 16) {
    int rem = a.M - m0;
    if (rem >= 9) launch_mc<XT, 16>(a, m0, st);
    else if (rem >= 5) launch_mc<XT, 8>(a, m0, st);
    else if (rem >= 3) launch_mc<XT, 4>(a, m0, st);
    else if (rem == 2) launch_mc<XT, 2>(a, m0, st);
    else launch_mc<XT, 1>(a, m0, st);
  }
}

}  // namespace

DGQ_EXPORT int32_t dgq_qlinear_forward(const void* x, int32_t x_dtype, int32_t M,
                                       const uint8_t* qweight, const void* scales_f16,
                                       const void* zeros_f16, const int32_t* g_idx,
                                       const void* bias, int32_t bias_dtype, int32_t N_out,
                                       int32_t K, int32_t n_groups, int32_t bits,
                                       int32_t group_size, void* y, void* stream) {
  DGQ_REQUIRE(x && qweight && scales_f16 && zeros_f16 && y, DGQ_ERR_ARG);
  DGQ_REQUIRE(M > 0 && N_out > 0 && K > 0 && n_groups > 0, DGQ_ERR_ARG);
  DGQ_REQUIRE(bits == 2 || bits == 3 || bits == 4 || bits == 8, DGQ_ERR_ARG);
  DGQ_REQUIRE(x_dtype >= DGQ_F32 && x_dtype <= DGQ_BF16, DGQ_ERR_ARG);
  DGQ_REQUIRE(!bias || (bias_dtype >= DGQ_F32 && bias_dtype <= DGQ_BF16), DGQ_ERR_ARG);
  if (g_idx == nullptr && n_groups > 1)
    DGQ_REQUIRE(group_size > 0 && dgq_cdiv(K, group_size) <= n_groups, DGQ_ERR_ARG);
  LinArgs a;
  a.x = x; a.y = y; a.qw = qweight;
  a.row_bytes = bits == 4 ? (K + 1) / 2 : K;
  a.scales = reinterpret_cast<const __half*>(scales_f16);
  a.zeros = reinterpret_cast<const __half*>(zeros_f16);
  a.g_idx = g_idx; a.bias = bias; a.bias_dtype = bias_dtype;
  a.M = M; a.N_out = N_out; a.K = K; a.n_groups = n_groups; a.group_size = group_size; a.bits = bits;
  a.vec16 = (a.row_bytes % 16 == 0 && dgq_aligned(qweight, 16)) ? 1 : 0;
  DGQ_REQUIRE(K % 8 != 0 || dgq_aligned(qweight, 8), DGQ_ERR_ALIGN);
  cudaStream_t st = dgq_stream(stream);
  if (x_dtype == DGQ_F32) launch_all<float>(a, st);
  else if (x_dtype == DGQ_F16) launch_all<__half>(a, st);
  else launch_all<__nv_bfloat16>(a, st);
  return dgq_launch_status(dgq_cdiv(M, 16));
}
