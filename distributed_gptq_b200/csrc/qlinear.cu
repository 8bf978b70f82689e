// y = x * dequant(qweight)^T + bias for small batches (the operator behind
// torch.ops.gptq.linear).  Bound by the HBM traffic of the packed weights: every
// weight byte is read exactly once, activations are staged in shared memory per
// 512-column slice and shared by all warps of the CTA.
//
// qlinear_mma_kernel is the main kernel (4-bit codes, 16-bit activations, K and the group
// size multiples of 128); qlinear_kernel (K a multiple of 8) covers fp32 activations, byte
// codes, small groups and g_idx on the CUDA cores; qlinear_generic_kernel covers ragged K.
// All accumulate up to 16 batch rows in fp32 and dequantize with the column's group
// scale/zero (through g_idx when given).
#include "common.cuh"
#include "qlinear_tc.cuh"

namespace {

constexpr int TC_MIN_ROWS = 33;     // fewer rows of activations: the kernels below, 16 rows a launch
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

// ---- tensor-core kernel -------------------------------------------------------------------------
// 4-bit codes, fp16 or bf16 activations, K a multiple of 128, groups that are whole multiples
// of 128 columns (or one group per row), no g_idx.  The kernel stays bound by the HBM traffic
// of the packed weights for up to 16 batch rows because a code costs about one and a half
// instructions: warp-level m16n8k16 multiply-accumulates take the dequantized weights
// straight from registers (no staging in shared or tensor memory), 16 output features by
// 8 batch rows at a time.
//
// A CTA owns 16 output features; its 8 warps take the 128-column steps of K round robin and
// are summed through shared memory at the end.  In a step, lane (g, t) loads 16 bytes = 32
// codes of feature rows g and g+8 (columns 32 t .. 32 t + 31 of the step) and the matching
// 64 bytes of activation row g (and g+8 for more than 8 batch rows).  A byte holds two
// adjacent columns; one byte permute (of the word and of the word shifted by 4) and one logic
// operation turn it into a pair of 16-bit floats (magic + low nibble, magic + high nibble),
// one packed addition per pair gives (code - zero), exactly when the zero point is an
// integer (a second subtraction is used when it is not).  Adjacent-column pairs are exactly the fragment layout of the
// multiply-accumulate, for the weights and for row-major activations alike.  The products
// accumulate in fp32 per step; the group's scale is applied to the step's sums.
template <typename T> struct MmaTraits;
template <> struct MmaTraits<__half> {
  static constexpr uint32_t MAGIC = 0x64006400u;   // (1024, 1024)
  static constexpr float BASE = 1024.f;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
    const __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <> struct MmaTraits<__nv_bfloat16> {
  static constexpr uint32_t MAGIC = 0x43004300u;   // (128, 128)
  static constexpr float BASE = 128.f;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                     *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  static __device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                     *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  static __device__ __forceinline__ void mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

// streamed once: do not keep the packed weights in L1, which holds the activations
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// eight 4-bit codes of one 32-bit word -> four pairs (code - zero) of adjacent columns
template <typename TR, bool TWO_STEP>
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t add2, uint32_t z2, uint32_t (&p)[4]) {
  const uint32_t w4 = w >> 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // byte i of w (low nibble = even column) and of w >> 4 (low nibble = odd column)
    const uint32_t b = __byte_perm(w, w4, ((4 + i) << 8) | i);
    p[i] = TR::add2((b & 0x000F000Fu) | TR::MAGIC, add2);
    if (TWO_STEP) p[i] = TR::sub2(p[i], z2);
  }
}

constexpr int MMA_WARPS = 8;
constexpr int MMA_STAGES = 4;   // 128-column steps of packed weights in flight per warp

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
               :: "r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

__device__ __forceinline__ void cp_async16_s(uint32_t smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t smem_src) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_src));
  return v;
}

template <typename T, int MT>
__global__ void __launch_bounds__(MMA_WARPS * 32, MT == 1 ? 4 : 2)
qlinear_mma_kernel(const LinArgs a, int m0, int n_tiles) {
  using TR = MmaTraits<T>;
  // per warp: a ring of steps of packed weights, filled by asynchronous copies that bypass the
  // registers and L1; every lane reads back exactly the 2 x 16 bytes it asked for
  __shared__ __align__(16) uint4 ring[MMA_WARPS][MMA_STAGES][2][32];
  __shared__ float red[MMA_WARPS][16][8 * MT + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int mrows = min(8 * MT, a.M - m0);
  const T* xbase = reinterpret_cast<const T*>(a.x) + (int64_t)m0 * a.K;
  const T* xrow[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) xrow[mt] = xbase + (int64_t)min(g + 8 * mt, mrows - 1) * a.K + t * 32;
  const int steps = a.K >> 7;
  const int steps_per_group = a.n_groups == 1 ? steps : (a.group_size >> 7);
  // The CTA walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ..; within a tile this warp takes
  // the contiguous steps s0 .. s0 + spw - 1.  The weight prefetch runs ahead across tiles.  The
  // per-step bookkeeping is kept to a few additions: this kernel is bound by instruction issue.
  const int spw = steps / MMA_WARPS + (warp < steps % MMA_WARPS ? 1 : 0);
  const int s0 = warp * (steps / MMA_WARPS) + min(warp, steps % MMA_WARPS);
  const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const uint32_t ring_lane = (uint32_t)__cvta_generic_to_shared(&ring[warp][0][0][lane]);
  constexpr uint32_t SLOT_BYTES = 2 * 32 * 16, HI_BYTES = 32 * 16;

  // byte offsets (below 2^32, checked by the host) of this lane's 16 bytes in rows g and g+8
  uint32_t pf_lo = 0, pf_hi = 0;
  int pf_tile = 0, pf_left = spw, pf_slot = 0;
  auto pf_enter_tile = [&]() {
    const int n_base = (blockIdx.x + pf_tile * gridDim.x) * 16;
    const uint32_t col = (uint32_t)(s0 * 64 + t * 16);
    pf_lo = (uint32_t)min(n_base + g, a.N_out - 1) * (uint32_t)a.row_bytes + col;
    pf_hi = (uint32_t)min(n_base + g + 8, a.N_out - 1) * (uint32_t)a.row_bytes + col;
  };
  const int pf_tiles = spw > 0 ? my_tiles : 0;
  if (pf_tiles > 0) pf_enter_tile();
  auto prefetch = [&]() {
    if (pf_tile < pf_tiles) {
      cp_async16_s(ring_lane + pf_slot * SLOT_BYTES, a.qw + pf_lo);
      cp_async16_s(ring_lane + pf_slot * SLOT_BYTES + HI_BYTES, a.qw + pf_hi);
      pf_lo += 64; pf_hi += 64;
      if (--pf_left == 0) {
        pf_left = spw;
        if (++pf_tile < pf_tiles) pf_enter_tile();
      }
    }
    pf_slot = (pf_slot + 1) & (MMA_STAGES - 1);
    cp_async_commit();          // committed even when empty: the group count stays uniform
  };
#pragma unroll
  for (int i = 0; i < MMA_STAGES - 1; ++i) prefetch();

  const __half2 k1024 = __float2half2_rn(1024.f), k64 = __float2half2_rn(64.f);
  int slot = 0;
  for (int ti = 0; ti < my_tiles; ++ti) {
    const int n_base = (blockIdx.x + ti * gridDim.x) * 16;
    // element offsets of the rows' group parameters, and the group of the first step
    const int so_lo = min(n_base + g, a.N_out - 1) * a.n_groups;
    const int so_hi = min(n_base + g + 8, a.N_out - 1) * a.n_groups;
    float yacc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) yacc[mt][e] = 0.f;

    for (int si = 0; si < spw; ++si) {
      const int step = s0 + si;
      prefetch();
      // activations and group parameters of this step (L1/L2 hits) are requested before the wait
      uint4 xv[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          xv[mt][j] = __ldg(reinterpret_cast<const uint4*>(xrow[mt] + step * 128) + j);
      const int grp = a.n_groups == 1 ? 0 : (steps_per_group == 1 ? step : step / steps_per_group);
      const __half hs_lo = a.scales[so_lo + grp], hs_hi = a.scales[so_hi + grp];
      const __half hz_lo = a.zeros[so_lo + grp], hz_hi = a.zeros[so_hi + grp];
      cp_async_wait<MMA_STAGES - 1>();
      const uint4 cl = lds16(ring_lane + slot * SLOT_BYTES);
      const uint4 ch = lds16(ring_lane + slot * SLOT_BYTES + HI_BYTES);
      slot = (slot + 1) & (MMA_STAGES - 1);
      float c[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) c[mt][e] = 0.f;
      // Integer zero points (every GPTQ zero is one) fold into the conversion's constant.  The
      // test runs on both rows at once in fp16: adding and removing 1024 leaves an integer alone.
      const __half2 zz = __halves2half2(hz_lo, hz_hi);
      const bool folded = __hbeq2(__hsub2(__hadd2(zz, k1024), k1024), zz) && __hble2(__habs2(zz), k64);
      const float cz_lo = __half2float(hz_lo), cz_hi = __half2float(hz_hi);
      const uint32_t wl4[4] = {cl.x, cl.y, cl.z, cl.w}, wh4[4] = {ch.x, ch.y, ch.z, ch.w};
      if (__all_sync(0xffffffffu, folded)) {
        const uint32_t add_lo = TR::pack(-(TR::BASE + cz_lo), -(TR::BASE + cz_lo));
        const uint32_t add_hi = TR::pack(-(TR::BASE + cz_hi), -(TR::BASE + cz_hi));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t pl[4], ph[4];
          dequant_word<TR, false>(wl4[j], add_lo, 0u, pl);
          dequant_word<TR, false>(wh4[j], add_hi, 0u, ph);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            TR::mma(c[mt], pl[0], ph[0], pl[1], ph[1], xv[mt][j].x, xv[mt][j].y);
            TR::mma(c[mt], pl[2], ph[2], pl[3], ph[3], xv[mt][j].z, xv[mt][j].w);
          }
        }
      } else {
        const uint32_t add = TR::pack(-TR::BASE, -TR::BASE);
        const uint32_t z2_lo = TR::pack(cz_lo, cz_lo), z2_hi = TR::pack(cz_hi, cz_hi);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t pl[4], ph[4];
          dequant_word<TR, true>(wl4[j], add, z2_lo, pl);
          dequant_word<TR, true>(wh4[j], add, z2_hi, ph);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            TR::mma(c[mt], pl[0], ph[0], pl[1], ph[1], xv[mt][j].x, xv[mt][j].y);
            TR::mma(c[mt], pl[2], ph[2], pl[3], ph[3], xv[mt][j].z, xv[mt][j].w);
          }
        }
      }
      const float cs_lo = __half2float(hs_lo), cs_hi = __half2float(hs_hi);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        yacc[mt][0] = fmaf(cs_lo, c[mt][0], yacc[mt][0]);
        yacc[mt][1] = fmaf(cs_lo, c[mt][1], yacc[mt][1]);
        yacc[mt][2] = fmaf(cs_hi, c[mt][2], yacc[mt][2]);
        yacc[mt][3] = fmaf(cs_hi, c[mt][3], yacc[mt][3]);
      }
    }
    // accumulator layout: [0], [1] = feature row g, batch rows 2t, 2t+1; [2], [3] = feature row g+8
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      red[warp][g][mt * 8 + 2 * t] = yacc[mt][0];
      red[warp][g][mt * 8 + 2 * t + 1] = yacc[mt][1];
      red[warp][g + 8][mt * 8 + 2 * t] = yacc[mt][2];
      red[warp][g + 8][mt * 8 + 2 * t + 1] = yacc[mt][3];
    }
    __syncthreads();
    T* y = reinterpret_cast<T*>(a.y);
    for (int idx = threadIdx.x; idx < 16 * 8 * MT; idx += MMA_WARPS * 32) {
      const int row = idx & 15, m = idx >> 4, n = n_base + row;
      if (n < a.N_out && m < mrows) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < MMA_WARPS; ++w) v += red[w][row][m];
        if (a.bias) v += load_bias<T>(a.bias, a.bias_dtype, n);
        y[(int64_t)(m0 + m) * a.N_out + n] = dgq_from_float<T>(v);
      }
    }
    __syncthreads();   // red is rewritten by the next tile
  }
  cp_async_wait<0>();
}

template <typename XT>
bool launch_mma(const LinArgs& a, int m0, cudaStream_t st) { return false; }

template <typename T>
bool launch_mma_typed(const LinArgs& a, int m0, cudaStream_t st) {
  const bool ok = a.bits == 4 && a.g_idx == nullptr && a.K % 128 == 0 && a.vec16 &&
                  dgq_aligned(a.x, 16) && (int64_t)a.N_out * a.row_bytes < ((int64_t)1 << 32) &&
                  (int64_t)a.N_out * a.n_groups < ((int64_t)1 << 31) &&
                  (a.n_groups == 1 || (a.group_size > 0 && a.group_size % 128 == 0));
  if (!ok) return false;
  // persistent CTAs: as many as fit on the device at once, every one with the same number of
  // 16-feature tiles (to within one)
  const int n_tiles = (int)dgq_cdiv(a.N_out, 16);
  const bool two = a.M - m0 > 8;
  static std::mutex mu;
  static int resident_of[DGQ_MAX_DEVICES][2] = {};   // per device: occupancy differs with the part
  const int dev = dgq_current_device();
  if (dev < 0) return false;
  int resident;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (resident_of[dev][two] == 0) {
      int per_sm = 0;
      const cudaError_t e = two
          ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qlinear_mma_kernel<T, 2>, MMA_WARPS * 32, 0)
          : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qlinear_mma_kernel<T, 1>, MMA_WARPS * 32, 0);
      if (e != cudaSuccess || per_sm <= 0) return false;
      resident_of[dev][two] = per_sm * dgq_sm_count();
    }
    resident = resident_of[dev][two];
  }
  const int rounds = (int)dgq_cdiv(n_tiles, resident);
  const unsigned grid = (unsigned)dgq_cdiv(n_tiles, rounds);
  if (two) qlinear_mma_kernel<T, 2><<<grid, MMA_WARPS * 32, 0, st>>>(a, m0, n_tiles);
  else qlinear_mma_kernel<T, 1><<<grid, MMA_WARPS * 32, 0, st>>>(a, m0, n_tiles);
  return true;
}
template <>
bool launch_mma<__half>(const LinArgs& a, int m0, cudaStream_t st) { return launch_mma_typed<__half>(a, m0, st); }
template <>
bool launch_mma<__nv_bfloat16>(const LinArgs& a, int m0, cudaStream_t st) {
  return launch_mma_typed<__nv_bfloat16>(a, m0, st);
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
    if (launch_mma<XT>(a, m0, st)) continue;
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
  if (M >= TC_MIN_ROWS && bits == 4 && g_idx == nullptr && x_dtype != DGQ_F32) {
    dgq::QLinearTcArgs t;
    t.x = x; t.y = y; t.dtype = x_dtype; t.qw = qweight; t.row_bytes = a.row_bytes;
    t.scales = a.scales; t.zeros = a.zeros; t.n_groups = n_groups; t.group_size = group_size;
    t.bias = bias; t.bias_dtype = bias_dtype; t.M = M; t.N_out = N_out; t.K = K; t.info = nullptr;
    if (dgq::qlinear_tc_supported(t) && dgq_device_check() == DGQ_OK) {
      if (!dgq::qlinear_tc_launch(t, st)) return DGQ_ERR_LAUNCH;
      return DGQ_OK;
    }
  }
  if (x_dtype == DGQ_F32) launch_all<float>(a, st);
  else if (x_dtype == DGQ_F16) launch_all<__half>(a, st);
  else launch_all<__nv_bfloat16>(a, st);
  return dgq_launch_status(dgq_cdiv(M, 16));
}
