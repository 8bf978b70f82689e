// HBM-bound helpers around the GPTQ core: dtype casts, the scale/zero and
// quantize formulas on their own, flat round-to-nearest, act-order permutation
// and Hessian preparation (scale, dead columns, damping).
#include "common.cuh"

namespace {

// ---- casts -------------------------------------------------------------------
template <typename ST>
__global__ void __launch_bounds__(256)
cast_to_bf16_kernel(const ST* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  // 8 elements per thread: 16-byte stores; the tail is handled element-wise
  const int64_t n8 = n / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
       i += (int64_t)gridDim.x * blockDim.x) {
    alignas(16) __nv_bfloat16 t[8];
    if (sizeof(ST) == 4) {
      float4 a = __ldg(reinterpret_cast<const float4*>(src) + 2 * i);
      float4 b = __ldg(reinterpret_cast<const float4*>(src) + 2 * i + 1);
      t[0] = __float2bfloat16_rn(a.x); t[1] = __float2bfloat16_rn(a.y);
      t[2] = __float2bfloat16_rn(a.z); t[3] = __float2bfloat16_rn(a.w);
      t[4] = __float2bfloat16_rn(b.x); t[5] = __float2bfloat16_rn(b.y);
      t[6] = __float2bfloat16_rn(b.z); t[7] = __float2bfloat16_rn(b.w);
    } else {
      alignas(16) ST s[8];
      *reinterpret_cast<uint4*>(s) = __ldg(reinterpret_cast<const uint4*>(src) + i);
#pragma unroll
      for (int j = 0; j < 8; ++j) t[j] = __float2bfloat16_rn(dgq_to_float<ST>(s[j]));
    }
    reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(t);
  }
  for (int64_t i = n8 * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(dgq_to_float<ST>(src[i]));
}

// ---- per-row scale/zero --------------------------------------------------------
// One warp per row: coalesced reads, shuffle reduction of min and max.
__global__ void __launch_bounds__(256)
find_params_kernel(const float* __restrict__ x, int64_t ldx, int rows, int cols, float maxq,
                   float* __restrict__ scale, float* __restrict__ zero) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < rows;
       r += gridDim.x * warps_per_cta) {
    const float* row = x + (int64_t)r * ldx;
    float mn = INFINITY, mx = -INFINITY;
    for (int c = lane; c < cols; c += 32) {
      float v = row[c];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) {
      float s, z;
      dgq_scale_zero(mn, mx, maxq, s, z);
      scale[r] = s;
      zero[r] = z;
    }
  }
}

__global__ void __launch_bounds__(256)
quantize_rows_kernel(const float* __restrict__ x, int64_t ldx, int rows, int cols, float maxq,
                     const float* __restrict__ scale, const float* __restrict__ zero,
                     uint8_t* __restrict__ q, int64_t ldq, float* __restrict__ xh, int64_t ldh) {
  const int64_t total = (int64_t)rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / cols;
    int64_t c = i - r * cols;
    float s = scale[r], z = zero[r];
    float lv = dgq_quant_level(x[r * ldx + c], s, z, maxq);
    if (q) q[r * ldq + c] = (uint8_t)lv;
    if (xh) xh[r * ldh + c] = dgq_dequant_level(lv, s, z);
  }
}

// ---- flat round-to-nearest -------------------------------------------------------
// One warp per group of group_size consecutive elements.
__global__ void __launch_bounds__(256)
rtn_find_params_kernel(const float* __restrict__ x, int64_t n, int group_size, float maxq,
                       float* __restrict__ scales, float* __restrict__ zeros, int64_t n_groups) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  for (int64_t g = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); g < n_groups;
       g += (int64_t)gridDim.x * warps_per_cta) {
    int64_t lo = g * group_size;
    int64_t hi = min(lo + group_size, n);
    float mn = INFINITY, mx = -INFINITY;
    for (int64_t i = lo + lane; i < hi; i += 32) {
      float v = x[i];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) {
      float s = __fdiv_rn(__fsub_rn(mx, mn), maxq);
      if (s == 0.f) s = 1.f;
      scales[g] = s;
      zeros[g] = __fdiv_rn(-mn, s);  // the flat helper keeps the zero point unrounded
    }
  }
}

__global__ void __launch_bounds__(256)
rtn_quantize_kernel(const float* __restrict__ x, int64_t n, int group_size, float maxq,
                    const float* __restrict__ scales, const float* __restrict__ zeros,
                    uint8_t* __restrict__ q) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t g = i / group_size;
    q[i] = (uint8_t)dgq_quant_level(x[i], scales[g], zeros[g], maxq);
  }
}

__global__ void __launch_bounds__(256)
rtn_dequantize_kernel(const uint8_t* __restrict__ q, int64_t n, int group_size,
                      const float* __restrict__ scales, const float* __restrict__ zeros,
                      float* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    int64_t g = i / group_size;
    out[i] = dgq_dequant_level((float)q[i], scales[g], zeros[g]);
  }
}

// perm[i], or i itself when there is no permutation or the entry is not a valid index (a
// caller's array that is not a permutation must not turn into an out-of-bounds access).
__device__ __forceinline__ int checked_index(const int32_t* __restrict__ perm, int i, int n) {
  if (!perm) return i;
  const int p = perm[i];
  return ((unsigned)p < (unsigned)n) ? p : i;
}

// ---- act-order ---------------------------------------------------------------------
// rank(i) = #{ j : d[j] > d[i]  or  (d[j] == d[i] and j < i) } is the position of i in
// a stable descending sort.  The key is the prepared diagonal: d = scale*H_ii, with a
// zero entry (dead column) replaced by 1, exactly what the damping step will see.
// A NaN entry (calibration activations that went non-finite) compares false with everything
// and would leave ranks unassigned, so the key maps NaN to +inf: with ties broken by index
// the ranks are a permutation for every input.  (The inverse factor then reports such a
// matrix as not positive definite.)
// K <= ~16K, so the K^2 comparisons are spread over the grid with the diagonal staged
// through shared memory.
__device__ __forceinline__ float actorder_key(float d) {
  if (d != d) return INFINITY;
  return d == 0.f ? 1.f : d;
}

__global__ void __launch_bounds__(256)
actorder_rank_kernel(const float* __restrict__ H, int64_t ldh, int K, float scale,
                     int32_t* __restrict__ perm, int32_t* __restrict__ invperm) {
  __shared__ float tile[256];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const float di = actorder_key((i < K) ? __fmul_rn(scale, H[(int64_t)i * ldh + i]) : 0.f);
  int rank = 0;
  for (int j0 = 0; j0 < K; j0 += 256) {
    int j = j0 + threadIdx.x;
    tile[threadIdx.x] = (j < K) ? actorder_key(__fmul_rn(scale, H[(int64_t)j * ldh + j])) : -INFINITY;
    __syncthreads();
    int lim = min(256, K - j0);
    for (int t = 0; t < lim; ++t) {
      float dj = tile[t];
      rank += (dj > di) || (dj == di && (j0 + t) < i);
    }
    __syncthreads();
  }
  if (i < K) {
    perm[rank] = i;
    invperm[i] = rank;
  }
}

// ---- Hessian preparation ---------------------------------------------------------------
// Pass 1: diag' = scale*diag (1 where zero) gathered through perm, dead mask, and
// sum(diag') accumulated into ws[0] (which the host zeroes beforehand).
__global__ void __launch_bounds__(256)
prepare_diag_kernel(const float* __restrict__ H, int64_t ldh, int K, float scale,
                    const int32_t* __restrict__ perm, uint8_t* __restrict__ dead,
                    float* __restrict__ diag_sum) {
  float local = 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < K; i += gridDim.x * blockDim.x) {
    const int p = checked_index(perm, i, K);
    float d = __fmul_rn(scale, H[(int64_t)p * ldh + p]);
    bool is_dead = (d == 0.f);
    if (is_dead) d = 1.f;
    if (dead) dead[i] = is_dead ? 1 : 0;
    local += d;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0 && local != 0.f) atomicAdd(diag_sum, local);
}

// Pass 2: Hout[i][j] = scale*H[p(i)][p(j)]; diagonal: (0 -> 1) + percdamp*mean(diag').
__global__ void __launch_bounds__(256)
prepare_gather_kernel(const float* __restrict__ H, int64_t ldh, float* __restrict__ Hout,
                      int64_t ldo, int K, float scale, float percdamp,
                      const int32_t* __restrict__ perm, const float* __restrict__ diag_sum) {
  const float damp = percdamp * (diag_sum[0] / (float)K);
  const int64_t total = (int64_t)K * K;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int i = (int)(idx / K);
    int j = (int)(idx - (int64_t)i * K);
    const int pi = checked_index(perm, i, K);
    const int pj = checked_index(perm, j, K);
    float v = __fmul_rn(scale, H[(int64_t)pi * ldh + pj]);
    if (i == j) {
      if (v == 0.f) v = 1.f;
      v += damp;
    }
    Hout[(int64_t)i * ldo + j] = v;
  }
}

__global__ void __launch_bounds__(256)
permute_cols_f32_kernel(const float* __restrict__ src, int64_t lds, float* __restrict__ dst,
                        int64_t ldd, int rows, int cols, const int32_t* __restrict__ perm,
                        const uint8_t* __restrict__ dead) {
  const int64_t total = (int64_t)rows * cols;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = idx / cols;
    int c = (int)(idx - r * cols);
    const int p = checked_index(perm, c, cols);
    float v = src[r * lds + p];
    if (dead && dead[c]) v = 0.f;
    dst[r * ldd + c] = v;
  }
}

__global__ void __launch_bounds__(256)
permute_cols_u8_kernel(const uint8_t* __restrict__ src, int64_t lds, uint8_t* __restrict__ dst,
                       int64_t ldd, int rows, int cols, const int32_t* __restrict__ perm) {
  const int64_t total = (int64_t)rows * cols;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = idx / cols;
    int c = (int)(idx - r * cols);
    dst[r * ldd + c] = src[r * lds + checked_index(perm, c, cols)];
  }
}

__global__ void __launch_bounds__(256)
permute_cols_u16_kernel(const uint16_t* __restrict__ src, int64_t lds, uint16_t* __restrict__ dst,
                        int64_t ldd, int rows, int cols, const int32_t* __restrict__ perm) {
  const int64_t total = (int64_t)rows * cols;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = idx / cols;
    int c = (int)(idx - r * cols);
    dst[r * ldd + c] = src[r * lds + checked_index(perm, c, cols)];
  }
}

bool valid_bits(int b) { return b == 2 || b == 3 || b == 4 || b == 8; }

}  // namespace

DGQ_EXPORT int32_t dgq_cast_f32_to_bf16(const float* src, void* dst, int64_t n, void* stream) {
  DGQ_REQUIRE(src && dst && n > 0, DGQ_ERR_ARG);
  DGQ_REQUIRE(dgq_aligned(src, 16) && dgq_aligned(dst, 16), DGQ_ERR_ALIGN);
  cast_to_bf16_kernel<float><<<dgq_grid(dgq_cdiv(n, 8), 256), 256, 0, dgq_stream(stream)>>>(
      src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_cast_f16_to_bf16(const void* src, void* dst, int64_t n, void* stream) {
  DGQ_REQUIRE(src && dst && n > 0, DGQ_ERR_ARG);
  DGQ_REQUIRE(dgq_aligned(src, 16) && dgq_aligned(dst, 16), DGQ_ERR_ALIGN);
  cast_to_bf16_kernel<__half><<<dgq_grid(dgq_cdiv(n, 8), 256), 256, 0, dgq_stream(stream)>>>(
      reinterpret_cast<const __half*>(src), reinterpret_cast<__nv_bfloat16*>(dst), n);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_find_params(const float* x, int64_t ldx, int32_t rows, int32_t cols,
                                   int32_t bits, float* scale, float* zero, void* stream) {
  DGQ_REQUIRE(x && scale && zero && rows > 0 && cols > 0 && ldx >= cols && valid_bits(bits),
              DGQ_ERR_ARG);
  unsigned grid = dgq_grid((int64_t)rows * 32, 256);
  find_params_kernel<<<grid, 256, 0, dgq_stream(stream)>>>(x, ldx, rows, cols,
                                                           (float)((1 << bits) - 1), scale, zero);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_quantize_rows(const float* x, int64_t ldx, int32_t rows, int32_t cols,
                                     int32_t bits, const float* scale, const float* zero,
                                     uint8_t* q, int64_t ldq, float* x_hat, int64_t ldh,
                                     void* stream) {
  DGQ_REQUIRE(x && scale && zero && (q || x_hat) && rows > 0 && cols > 0 && ldx >= cols &&
                  valid_bits(bits),
              DGQ_ERR_ARG);
  DGQ_REQUIRE((!q || ldq >= cols) && (!x_hat || ldh >= cols), DGQ_ERR_ARG);
  quantize_rows_kernel<<<dgq_grid((int64_t)rows * cols, 256), 256, 0, dgq_stream(stream)>>>(
      x, ldx, rows, cols, (float)((1 << bits) - 1), scale, zero, q, ldq, x_hat, ldh);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_rtn_find_params(const float* x, int64_t n, int32_t bits, int32_t group_size,
                                       float* scales, float* zeros, void* stream) {
  DGQ_REQUIRE(x && scales && zeros && n > 0 && group_size > 0 && valid_bits(bits), DGQ_ERR_ARG);
  int64_t ng = dgq_cdiv(n, group_size);
  rtn_find_params_kernel<<<dgq_grid(ng * 32, 256), 256, 0, dgq_stream(stream)>>>(
      x, n, group_size, (float)((1 << bits) - 1), scales, zeros, ng);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_rtn_quantize(const float* x, int64_t n, int32_t bits, int32_t group_size,
                                    const float* scales, const float* zeros, uint8_t* q,
                                    void* stream) {
  DGQ_REQUIRE(x && scales && zeros && q && n > 0 && group_size > 0 && valid_bits(bits), DGQ_ERR_ARG);
  rtn_quantize_kernel<<<dgq_grid(n, 256), 256, 0, dgq_stream(stream)>>>(
      x, n, group_size, (float)((1 << bits) - 1), scales, zeros, q);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_rtn_dequantize(const uint8_t* q, int64_t n, int32_t group_size,
                                      const float* scales, const float* zeros, float* out,
                                      void* stream) {
  DGQ_REQUIRE(q && scales && zeros && out && n > 0 && group_size > 0, DGQ_ERR_ARG);
  rtn_dequantize_kernel<<<dgq_grid(n, 256), 256, 0, dgq_stream(stream)>>>(q, n, group_size, scales,
                                                                         zeros, out);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_actorder_perm(const float* H, int32_t K, int64_t ldh, float scale,
                                     int32_t* perm, int32_t* invperm, void* stream) {
  DGQ_REQUIRE(H && perm && invperm && K > 0 && ldh >= K, DGQ_ERR_ARG);
  actorder_rank_kernel<<<(unsigned)dgq_cdiv(K, 256), 256, 0, dgq_stream(stream)>>>(H, ldh, K, scale,
                                                                                   perm, invperm);
  return dgq_launch_status();
}

DGQ_EXPORT int64_t dgq_hessian_prepare_workspace_bytes(int32_t K) {
  return K > 0 ? 256 : DGQ_ERR_ARG;
}

DGQ_EXPORT int32_t dgq_hessian_prepare(const float* H, int64_t ldh, float* Hout, int64_t ldo,
                                       int32_t K, float scale, float percdamp, const int32_t* perm,
                                       uint8_t* dead_out, void* ws, int64_t ws_bytes, void* stream) {
  DGQ_REQUIRE(H && Hout && ws && K > 0 && ldh >= K && ldo >= K, DGQ_ERR_ARG);
  DGQ_REQUIRE(ws_bytes >= dgq_hessian_prepare_workspace_bytes(K), DGQ_ERR_WORKSPACE);
  DGQ_REQUIRE(dgq_aligned(ws, 16), DGQ_ERR_ALIGN);
  cudaStream_t st = dgq_stream(stream);
  float* diag_sum = reinterpret_cast<float*>(ws);
  if (cudaMemsetAsync(diag_sum, 0, sizeof(float), st) != cudaSuccess) return DGQ_ERR_LAUNCH;
  // a single CTA keeps the diagonal sum's order of additions fixed
  prepare_diag_kernel<<<1, 256, 0, st>>>(H, ldh, K, scale, perm, dead_out, diag_sum);
  prepare_gather_kernel<<<dgq_grid((int64_t)K * K, 256), 256, 0, st>>>(H, ldh, Hout, ldo, K, scale,
                                                                      percdamp, perm, diag_sum);
  return dgq_launch_status(2);
}

DGQ_EXPORT int32_t dgq_permute_cols_f32(const float* src, int64_t lds, float* dst, int64_t ldd,
                                        int32_t rows, int32_t cols, const int32_t* perm,
                                        const uint8_t* dead, void* stream) {
  DGQ_REQUIRE(src && dst && rows > 0 && cols > 0 && lds >= cols && ldd >= cols, DGQ_ERR_ARG);
  permute_cols_f32_kernel<<<dgq_grid((int64_t)rows * cols, 256), 256, 0, dgq_stream(stream)>>>(
      src, lds, dst, ldd, rows, cols, perm, dead);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_permute_cols_u8(const uint8_t* src, int64_t lds, uint8_t* dst, int64_t ldd,
                                       int32_t rows, int32_t cols, const int32_t* perm,
                                       void* stream) {
  DGQ_REQUIRE(src && dst && perm && rows > 0 && cols > 0 && lds >= cols && ldd >= cols, DGQ_ERR_ARG);
  permute_cols_u8_kernel<<<dgq_grid((int64_t)rows * cols, 256), 256, 0, dgq_stream(stream)>>>(
      src, lds, dst, ldd, rows, cols, perm);
  return dgq_launch_status();
}

DGQ_EXPORT int32_t dgq_permute_cols_u16(const void* src, int64_t lds, void* dst, int64_t ldd,
                                        int32_t rows, int32_t cols, const int32_t* perm,
                                        void* stream) {
  DGQ_REQUIRE(src && dst && perm && rows > 0 && cols > 0 && lds >= cols && ldd >= cols, DGQ_ERR_ARG);
  permute_cols_u16_kernel<<<dgq_grid((int64_t)rows * cols, 256), 256, 0, dgq_stream(stream)>>>(
      reinterpret_cast<const uint16_t*>(src), lds, reinterpret_cast<uint16_t*>(dst), ldd, rows,
      cols, perm);
  return dgq_launch_status();
}
