// Blockwise GPTQ quantization of one weight matrix given the inverse-Hessian factor.
//
// For every block of `blocksize` (<= 128) columns:
//   1. gptq_block8_kernel - eight lanes per weight row, four rows per warp.  A lane
//      keeps 16 columns of the 128-column block in registers (four float4 chunks,
//      interleaved over the lanes so that shared-memory reads of the block of U are
//      conflict free).  Columns are visited in order: the
//      owning lane's value is broadcast inside its group of eight with a shuffle,
//      every lane of the group evaluates the quantize/dequantize formulas on it (so
//      the scaled error needs no second broadcast) and applies the error feedback
//      to the columns it holds.  Codes, dequantized values and the scaled errors
//      leave through 16-byte stores.  (gptq_block_kernel, one warp per row, is the
//      general variant for ragged blocks and groups narrower than 32 columns.)
//   2. trailing update - W[:, i2:] -= Err * U[i1:i2, i2:], an fp32-accurate product on
//      the tensor cores (tgemm.cu; on the CUDA cores for ragged or tiny shapes), applied
//      in two levels: at once to the rest of the current 256-column super-block, and once
//      per super-block (reduction length 256) to all columns beyond it.  (512 columns moved
//      less data, but the tensor core's accumulator truncates and the error of a 512-deep
//      update, whose terms cancel to a result far smaller than their magnitudes, showed as
//      code mismatches at K = 11008; cutting that product into two chunks cost more time than
//      the narrower window.)
//
// Group scale/zero are taken from W as it stands when the group's first column is
// reached by the block loop (all earlier blocks' trailing updates applied, none of
// the current block's in-block updates), which for groups that start inside a block
// means the values the block had at entry.
#include <algorithm>

#include "common.cuh"
#include "sgemm_view.cuh"
#include "tgemm.cuh"

namespace {

constexpr int MAX_BLOCK = 128;
constexpr int SUPER_BLOCK = 256;   // columns whose updates of far columns are applied together
constexpr int ROWS_PER_CTA = 16;  // one warp each

struct QuantArgs {
  float* W; int64_t ldw;
  const float* U; int64_t ldu;
  uint8_t* codes; int64_t ldc;
  float* scales; float* zeros; int n_groups;
  float* err;            // (N_out, err_ld): scaled errors of the current super-block
  int64_t err_ld; int err_off;  // row stride and first column of the current block in it
  double* total_error;
  double* row_error;     // optional (N_out): sum of squared scaled errors of every row
  int N_out, K, i1, bw;  // block start and width
  int group;             // effective group size (K for per-channel)
  float maxq;
};

__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
gptq_block_kernel(const QuantArgs a) {
  extern __shared__ float Us[];  // bw x MAX_BLOCK, row j = U[i1 + j][i1 .. i1 + bw)
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  // U is an input of the entry point, complete before its first launch (a memset precedes
  // that launch in the stream), so its block may be staged while the preceding trailing
  // update, which only writes W, is still running; W and the error buffer wait for it.
  dgq_chain_release();
  for (int idx = threadIdx.x; idx < a.bw * MAX_BLOCK; idx += blockDim.x) {
    int j = idx / MAX_BLOCK, c = idx % MAX_BLOCK;
    Us[idx] = (c < a.bw && c >= j) ? a.U[(int64_t)(a.i1 + j) * a.ldu + a.i1 + c] : 0.f;
  }
  __syncthreads();
  dgq_chain_wait();

  double err_sq = 0.0;
  for (int row = blockIdx.x * ROWS_PER_CTA + warp; row < a.N_out; row += gridDim.x * ROWS_PER_CTA) {
    float* wrow = a.W + (int64_t)row * a.ldw + a.i1;
    float w[4], s_c[4], z_c[4], what[4], ev[4];
    uint32_t code[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      int c = t * 32 + lane;
      w[t] = (c < a.bw) ? wrow[c] : 0.f;
      what[t] = 0.f; ev[t] = 0.f; code[t] = 0;
    }
    // ---- scale / zero of every column this lane holds
    if (a.group >= a.bw) {
      // the group spans this whole block (and possibly more): one pair for the row
      const int g = a.i1 / a.group;
      float s, z;
      if (a.i1 % a.group == 0) {
        // the group starts here: min/max over W[row][i1 .. i1+group)
        float mn = INFINITY, mx = -INFINITY;
        const int gend = min(a.group, a.K - a.i1);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          int c = t * 32 + lane;
          if (c < a.bw) { mn = fminf(mn, w[t]); mx = fmaxf(mx, w[t]); }
        }
        for (int c = a.bw + lane; c < gend; c += 32) {
          float v = wrow[c];
          mn = fminf(mn, v); mx = fmaxf(mx, v);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        dgq_scale_zero(mn, mx, a.maxq, s, z);
        if (lane == 0) {
          a.scales[(int64_t)row * a.n_groups + g] = s;
          a.zeros[(int64_t)row * a.n_groups + g] = z;
        }
      } else {
        s = a.scales[(int64_t)row * a.n_groups + g];
        z = a.zeros[(int64_t)row * a.n_groups + g];
      }
#pragma unroll
      for (int t = 0; t < 4; ++t) { s_c[t] = s; z_c[t] = z; }
    } else {
      // groups start inside the block, at multiples of `group` (i1 is one too)
      const int g0 = a.i1 / a.group;
      if (a.group >= 32) {
        // a group covers group/32 whole register slots
        const int slots = a.group / 32;
#pragma unroll
        for (int t0 = 0; t0 < 4; t0 += 1) {
          if (t0 % slots != 0) continue;
          float mn = INFINITY, mx = -INFINITY;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            if (t >= t0 && t < t0 + slots) {
              int c = t * 32 + lane;
              if (c < a.bw) { mn = fminf(mn, w[t]); mx = fmaxf(mx, w[t]); }
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          }
          float s, z;
          dgq_scale_zero(mn, mx, a.maxq, s, z);
          const int gi = g0 + (t0 * 32) / a.group;
          if (lane == 0 && t0 * 32 < a.bw) {
            a.scales[(int64_t)row * a.n_groups + gi] = s;
            a.zeros[(int64_t)row * a.n_groups + gi] = z;
          }
#pragma unroll
          for (int t = 0; t < 4; ++t)
            if (t >= t0 && t < t0 + slots) { s_c[t] = s; z_c[t] = z; }
        }
      } else {
        // several groups per slot: segmented reduction over `group` adjacent lanes
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          int c = t * 32 + lane;
          float mn = (c < a.bw) ? w[t] : INFINITY, mx = (c < a.bw) ? w[t] : -INFINITY;
          for (int o = a.group >> 1; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          }
          float s, z;
          dgq_scale_zero(mn, mx, a.maxq, s, z);
          s_c[t] = s; z_c[t] = z;
          if (c < a.bw && (lane % a.group) == 0) {
            a.scales[(int64_t)row * a.n_groups + g0 + c / a.group] = s;
            a.zeros[(int64_t)row * a.n_groups + g0 + c / a.group] = z;
          }
        }
      }
    }
    // ---- the column loop
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (t * 32 >= a.bw) break;
      const int jn = min(32, a.bw - t * 32);
      for (int jl = 0; jl < jn; ++jl) {
        const int j = t * 32 + jl;
        const float wj = __shfl_sync(0xffffffffu, w[t], jl);
        const float sj = __shfl_sync(0xffffffffu, s_c[t], jl);
        const float zj = __shfl_sync(0xffffffffu, z_c[t], jl);
        const float* urow = Us + j * MAX_BLOCK;
        const float q = dgq_quant_level(wj, sj, zj, a.maxq);
        const float wh = dgq_dequant_level(q, sj, zj);
        const float e = __fdiv_rn(__fsub_rn(wj, wh), urow[j]);
        if (lane == jl) {
          code[t] = (uint32_t)q;
          what[t] = wh;
          ev[t] = e;
        }
        // error feedback on the columns to the right (separate multiply and subtract,
        // the order of operations of an outer-product update)
        if (lane > jl) w[t] = __fsub_rn(w[t], __fmul_rn(e, urow[t * 32 + lane]));
#pragma unroll
        for (int u = t + 1; u < 4; ++u) w[u] = __fsub_rn(w[u], __fmul_rn(e, urow[u * 32 + lane]));
      }
    }
    // ---- outputs
    float* erow = a.err + (int64_t)row * a.err_ld + a.err_off;
    uint8_t* crow = a.codes + (int64_t)row * a.ldc + a.i1;
    double row_sq = 0.0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      int c = t * 32 + lane;
      if (c < a.bw) {
        wrow[c] = what[t];
        crow[c] = (uint8_t)code[t];
        erow[c] = ev[t];
        row_sq += (double)ev[t] * (double)ev[t];
      }
    }
    err_sq += row_sq;
    if (a.row_error) {   // one warp per row and one launch per block: no other writer
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) row_sq += __shfl_xor_sync(0xffffffffu, row_sq, o);
      if (lane == 0) a.row_error[row] += row_sq;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) err_sq += __shfl_xor_sync(0xffffffffu, err_sq, o);
  if (lane == 0 && err_sq != 0.0) atomicAdd(a.total_error, err_sq);
}

// ---- fast variant: full 128-column blocks, groups of 32 / 64 / >= 128 columns ----------------
constexpr int F_WARPS = 8;
constexpr int F_ROWS_PER_CTA = F_WARPS * 4;

template <int GPB /* groups per block: 1, 2 or 4 */>
__global__ void __launch_bounds__(F_WARPS * 32)
gptq_block8_kernel(const QuantArgs a) {
  extern __shared__ float Us[];  // 128 x 128, row j = U[i1 + j][i1 .. i1 + 128), zeros left of the diagonal
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane & 7;   // lane inside the row's group of eight
  const int rg = lane >> 3;   // row inside the warp
  // U is an input of the entry point, complete before its first launch (a memset precedes
  // that launch in the stream), so its block may be staged while the preceding trailing
  // update, which only writes W, is still running; W and the error buffer wait for it.
  dgq_chain_release();
  for (int idx = threadIdx.x; idx < MAX_BLOCK * MAX_BLOCK / 4; idx += blockDim.x) {
    const int j = idx / (MAX_BLOCK / 4), c4 = (idx % (MAX_BLOCK / 4)) * 4;
    const float4 u = *reinterpret_cast<const float4*>(a.U + (int64_t)(a.i1 + j) * a.ldu + a.i1 + c4);
    float4 v;
    v.x = (c4 + 0 >= j) ? u.x : 0.f; v.y = (c4 + 1 >= j) ? u.y : 0.f;
    v.z = (c4 + 2 >= j) ? u.z : 0.f; v.w = (c4 + 3 >= j) ? u.w : 0.f;
    reinterpret_cast<float4*>(Us)[idx] = v;
  }
  __syncthreads();
  dgq_chain_wait();
  const float4* Us4 = reinterpret_cast<const float4*>(Us);
  constexpr int GW = MAX_BLOCK / GPB;  // columns per group inside the block

  double err_sq = 0.0;
  for (int row0 = blockIdx.x * F_ROWS_PER_CTA + warp * 4; row0 < a.N_out;
       row0 += gridDim.x * F_ROWS_PER_CTA) {
    const int row = row0 + rg;
    const bool live = row < a.N_out;
    const int rrow = live ? row : a.N_out - 1;  // idle lanes shadow the last row, never store
    float* wrow = a.W + (int64_t)rrow * a.ldw + a.i1;
    float w[16], what[16], ev[16];
    uint32_t code[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 t = *reinterpret_cast<const float4*>(wrow + 4 * (sub + 8 * i));
      w[4 * i] = t.x; w[4 * i + 1] = t.y; w[4 * i + 2] = t.z; w[4 * i + 3] = t.w;
    }
    // ---- scale / zero of the groups of this block
    float sg[GPB], zg[GPB];
    if (GPB == 1 && a.group > MAX_BLOCK && (a.i1 % a.group) != 0) {
      sg[0] = a.scales[(int64_t)rrow * a.n_groups + a.i1 / a.group];
      zg[0] = a.zeros[(int64_t)rrow * a.n_groups + a.i1 / a.group];
    } else {
#pragma unroll
      for (int g = 0; g < GPB; ++g) {
        float mn = INFINITY, mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if ((32 * i) / GW == g) {
#pragma unroll
            for (int e = 0; e < 4; ++e) { mn = fminf(mn, w[4 * i + e]); mx = fmaxf(mx, w[4 * i + e]); }
          }
        }
        if (GPB == 1 && a.group > MAX_BLOCK) {
          // the group continues past this block: the rest of it is read from W
          const int gend = min(a.group, a.K - a.i1);
          for (int c = MAX_BLOCK + sub; c < gend; c += 8) {
            const float v = wrow[c];
            mn = fminf(mn, v); mx = fmaxf(mx, v);
          }
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        dgq_scale_zero(mn, mx, a.maxq, sg[g], zg[g]);
        if (live && sub == 0) {
          const int gi = a.i1 / a.group + g;
          a.scales[(int64_t)row * a.n_groups + gi] = sg[g];
          a.zeros[(int64_t)row * a.n_groups + gi] = zg[g];
        }
      }
    }
    // ---- the column loop.  Columns are visited in order j = 32*ij + 4*owner + e.  The
    // loops over ij (which of the lane's chunks) and e (element of the chunk) are unrolled
    // so that every register index is a constant; the loop over the owning lane is a real
    // loop, which keeps the code small enough to stay in the instruction cache.
#pragma unroll
    for (int ij = 0; ij < 4; ++ij) {
#pragma unroll 1
      for (int owner = 0; owner < 8; ++owner) {
#pragma unroll
        for (int e4 = 0; e4 < 4; ++e4) {
          const int j = 32 * ij + 4 * owner + e4;
          const int reg = 4 * ij + e4;
          const float wj = __shfl_sync(0xffffffffu, w[reg], owner, 8);
          const float sj = sg[(32 * ij) / GW], zj = zg[(32 * ij) / GW];
          const float q = dgq_quant_level(wj, sj, zj, a.maxq);
          const float wh = dgq_dequant_level(q, sj, zj);
          const float e = __fdiv_rn(__fsub_rn(wj, wh), Us[j * MAX_BLOCK + j]);
          if (sub == owner) {
            what[reg] = wh;
            ev[reg] = e;
            code[ij] |= ((uint32_t)q) << (8 * e4);
          }
          // error feedback; U is zero left of the diagonal, so columns already done are untouched
#pragma unroll
          for (int i = ij; i < 4; ++i) {
            const float4 u = Us4[j * (MAX_BLOCK / 4) + sub + 8 * i];
            w[4 * i + 0] = fmaf(-e, u.x, w[4 * i + 0]);
            w[4 * i + 1] = fmaf(-e, u.y, w[4 * i + 1]);
            w[4 * i + 2] = fmaf(-e, u.z, w[4 * i + 2]);
            w[4 * i + 3] = fmaf(-e, u.w, w[4 * i + 3]);
          }
        }
      }
    }
    // ---- outputs
    double row_sq = 0.0;
    if (live) {
      float* erow = a.err + (int64_t)row * a.err_ld + a.err_off;
      uint8_t* crow = a.codes + (int64_t)row * a.ldc + a.i1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 4 * (sub + 8 * i);
        *reinterpret_cast<float4*>(wrow + c) =
            make_float4(what[4 * i], what[4 * i + 1], what[4 * i + 2], what[4 * i + 3]);
        *reinterpret_cast<float4*>(erow + c) =
            make_float4(ev[4 * i], ev[4 * i + 1], ev[4 * i + 2], ev[4 * i + 3]);
        *reinterpret_cast<uint32_t*>(crow + c) = code[i];
#pragma unroll
        for (int e = 0; e < 4; ++e) row_sq += (double)ev[4 * i + e] * (double)ev[4 * i + e];
      }
    }
    err_sq += row_sq;
    if (a.row_error) {   // eight lanes per row and one launch per block: no other writer
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) row_sq += __shfl_xor_sync(0xffffffffu, row_sq, o);
      if (live && sub == 0) a.row_error[row] += row_sq;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) err_sq += __shfl_xor_sync(0xffffffffu, err_sq, o);
  if (lane == 0 && err_sq != 0.0) atomicAdd(a.total_error, err_sq);
}

bool valid_bits(int b) { return b == 2 || b == 3 || b == 4 || b == 8; }

}  // namespace

DGQ_EXPORT int64_t dgq_gptq_quantize_workspace_bytes(int32_t N_out, int32_t K, int32_t blocksize) {
  if (N_out <= 0 || K <= 0 || blocksize <= 0 || blocksize > MAX_BLOCK) return DGQ_ERR_ARG;
  // room for the scaled errors of a whole super-block; a quarter of this (one block's
  // worth) is the minimum dgq_gptq_quantize accepts, at the price of more trailing updates
  return (int64_t)N_out * SUPER_BLOCK * (int64_t)sizeof(float);
}

DGQ_EXPORT int32_t dgq_gptq_quantize(float* W, int64_t ldw, const float* U, int64_t ldu,
                                     int32_t N_out, int32_t K, int32_t bits, int32_t group_size,
                                     int32_t blocksize, uint8_t* codes, int64_t ldc, float* scales,
                                     float* zeros, double* total_error, void* ws, int64_t ws_bytes,
                                     void* stream) {
  return dgq_gptq_quantize_rows(W, ldw, U, ldu, N_out, K, bits, group_size, blocksize, codes, ldc,
                                scales, zeros, total_error, nullptr, ws, ws_bytes, stream);
}

DGQ_EXPORT int32_t dgq_gptq_quantize_rows(float* W, int64_t ldw, const float* U, int64_t ldu,
                                          int32_t N_out, int32_t K, int32_t bits,
                                          int32_t group_size, int32_t blocksize, uint8_t* codes,
                                          int64_t ldc, float* scales, float* zeros,
                                          double* total_error, double* row_error, void* ws,
                                          int64_t ws_bytes, void* stream) {
  DGQ_REQUIRE(W && U && codes && scales && zeros && total_error && ws, DGQ_ERR_ARG);
  DGQ_REQUIRE(N_out > 0 && K > 0 && ldw >= K && ldu >= K && ldc >= K && valid_bits(bits), DGQ_ERR_ARG);
  DGQ_REQUIRE(blocksize > 0 && blocksize <= MAX_BLOCK, DGQ_ERR_UNSUPPORTED);
  const bool per_channel = group_size <= 0 || group_size >= K;
  const int group = per_channel ? K : group_size;
  if (!per_channel) {
    const bool divides = blocksize % group == 0 && (group >= 32 ? group % 32 == 0
                                                                 : (group & (group - 1)) == 0);
    const bool multiple = group % blocksize == 0;
    DGQ_REQUIRE(divides || multiple, DGQ_ERR_UNSUPPORTED);
  }
  DGQ_REQUIRE(ws_bytes >= (int64_t)N_out * MAX_BLOCK * (int64_t)sizeof(float), DGQ_ERR_WORKSPACE);
  DGQ_REQUIRE(dgq_aligned(ws, 16), DGQ_ERR_ALIGN);
  cudaStream_t st = dgq_stream(stream);

  constexpr size_t smem = (size_t)MAX_BLOCK * MAX_BLOCK * sizeof(float);
  static DgqDeviceOnce once;
  if (!once.run([] {
        const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
        return cudaFuncSetAttribute(gptq_block_kernel, at, (int)smem) == cudaSuccess &&
               cudaFuncSetAttribute(gptq_block8_kernel<1>, at, (int)smem) == cudaSuccess &&
               cudaFuncSetAttribute(gptq_block8_kernel<2>, at, (int)smem) == cudaSuccess &&
               cudaFuncSetAttribute(gptq_block8_kernel<4>, at, (int)smem) == cudaSuccess;
      }))
    return DGQ_ERR_LAUNCH;
  // the fast kernel takes full 128-column blocks with 16-byte aligned rows
  const bool fast_layout = blocksize == MAX_BLOCK && ldw % 4 == 0 && ldu % 4 == 0 && ldc % 4 == 0 &&
                           dgq_aligned(W, 16) && dgq_aligned(U, 16) && dgq_aligned(codes, 4);
  int gpb = 0;  // groups per block for the fast kernel, 0 = not eligible
  if (group >= MAX_BLOCK) gpb = (group % MAX_BLOCK == 0 || per_channel) ? 1 : 0;
  else if (group == 64) gpb = 2;
  else if (group == 32) gpb = 4;
  if (cudaMemsetAsync(total_error, 0, sizeof(double), st) != cudaSuccess) return DGQ_ERR_LAUNCH;
  if (row_error &&
      cudaMemsetAsync(row_error, 0, sizeof(double) * (size_t)N_out, st) != cudaSuccess)
    return DGQ_ERR_LAUNCH;

  QuantArgs a;
  a.W = W; a.ldw = ldw; a.U = U; a.ldu = ldu; a.codes = codes; a.ldc = ldc;
  a.scales = scales; a.zeros = zeros;
  a.n_groups = per_channel ? 1 : (int)dgq_cdiv(K, group);
  a.err = reinterpret_cast<float*>(ws);
  a.total_error = total_error;
  a.row_error = row_error;
  a.N_out = N_out; a.K = K; a.group = group; a.maxq = (float)((1 << bits) - 1);
  const unsigned grid = (unsigned)std::min<int64_t>(dgq_cdiv(N_out, ROWS_PER_CTA),
                                                    (int64_t)dgq_sm_count() * 2);
  const bool use_tensor = dgq_use_tensor_gemm();
  // Two-level lazy update: inside a super-block every block's errors update only the
  // super-block's remaining columns; the columns beyond it receive one update per
  // super-block with a reduction as long as the super-block is wide.  This cuts the
  // read-modify-write traffic over W by the number of blocks per super-block.
  int super_cols = (int)std::min<int64_t>(SUPER_BLOCK, ws_bytes / ((int64_t)N_out * sizeof(float)));
  super_cols = std::max(MAX_BLOCK, super_cols / MAX_BLOCK * MAX_BLOCK);
  super_cols = super_cols / blocksize * blocksize;  // block boundaries stay multiples of blocksize
  // A group wider than a block takes its min/max over all its columns when its first column
  // is reached, so by then every one of them must have received all earlier updates: the
  // group either lies inside one super-block or starts where a super-block starts.
  if (!per_channel && group > blocksize) {
    if (group <= super_cols) super_cols = super_cols / group * group;
    else
      while (group % super_cols != 0) super_cols -= blocksize;   // ends at blocksize at the latest
  }
  a.err_ld = super_cols;
  // W[:, c0:c1] -= Err[:, e0:e0+k] * U[r0:r0+k, c0:c1]
  auto update = [&](int e0, int k, int r0, int c0, int c1) {
    if (c1 <= c0 || k <= 0) return;
    bool done = false;
    if (use_tensor && k % 32 == 0 && e0 % 4 == 0 && N_out >= dgq::TGEMM_TILE) {
      dgq::TGemmArgs t = {};
      t.a = a.err + e0; t.lda = a.err_ld;
      t.b = U + (int64_t)r0 * ldu + c0; t.ldb = ldu; t.b_is_kn = 1;
      t.c = W + c0; t.ldc = ldw;
      t.m = N_out; t.n = c1 - c0; t.k = k; t.alpha = -1.f; t.beta = 1.f;
      t.info = nullptr;
      done = dgq::tgemm_supported(t) && dgq::tgemm_launch(t, st);
    }
    if (!done) {
      GemmArgs g = gemm_args(a.err + e0, a.err_ld, 1, U + (int64_t)r0 * ldu + c0, ldu, 1,
                             W + c0, ldw, 1, N_out, c1 - c0, k, -1.f, 1.f);
      launch_gemm(g, st);
    }
  };
  for (int s0 = 0; s0 < K; s0 += super_cols) {
    const int s1 = std::min(K, s0 + super_cols);
    for (int i1 = s0; i1 < s1; i1 += blocksize) {
      a.i1 = i1;
      a.bw = std::min(blocksize, s1 - i1);
      a.err_off = i1 - s0;
      if (fast_layout && gpb != 0 && a.bw == MAX_BLOCK) {
        const unsigned fgrid = (unsigned)std::min<int64_t>(dgq_cdiv(N_out, F_ROWS_PER_CTA),
                                                           (int64_t)dgq_sm_count() * 3);
        const dim3 fg(fgrid), fb(F_WARPS * 32);
        cudaError_t e;
        if (gpb == 1) e = dgq_launch_chained(gptq_block8_kernel<1>, fg, fb, smem, st, a);
        else if (gpb == 2) e = dgq_launch_chained(gptq_block8_kernel<2>, fg, fb, smem, st, a);
        else e = dgq_launch_chained(gptq_block8_kernel<4>, fg, fb, smem, st, a);
        if (e != cudaSuccess) return DGQ_ERR_LAUNCH;
      } else {
        if (dgq_launch_chained(gptq_block_kernel, dim3(grid), dim3(ROWS_PER_CTA * 32),
                               (size_t)a.bw * MAX_BLOCK * sizeof(float), st, a) != cudaSuccess)
          return DGQ_ERR_LAUNCH;
      }
      update(a.err_off, a.bw, i1, i1 + a.bw, s1);      // rest of this super-block
    }
    update(0, s1 - s0, s0, s1, K);                      // everything beyond it
  }
  return dgq_launch_status(dgq_cdiv(K, blocksize));
}

// ---- variant for callers that cannot allocate ---------------------------------------------------
// Scratch for dgq_gptq_quantize_noalloc: the (rows x 128) buffer of scaled errors that the
// block kernel hands to the trailing update.  It lives in the library's device image, so
// every GPU that loads the library holds these 8 MiB until the process exits.
constexpr int NOALLOC_MAX_ROWS = 16384;
static __device__ __align__(256) float g_noalloc_err[(size_t)NOALLOC_MAX_ROWS * MAX_BLOCK];

DGQ_EXPORT int32_t dgq_gptq_quantize_noalloc_max_rows(void) { return NOALLOC_MAX_ROWS; }

DGQ_EXPORT int32_t dgq_gptq_quantize_noalloc(float* W, int64_t ldw, const float* U, int64_t ldu,
                                             int32_t N_out, int32_t K, int32_t bits,
                                             int32_t group_size, int32_t blocksize, uint8_t* codes,
                                             int64_t ldc, float* scales, float* zeros,
                                             double* total_error, void* stream) {
  DGQ_REQUIRE(N_out > 0, DGQ_ERR_ARG);
  DGQ_REQUIRE(N_out <= NOALLOC_MAX_ROWS, DGQ_ERR_SIZE);
  // In host code the array's name is only a handle: the device address has to be asked
  // for, once per device, with that device current.
  constexpr int MAX_DEVICES = 64;
  static float* scratch_of_device[MAX_DEVICES] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return DGQ_ERR_LAUNCH;
  if (scratch_of_device[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_err) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return DGQ_ERR_LAUNCH;
    }
    scratch_of_device[dev] = static_cast<float*>(p);
  }
  return dgq_gptq_quantize(W, ldw, U, ldu, N_out, K, bits, group_size, blocksize, codes, ldc,
                           scales, zeros, total_error, scratch_of_device[dev],
                           (int64_t)sizeof(float) * NOALLOC_MAX_ROWS * MAX_BLOCK, stream);
}
