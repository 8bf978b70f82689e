// Quantized linear for many rows of activations (prefill-sized M) on the sm_100a tensor cores:
//
//   y(M x N_out) = x(M x K) * dequant(Wq)(N_out x K)^T + bias      x, y fp16 or bf16
//
// 4-bit codes, two per byte with the even column in the low nibble (the QuantizedLinear
// layout, models/layers.py:76-93), one fp16 scale/zero per output feature and group of
// `group_size` consecutive columns (a multiple of 64).  The weights never exist in 16-bit
// form in global memory: a CTA works on a 128-row x 128-feature tile of y and walks K in
// slices of 64 columns; per slice
//   - warp 0 fetches the 128 x 64 slice of x with one TMA box (128-byte swizzle): operand A;
//   - warps 2-5 ("converters", one thread per output feature) read the feature's 32 bytes of
//     packed codes straight from global memory (prefetched one slice ahead), turn them into
//     64 values (code - zero) * scale of the activation type and store them as the feature's
//     128-byte row of operand B, in the same swizzled layout a TMA box would have produced;
//   - warp 1 issues four tcgen05.mma kind::f16 (M = 128 rows, N = 128 features, K = 16) into
//     a 128-column fp32 accumulator in tensor memory;
// and warps 6-9 drain finished accumulators (two alternate), add the bias, round and store.
// CTAs are persistent; tiles are ordered with the row tile running fastest, so the CTAs
// running at one time share packed weights through L2.
//
// Rounding: (code - zero) * scale is rounded once to the activation type (relative 2^-11 for
// fp16, 2^-8 for bf16) before the product, which is what dequantize-then-matmul in that type
// does (models/layers.py:155-157); products are exact and accumulate in fp32.
//
// Every wait on an mbarrier is bounded, as in the other tensor-core kernels of this library.
#include <algorithm>

#include "common.cuh"
#include "qlinear_tc.cuh"
#include "tc05.cuh"

namespace {

constexpr int TILE_M = 128, TILE_N = 128, BK = 64;
constexpr int A_BYTES = TILE_M * BK * 2, B_BYTES = TILE_N * BK * 2;     // 16 KB each
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4;
constexpr int THREADS = 320;
constexpr uint32_t TMEM_COLS = 256;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 + 256;

struct Control {
  uint64_t full[STAGES], conv[STAGES], empty[STAGES];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};

struct Params {
  dgq::QLinearTcArgs a;
  int tiles_m, tiles_n, n_tiles, n_slices;
};

template <typename T> struct Cvt;
template <> struct Cvt<__half> {
  static constexpr uint32_t FMT = tc05::FMT_F16;
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <> struct Cvt<__nv_bfloat16> {
  static constexpr uint32_t FMT = tc05::FMT_BF16;
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};

__device__ __forceinline__ float bias_at(const void* b, int dt, int n) {
  if (dt == DGQ_F32) return reinterpret_cast<const float*>(b)[n];
  if (dt == DGQ_F16) return __half2float(reinterpret_cast<const __half*>(b)[n]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[n]);
}

template <typename T>
__global__ void __launch_bounds__(THREADS, 1)
qlinear_tc_kernel(const __grid_constant__ CUtensorMap map_x, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stages = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Control* ctl = reinterpret_cast<Control*>(stages + (size_t)STAGES * STAGE_BYTES);
  volatile int* abort_flag = &ctl->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const dgq::QLinearTcArgs& a = p.a;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc05::mbar_init(&ctl->full[s], 1);
      tc05::mbar_init(&ctl->conv[s], 4);
      tc05::mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc05::mbar_init(&ctl->tmem_full[b], 1);
      tc05::mbar_init(&ctl->tmem_empty[b], 4);
    }
    ctl->abort = 0;
    tc05::fence_mbar_init();
    tc05::prefetch_tensormap(&map_x);
  }
  if (warp == 0) {
    __syncwarp();
    tc05::tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tc05::tmem_relinquish();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (x)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
        const int tm = t % p.tiles_m;
        for (int s_ = 0; s_ < p.n_slices; ++s_, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!tc05::mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag)) {
            if (a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 21; }
            ok = false;
            break;
          }
          tc05::mbar_expect_tx(&ctl->full[s], A_BYTES);
          tc05::tma_load_2d(stages + (size_t)s * STAGE_BYTES, &map_x, s_ * BK, tm * TILE_M,
                            &ctl->full[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = tc05::make_instr_desc(Cvt<T>::FMT, false, false, TILE_M, TILE_N);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++lt) {
        const uint32_t ab = lt & 1, aph = (lt >> 1) & 1;
        if (!tc05::mbar_wait_bounded(&ctl->tmem_empty[ab], aph ^ 1, abort_flag)) {
          if (a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 22; }
          break;
        }
        tc05::fence_after_sync();
        const uint32_t acc = tmem_base + ab * TILE_N;
        for (int s_ = 0; s_ < p.n_slices; ++s_, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!tc05::mbar_wait_bounded(&ctl->full[s], ph, abort_flag) ||
              !tc05::mbar_wait_bounded(&ctl->conv[s], ph, abort_flag)) {
            if (a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 23; }
            ok = false;
            break;
          }
          tc05::fence_after_sync();
          const uint32_t a_base = tc05::smem_u32(stages + (size_t)s * STAGE_BYTES);
          const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // both operands are K-major rows of 128 bytes: 16 elements = 32 bytes further along
            const uint64_t da = tc05::make_smem_desc(a_base + k * 32, 0, 1024);
            const uint64_t db = tc05::make_smem_desc(b_base + k * 32, 0, 1024);
            tc05::umma_bf16(acc, da, db, idesc, (s_ | k) != 0 ? 1u : 0u);
          }
          tc05::umma_commit(&ctl->empty[s]);
        }
        if (ok) tc05::umma_commit(&ctl->tmem_full[ab]);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------------ converters (weights)
    const int f = threadIdx.x - 64;                  // feature row of the tile, 0..127
    const int slices_per_group = a.n_groups == 1 ? p.n_slices : a.group_size / BK;
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
      const int tn = t / p.tiles_m;
      const int n = min(tn * TILE_N + f, a.N_out - 1);       // rows past the end repeat the last
      const uint8_t* wrow = a.qw + (int64_t)n * a.row_bytes;
      const __half* srow = a.scales + (int64_t)n * a.n_groups;
      const __half* zrow = a.zeros + (int64_t)n * a.n_groups;
      uint4 c0 = *reinterpret_cast<const uint4*>(wrow);      // slice 0: columns 0..63 = 32 bytes
      uint4 c1 = *reinterpret_cast<const uint4*>(wrow + 16);
      float sc = 0.f, zs = 0.f;
      for (int s_ = 0; s_ < p.n_slices; ++s_, ++it) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
        if (s_ % slices_per_group == 0) {
          const int g = s_ / slices_per_group;
          sc = __half2float(srow[g]);
          zs = __half2float(zrow[g]) * sc;                   // w = code * scale - zero * scale
        }
        const uint4 cur0 = c0, cur1 = c1;
        if (s_ + 1 < p.n_slices) {                           // next slice's codes, in flight
          c0 = *reinterpret_cast<const uint4*>(wrow + (s_ + 1) * 32);
          c1 = *reinterpret_cast<const uint4*>(wrow + (s_ + 1) * 32 + 16);
        }
        const bool got = tc05::mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 24; }
          ok = false;
          break;
        }
        // row f of operand B: eight 16-byte pieces, piece c stored at position c ^ (f % 8)
        uint4* brow = reinterpret_cast<uint4*>(stages + (size_t)s * STAGE_BYTES + A_BYTES) + f * 8;
        const uint32_t words[8] = {cur0.x, cur0.y, cur0.z, cur0.w, cur1.x, cur1.y, cur1.z, cur1.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          // one 32-bit word = 4 bytes = 8 codes = columns 8c .. 8c+7 of the slice
          const uint32_t w = words[c];
          uint32_t o[4];
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const float lo = (float)((w >> (8 * b)) & 15u), hi = (float)((w >> (8 * b + 4)) & 15u);
            o[b] = Cvt<T>::pack2(fmaf(lo, sc, -zs), fmaf(hi, sc, -zs));
          }
          brow[c ^ (f & 7)] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        // make the generic-proxy writes visible to the tensor core's (async proxy) reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) tc05::mbar_arrive(&ctl->conv[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    uint32_t lt = 0;
    T* y = reinterpret_cast<T*>(a.y);
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++lt) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      const uint32_t ab = lt & 1, aph = (lt >> 1) & 1;
      const bool got = tc05::mbar_wait_bounded(&ctl->tmem_full[ab], aph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0 && a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 25; }
        break;
      }
      tc05::fence_after_sync();
      const int row = tm * TILE_M + q * 32 + lane;           // this thread's row of y
#pragma unroll 1
      for (int chunk = 0; chunk < TILE_N / 32; ++chunk) {
        uint32_t v[32];
        tc05::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + ab * TILE_N + chunk * 32, v);
        tc05::tmem_ld_wait();
        const int n0 = tn * TILE_N + chunk * 32;
        if (row < a.M && n0 < a.N_out) {
          T* dst = y + (int64_t)row * a.N_out + n0;
          if (n0 + 32 <= a.N_out && (a.N_out % 8) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float lo = __uint_as_float(v[j + 2 * e]), hi = __uint_as_float(v[j + 2 * e + 1]);
                if (a.bias) {
                  lo += bias_at(a.bias, a.bias_dtype, n0 + j + 2 * e);
                  hi += bias_at(a.bias, a.bias_dtype, n0 + j + 2 * e + 1);
                }
                o[e] = Cvt<T>::pack2(lo, hi);
              }
              *reinterpret_cast<uint4*>(dst + j) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          } else {
            for (int j = 0; j < 32 && n0 + j < a.N_out; ++j) {
              float val = __uint_as_float(v[j]);
              if (a.bias) val += bias_at(a.bias, a.bias_dtype, n0 + j);
              dst[j] = dgq_from_float<T>(val);
            }
          }
        }
      }
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty[ab]);
    }
  }

  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

namespace dgq {

bool qlinear_tc_supported(const QLinearTcArgs& a) {
  if (a.dtype != DGQ_F16 && a.dtype != DGQ_BF16) return false;
  if (a.M <= 0 || a.N_out <= 0 || a.K < BK || a.K % BK != 0) return false;
  if (a.n_groups != 1 && (a.group_size <= 0 || a.group_size % BK != 0 ||
                          (int64_t)a.n_groups * a.group_size < a.K))
    return false;
  if (a.row_bytes % 16 != 0 || !dgq_aligned(a.qw, 16)) return false;   // 16-byte loads of codes
  if (!dgq_aligned(a.x, 16) || !dgq_aligned(a.y, 16)) return false;     // TMA base, 16-byte stores
  return true;
}

bool qlinear_tc_launch(const QLinearTcArgs& a, cudaStream_t st) {
  static DgqDeviceOnce once;
  if (!once.run([] {
        const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
        return cudaFuncSetAttribute(qlinear_tc_kernel<__half>, at, (int)SMEM_BYTES) == cudaSuccess &&
               cudaFuncSetAttribute(qlinear_tc_kernel<__nv_bfloat16>, at, (int)SMEM_BYTES) == cudaSuccess;
      }))
    return false;
  CUtensorMap map_x;
  const CUtensorMapDataType dt = a.dtype == DGQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!tc05::make_tensor_map_2d(&map_x, dt, 2, a.x, (uint64_t)a.M, (uint64_t)a.K,
                                (uint64_t)a.K * 2, TILE_M, BK))
    return false;
  Params p;
  p.a = a;
  p.tiles_m = (int)dgq_cdiv(a.M, TILE_M);
  p.tiles_n = (int)dgq_cdiv(a.N_out, TILE_N);
  p.n_tiles = p.tiles_m * p.tiles_n;
  p.n_slices = a.K / BK;
  const unsigned grid = (unsigned)std::min(p.n_tiles, dgq_sm_count());
  if (a.dtype == DGQ_F16)
    qlinear_tc_kernel<__half><<<grid, THREADS, SMEM_BYTES, st>>>(map_x, p);
  else
    qlinear_tc_kernel<__nv_bfloat16><<<grid, THREADS, SMEM_BYTES, st>>>(map_x, p);
  dgq_note_launches(1);
  return cudaGetLastError() == cudaSuccess;
}

}  // namespace dgq
