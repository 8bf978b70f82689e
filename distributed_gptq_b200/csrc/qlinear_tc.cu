// Quantized linear for many rows of activations (prefill-sized M) on the sm_100a tensor cores:
//
//   y(M x N_out) = x(M x K) * dequant(Wq)(N_out x K)^T + bias      x, y fp16 or bf16
//
// 4-bit codes, two per byte with the even column in the low nibble (the QuantizedLinear
// layout, models/layers.py:76-93), one fp16 scale/zero per output feature and group of
// `group_size` consecutive columns (a multiple of 64).  The weights never exist in 16-bit
// form in global memory: a CTA works on a tile of y of 128 features x 128 rows (M <= 128),
// 128 features x 256 rows (two sub-tiles that share the converted weights) or, when there are
// enough tiles, 256 features x 256 rows, and walks K in slices of 64 columns; per slice
//   - warp 0 fetches the slice of x with one TMA box (128-byte swizzle): operand A;
//   - warps 2-17 ("converters", one thread per output feature and slice; with 128 features per
//     tile four groups of four warps, with 256 two groups of eight, each group taking every
//     fourth / second slice) read the feature's 32 bytes of packed codes straight from global
//     memory (two own slices ahead: a load takes longer than a slice), turn them into 64
//     values (code - zero) * scale of the activation type and store them as the feature's
//     128-byte row of operand B, in the same swizzled layout a TMA box would have produced;
//   - warp 1 issues four tcgen05.mma kind::f16 (M = 128 rows, N = 128 features, K = 16) per
//     sub-tile into that sub-tile's 128-column fp32 accumulator in tensor memory;
// and warps 18-21 drain finished accumulators (two sets alternate where they fit), add the
// bias, round and store.
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

constexpr int SUB_M = 128, SUB_N = 128, BK = 64;
constexpr int SUB_A_BYTES = SUB_M * BK * 2, SUB_B_BYTES = SUB_N * BK * 2;   // 16 KB each
constexpr int MAX_STAGES = 6;
constexpr int CONV_WARPS = 16;
constexpr int CONV_THREADS = 32 * CONV_WARPS;
constexpr int THREADS = 32 * (2 + CONV_WARPS + 4);

// A tile of y is MT sub-tiles of 128 rows against NT sub-tiles of 128 features.  MT = 2: the
// converted slice of weights (the expensive operand) serves two products.  NT = 2: the slice of
// activations does, and one product instruction covers 256 features (with the conversion left
// out, the 256 x 128 pipeline runs at 1.0 PFLOP/s, the 256 x 256 one at 1.4-1.5), at the price
// of a single set of accumulators (all 512 columns of tensor memory), i.e. an epilogue the next
// tile's products wait for.  192 KB of stages in every shape.
template <int MT, int NT> struct Shape {
  static constexpr int TILE_M = SUB_M * MT, TILE_N = SUB_N * NT;
  static constexpr int A_BYTES = SUB_A_BYTES * MT, B_BYTES = SUB_B_BYTES * NT;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;  // 6, 4, 3
  static constexpr uint32_t ACC_COLS = SUB_N * NT * MT;      // one accumulator set
  static constexpr int ACC_SETS = ACC_COLS * 2 <= 512 ? 2 : 1;
  static constexpr uint32_t TMEM_COLS = ACC_SETS * ACC_COLS;
  // converter threads per slice: one per feature row; the groups take alternate slices
  static constexpr int GROUPS = CONV_THREADS / TILE_N;
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
  static_assert(STAGES <= MAX_STAGES && STAGES >= 2 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "shape");
};

struct Control {
  uint64_t full[MAX_STAGES], conv[MAX_STAGES], empty[MAX_STAGES];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};

struct Params {
  dgq::QLinearTcArgs a;
  int tiles_m, tiles_n, n_tiles, n_slices;
};

// Per activation type: packing of two floats, and the arithmetic of the short dequantization.
// A 4-bit code c OR-ed into the mantissa of BASE (1024 in fp16, 128 in bf16) is the number
// BASE + c; subtracting BASE + zero is exact for an integer zero point, and one multiplication
// by the scale rounds once - the same value as rounding (c - zero) * scale computed in fp32.
template <typename T> struct Cvt;
template <> struct Cvt<__half> {
  static constexpr uint32_t FMT = tc05::FMT_F16;
  static constexpr uint32_t MAGIC = 0x64006400u;
  static constexpr float BASE = 1024.f;
  static constexpr float MAX_ZERO = 64.f;      // largest |zero| the short conversion is exact for
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  // the scale as a pair of T, and what T cannot hold of it (nothing: the scale is fp16)
  static __device__ __forceinline__ void scale_pairs(float sc, uint32_t& hi2, uint32_t& lo2) {
    hi2 = pack2(sc, sc);
    lo2 = 0u;
  }
  // (BASE + c) - (BASE + zero) is exact, the scale is an fp16 number: one rounding
  static __device__ __forceinline__ uint32_t dequant_pair(uint32_t v, uint32_t sub, uint32_t mul,
                                                          uint32_t) {
    const __half2 r = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&v),
                                      *reinterpret_cast<const __half2*>(&sub)),
                              *reinterpret_cast<const __half2*>(&mul));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
};
template <> struct Cvt<__nv_bfloat16> {
  static constexpr uint32_t FMT = tc05::FMT_BF16;
  static constexpr uint32_t MAGIC = 0x43004300u;
  static constexpr float BASE = 128.f;
  static constexpr float MAX_ZERO = 16.f;      // |d| <= 31: 5 bits, times the 3 bits of lo = 8
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  // The fp16 scale (11 significant bits) is not a bf16 number (8): it is split into
  // hi = bf16(scale) and lo = scale - hi, which has at most 3 significant bits and is a bf16
  // number too.
  static __device__ __forceinline__ void scale_pairs(float sc, uint32_t& hi2, uint32_t& lo2) {
    const float hi = __bfloat162float(__float2bfloat16_rn(sc));
    hi2 = pack2(hi, hi);
    lo2 = pack2(sc - hi, sc - hi);
  }
  // d = (BASE + c) - (BASE + zero) is exact and at most 5 bits wide (|zero| <= MAX_ZERO), so
  // d * lo is exact in bf16 and fma(d, hi, d * lo) is the exact product d * scale rounded
  // once - the value rounding (c - zero) * scale computed in fp32 gives.
  static __device__ __forceinline__ uint32_t dequant_pair(uint32_t v, uint32_t sub, uint32_t mul,
                                                          uint32_t mul_lo) {
    const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&v),
                                     *reinterpret_cast<const __nv_bfloat162*>(&sub));
    const __nv_bfloat162 t = __hmul2(d, *reinterpret_cast<const __nv_bfloat162*>(&mul_lo));
    const __nv_bfloat162 r = __hfma2(d, *reinterpret_cast<const __nv_bfloat162*>(&mul), t);
    return *reinterpret_cast<const uint32_t*>(&r);
  }
};

__device__ __forceinline__ float bias_at(const void* b, int dt, int n) {
  if (dt == DGQ_F32) return reinterpret_cast<const float*>(b)[n];
  if (dt == DGQ_F16) return __half2float(reinterpret_cast<const __half*>(b)[n]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[n]);
}

template <typename T, int MT, int NT>
__global__ void __launch_bounds__(THREADS, 1)
qlinear_tc_kernel(const __grid_constant__ CUtensorMap map_x, const Params p) {
  using S = Shape<MT, NT>;
  constexpr int TILE_M = S::TILE_M, TILE_N = S::TILE_N, A_BYTES = S::A_BYTES;
  constexpr int STAGE_BYTES = S::STAGE_BYTES, STAGES = S::STAGES;
  constexpr int ACC_SETS = S::ACC_SETS, GROUPS = S::GROUPS;
  constexpr uint32_t TMEM_COLS = S::TMEM_COLS, ACC_COLS = S::ACC_COLS;
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
      tc05::mbar_init(&ctl->conv[s], CONV_WARPS / GROUPS); // the warps of one group
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
      // one instruction covers all NT sub-tiles of features: their rows follow each other in
      // operand B (128 bytes each, 1024 bytes per group of eight)
      constexpr uint32_t idesc = tc05::make_instr_desc(Cvt<T>::FMT, false, false, SUB_M, TILE_N);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, ++lt) {
        const uint32_t ab = lt % ACC_SETS, aph = (lt / ACC_SETS) & 1;
        if (!tc05::mbar_wait_bounded(&ctl->tmem_empty[ab], aph ^ 1, abort_flag)) {
          if (a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 22; }
          break;
        }
        tc05::fence_after_sync();
        const uint32_t acc = tmem_base + ab * ACC_COLS;
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
            const uint64_t db = tc05::make_smem_desc(b_base + k * 32, 0, 1024);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              // sub-tile mt: rows 128 mt .. of the box, 16 KB further; its own TILE_N columns
              const uint64_t da = tc05::make_smem_desc(a_base + mt * SUB_A_BYTES + k * 32, 0, 1024);
              tc05::umma_bf16(acc + mt * TILE_N, da, db, idesc, (s_ | k) != 0 ? 1u : 0u);
            }
          }
          tc05::umma_commit(&ctl->empty[s]);
        }
        if (ok) tc05::umma_commit(&ctl->tmem_full[ab]);
      }
    }
    __syncwarp();
  } else if (warp < 2 + CONV_WARPS) {
    // ------------------------------------------------------------------ converters (weights)
    // GROUPS groups of converter warps take every GROUPS-th slice (group = running slice count
    // mod GROUPS), one thread per feature row: a slice's conversion is a chain of dependent
    // steps (wait for the stage, convert, store, proxy fence, arrive) whose latency, not its
    // instruction count, bounds a group (with the conversion left out the same pipeline runs
    // at 1.4-1.5 PFLOP/s); several slices in flight hide part of it.
    const int ct = threadIdx.x - 64;                 // 0..CONV_THREADS-1
    const int f = ct % TILE_N;                       // feature row of the tile
    const int grp = ct / TILE_N;                     // takes the slices whose running count is grp mod GROUPS
    const int slices_per_group = a.n_groups == 1 ? p.n_slices : a.group_size / BK;
    uint32_t it0 = 0;                                // slices of the tiles before this one
    bool ok = true;
    for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, it0 += p.n_slices) {
      const int tn = t / p.tiles_m;
      const int n = min(tn * TILE_N + f, a.N_out - 1);       // rows past the end repeat the last
      const uint8_t* wrow = a.qw + (int64_t)n * a.row_bytes;
      const __half* srow = a.scales + (int64_t)n * a.n_groups;
      const __half* zrow = a.zeros + (int64_t)n * a.n_groups;
      struct Codes { uint4 lo, hi; };                 // the slice's 32 bytes of this row
      auto fetch = [&](int sl) -> Codes {
        Codes c;
        if (sl < p.n_slices) {
          const uint4* src = reinterpret_cast<const uint4*>(wrow + (int64_t)sl * 32);
          c.lo = src[0];
          c.hi = src[1];
        } else {
          c.lo = c.hi = make_uint4(0u, 0u, 0u, 0u);
        }
        return c;
      };
      // this group's first slice of the tile: (it0 + first) % GROUPS == grp
      const int first = (int)(((uint32_t)grp + GROUPS - it0 % GROUPS) % GROUPS);
      Codes qa = fetch(first), qb = fetch(first + GROUPS);
      // scale and zero of the group of the next own slice are fetched a slice ahead as well: a
      // load that is needed at once would stall the warp for longer than a slice takes
      int cur_g = -1, pre_g = -1;
      __half s_pre = __float2half(0.f), z_pre = __float2half(0.f);
      float sc = 0.f, zs = 0.f;
      uint32_t sub2 = 0u, mul2 = 0u, mul_lo2 = 0u;   // (BASE + zero) x 2, scale x 2 (and its rest) as pairs of T
      bool short_path = false;
      // one slice: the row's 32 bytes of codes -> 64 values -> the eight 16-byte pieces of row f
      auto step = [&](int sl, const Codes& codes) -> bool {
        const uint32_t it = it0 + (uint32_t)sl;
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
        const int g = a.n_groups == 1 ? 0 : sl / slices_per_group;
        if (g != cur_g) {
          const __half sv = g == pre_g ? s_pre : srow[g], zv = g == pre_g ? z_pre : zrow[g];
          cur_g = g;
          sc = __half2float(sv);
          const float z = __half2float(zv);
          zs = z * sc;                                       // w = code * scale - zero * scale
          // integer zero points (every GPTQ zero is one) take the short path
          short_path = (z == rintf(z)) && fabsf(z) <= Cvt<T>::MAX_ZERO;
          sub2 = Cvt<T>::pack2(Cvt<T>::BASE + z, Cvt<T>::BASE + z);
          Cvt<T>::scale_pairs(sc, mul2, mul_lo2);
        }
        const int gn = a.n_groups == 1 ? 0 : min((sl + GROUPS) / slices_per_group, a.n_groups - 1);
        if (gn != cur_g && gn != pre_g) {
          s_pre = srow[gn];
          z_pre = zrow[gn];
          pre_g = gn;
        }
        const bool got = tc05::mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 24; }
          return false;
        }
        // row f of operand B: eight 16-byte pieces, piece c stored at position c ^ (f % 8)
        uint4* brow = reinterpret_cast<uint4*>(stages + (size_t)s * STAGE_BYTES + A_BYTES) + f * 8;
        const uint32_t words[8] = {codes.lo.x, codes.lo.y, codes.lo.z, codes.lo.w,
                                   codes.hi.x, codes.hi.y, codes.hi.z, codes.hi.w};
        const bool fast = __all_sync(0xffffffffu, short_path);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          // one 32-bit word = 4 bytes = 8 codes = columns 8 c .. 8 c + 7 of the slice
          const uint32_t w = words[c], w4 = w >> 4;
          uint32_t o[4];
          if (fast) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              // byte b of w (low nibble = even column) and of w >> 4 (low nibble = odd column)
              const uint32_t pr = __byte_perm(w, w4, ((4 + b) << 8) | b);
              o[b] = Cvt<T>::dequant_pair((pr & 0x000F000Fu) | Cvt<T>::MAGIC, sub2, mul2, mul_lo2);
            }
          } else {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const float lo = (float)((w >> (8 * b)) & 15u), hi = (float)((w >> (8 * b + 4)) & 15u);
              o[b] = Cvt<T>::pack2(fmaf(lo, sc, -zs), fmaf(hi, sc, -zs));
            }
          }
          brow[c ^ (f & 7)] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        // make the generic-proxy writes visible to the tensor core's (async proxy) reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) tc05::mbar_arrive(&ctl->conv[s]);
        return true;
      };
      for (int s_ = first; s_ < p.n_slices && ok; s_ += 2 * GROUPS) {
        // two own slices per turn so that the code registers have fixed names; each is
        // refilled, for the own slice after the next, as soon as it has been used
        ok = step(s_, qa);
        qa = fetch(s_ + 2 * GROUPS);
        if (ok && s_ + GROUPS < p.n_slices) { ok = step(s_ + GROUPS, qb); qb = fetch(s_ + 3 * GROUPS); }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;
    uint32_t lt = 0;
    T* y = reinterpret_cast<T*>(a.y);
    for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++lt) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      const uint32_t ab = lt % ACC_SETS, aph = (lt / ACC_SETS) & 1;
      const bool got = tc05::mbar_wait_bounded(&ctl->tmem_full[ab], aph, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0 && a.info) { a.info[0] = DGQ_INFO_WAIT_TIMEOUT; a.info[1] = 25; }
        break;
      }
      tc05::fence_after_sync();
#pragma unroll 1
      for (int cc = 0; cc < MT * (TILE_N / 32); ++cc) {
        const int mt = cc / (TILE_N / 32), chunk = cc % (TILE_N / 32);
        const int row = tm * TILE_M + mt * SUB_M + q * 32 + lane;   // this thread's row of y
        uint32_t v[32];
        tc05::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + ab * ACC_COLS + mt * TILE_N +
                                chunk * 32, v);
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

namespace {

template <int MT, int NT>
bool launch_shape(const QLinearTcArgs& a, cudaStream_t st) {
  using S = Shape<MT, NT>;
  CUtensorMap map_x;
  const CUtensorMapDataType dt = a.dtype == DGQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!tc05::make_tensor_map_2d(&map_x, dt, 2, a.x, (uint64_t)a.M, (uint64_t)a.K,
                                (uint64_t)a.K * 2, S::TILE_M, BK))
    return false;
  Params p;
  p.a = a;
  p.tiles_m = (int)dgq_cdiv(a.M, S::TILE_M);
  p.tiles_n = (int)dgq_cdiv(a.N_out, S::TILE_N);
  p.n_tiles = p.tiles_m * p.tiles_n;
  p.n_slices = a.K / BK;
  const unsigned grid = (unsigned)std::min(p.n_tiles, dgq_sm_count());
  if (a.dtype == DGQ_F16)
    qlinear_tc_kernel<__half, MT, NT><<<grid, THREADS, S::SMEM_BYTES, st>>>(map_x, p);
  else
    qlinear_tc_kernel<__nv_bfloat16, MT, NT><<<grid, THREADS, S::SMEM_BYTES, st>>>(map_x, p);
  dgq_note_launches(1);
  return cudaGetLastError() == cudaSuccess;
}

template <int MT, int NT>
bool set_smem() {
  const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
  const int bytes = (int)Shape<MT, NT>::SMEM_BYTES;
  return cudaFuncSetAttribute(qlinear_tc_kernel<__half, MT, NT>, at, bytes) == cudaSuccess &&
         cudaFuncSetAttribute(qlinear_tc_kernel<__nv_bfloat16, MT, NT>, at, bytes) == cudaSuccess;
}

}  // namespace

bool qlinear_tc_launch(const QLinearTcArgs& a, cudaStream_t st) {
  static DgqDeviceOnce once;
  if (!once.run([] { return set_smem<1, 1>() && set_smem<2, 1>() && set_smem<2, 2>(); }))
    return false;
  if (a.M <= SUB_M) return launch_shape<1, 1>(a, st);
  // Above one sub-tile of rows the 256-row tile halves the conversions per product, and the
  // 256-feature tile halves the activation bytes per product too (measured 1090 against 910
  // TFLOP/s with every SM busy) - but a persistent grid's last round is partly idle, and
  // with few tiles the larger tile loses more to that than it gains.
  const int64_t sms = dgq_sm_count();
  auto busy = [&](int64_t tiles) { return (double)tiles / (double)(dgq_cdiv(tiles, sms) * sms); };
  const int64_t tiles_m = dgq_cdiv(a.M, 2 * SUB_M);
  const double wide = busy(tiles_m * dgq_cdiv(a.N_out, 2 * SUB_N));
  const double narrow = busy(tiles_m * dgq_cdiv(a.N_out, SUB_N));
  if (wide * 1090.0 > narrow * 910.0) return launch_shape<2, 2>(a, st);
  return launch_shape<2, 1>(a, st);
}

}  // namespace dgq
