// fp32-accurate matrix product on the sm_100a tensor cores:  C = alpha * A * B + beta * C.
//
// Data path per 32-wide reduction slice: TMA brings the fp32 tiles of A (128 x 32) and of
// B (128 x 32, or 32 x 128 as four 32 x 32 panels) into 128-byte-swizzled shared memory
// (32-byte swizzle atoms for the n-contiguous form of B, as tf32 operands require);
// four converter warps split every element x into hi = tf32(x) (round to nearest) and
// lo = x - hi.  For B, hi is written in place and lo into a twin buffer at the same
// (swizzled) offset.  For A, converter thread r owns row r of the tile and writes hi and lo
// into tensor memory (32 columns each per stage), from where the products read their A
// operand: the kernel is bound by shared-memory bandwidth (TMA writes, converter traffic and
// the operand reads of three products per slice), and this takes A's converter writes and
// all A operand reads off it (224 -> 144 KB of shared-memory traffic per slice; 4096^3:
// 165 -> 205 TFLOP/s fp32-equivalent).  One thread then issues, per 8 reduction steps, three
// tcgen05.mma kind::tf32 instructions (lo*hi, hi*lo, hi*hi) into a 128 x 128 fp32
// accumulator in tensor memory.
// Accumulators are double buffered so that the epilogue warps (TMEM -> registers -> a
// warp-private swizzled staging tile in shared memory -> alpha/beta update with whole
// 128-byte lines of C per row) overlap the next tile's main loop.  CTAs are persistent
// over the output tiles.
//
// Warps: 0 TMA producer (+ TMEM allocation), 1 MMA issuer, 2-5 converters, 6-9 epilogue.
// Every mbarrier wait is bounded; on a timeout the CTA raises an abort flag, reports
// DGQ_INFO_WAIT_TIMEOUT, waits for copies in flight, frees its tensor memory and returns.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "tc05.cuh"
#include "tgemm.cuh"

namespace {

constexpr int TILE = dgq::TGEMM_TILE;   // 128 x 128 output tile
constexpr int BK = 32;                  // fp32 elements per slice = one 128-byte swizzle row
constexpr int OPERAND_BYTES = TILE * BK * 4;       // 16 KB
constexpr int STAGE_BYTES = 4 * OPERAND_BYTES;     // A hi, A lo, B hi, B lo
constexpr int STAGES = 3;
// The tensor core adds into its fp32 accumulator with truncation, not rounding: measured on
// B200, every 8-deep step of a product shrinks the sum by about 2^-25 of its value, always in
// the same direction, so the relative error of a product grows linearly with the reduction
// length (1e-6 at 128, 3e-5 at 4096 - a hundred times torch's fp32 product).  The reduction is
// therefore cut into chunks of KC_SLICES slices when it is long (the inverse factor's products,
// whose errors are amplified by the conditioning of the matrix); the epilogue warps add the
// chunks' partial sums in registers with ordinary round-to-nearest fp32 additions, which bounds
// the truncation error by that of one chunk whatever the length.  A drain is not free: loads
// from tensor memory queue behind the products already issued, so a chunk costs its products
// plus about 1.3 us (measured: +35 % on a long product with chunks of 128, the price of an
// inverse factor within 3x of LAPACK's fp32 accuracy).  Reductions up to 256 are left in one
// piece (error <= 2e-6); the 512-deep trailing updates of the block quantization take two
// chunks: their terms cancel to a result much smaller than their magnitudes, and with a
// single chunk the truncation showed as code mismatches at K = 11008.
constexpr int KC_SLICES = 4;            // long reductions: 4 slices x 32 = 128 elements of k per chunk
constexpr int KC_SLICES_SHORT = 8;      // reductions of 257..512: two chunks of at most 256
constexpr int CHUNK_FROM_K = 256;       // reductions up to this length stay in tensor memory throughout
constexpr int THREADS = 320;
constexpr uint32_t TMEM_COLS = 256;                // two 128-column accumulators
constexpr uint32_t TMEM_COLS_TS = 512;             // + per stage 32 columns of A hi and 32 of A lo
constexpr uint32_t TS_A_COL0 = 256, TS_A_STAGE_COLS = 64;
constexpr int EPI_STAGE_BYTES = 4 * 32 * 128;        // per epilogue warp: 32 rows x 32 fp32 columns
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + EPI_STAGE_BYTES + 1024 + 256;

struct Control {
  uint64_t full[STAGES], conv[STAGES], empty[STAGES];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort;
};

struct Params {
  float* c; int64_t ldc;
  int m, n, k;
  float alpha, beta;
  int b_is_kn, lo_from_j, hi_from_j, hi_from_i, lower_only;
  int tiles_m, tiles_n, n_tiles;
  int kc_slices;         // slices per chunk of the reduction (chunked kernel)
  int32_t* info;
};

struct TileWork { int ti, tj, k_lo, n_slices; };

__device__ __forceinline__ TileWork decode_tile(const Params& p, int t) {
  TileWork w;
  if (p.lower_only) {
    // row ti holds min(ti + 1, tiles_n) tiles
    int ti = 0, rem = t;
    while (true) {
      int in_row = min(ti + 1, p.tiles_n);
      if (rem < in_row) break;
      rem -= in_row;
      ++ti;
    }
    w.ti = ti; w.tj = rem;
  } else {
    w.ti = t / p.tiles_n;
    w.tj = t - w.ti * p.tiles_n;
  }
  w.k_lo = p.lo_from_j ? w.tj * TILE : 0;
  int k_hi = p.k;
  if (p.hi_from_j) k_hi = min(k_hi, w.tj * TILE + TILE);
  else if (p.hi_from_i) k_hi = min(k_hi, w.ti * TILE + TILE);
  w.n_slices = max(1, (k_hi - w.k_lo + BK - 1) / BK);
  return w;
}

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

template <bool TS /* A operand of the products from tensor memory */,
          bool CHUNKED /* reduction cut into chunks that are summed outside the tensor core */>
__global__ void __launch_bounds__(THREADS, 1)
tgemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* stages = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* epi_stage = stages + (size_t)STAGES * STAGE_BYTES;
  Control* ctl = reinterpret_cast<Control*>(epi_stage + EPI_STAGE_BYTES);
  volatile int* abort_flag = &ctl->abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  dgq_chain_release();   // the next kernel of a chain may start its own set-up

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
    tc05::prefetch_tensormap(&map_a);
    tc05::prefetch_tensormap(&map_b);
  }
  if (warp == 0) {
    __syncwarp();
    tc05::tmem_alloc(&ctl->tmem_base, TS ? TMEM_COLS_TS : TMEM_COLS);
    tc05::tmem_relinquish();
  }
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  // set-up done; global memory is touched only after the predecessor in the stream is complete
  dgq_chain_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
        const TileWork w = decode_tile(p, t);
        for (int s_ = 0; s_ < w.n_slices; ++s_, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!tc05::mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag)) {
            if (p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 11; }
            ok = false;
            break;
          }
          uint8_t* a_hi = stages + (size_t)s * STAGE_BYTES;
          uint8_t* b_hi = a_hi + 2 * OPERAND_BYTES;
          const int k0 = w.k_lo + s_ * BK;
          tc05::mbar_expect_tx(&ctl->full[s], 2 * OPERAND_BYTES);
          tc05::tma_load_2d(a_hi, &map_a, k0, w.ti * TILE, &ctl->full[s]);
          if (!p.b_is_kn) {
            tc05::tma_load_2d(b_hi, &map_b, k0, w.tj * TILE, &ctl->full[s]);
          } else {
#pragma unroll
            for (int pn = 0; pn < TILE / 32; ++pn)
              tc05::tma_load_2d(b_hi + pn * (32 * 128), &map_b, w.tj * TILE + pn * 32, k0,
                                &ctl->full[s]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_nt = tc05::make_instr_desc(tc05::FMT_TF32, false, false, TILE, TILE);
      const uint32_t idesc_nn = tc05::make_instr_desc(tc05::FMT_TF32, false, true, TILE, TILE);
      const uint32_t idesc = p.b_is_kn ? idesc_nn : idesc_nt;
      uint32_t it = 0, ct = 0;   // slices and chunks issued so far
      bool ok = true;
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
        const TileWork w = decode_tile(p, t);
        const int kc_len = CHUNKED ? p.kc_slices : w.n_slices;
        for (int c0s = 0; c0s < w.n_slices && ok; c0s += kc_len, ++ct) {
          // one chunk of the reduction into one of the two accumulators; the epilogue warps
          // drain it while the next chunk goes into the other
          const uint32_t ab = ct & 1, aph = (ct >> 1) & 1;
          if (!tc05::mbar_wait_bounded(&ctl->tmem_empty[ab], aph ^ 1, abort_flag)) {
            if (p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 12; }
            ok = false;
            break;
          }
          tc05::fence_after_sync();
          const uint32_t acc = tmem_base + ab * TILE;
          const int s_end = min(w.n_slices, c0s + kc_len);
          for (int s_ = c0s; s_ < s_end; ++s_, ++it) {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
            if (!tc05::mbar_wait_bounded(&ctl->conv[s], ph, abort_flag)) {
              if (p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 13; }
              ok = false;
              break;
            }
            tc05::fence_after_sync();
            const uint32_t a_hi = tc05::smem_u32(stages + (size_t)s * STAGE_BYTES);
            const uint32_t a_lo = a_hi + OPERAND_BYTES;
            const uint32_t b_hi = a_hi + 2 * OPERAND_BYTES;
            const uint32_t b_lo = a_hi + 3 * OPERAND_BYTES;
#pragma unroll
            for (int k8 = 0; k8 < BK / 8; ++k8) {
              // A (and B in NT form): rows of 128 bytes along k -> step 8 floats = 32 bytes
              // B in NN form: four panels of 32 k-rows x 128 bytes -> step 8 rows = 1024 bytes
              const uint32_t a_off = k8 * 32;
              const uint32_t b_off = p.b_is_kn ? k8 * 1024 : k8 * 32;
              // (n-contiguous fp32 uses the 32-byte-atom swizzle: groups of 4 k-rows, 512 bytes apart)
              const uint32_t b_lbo = p.b_is_kn ? 32 * 128 : 0;
              const uint32_t b_sbo = p.b_is_kn ? 512 : 1024;
              const uint64_t b_layout = p.b_is_kn ? tc05::SWIZZLE_128B_BASE32B : tc05::SWIZZLE_128B;
              const uint64_t da_hi = tc05::make_smem_desc(a_hi + a_off, 0, 1024);
              const uint64_t da_lo = tc05::make_smem_desc(a_lo + a_off, 0, 1024);
              const uint64_t db_hi = tc05::make_smem_desc(b_hi + b_off, b_lbo, b_sbo, b_layout);
              const uint64_t db_lo = tc05::make_smem_desc(b_lo + b_off, b_lbo, b_sbo, b_layout);
              const uint32_t first = (s_ != c0s || k8 != 0) ? 1u : 0u;   // 0: overwrite the accumulator
              if (TS) {
                const uint32_t ta_hi = tmem_base + TS_A_COL0 + s * TS_A_STAGE_COLS + k8 * 8;
                const uint32_t ta_lo = ta_hi + 32;
                tc05::umma_tf32_ts(acc, ta_lo, db_hi, idesc, first);
                tc05::umma_tf32_ts(acc, ta_hi, db_lo, idesc, 1u);
                tc05::umma_tf32_ts(acc, ta_hi, db_hi, idesc, 1u);
              } else {
                tc05::umma_tf32(acc, da_lo, db_hi, idesc, first);
                tc05::umma_tf32(acc, da_hi, db_lo, idesc, 1u);
                tc05::umma_tf32(acc, da_hi, db_hi, idesc, 1u);
              }
            }
            tc05::umma_commit(&ctl->empty[s]);
          }
          if (ok) tc05::umma_commit(&ctl->tmem_full[ab]);
        }
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------------ hi/lo converters
    const int ct = threadIdx.x - 64;  // 0..127
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
      const TileWork w = decode_tile(p, t);
      for (int s_ = 0; s_ < w.n_slices; ++s_, ++it) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
        const bool got = tc05::mbar_wait_bounded(&ctl->full[s], ph, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 14; }
          ok = false;
          break;
        }
        float4* hi_a = reinterpret_cast<float4*>(stages + (size_t)s * STAGE_BYTES);
        float4* lo_a = hi_a + OPERAND_BYTES / 16;
        float4* hi_b = hi_a + 2 * (OPERAND_BYTES / 16);
        float4* lo_b = hi_a + 3 * (OPERAND_BYTES / 16);
        if (TS) {
          // B is split in shared memory as below; A goes to tensor memory: this thread owns row
          // (32 * (warp % 4) + lane) of the tile, reads its 128 bytes (eight 16-byte pieces,
          // XOR-swizzled by the row) and writes 32 columns of hi and 32 of lo.
#pragma unroll
          for (int r = 0; r < OPERAND_BYTES / 16 / 128; ++r) {
            const int idx = ct + r * 128;
            const float4 xb = hi_b[idx];
            float4 hb, lb;
            hb.x = to_tf32(xb.x); hb.y = to_tf32(xb.y); hb.z = to_tf32(xb.z); hb.w = to_tf32(xb.w);
            lb.x = xb.x - hb.x; lb.y = xb.y - hb.y; lb.z = xb.z - hb.z; lb.w = xb.w - hb.w;
            hi_b[idx] = hb; lo_b[idx] = lb;
          }
          const int row = (warp & 3) * 32 + lane;
          uint32_t hi[32], lo[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 v = hi_a[row * 8 + (c ^ (row & 7))];
            const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float h = to_tf32(x[e]);
              hi[4 * c + e] = __float_as_uint(h);
              lo[4 * c + e] = __float_as_uint(x[e] - h);
            }
          }
          const uint32_t ta = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + TS_A_COL0 +
                              s * TS_A_STAGE_COLS;
          tc05::tmem_st_32x32(ta, hi);
          tc05::tmem_st_32x32(ta + 32, lo);
          tc05::tmem_st_wait();
          tc05::fence_before_sync();
        } else {
#pragma unroll
        for (int r = 0; r < OPERAND_BYTES / 16 / 128; ++r) {
          const int idx = ct + r * 128;
          const float4 xa = hi_a[idx], xb = hi_b[idx];
          float4 ha, la, hb, lb;
          ha.x = to_tf32(xa.x); ha.y = to_tf32(xa.y); ha.z = to_tf32(xa.z); ha.w = to_tf32(xa.w);
          la.x = xa.x - ha.x; la.y = xa.y - ha.y; la.z = xa.z - ha.z; la.w = xa.w - ha.w;
          hb.x = to_tf32(xb.x); hb.y = to_tf32(xb.y); hb.z = to_tf32(xb.z); hb.w = to_tf32(xb.w);
          lb.x = xb.x - hb.x; lb.y = xb.y - hb.y; lb.z = xb.z - hb.z; lb.w = xb.w - hb.w;
          hi_a[idx] = ha; lo_a[idx] = la; hi_b[idx] = hb; lo_b[idx] = lb;
        }
        }
        // make the generic-proxy writes visible to the tensor core's (async proxy) reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) tc05::mbar_arrive(&ctl->conv[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    if constexpr (!CHUNKED) {
      // ---- short reductions: the whole sum stays in tensor memory, one drain per tile
      const int q = warp & 3;
      uint32_t lt = 0;
      for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, ++lt) {
        const TileWork w = decode_tile(p, t);
        const uint32_t ab = lt & 1, aph = (lt >> 1) & 1;
        const bool got = tc05::mbar_wait_bounded(&ctl->tmem_full[ab], aph, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0 && p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 15; }
          break;
        }
        tc05::fence_after_sync();
        // Each warp drains its 32 accumulator rows 32 columns at a time: TMEM -> registers
        // (one row per lane) -> this warp's 4 KB of shared memory (16-byte pieces XOR-swizzled
        // by the row so that neither side has bank conflicts) -> global memory with eight
        // lanes per row, i.e. every load/store instruction touches four whole 128-byte lines.
        float4* mine = reinterpret_cast<float4*>(epi_stage) + (warp - 6) * (32 * 8);
        const int row0 = w.ti * TILE + q * 32;
#pragma unroll 1
        for (int chunk = 0; chunk < TILE / 32; ++chunk) {
          const int c0 = w.tj * TILE + chunk * 32;
          const bool live = (row0 < p.m && c0 < p.n);   // uniform across the warp
          // this lane's eight 16-byte pieces of C: rows row0 + 4 it + lane/8, columns c0 + 4 (lane%8)
          const int c = c0 + 4 * (lane & 7);
          float4 old[8];
          bool ok[8];
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = row0 + it * 4 + (lane >> 3);
            // whole float4 inside the matrix (and, for a lower-triangular result, not right of
            // the diagonal); ragged pieces take the scalar path below
            ok[it] = live && row < p.m && c + 3 < p.n && (!p.lower_only || c + 3 <= row);
            old[it] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
          if (p.beta != 0.f) {
            // all loads of the chunk are issued before anything waits on them
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int row = row0 + it * 4 + (lane >> 3);
              if (ok[it]) old[it] = *reinterpret_cast<const float4*>(p.c + (int64_t)row * p.ldc + c);
            }
          }
          uint32_t v[32];
          tc05::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + ab * TILE + chunk * 32, v);
          tc05::tmem_ld_wait();
          if (!live) continue;
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)
            mine[lane * 8 + (c4 ^ (lane & 7))] =
                make_float4(__uint_as_float(v[4 * c4]), __uint_as_float(v[4 * c4 + 1]),
                            __uint_as_float(v[4 * c4 + 2]), __uint_as_float(v[4 * c4 + 3]));
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3), c4 = lane & 7;
            const int row = row0 + rr;
            const float4 acc = mine[rr * 8 + (c4 ^ (rr & 7))];
            float* cp = p.c + (int64_t)row * p.ldc + c;
            if (ok[it]) {
              *reinterpret_cast<float4*>(cp) =
                  make_float4(fmaf(p.alpha, acc.x, p.beta * old[it].x), fmaf(p.alpha, acc.y, p.beta * old[it].y),
                              fmaf(p.alpha, acc.z, p.beta * old[it].z), fmaf(p.alpha, acc.w, p.beta * old[it].w));
            } else if (row < p.m && c < p.n) {
              const float o[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (c + e < p.n && (!p.lower_only || c + e <= row)) {
                  float val = p.alpha * o[e];
                  if (p.beta != 0.f) val += p.beta * cp[e];
                  cp[e] = val;
                }
              }
            }
          }
          __syncwarp();   // the staging rows are rewritten by the next chunk
        }
        tc05::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty[ab]);
      }

    } else {
      // ---- long reductions: chunks of KC_SLICES slices, summed in registers
      const int q = warp & 3;
      uint32_t ct = 0;            // chunks drained so far
      bool alive = true;
      for (int t = blockIdx.x; t < p.n_tiles && alive; t += gridDim.x) {
        const TileWork w = decode_tile(p, t);
        // ---- this thread's row of the tile: the chunks' partial sums are added here
        float acc[TILE];
        const int n_chunks = (w.n_slices + p.kc_slices - 1) / p.kc_slices;
        for (int kc = 0; kc < n_chunks; ++kc, ++ct) {
          const uint32_t ab = ct & 1, aph = (ct >> 1) & 1;
          const bool got = tc05::mbar_wait_bounded(&ctl->tmem_full[ab], aph, abort_flag);
          if (!__all_sync(0xffffffffu, got)) {
            if (lane == 0 && p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 15; }
            alive = false;
            break;
          }
          tc05::fence_after_sync();
          // 16 columns at a time: the row's 128 running sums already take most of the registers
          // (ten warps share the register file, 168 registers per thread at most)
#pragma unroll
          for (int piece = 0; piece < TILE / 16; ++piece) {
            uint32_t v[16];
            tc05::tmem_ld_32x16(tmem_base + ((uint32_t)(q * 32) << 16) + ab * TILE + piece * 16, v);
            tc05::tmem_ld_wait();
            if (kc == 0) {
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[piece * 16 + j] = __uint_as_float(v[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[piece * 16 + j] += __uint_as_float(v[j]);
            }
          }
          tc05::fence_before_sync();
          __syncwarp();
          if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty[ab]);
        }
        if (!alive) break;
        // ---- output.  Each warp writes its 32 rows 32 columns at a time: registers (one row
        // per lane) -> this warp's 4 KB of shared memory (16-byte pieces XOR-swizzled by the row
        // so that neither side has bank conflicts) -> global memory with eight lanes per row,
        // i.e. every load/store instruction touches four whole 128-byte lines.
        float4* mine = reinterpret_cast<float4*>(epi_stage) + (warp - 6) * (32 * 8);
        const int row0 = w.ti * TILE + q * 32;
#pragma unroll
        for (int chunk = 0; chunk < TILE / 32; ++chunk) {
          const int c0 = w.tj * TILE + chunk * 32;
          const bool live = (row0 < p.m && c0 < p.n);   // uniform across the warp
          if (!live) continue;
          // this lane's eight 16-byte pieces of C: rows row0 + 4 it + lane/8, columns c0 + 4 (lane%8)
          const int c = c0 + 4 * (lane & 7);
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)
            mine[lane * 8 + (c4 ^ (lane & 7))] =
                make_float4(acc[chunk * 32 + 4 * c4], acc[chunk * 32 + 4 * c4 + 1],
                            acc[chunk * 32 + 4 * c4 + 2], acc[chunk * 32 + 4 * c4 + 3]);
          __syncwarp();
          // the chunk's 32 sums are in shared memory now and their registers are free: all
          // loads of C are issued before anything waits on them
          float4 old[8];
          bool whole[8];
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = row0 + it * 4 + (lane >> 3);
            // whole float4 inside the matrix (and, for a lower-triangular result, not right of
            // the diagonal); ragged pieces take the scalar path below
            whole[it] = row < p.m && c + 3 < p.n && (!p.lower_only || c + 3 <= row);
            old[it] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
          if (p.beta != 0.f) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int row = row0 + it * 4 + (lane >> 3);
              if (whole[it]) old[it] = *reinterpret_cast<const float4*>(p.c + (int64_t)row * p.ldc + c);
            }
          }
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3), c4 = lane & 7;
            const int row = row0 + rr;
            const float4 a4 = mine[rr * 8 + (c4 ^ (rr & 7))];
            float* cp = p.c + (int64_t)row * p.ldc + c;
            if (whole[it]) {
              *reinterpret_cast<float4*>(cp) =
                  make_float4(fmaf(p.alpha, a4.x, p.beta * old[it].x), fmaf(p.alpha, a4.y, p.beta * old[it].y),
                              fmaf(p.alpha, a4.z, p.beta * old[it].z), fmaf(p.alpha, a4.w, p.beta * old[it].w));
            } else if (row < p.m && c < p.n) {
              const float o[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (c + e < p.n && (!p.lower_only || c + e <= row)) {
                  float val = p.alpha * o[e];
                  if (p.beta != 0.f) val += p.beta * cp[e];
                  cp[e] = val;
                }
              }
            }
          }
          __syncwarp();   // the staging rows are rewritten by the next chunk
        }
      }

    }
  }

  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem_base, TS ? TMEM_COLS_TS : TMEM_COLS);
  }
}

}  // namespace

namespace dgq {

bool tgemm_supported(const TGemmArgs& g) {
  if (g.m <= 0 || g.n <= 0 || g.k <= 0) return false;
  if (!dgq_aligned(g.a, 16) || !dgq_aligned(g.b, 16) || !dgq_aligned(g.c, 16)) return false;
  if (g.lda % 4 || g.ldb % 4 || g.ldc % 4) return false;
  if (g.lo_from_j && (int64_t)(dgq_cdiv(g.n, TILE) - 1) * TILE >= g.k) return false;
  return true;
}

bool tgemm_launch(const TGemmArgs& g, cudaStream_t st) {
  static DgqDeviceOnce once;
  if (!once.run([] {
        const cudaFuncAttribute at = cudaFuncAttributeMaxDynamicSharedMemorySize;
        return cudaFuncSetAttribute(tgemm_kernel<false, false>, at, (int)SMEM_BYTES) == cudaSuccess &&
               cudaFuncSetAttribute(tgemm_kernel<true, false>, at, (int)SMEM_BYTES) == cudaSuccess &&
               cudaFuncSetAttribute(tgemm_kernel<false, true>, at, (int)SMEM_BYTES) == cudaSuccess &&
               cudaFuncSetAttribute(tgemm_kernel<true, true>, at, (int)SMEM_BYTES) == cudaSuccess;
      }))
    return false;
  CUtensorMap map_a, map_b;
  if (!tc05::make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, g.a, (uint64_t)g.m,
                                (uint64_t)g.k, (uint64_t)g.lda * 4, TILE, BK))
    return false;
  const bool ok_b = g.b_is_kn
      ? tc05::make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, g.b, (uint64_t)g.k,
                                 (uint64_t)g.n, (uint64_t)g.ldb * 4, BK, 32,
                                 CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
      : tc05::make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, g.b, (uint64_t)g.n,
                                 (uint64_t)g.k, (uint64_t)g.ldb * 4, TILE, BK);
  if (!ok_b) return false;
  Params p;
  p.c = g.c; p.ldc = g.ldc; p.m = g.m; p.n = g.n; p.k = g.k;
  p.alpha = g.alpha; p.beta = g.beta;
  p.b_is_kn = g.b_is_kn; p.lo_from_j = g.lo_from_j; p.hi_from_j = g.hi_from_j;
  p.hi_from_i = g.hi_from_i; p.lower_only = g.lower_only;
  p.tiles_m = (int)dgq_cdiv(g.m, TILE);
  p.tiles_n = (int)dgq_cdiv(g.n, TILE);
  if (g.lower_only) {
    int64_t cnt = 0;
    for (int ti = 0; ti < p.tiles_m; ++ti) cnt += std::min(ti + 1, p.tiles_n);
    p.n_tiles = (int)cnt;
  } else {
    p.n_tiles = p.tiles_m * p.tiles_n;
  }
  p.info = g.info;
  const unsigned grid = (unsigned)std::min(p.n_tiles, dgq_sm_count());
  // A operand from tensor memory unless DGQ_TGEMM_SS is set to a non-zero value (then both
  // operands of every product come from shared memory)
  static const bool a_from_tmem = [] {
    const char* v = std::getenv("DGQ_TGEMM_SS");
    return !(v && v[0] != '\0' && v[0] != '0');
  }();
  // reductions longer than CHUNK_FROM_K are cut into chunks (see KC_SLICES): up to that length
  // the accumulator's truncation stays below 2e-6 of the result, beyond it it would keep growing
  const bool chunked = g.k > CHUNK_FROM_K;
  p.kc_slices = g.k <= 512 ? KC_SLICES_SHORT : KC_SLICES;
  const dim3 gd(grid), bd(THREADS);
  cudaError_t e;
  if (a_from_tmem)
    e = chunked ? dgq_launch_chained(tgemm_kernel<true, true>, gd, bd, SMEM_BYTES, st, map_a, map_b, p)
                : dgq_launch_chained(tgemm_kernel<true, false>, gd, bd, SMEM_BYTES, st, map_a, map_b, p);
  else
    e = chunked ? dgq_launch_chained(tgemm_kernel<false, true>, gd, bd, SMEM_BYTES, st, map_a, map_b, p)
                : dgq_launch_chained(tgemm_kernel<false, false>, gd, bd, SMEM_BYTES, st, map_a, map_b, p);
  dgq_note_launches(1);
  return e == cudaSuccess && cudaGetLastError() == cudaSuccess;
}

}  // namespace dgq

// ---- C ABI ---------------------------------------------------------------------------------
DGQ_EXPORT int32_t dgq_gemm_f32(const float* a, int64_t lda, const float* b, int64_t ldb,
                                int32_t b_is_kn, float* c, int64_t ldc, int32_t m, int32_t n,
                                int32_t k, float alpha, float beta, int32_t lower_only,
                                int32_t* info, void* stream) {
  DGQ_REQUIRE(a && b && c && m > 0 && n > 0 && k > 0, DGQ_ERR_ARG);
  DGQ_REQUIRE(lda >= k && ldc >= n && ldb >= (b_is_kn ? n : k), DGQ_ERR_ARG);
  int32_t arch = dgq_device_check();
  if (arch != DGQ_OK) return arch;
  dgq::TGemmArgs t = {};
  t.a = a; t.lda = lda; t.b = b; t.ldb = ldb; t.c = c; t.ldc = ldc;
  t.m = m; t.n = n; t.k = k; t.alpha = alpha; t.beta = beta;
  t.b_is_kn = b_is_kn ? 1 : 0; t.lower_only = lower_only ? 1 : 0; t.info = info;
  DGQ_REQUIRE(dgq::tgemm_supported(t), DGQ_ERR_ALIGN);
  return dgq::tgemm_launch(t, dgq_stream(stream)) ? DGQ_OK : DGQ_ERR_LAUNCH;
}
