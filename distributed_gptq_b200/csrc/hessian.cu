// Hessian accumulation  H += alpha * X^T X  on the sm_100a tensor cores.
//
// X is (T tokens, K features) bf16 row-major, so both MMA operands of X^T X are
// "MN-major": a 64-feature x BK-token box of X is fetched by TMA with the
// 128-byte swizzle and used, unchanged, as a panel of A (features = M) or of B
// (features = N); the token axis is the reduction axis.
//
// Work decomposition: H is cut into 256 x 256 macro-tiles, only those on or above
// the diagonal are computed, and the token axis is optionally cut into `splits`
// ranges.  A work item (tile, range) is owned by one CTA, which keeps the whole
// 256 x 256 fp32 accumulator in tensor memory (2 halves of 128 lanes x 256
// columns = all 512 columns), streams its token range through a 3-stage TMA
// pipeline and finally adds the tile into H - and its transpose into the mirrored
// position - with fp32 reductions.  CTAs are persistent: grid = SM count, work
// items are taken round-robin, ordered so that CTAs running at the same time read
// the same token range (shared through L2).
//
// Warp roles (10 warps): 0 = TMA producer, 1 = MMA issuer, 2..9 = epilogue
// (warp w reads TMEM lane quadrant w % 4 of accumulator half (w - 2) / 4).
// Every wait on an mbarrier is bounded; when one runs out the CTA raises an abort
// flag, reports DGQ_INFO_WAIT_TIMEOUT, lets its copies land, frees its tensor
// memory and returns.
#include <algorithm>

#include "common.cuh"
#include "tc05.cuh"

namespace {

constexpr int BK = 64;                          // tokens per pipeline stage
constexpr int TILE = 256;                       // macro-tile edge (features)
constexpr int PANEL = 64;                       // features per TMA box (128 bytes of bf16)
constexpr int PANEL_BYTES = BK * 128;           // one box in shared memory
constexpr int OPERAND_BYTES = (TILE / PANEL) * PANEL_BYTES;  // 256 features x BK tokens
constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;  // A and B operands
constexpr int STAGES = 3;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int UMMA_K = 16;                      // bf16 elements along K per instruction
constexpr uint32_t TMEM_COLS = 512;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;

struct Control {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  uint32_t tmem_base;
  int abort;
};

struct Params {
  float* H;
  int64_t ldh;
  int K;
  int64_t T;
  float alpha;
  int P;                 // macro-tiles per dimension
  int n_tiles;           // P (P + 1) / 2
  int n_work;            // n_tiles * splits
  int64_t split_tokens;  // tokens per range, a multiple of BK
  int32_t* info;
  int mirror;            // 1: also add the transposed tile below the diagonal
};

__device__ __forceinline__ void decode_work(const Params& p, int w, int& I, int& J, int64_t& t0,
                                            int& nkb) {
  int split = w / p.n_tiles;
  int rem = w - split * p.n_tiles;
  I = 0;
  while (rem >= p.P - I) {
    rem -= p.P - I;
    ++I;
  }
  J = I + rem;
  t0 = (int64_t)split * p.split_tokens;
  int64_t t1 = min(p.T, t0 + p.split_tokens);
  nkb = (int)((t1 - t0 + BK - 1) / BK);
}

__global__ void __launch_bounds__(THREADS, 1)
hessian_syrk_kernel(const __grid_constant__ CUtensorMap tmap, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // the 128-byte swizzle pattern repeats every 1024 bytes: stage bases must be 1024-aligned
  uint8_t* stages = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Control* ctl = reinterpret_cast<Control*>(stages + (size_t)STAGES * STAGE_BYTES);
  volatile int* abort_flag = &ctl->abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      tc05::mbar_init(&ctl->full[s], 1);
      tc05::mbar_init(&ctl->empty[s], 1);
    }
    tc05::mbar_init(&ctl->tmem_full, 1);
    tc05::mbar_init(&ctl->tmem_empty, EPI_WARPS);
    ctl->abort = 0;
    tc05::fence_mbar_init();
    tc05::prefetch_tensormap(&tmap);
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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.n_work && ok; w += gridDim.x) {
        int I, J, nkb;
        int64_t t0;
        decode_work(p, w, I, J, t0, nkb);
        const bool diag = (I == J);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!tc05::mbar_wait_bounded(&ctl->empty[s], ph ^ 1, abort_flag)) {
            if (p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 1; }
            ok = false;
            break;
          }
          uint8_t* a = stages + (size_t)s * STAGE_BYTES;
          uint8_t* b = a + OPERAND_BYTES;
          tc05::mbar_expect_tx(&ctl->full[s], diag ? OPERAND_BYTES : STAGE_BYTES);
          const int32_t tok = (int32_t)(t0 + (int64_t)kb * BK);
#pragma unroll
          for (int c = 0; c < TILE / PANEL; ++c)
            tc05::tma_load_2d(a + c * PANEL_BYTES, &tmap, I * TILE + c * PANEL, tok, &ctl->full[s]);
          if (!diag) {
#pragma unroll
            for (int c = 0; c < TILE / PANEL; ++c)
              tc05::tma_load_2d(b + c * PANEL_BYTES, &tmap, J * TILE + c * PANEL, tok,
                                &ctl->full[s]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = tc05::make_instr_desc(tc05::FMT_BF16, true, true, 128, 256);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.n_work && ok; w += gridDim.x, ++lt) {
        int I, J, nkb;
        int64_t t0;
        decode_work(p, w, I, J, t0, nkb);
        const bool diag = (I == J);
        // the epilogue of the previous tile must have drained the accumulator
        if (!tc05::mbar_wait_bounded(&ctl->tmem_empty, (lt & 1) ^ 1, abort_flag)) {
          if (p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 2; }
          break;
        }
        tc05::fence_after_sync();
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!tc05::mbar_wait_bounded(&ctl->full[s], ph, abort_flag)) {
            if (p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 3; }
            ok = false;
            break;
          }
          tc05::fence_after_sync();
          const uint32_t a_base = tc05::smem_u32(stages + (size_t)s * STAGE_BYTES);
          const uint32_t b_base = diag ? a_base : a_base + OPERAND_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // 16 tokens = 16 rows of 128 bytes further down every panel
            const uint32_t koff = k * UMMA_K * 128;
            const uint64_t bdesc = tc05::make_smem_desc(b_base + koff, PANEL_BYTES, 1024);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint64_t adesc =
                  tc05::make_smem_desc(a_base + h * 2 * PANEL_BYTES + koff, PANEL_BYTES, 1024);
              tc05::umma_bf16(tmem_base + h * 256, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          tc05::umma_commit(&ctl->empty[s]);  // the stage is free once these MMAs retire
        }
        if (ok) tc05::umma_commit(&ctl->tmem_full);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue
    const int e = warp - 2;
    const int h = e >> 2;         // accumulator half (rows 128 h .. 128 h + 127 of the tile)
    const int q = warp & 3;       // TMEM lane quadrant this warp may read
    uint32_t lt = 0;
    for (int w = blockIdx.x; w < p.n_work; w += gridDim.x, ++lt) {
      int I, J, nkb;
      int64_t t0;
      decode_work(p, w, I, J, t0, nkb);
      // every lane waits (each needs the barrier's acquire), then the warp agrees on
      // the outcome so that the .aligned TMEM loads below are never partially taken
      const bool got = tc05::mbar_wait_bounded(&ctl->tmem_full, lt & 1, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0 && p.info) { p.info[0] = DGQ_INFO_WAIT_TIMEOUT; p.info[1] = 4; }
        break;
      }
      tc05::fence_after_sync();
      const int r = I * TILE + h * 128 + q * 32 + lane;
      const bool diag = (I == J);
      float* Hrow = p.H + (int64_t)r * p.ldh;
#pragma unroll 1
      for (int chunk = 0; chunk < TILE / 32; ++chunk) {
        uint32_t v[32];
        tc05::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + h * 256 + chunk * 32, v);
        tc05::tmem_ld_wait();
        const int c0 = J * TILE + chunk * 32;
        if (c0 >= p.K) continue;  // uniform across the warp
        if (!diag) {
          // strictly above the diagonal: c > r for every element of the tile
          if (r < p.K) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (c0 + j < p.K)
                tc05::red_add_v4_f32(Hrow + c0 + j, p.alpha * __uint_as_float(v[j]),
                                     p.alpha * __uint_as_float(v[j + 1]),
                                     p.alpha * __uint_as_float(v[j + 2]),
                                     p.alpha * __uint_as_float(v[j + 3]));
            }
          }
          // mirrored element H[c][r]: consecutive lanes hold consecutive r -> coalesced
          if (p.mirror) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (r < p.K && c0 + j < p.K)
                tc05::red_add_f32(p.H + (int64_t)(c0 + j) * p.ldh + r,
                                  p.alpha * __uint_as_float(v[j]));
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int c = c0 + j;
            if (r < p.K && c < p.K && c >= r) {
              const float val = p.alpha * __uint_as_float(v[j]);
              tc05::red_add_f32(Hrow + c, val);
              if (c > r && p.mirror) tc05::red_add_f32(p.H + (int64_t)c * p.ldh + r, val);
            }
          }
        }
      }
      tc05::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc05::mbar_arrive(&ctl->tmem_empty);
    }
  }

  // ---- teardown: everyone meets here, also after an abort
  __syncthreads();
  if (*abort_flag) {
    // give copies and MMAs that may still be in flight time to land before the
    // shared and tensor memory they target is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc05::fence_after_sync();
    tc05::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Chooses how many token ranges to cut the work into: the fewest that fills the
// last wave of CTAs well, keeping every range at least `min_tokens` long.
int choose_splits(int n_tiles, int64_t T, int sms) {
  // Cost of a split count s, in token-times of one tile: every wave of CTAs streams
  // T/s tokens and then pays one epilogue, which is not overlapped with the next tile
  // and costs about as much as streaming EPILOGUE_TOKENS tokens (measured on B200).
  const double EPILOGUE_TOKENS = 1700.0;
  const int64_t min_tokens = 2048;
  int max_splits = (int)std::max<int64_t>(1, T / min_tokens);
  if (max_splits > 64) max_splits = 64;
  int best = 1;
  double best_cost = 0.0;
  for (int s = 1; s <= max_splits; ++s) {
    const int64_t items = (int64_t)n_tiles * s;
    const int64_t waves = dgq_cdiv(items, sms);
    const double cost = (double)waves * ((double)T / s + EPILOGUE_TOKENS);
    if (s == 1 || cost < 0.97 * best_cost) {  // prefer fewer splits unless clearly better
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

}  // namespace

namespace {
int32_t hessian_accum(const void* X, int64_t T, int32_t K, int64_t ldx, float* H, int64_t ldh,
                      float alpha, int32_t splits, int32_t* info, void* stream, int mirror) {
  DGQ_REQUIRE(X && H && T > 0 && K >= 8 && ldx >= K && ldh >= K && splits >= 0, DGQ_ERR_ARG);
  DGQ_REQUIRE(T < (1ll << 31), DGQ_ERR_SIZE);
  DGQ_REQUIRE(dgq_aligned(X, 16) && dgq_aligned(H, 16) && ldx % 8 == 0 && ldh % 4 == 0 && K % 8 == 0,
              DGQ_ERR_ALIGN);
  int32_t arch = dgq_device_check();
  if (arch != DGQ_OK) return arch;

  static DgqDeviceOnce once;
  if (!once.run([] {
        return cudaFuncSetAttribute(hessian_syrk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)SMEM_BYTES) == cudaSuccess;
      }))
    return DGQ_ERR_LAUNCH;

  CUtensorMap tmap;
  if (!tc05::make_tensor_map_2d(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, (uint64_t)T,
                                (uint64_t)K, (uint64_t)ldx * 2, BK, PANEL))
    return DGQ_ERR_LAUNCH;

  Params p;
  p.H = H;
  p.ldh = ldh;
  p.K = K;
  p.T = T;
  p.alpha = alpha;
  p.P = (int)dgq_cdiv(K, TILE);
  p.n_tiles = p.P * (p.P + 1) / 2;
  const int sms = dgq_sm_count();
  int s = splits > 0 ? splits : choose_splits(p.n_tiles, T, sms);
  int64_t kblocks = dgq_cdiv(T, BK);
  p.split_tokens = dgq_cdiv(kblocks, s) * BK;
  s = (int)dgq_cdiv(T, p.split_tokens);  // drop ranges that would be empty
  p.n_work = p.n_tiles * s;
  p.info = info;
  p.mirror = mirror;

  // Work items are dealt round robin, so the kernel lasts as long as the CTA with the most
  // items: the smallest grid with that many rounds is as fast as one CTA per SM and leaves
  // the other SMs to kernels on other streams (K = 11008: 946 items, 7 rounds, 136 CTAs).
  const int64_t rounds = dgq_cdiv(p.n_work, sms);
  unsigned grid = (unsigned)dgq_cdiv(p.n_work, rounds);
  hessian_syrk_kernel<<<grid, THREADS, SMEM_BYTES, dgq_stream(stream)>>>(tmap, p);
  return dgq_launch_status();
}

// Copies the part of H above the diagonal to below it (32 x 32 tiles through shared memory,
// so that both the reads and the writes are coalesced).
__global__ void __launch_bounds__(256)
mirror_upper_kernel(float* __restrict__ H, int64_t ldh, int K) {
  __shared__ float tile[32][33];
  const int nt = (K + 31) / 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int64_t t = blockIdx.x; t < (int64_t)nt * nt; t += gridDim.x) {
    const int bi = (int)(t / nt), bj = (int)(t % nt);
    if (bj < bi) continue;                                   // tiles on or above the diagonal
    for (int y = ty; y < 32; y += 8) {
      const int r = bi * 32 + y, c = bj * 32 + tx;
      tile[y][tx] = (r < K && c < K) ? H[(int64_t)r * ldh + c] : 0.f;
    }
    __syncthreads();
    for (int y = ty; y < 32; y += 8) {
      const int r = bj * 32 + y, c = bi * 32 + tx;           // destination H[r][c] = source[c'][r']
      if (r < K && c < K && r > c) H[(int64_t)r * ldh + c] = tile[tx][y];
    }
    __syncthreads();
  }
}
}  // namespace

DGQ_EXPORT int32_t dgq_hessian_accum(const void* X, int64_t T, int32_t K, int64_t ldx, float* H,
                                     int64_t ldh, float alpha, int32_t splits, int32_t* info,
                                     void* stream) {
  return hessian_accum(X, T, K, ldx, H, ldh, alpha, splits, info, stream, 1);
}

DGQ_EXPORT int32_t dgq_hessian_accum_upper(const void* X, int64_t T, int32_t K, int64_t ldx,
                                           float* H, int64_t ldh, float alpha, int32_t splits,
                                           int32_t* info, void* stream) {
  return hessian_accum(X, T, K, ldx, H, ldh, alpha, splits, info, stream, 0);
}

DGQ_EXPORT int32_t dgq_hessian_mirror(float* H, int32_t K, int64_t ldh, void* stream) {
  DGQ_REQUIRE(H && K > 0 && ldh >= K, DGQ_ERR_ARG);
  const int64_t nt = dgq_cdiv(K, 32);
  const unsigned grid = (unsigned)std::min<int64_t>(nt * nt, (int64_t)dgq_sm_count() * 16);
  mirror_upper_kernel<<<grid, 256, 0, dgq_stream(stream)>>>(H, ldh, K);
  return dgq_launch_status();
}
