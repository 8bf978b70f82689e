// Shared host/device helpers for the dgq_* entry points.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <mutex>

#include "dgq.h"

#define DGQ_EXPORT extern "C" __attribute__((visibility("default")))

#define DGQ_REQUIRE(cond, code) \
  do {                          \
    if (!(cond)) return (code); \
  } while (0)

static inline cudaStream_t dgq_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Process-wide count of kernels this library has launched (defined in abi.cu).
void dgq_note_launches(int64_t n);

// Status of the launches an entry point has just made; `launched` is how many.
static inline int32_t dgq_launch_status(int64_t launched = 1) {
  dgq_note_launches(launched);
  return cudaGetLastError() == cudaSuccess ? DGQ_OK : DGQ_ERR_LAUNCH;
}

// False when the environment variable DGQ_SIMT_GEMM is set to a non-zero value: the fp32
// products of the inverse factor and of the trailing update then stay on the CUDA cores.
bool dgq_use_tensor_gemm();

// False when the environment variable DGQ_NO_PDL is set to a non-zero value: the kernels of
// the latency-bound chains (inverse factor, block quantization) are then launched without
// programmatic dependent launch.
bool dgq_use_pdl();

// Programmatic dependent launch for chains of short dependent kernels.  A kernel launched
// through dgq_launch_chained may be scheduled while its predecessor in the stream is still
// running; it does its set-up (shared memory, barriers, tensor memory), and must execute
// dgq_chain_wait() before its first access to global memory: the wait returns when the
// predecessor has completed and its writes are visible.  dgq_chain_release() lets the next
// kernel of the chain be scheduled early in the same way.  Both are no-ops for a kernel that
// was launched the ordinary way.
constexpr unsigned DGQ_CHAIN_EARLY_MAX_CTAS = 16;
#ifdef __CUDACC__
__device__ __forceinline__ void dgq_chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dgq_chain_release() { asm volatile("griddepcontrol.launch_dependents;"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t dgq_launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                             size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // Only small grids are launched early: the CTAs of an early kernel sit on their SMs until its
  // predecessor is done, which is harmless for a handful of CTAs and would shut other streams
  // out of the machine for a grid that covers it.
  const unsigned ctas = grid.x * grid.y * grid.z;
  cfg.numAttrs = (dgq_use_pdl() && ctas <= DGQ_CHAIN_EARLY_MAX_CTAS) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

static inline bool dgq_aligned(const void* p, uintptr_t a) {
  return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0;
}

static inline int64_t dgq_cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- per-device state ----------------------------------------------------------------------
// Function attributes (the dynamic shared-memory limit), occupancy figures and the SM count
// belong to a device, and one process may drive several (one host thread per GPU, or one
// thread that switches devices).  Everything cached is therefore indexed by the current
// device and guarded by a mutex, since entry points may be called from several host threads.
constexpr int DGQ_MAX_DEVICES = 64;

static inline int dgq_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  return (dev >= 0 && dev < DGQ_MAX_DEVICES) ? dev : -1;
}

// Runs `setup` (a callable returning true on success) at most once per device, with that
// device current; returns false if the device is unknown or the set-up failed (it is then
// tried again by the next call).
struct DgqDeviceOnce {
  std::mutex mu;
  bool done[DGQ_MAX_DEVICES] = {};
  template <typename F>
  bool run(F&& setup) {
    const int dev = dgq_current_device();
    if (dev < 0) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (done[dev]) return true;
    if (!setup()) {
      (void)cudaGetLastError();
      return false;
    }
    done[dev] = true;
    return true;
  }
};

// Number of SMs of the current device (148 on B200); looked up once per device (abi.cu).
int dgq_sm_count();

// Grid for a grid-stride kernel: enough CTAs to fill the machine a few times
// over, rounded to a multiple of the SM count, never more than the work needs.
static inline unsigned dgq_grid(int64_t work_items, int threads, int ctas_per_sm = 8) {
  int64_t need = dgq_cdiv(work_items, threads);
  int64_t cap = (int64_t)dgq_sm_count() * ctas_per_sm;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

// ---- the scalar formulas of the path --------------------------------------
// q = clamp(round(w/scale + zero), 0, maxq) with true division and round-half-even.
__device__ __forceinline__ float dgq_quant_level(float w, float scale, float zero, float maxq) {
  float q = rintf(__fadd_rn(__fdiv_rn(w, scale), zero));
  return fminf(fmaxf(q, 0.f), maxq);
}
__device__ __forceinline__ float dgq_dequant_level(float q, float scale, float zero) {
  return __fmul_rn(__fsub_rn(q, zero), scale);
}
// scale = (max-min)/maxq (1 if zero), zero = round(-min/scale)
__device__ __forceinline__ void dgq_scale_zero(float mn, float mx, float maxq, float& scale,
                                               float& zero) {
  float s = __fdiv_rn(__fsub_rn(mx, mn), maxq);
  if (s == 0.f) s = 1.f;
  scale = s;
  zero = rintf(__fdiv_rn(-mn, s));
}

template <typename T>
__device__ __forceinline__ float dgq_to_float(T v);
template <>
__device__ __forceinline__ float dgq_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float dgq_to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float dgq_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T>
__device__ __forceinline__ T dgq_from_float(float v);
template <>
__device__ __forceinline__ float dgq_from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half dgq_from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 dgq_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
