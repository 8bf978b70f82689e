// Library-wide entry points: version, status strings, device check.
#include <atomic>
#include <cstdlib>

#include "common.cuh"

static std::atomic<int64_t> g_launches{0};
void dgq_note_launches(int64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

bool dgq_use_tensor_gemm() {
  const char* e = std::getenv("DGQ_SIMT_GEMM");
  return !(e && e[0] != '\0' && e[0] != '0');
}

bool dgq_use_pdl() {
  static const bool on = [] {
    const char* e = std::getenv("DGQ_NO_PDL");
    return !(e && e[0] != '\0' && e[0] != '0');
  }();
  return on;
}

DGQ_EXPORT int64_t dgq_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

DGQ_EXPORT int32_t dgq_version(void) { return 100; }

DGQ_EXPORT const char* dgq_status_string(int32_t status) {
  switch (status) {
    case DGQ_OK: return "ok";
    case DGQ_ERR_ARG: return "invalid argument (null pointer, non-positive size or unknown enum)";
    case DGQ_ERR_ALIGN: return "pointer or leading dimension not aligned as documented";
    case DGQ_ERR_WORKSPACE: return "workspace too small";
    case DGQ_ERR_ARCH: return "the current CUDA device is not compute capability 10.x (B200)";
    case DGQ_ERR_LAUNCH: return "the CUDA runtime refused a launch or a set-up call";
    case DGQ_ERR_UNSUPPORTED: return "request outside what this build implements";
    case DGQ_ERR_SIZE: return "size beyond a documented maximum";
    default: return "unknown status";
  }
}

DGQ_EXPORT int32_t dgq_device_check(void) {
  static int cached_dev = -1;
  static int32_t cached = DGQ_ERR_ARCH;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return DGQ_ERR_ARCH;
  }
  if (dev == cached_dev) return cached;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return DGQ_ERR_ARCH;
  }
  cached_dev = dev;
  cached = (major == 10) ? DGQ_OK : DGQ_ERR_ARCH;
  return cached;
}
