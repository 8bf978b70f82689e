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

int dgq_sm_count() {
  static std::mutex mu;
  static int cached[DGQ_MAX_DEVICES] = {};
  const int dev = dgq_current_device();
  if (dev < 0) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return 148;
    }
    cached[dev] = n;
  }
  return cached[dev];
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
  static std::mutex mu;
  static int8_t known[DGQ_MAX_DEVICES] = {};   // 0 = not asked yet, 1 = sm_10x, 2 = other
  const int dev = dgq_current_device();
  if (dev < 0) return DGQ_ERR_ARCH;
  std::lock_guard<std::mutex> lock(mu);
  if (known[dev] == 0) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
      (void)cudaGetLastError();
      return DGQ_ERR_ARCH;
    }
    known[dev] = (major == 10) ? 1 : 2;
  }
  return known[dev] == 1 ? DGQ_OK : DGQ_ERR_ARCH;
}
