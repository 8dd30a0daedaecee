// Process-wide state of the library (error code, launch counter, device facts) and
// the small query entry points of the C ABI.
#include "ftb_host.h"
#include "ftb_ptx.cuh"

#include <atomic>
#include <mutex>

namespace ftb {

static std::atomic<int> g_last_cuda_error{0};
static std::atomic<long long> g_launches{0};
__device__ int g_status_word;  // receives FTB_DEV_* bits when the caller passes no status pointer

void set_last_cuda_error(int code) { g_last_cuda_error.store(code); }
void count_launch() { g_launches.fetch_add(1); }

constexpr int kMaxDevices = 64;
static std::mutex g_dev_mutex;
static int g_dev_major[kMaxDevices];
static int g_dev_sms[kMaxDevices];
static int* g_dev_status[kMaxDevices];
static bool g_dev_known[kMaxDevices];

static int probe_device(int* dev_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return FTB_E_NO_DEVICE;
  }
  if (dev < 0 || dev >= kMaxDevices) return FTB_E_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!g_dev_known[dev]) {
    int major = 0, sms = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    void* addr = nullptr;
    if (e == cudaSuccess && major == 10) e = cudaGetSymbolAddress(&addr, g_status_word);
    if (e != cudaSuccess) {
      set_last_cuda_error(static_cast<int>(e));
      return FTB_E_CUDA;
    }
    g_dev_major[dev] = major;
    g_dev_sms[dev] = sms;
    g_dev_status[dev] = static_cast<int*>(addr);
    g_dev_known[dev] = true;
  }
  *dev_out = dev;
  return FTB_OK;
}

int device_ok() {
  int dev;
  int rc = probe_device(&dev);
  if (rc) return rc;
  return g_dev_major[dev] == 10 ? FTB_OK : FTB_E_NO_DEVICE;
}

int sm_count() {
  int dev;
  if (probe_device(&dev)) return 1;
  return g_dev_sms[dev] > 0 ? g_dev_sms[dev] : 1;
}

int* fallback_status() {
  int dev;
  if (probe_device(&dev)) return nullptr;
  return g_dev_status[dev];
}

// One thread waits, with the kernels' own bounded wait, on a barrier that nothing ever
// completes: the wait must run out, set its status bit and return normally.
__global__ void selftest_wait_kernel(int* status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
    if (!mbar_wait(smem_u32(&bar), 0, &abort_flag)) atomicOr(status, FTB_DEV_WAIT_FULL);
  }
}

}  // namespace ftb

extern "C" {

int ftb_selftest_bounded_wait(int* status, void* stream) {
  if (!status) return FTB_E_BAD_ARG;
  int rc = ftb::device_ok();
  if (rc) return rc;
  ftb::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status);
  ftb::count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    ftb::set_last_cuda_error(static_cast<int>(e));
    return FTB_E_CUDA;
  }
  return FTB_OK;
}

int ftb_version(void) { return FTB_VERSION; }

const char* ftb_strerror(int code) {
  switch (code) {
    case FTB_OK: return "ok";
    case FTB_E_BAD_ARG: return "bad argument";
    case FTB_E_UNSUPPORTED: return "unsupported shape or alignment";
    case FTB_E_BAD_CONFIG: return "bad kernel configuration";
    case FTB_E_WORKSPACE: return "workspace missing, misaligned or too small";
    case FTB_E_CUDA: return "CUDA call failed";
    case FTB_E_NO_DEVICE: return "no sm_100 device is current";
    case FTB_E_TOO_LARGE: return "size beyond the supported maximum";
    default: return "unknown error";
  }
}

int ftb_last_cuda_error(void) { return ftb::g_last_cuda_error.load(); }

int ftb_device_check(void) { return ftb::device_ok(); }

int64_t ftb_launch_count(void) { return ftb::g_launches.load(); }

int ftb_validate(int op, const ftb_config* cfg, int64_t m, int64_t n, int64_t k) {
  if (op < 0 || op > 4) return FTB_E_BAD_ARG;
  if (m <= 0 || n <= 0 || k <= 0) return FTB_E_BAD_ARG;
  if (!cfg) return FTB_OK;
  if (op == 4) {
    if (cfg->tile_h < 0 || cfg->tile_h > 256) return FTB_E_BAD_CONFIG;
    if (cfg->threads != 0 && (cfg->threads < 32 || cfg->threads > 1024 || cfg->threads % 32)) return FTB_E_BAD_CONFIG;
    return FTB_OK;
  }
  const int esize = op == 1 ? 2 : (op == 2 ? 1 : 4);
  const bool split3 = (op == 0 || op == 3) && cfg->fp32_mode == 1;
  if (cfg->fp32_mode < 0 || cfg->fp32_mode > 1) return FTB_E_BAD_CONFIG;
  if (cfg->tile_n == 512) {
    // 256 x 512 tile of a CTA pair: plain GEMMs only
    if (cfg->cluster != 2 || op == 3 || split3) return FTB_E_BAD_CONFIG;
  } else if (cfg->tile_n != 0 && cfg->tile_n != 32 && cfg->tile_n != 64 && cfg->tile_n != 128 && cfg->tile_n != 256) {
    return FTB_E_BAD_CONFIG;
  }
  if (cfg->stages != 0 && (cfg->stages < 2 || cfg->stages > 8)) return FTB_E_BAD_CONFIG;
  if (cfg->cluster < 0 || cfg->cluster > 2) return FTB_E_BAD_CONFIG;
  if (cfg->cluster == 2 && split3) return FTB_E_BAD_CONFIG;
  if (cfg->cluster == 2 && cfg->tile_n != 0 && cfg->tile_n < 64) return FTB_E_BAD_CONFIG;
  if (cfg->tile_n != 0 && cfg->stages != 0) {
    const size_t per_cta = static_cast<size_t>(cfg->tile_n) / (cfg->cluster == 2 ? 2 : 1);
    // GEMM kernels also hold two 16 KB output slabs for the bulk-store epilogue
    const size_t smem = static_cast<size_t>(cfg->stages) * (16384 + per_cta * 128) * (split3 ? 2 : 1) + 1024 +
                        (op == 3 ? 0 : 32768);
    if (smem > 227 * 1024 - 2048) return FTB_E_BAD_CONFIG;
  }
  if (cfg->raster < 0 || cfg->raster > 3 || cfg->group_m < 0) return FTB_E_BAD_CONFIG;
  const int64_t kblk = 128 / esize;
  const int64_t num_kb = (k + kblk - 1) / kblk;
  if (cfg->split_k != 0 && (cfg->split_k < 1 || cfg->split_k > 64 || cfg->split_k > num_kb)) return FTB_E_BAD_CONFIG;
  if (cfg->split_k > 1 && (op == 1 || op == 2)) return FTB_E_BAD_CONFIG;
  if (cfg->ctas < 0) return FTB_E_BAD_CONFIG;
  return FTB_OK;
}

}  // extern "C"
