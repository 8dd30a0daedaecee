// conv2d for callers that must not allocate device memory.
//
// The regular conv2d entry point needs a caller-provided workspace (the channels-last copy
// of the input and the packed weights).  Some callers cannot provide one: a plugin that is
// handed its input and output buffers by another runtime and owns no allocator, or a serving
// loop that forbids allocation after start-up because cudaMalloc synchronises the device and
// can fail under memory pressure.  For them the workspace lives here, in a fixed array in
// device global memory that exists from the moment the library is loaded on a device until
// the process exits.
#include "ftb_host.h"

#include <mutex>

namespace ftb {

// The scratch itself.  Every GPU that loads the library holds FTB_NOALLOC_SCRATCH_BYTES of
// it.  In host code this name is only a handle for the runtime, not a device address: the
// address the kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_conv_scratch[FTB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mutex;
static void* g_scratch_ptr[kMaxDevices];  // device address of g_conv_scratch, per device

// Looks up (once per device, with that device current) where the array lives on the device.
static int scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return FTB_E_NO_DEVICE;
  }
  if (dev < 0 || dev >= kMaxDevices) return FTB_E_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_conv_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_last_cuda_error(static_cast<int>(e));
      return FTB_E_CUDA;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return FTB_OK;
}

}  // namespace ftb

extern "C" int ftb_conv2d_nchw_f32_noalloc(const float* in, const float* weight, const float* bias, float* out,
                                           int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                                           int64_t s, int stride_h, int stride_w, int pad_h, int pad_w,
                                           int dil_h, int dil_w, int groups, const ftb_config* cfg,
                                           int* status, void* stream) {
  using namespace ftb;
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || k <= 0 || r <= 0 || s <= 0 || groups <= 0) return FTB_E_BAD_ARG;
  // Sizes whose workspace does not fit the fixed array are refused before any device work.
  const size_t need = ftb_conv2d_workspace_bytes(n, c, h, w, k, r, s, groups);
  if (need == 0) return FTB_E_BAD_ARG;
  if (need > static_cast<size_t>(FTB_NOALLOC_SCRATCH_BYTES)) return FTB_E_TOO_LARGE;
  int rc = device_ok();
  if (rc) return rc;
  void* scratch = nullptr;
  rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: the pre-pass writes every byte the main kernel
  // reads (padding channels and padded weights included), so what an earlier call left is harmless.
  return conv2d_generic(in, weight, bias, out, n, c, h, w, k, r, s, stride_h, stride_w, pad_h, pad_w, dil_h,
                        dil_w, groups, cfg, scratch, static_cast<size_t>(FTB_NOALLOC_SCRATCH_BYTES), status,
                        stream);
}
