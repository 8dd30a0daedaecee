// Host-side helpers shared by the translation units of the library.
#pragma once
#include "../../include/ftb200.h"
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace ftb {

void set_last_cuda_error(int code);
void count_launch();
// FTB_OK when the current device is compute capability 10.x.
int device_ok();
// SM count of the current device (cached per device).
int sm_count();
// Device address of the library's own status word, used when the caller passes none.
int* fallback_status();

// Options of gemm_generic beyond the plain (batched) product.
struct GemmExtras {
  int a_broadcast;        // 1: every batch entry multiplies the same A (A holds one matrix)
  const float* row_bias;  // fp32 output only: bias[i] added to row i of every result, may be null
};

// `extra_dst`: further buffers (num_extra of them) that receive the same result as `c`.
int gemm_generic(int kind, int out, const void* a, const void* b, void* c, int64_t batch, int64_t m,
                 int64_t n, int64_t k, int trans_a, int trans_b, const ftb_config* user, int* status,
                 void* stream, void* const* extra_dst, int num_extra, const GemmExtras* extras = nullptr);

// CUDA-core GEMM for operands whose pitches or bases break the 16-byte rules of TMA.
int simt_gemm(int kind, int out, const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n,
              int64_t k, int trans_a, int trans_b, void* stream);

int conv2d_generic(const float* in, const float* weight, const float* bias, float* out, int64_t n,
                   int64_t c, int64_t h, int64_t w, int64_t k, int64_t r, int64_t s, int stride_h,
                   int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups,
                   const ftb_config* user, void* workspace, size_t workspace_bytes, int* status,
                   void* stream, float* const* extra_dst = nullptr, int num_extra = 0, int filter_mode = 0,
                   int layout = 0);

}  // namespace ftb
