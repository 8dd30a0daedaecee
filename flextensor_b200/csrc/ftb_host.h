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

int gemm_generic(int kind, int out, const void* a, const void* b, void* c, int64_t batch, int64_t m,
                 int64_t n, int64_t k, int trans_a, int trans_b, const ftb_config* user, int* status,
                 void* stream);

}  // namespace ftb
