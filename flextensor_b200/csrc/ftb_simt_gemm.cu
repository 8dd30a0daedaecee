// CUDA-core GEMM for operands the TMA path cannot address.
//
// A tiled TMA copy needs 16-byte aligned base addresses and row pitches; a GEMM whose K (or N,
// for an N-contiguous B) times the element size is not a multiple of 16 bytes - e.g. a bf16
// batch with N = 28 - cannot be fed to the tensor-core kernel without re-laying it out.  Those
// shapes run here instead: a plain shared-memory tiled kernel, 64 x 64 outputs per CTA, 4 x 4
// per thread, fp32 (or int32) accumulation, any transposition through element strides, every
// access bounds-checked.  It is a correctness path, an order of magnitude slower than the
// tcgen05 kernel, and is only ever chosen when the alignment rules fail.
#include "ftb_host.h"

#include <cuda_bf16.h>
#include <type_traits>

namespace ftb {

template <typename T>
__device__ __forceinline__ float to_acc_f(T v);
template <>
__device__ __forceinline__ float to_acc_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_acc_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename TIn, typename TAcc, typename TOut>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const TIn* __restrict__ A, const TIn* __restrict__ B, TOut* __restrict__ C, int M, int N, int K,
                 long long a_rs, long long a_cs, long long b_rs, long long b_cs, long long a_bs,
                 long long b_bs, long long c_bs) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ TAcc As[TK][TM + 1];
  __shared__ TAcc Bs[TK][TN + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const TIn* Ab = A + blockIdx.z * a_bs;
  const TIn* Bb = B + blockIdx.z * b_bs;
  TOut* Cb = C + blockIdx.z * c_bs;
  TAcc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = TAcc(0);

  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int m = i % TM, k = i / TM;
      const int gm = m0 + m, gk = k0 + k;
      TAcc v = TAcc(0);
      if (gm < M && gk < K) {
        if constexpr (sizeof(TAcc) == 4 && !std::is_integral<TAcc>::value) v = to_acc_f<TIn>(Ab[gm * a_rs + gk * a_cs]);
        else v = static_cast<TAcc>(Ab[gm * a_rs + gk * a_cs]);
      }
      As[k][m] = v;
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      const int n = i % TN, k = i / TN;
      const int gn = n0 + n, gk = k0 + k;
      TAcc v = TAcc(0);
      if (gn < N && gk < K) {
        if constexpr (sizeof(TAcc) == 4 && !std::is_integral<TAcc>::value) v = to_acc_f<TIn>(Bb[gk * b_rs + gn * b_cs]);
        else v = static_cast<TAcc>(Bb[gk * b_rs + gn * b_cs]);
      }
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      TAcc a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < M && gn < N) {
        if constexpr (std::is_same<TOut, __nv_bfloat16>::value) Cb[static_cast<long long>(gm) * N + gn] = __float2bfloat16_rn(acc[i][j]);
        else Cb[static_cast<long long>(gm) * N + gn] = static_cast<TOut>(acc[i][j]);
      }
    }
}

template <typename TIn, typename TAcc, typename TOut>
static int launch_simt(const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                       int trans_a, int trans_b, cudaStream_t stream) {
  const long long a_rs = trans_a ? 1 : k, a_cs = trans_a ? m : 1;  // A(i,k): [M,K] or stored [K,M]
  const long long b_rs = trans_b ? 1 : n, b_cs = trans_b ? k : 1;  // B(k,j): [K,N] or stored [N,K]
  dim3 grid(static_cast<unsigned>((n + 63) / 64), static_cast<unsigned>((m + 63) / 64), static_cast<unsigned>(batch));
  if (grid.y > 65535 || grid.z > 65535) return FTB_E_TOO_LARGE;
  simt_gemm_kernel<TIn, TAcc, TOut><<<grid, 256, 0, stream>>>(
      static_cast<const TIn*>(a), static_cast<const TIn*>(b), static_cast<TOut*>(c), static_cast<int>(m),
      static_cast<int>(n), static_cast<int>(k), a_rs, a_cs, b_rs, b_cs, m * k, k * n, m * n);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return FTB_E_CUDA;
  }
  return FTB_OK;
}

// kind: 0 bf16, 1 fp32, 2 int8; out: 0 bf16, 1 fp32, 2 int32 (the codes of the tensor-core path)
int simt_gemm(int kind, int out, const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n,
              int64_t k, int trans_a, int trans_b, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (kind == 0 && out == 0) return launch_simt<__nv_bfloat16, float, __nv_bfloat16>(a, b, c, batch, m, n, k, trans_a, trans_b, stream);
  if (kind == 0 && out == 1) return launch_simt<__nv_bfloat16, float, float>(a, b, c, batch, m, n, k, trans_a, trans_b, stream);
  if (kind == 1 && out == 1) return launch_simt<float, float, float>(a, b, c, batch, m, n, k, trans_a, trans_b, stream);
  if (kind == 2 && out == 2) return launch_simt<int8_t, int32_t, int32_t>(a, b, c, batch, m, n, k, trans_a, trans_b, stream);
  return FTB_E_BAD_ARG;
}

}  // namespace ftb
