// Depthwise conv2d NCHW fp32: a bandwidth-bound stencil, no tensor cores.
//
// One CTA owns a strip of `strip_h` output rows of one input plane (n, c) and produces
// the strip for all `factor` output channels fed by that plane.  The input rows the
// strip needs are staged once in shared memory with 16-byte loads, zero padding is
// written into the staging tile (the reference's separate padding op disappears),
// each thread then produces four adjacent outputs of a row and stores them as one
// 16-byte vector.  Algorithmic traffic: input read once, output written once.
#include "ftb_host.h"

namespace ftb {

constexpr int kMaxTaps = 49;

struct DwParams {
  const float* in;
  const float* w;
  const float* bias;
  float* out;
  int N, C, H, W, F, R, S, P, Q;
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int strip_h, strips;  // output rows per CTA, strips per plane
  int tile_rows;        // input rows staged per strip
  int tile_pitch;       // floats per staged row (multiple of 4)
  int lead;             // staged column of input column 0 (multiple of 4, >= pad_w)
  // Further buffers that receive the same result (same layout as `out`): this GPU's memory or a
  // peer GPU's mapped buffer.  The batch-sharded path uses them to place a rank's slice in every
  // rank's gathered output with plain stores.
  float* extra[7];
  int num_extra;
  int relu;  // clamp the result at zero after the bias
};

// Byte distance from `out` to the d-th extra destination is the same for every element.
// MULTI = false is the common case (one destination, no clamp): its kernels carry none of the
// extra code or registers.
template <bool MULTI>
__device__ __forceinline__ void dw_store4(const DwParams& p, float* dst, float4 v) {
  if constexpr (!MULTI) {
    *reinterpret_cast<float4*>(dst) = v;
    return;
  }
  if (p.relu) v = make_float4(fmaxf(v.x, 0.f), fmaxf(v.y, 0.f), fmaxf(v.z, 0.f), fmaxf(v.w, 0.f));
  *reinterpret_cast<float4*>(dst) = v;
  const long long off = dst - p.out;
  for (int d = 0; d < p.num_extra; ++d) *reinterpret_cast<float4*>(p.extra[d] + off) = v;
}
template <bool MULTI>
__device__ __forceinline__ void dw_store1(const DwParams& p, float* dst, float v) {
  if constexpr (!MULTI) {
    *dst = v;
    return;
  }
  if (p.relu) v = fmaxf(v, 0.f);
  *dst = v;
  const long long off = dst - p.out;
  for (int d = 0; d < p.num_extra; ++d) p.extra[d][off] = v;
}

// Staging tile: row i holds input row (h_in0 + i); column (lead + x) holds input column x.
template <bool K3S1, bool MULTI>
__global__ void dwconv_kernel(const DwParams p) {
  extern __shared__ __align__(16) float tile[];
  __shared__ float wsm[kMaxTaps];

  const int strip = blockIdx.x % p.strips;
  const int plane = blockIdx.x / p.strips;  // n * C + c
  const int c = plane % p.C;
  const int n = plane / p.C;
  const int oh0 = strip * p.strip_h;
  const int h_in0 = oh0 * p.stride_h - p.pad_h;
  const float* src = p.in + static_cast<long long>(plane) * p.H * p.W;

  // ---- stage input rows (zero outside the image)
  const bool vec_in = (p.W % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 15) == 0);
  const int pitch4 = p.tile_pitch / 4;
  for (int i = threadIdx.x; i < p.tile_rows * pitch4; i += blockDim.x) {
    const int row = i / pitch4;
    const int col = (i - row * pitch4) * 4;  // staged column of this 4-wide group
    const int h = h_in0 + row;
    const int x = col - p.lead;              // input column of the group's first element
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (h >= 0 && h < p.H) {
      const float* rp = src + static_cast<long long>(h) * p.W;
      if (vec_in && x >= 0 && x + 3 < p.W) {
        v = __ldg(reinterpret_cast<const float4*>(rp + x));
      } else {
        if (x >= 0 && x < p.W) v.x = __ldg(rp + x);
        if (x + 1 >= 0 && x + 1 < p.W) v.y = __ldg(rp + x + 1);
        if (x + 2 >= 0 && x + 2 < p.W) v.z = __ldg(rp + x + 2);
        if (x + 3 >= 0 && x + 3 < p.W) v.w = __ldg(rp + x + 3);
      }
    }
    *reinterpret_cast<float4*>(tile + row * p.tile_pitch + col) = v;
  }

  const int rows_here = min(p.strip_h, p.P - oh0);
  const int q4 = (p.Q + 3) / 4;
  const bool vec_out = (p.Q % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);

  for (int f = 0; f < p.F; ++f) {
    __syncthreads();  // tile staged (f == 0) / previous weights consumed (f > 0)
    if (threadIdx.x < p.R * p.S)
      wsm[threadIdx.x] = p.w[(static_cast<long long>(c) * p.F + f) * p.R * p.S + threadIdx.x];
    __syncthreads();
    const int co = c * p.F + f;
    const float b = p.bias ? p.bias[co] : 0.f;
    float* dst_plane = p.out + (static_cast<long long>(n) * p.C * p.F + co) * p.P * p.Q;

    for (int i = threadIdx.x; i < rows_here * q4; i += blockDim.x) {
      const int orow = i / q4;
      const int ow = (i - orow * q4) * 4;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if constexpr (K3S1) {
        // 3x3, stride 1, dilation 1: six staged values per row feed four outputs.
        const int col0 = ow - p.pad_w + p.lead;  // staged column of tap s = 0 for output ow
#pragma unroll
        for (int r = 0; r < 3; ++r) {
          const float* tr = tile + (orow + r) * p.tile_pitch + col0;
          float x[6];
#pragma unroll
          for (int j = 0; j < 6; ++j) x[j] = tr[j];
#pragma unroll
          for (int s = 0; s < 3; ++s) {
            const float wv = wsm[r * 3 + s];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(x[j + s], wv, acc[j]);
          }
        }
      } else {
        for (int r = 0; r < p.R; ++r) {
          const float* tr = tile + (orow * p.stride_h + r * p.dil_h) * p.tile_pitch + p.lead - p.pad_w;
          for (int s = 0; s < p.S; ++s) {
            const float wv = wsm[r * p.S + s];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // Outputs past Q read staged zeros or neighbours; they are never stored.
              const int col = (ow + j) * p.stride_w + s * p.dil_w;
              acc[j] = fmaf(tr[col], wv, acc[j]);
            }
          }
        }
      }
      float* dst = dst_plane + static_cast<long long>(oh0 + orow) * p.Q + ow;
      if (vec_out) {
        dw_store4<MULTI>(p, dst, make_float4(acc[0] + b, acc[1] + b, acc[2] + b, acc[3] + b));
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (ow + j < p.Q) dw_store1<MULTI>(p, dst + j, acc[j] + b);
      }
    }
  }
}

// 3x3, stride 1, dilation 1, pad_w = 1, W % 4 == 0: no staging at all.  A thread owns a
// 4-wide, RH-tall block of outputs of one input plane: it loads RH + 2 input rows as one
// aligned 16-byte vector each plus the two halo scalars (which hit in L1: the neighbouring
// threads load those lines as vectors), keeps them in registers and writes RH vectors.  Every
// load of a thread is issued before the first use, so a CTA keeps (RH + 2) * 16 B per thread in
// flight - what a bandwidth-bound kernel needs - and there is no barrier anywhere.
template <int RH, bool MULTI>
__global__ void __launch_bounds__(256) dwconv3x3_direct_kernel(const DwParams p, long long items, int vcols,
                                                               int rblocks) {
  const long long item = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= items) return;
  const int vc = static_cast<int>(item % vcols);
  const int rb = static_cast<int>((item / vcols) % rblocks);
  const long long plane = item / (static_cast<long long>(vcols) * rblocks);  // n * C + c
  const int c = static_cast<int>(plane % p.C);
  const long long n = plane / p.C;
  const int ow = vc * 4;
  const int oh0 = rb * RH;
  const float* src = p.in + plane * p.H * p.W;

  float x[RH + 2][6];
#pragma unroll
  for (int i = 0; i < RH + 2; ++i) {
    const int h = oh0 + i - p.pad_h;
    const bool row_ok = h >= 0 && h < p.H && (oh0 + i - 2 < p.P);  // rows past the last output are not needed
    const float* rp = src + static_cast<long long>(row_ok ? h : 0) * p.W + ow;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    float left = 0.f, right = 0.f;
    if (row_ok) {
      v = __ldg(reinterpret_cast<const float4*>(rp));
      if (ow > 0) left = __ldg(rp - 1);
      if (ow + 4 < p.W) right = __ldg(rp + 4);
    }
    x[i][0] = left; x[i][1] = v.x; x[i][2] = v.y; x[i][3] = v.z; x[i][4] = v.w; x[i][5] = right;
  }

  for (int f = 0; f < p.F; ++f) {
    const int co = c * p.F + f;
    float wv[9];
#pragma unroll
    for (int t = 0; t < 9; ++t) wv[t] = __ldg(p.w + static_cast<long long>(co) * 9 + t);
    const float b = p.bias ? __ldg(p.bias + co) : 0.f;
    float* dst = p.out + ((n * p.C * p.F + co) * p.P + oh0) * p.Q + ow;
#pragma unroll
    for (int i = 0; i < RH; ++i) {
      if (oh0 + i >= p.P) break;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int s = 0; s < 3; ++s)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] = fmaf(x[i + r][j + s], wv[r * 3 + s], acc[j]);
      dw_store4<MULTI>(p, dst + static_cast<long long>(i) * p.Q, make_float4(acc[0] + b, acc[1] + b, acc[2] + b, acc[3] + b));
    }
  }
}

// Square filters of 3 or 5 taps a side at stride 1 or 2 (dilation 1) that the kernel above does not take
// (stride 2, 5x5, rows that are no multiple of 16 bytes, planes of a few pixels): still no staging
// and no barrier.  A thread owns four adjacent outputs of one row, reads the K x ((4-1)*STRIDE + K)
// input window they share straight from global memory (neighbouring threads hit the same lines in
// L1; out-of-image taps read as zero) and serves every output channel of its input plane from it.
template <int K, int STRIDE, bool MULTI>
__global__ void __launch_bounds__(256) dwconv_window_kernel(const DwParams p, long long items, int groups_w) {
  const long long item = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= items) return;
  constexpr int SPAN = 3 * STRIDE + K;
  const int g = static_cast<int>(item % groups_w);
  const int oh = static_cast<int>((item / groups_w) % p.P);
  const long long plane = item / (static_cast<long long>(groups_w) * p.P);  // n * C + c
  const int c = static_cast<int>(plane % p.C);
  const long long n = plane / p.C;
  const int ow = g * 4;
  const float* src = p.in + plane * p.H * p.W;
  const int ih0 = oh * STRIDE - p.pad_h, iw0 = ow * STRIDE - p.pad_w;

  float x[K][SPAN];
#pragma unroll
  for (int r = 0; r < K; ++r) {
    const int ih = ih0 + r;
    const bool row_ok = ih >= 0 && ih < p.H;
    const float* rp = src + static_cast<long long>(row_ok ? ih : 0) * p.W;
#pragma unroll
    for (int j = 0; j < SPAN; ++j) {
      const int iw = iw0 + j;
      x[r][j] = (row_ok && iw >= 0 && iw < p.W) ? __ldg(rp + iw) : 0.f;
    }
  }
  for (int f = 0; f < p.F; ++f) {
    const int co = c * p.F + f;
    const float* wp = p.w + static_cast<long long>(co) * K * K;
    float acc[4];
    const float b = p.bias ? __ldg(p.bias + co) : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = b;
#pragma unroll
    for (int r = 0; r < K; ++r)
#pragma unroll
      for (int t = 0; t < K; ++t) {
        const float wv = __ldg(wp + r * K + t);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = fmaf(x[r][j * STRIDE + t], wv, acc[j]);
      }
    float* dst = p.out + ((n * p.C * p.F + co) * p.P + oh) * p.Q + ow;
    if (ow + 3 < p.Q && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
      dw_store4<MULTI>(p, dst, make_float4(acc[0], acc[1], acc[2], acc[3]));
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (ow + j < p.Q) dw_store1<MULTI>(p, dst + j, acc[j]);
    }
  }
}

}  // namespace ftb

namespace ftb {
static int dwconv_generic(const float* in, const float* weight, const float* bias, float* out, float* const* extra,
                          int num_extra, int64_t n, int64_t c, int64_t h, int64_t w, int64_t factor, int64_t r,
                          int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                          const ftb_config* cfg, int* status, void* stream_v);
}

extern "C" int ftb_dwconv2d_nchw_f32(const float* in, const float* weight, const float* bias, float* out,
                                     int64_t n, int64_t c, int64_t h, int64_t w, int64_t factor, int64_t r,
                                     int64_t s, int stride_h, int stride_w, int pad_h, int pad_w,
                                     int dil_h, int dil_w, const ftb_config* cfg, int* status,
                                     void* stream_v) {
  return ftb::dwconv_generic(in, weight, bias, out, nullptr, 0, n, c, h, w, factor, r, s, stride_h, stride_w, pad_h,
                             pad_w, dil_h, dil_w, cfg, status, stream_v);
}

extern "C" int ftb_dwconv2d_nchw_f32_multi(const float* in, const float* weight, const float* bias,
                                           float* const* out_dst, int num_dst, int64_t n, int64_t c, int64_t h,
                                           int64_t w, int64_t factor, int64_t r, int64_t s, int stride_h,
                                           int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                                           const ftb_config* cfg, int* status, void* stream_v) {
  if (!out_dst || num_dst < 1 || num_dst > 8) return FTB_E_BAD_ARG;
  for (int d = 0; d < num_dst; ++d)
    if (!out_dst[d]) return FTB_E_BAD_ARG;
  return ftb::dwconv_generic(in, weight, bias, out_dst[0], out_dst + 1, num_dst - 1, n, c, h, w, factor, r, s,
                             stride_h, stride_w, pad_h, pad_w, dil_h, dil_w, cfg, status, stream_v);
}

namespace ftb {
static int dwconv_generic(const float* in, const float* weight, const float* bias, float* out, float* const* extra,
                          int num_extra, int64_t n, int64_t c, int64_t h, int64_t w, int64_t factor, int64_t r,
                          int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                          const ftb_config* cfg, int* status, void* stream_v) {
  (void)status;  // no in-kernel waits: nothing to report
  if (!in || !weight || !out) return FTB_E_BAD_ARG;
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || factor <= 0 || r <= 0 || s <= 0) return FTB_E_BAD_ARG;
  if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0 || pad_h < 0 || pad_w < 0) return FTB_E_BAD_ARG;
  if (r * s > kMaxTaps) return FTB_E_UNSUPPORTED;
  const int64_t P = (h + 2 * pad_h - dil_h * (r - 1) - 1) / stride_h + 1;
  const int64_t Q = (w + 2 * pad_w - dil_w * (s - 1) - 1) / stride_w + 1;
  if (P <= 0 || Q <= 0) return FTB_E_BAD_ARG;
  if (n * c * h * w > (1ll << 31) || n * c * factor * P * Q > (1ll << 31)) return FTB_E_TOO_LARGE;
  int rc = device_ok();
  if (rc) return rc;

  DwParams p;
  memset(&p, 0, sizeof(p));
  p.in = in; p.w = weight; p.bias = bias; p.out = out;
  if (cfg && (cfg->relu < 0 || cfg->relu > 1)) return FTB_E_BAD_CONFIG;
  p.relu = cfg ? cfg->relu : 0;
  p.num_extra = num_extra;
  const bool multi = p.relu != 0 || num_extra > 0;  // selects the kernels that clamp and write several destinations
  for (int d = 0; d < num_extra; ++d) {
    // the vector stores need every destination as aligned as the first
    if ((reinterpret_cast<uintptr_t>(extra[d]) & 15) != (reinterpret_cast<uintptr_t>(out) & 15)) return FTB_E_BAD_ARG;
    p.extra[d] = extra[d];
  }
  p.N = static_cast<int>(n); p.C = static_cast<int>(c); p.H = static_cast<int>(h); p.W = static_cast<int>(w);
  p.F = static_cast<int>(factor); p.R = static_cast<int>(r); p.S = static_cast<int>(s);
  p.P = static_cast<int>(P); p.Q = static_cast<int>(Q);
  p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w;
  p.dil_h = dil_h; p.dil_w = dil_w;

  // Staged row: [lead zeros/halo | W input columns | right halo], wide enough for the
  // last 4-output group (which may run past Q) and rounded to 16 bytes.
  p.lead = (pad_w + 3) / 4 * 4;
  const int q_pad = static_cast<int>((Q + 3) / 4 * 4);
  const int max_col = p.lead - pad_w + (q_pad - 1) * stride_w + (p.S - 1) * dil_w;
  int pitch = max_col + 1;
  if (pitch < p.lead + p.W) pitch = p.lead + p.W;
  p.tile_pitch = (pitch + 3) / 4 * 4;

  // Register-tiled path: 3x3, stride 1, dilation 1, pad_w 1, 16-byte aligned rows.
  // cfg->tile_h selects the rows per thread (4 or 8; other values keep the staged kernel).
  const bool direct_ok = r == 3 && s == 3 && stride_h == 1 && stride_w == 1 && dil_h == 1 && dil_w == 1 &&
                         pad_w == 1 && (w % 4 == 0) && Q == w &&
                         ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const int want_rows = cfg ? cfg->tile_h : 0;
  if (direct_ok && (want_rows == 0 || want_rows == 4 || want_rows == 8)) {
    int threads_d = cfg && cfg->threads > 0 ? cfg->threads : 128;
    if (threads_d < 32 || threads_d > 256 || threads_d % 32) return FTB_E_BAD_CONFIG;
    const int vcols = p.W / 4;
    // 8 rows per thread reuse more of what they load; on a small problem 4 rows give twice the threads
    // to hide the latency with (chosen when 8 rows would leave fewer than four CTAs per SM)
    int rh = want_rows == 4 ? 4 : 8;
    if (want_rows == 0 &&
        static_cast<long long>(n) * c * vcols * ((p.P + 7) / 8) < 4ll * sm_count() * threads_d)
      rh = 4;
    const int rblocks = (p.P + rh - 1) / rh;
    const long long items = static_cast<long long>(n) * c * vcols * rblocks;
    const long long blocks_d = (items + threads_d - 1) / threads_d;
    if (blocks_d > 0x7fffffffll) return FTB_E_TOO_LARGE;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const unsigned gd = static_cast<unsigned>(blocks_d);
    if (rh == 4 && !multi) dwconv3x3_direct_kernel<4, false><<<gd, threads_d, 0, stream>>>(p, items, vcols, rblocks);
    else if (rh == 4) dwconv3x3_direct_kernel<4, true><<<gd, threads_d, 0, stream>>>(p, items, vcols, rblocks);
    else if (!multi) dwconv3x3_direct_kernel<8, false><<<gd, threads_d, 0, stream>>>(p, items, vcols, rblocks);
    else dwconv3x3_direct_kernel<8, true><<<gd, threads_d, 0, stream>>>(p, items, vcols, rblocks);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_last_cuda_error(static_cast<int>(e));
      return FTB_E_CUDA;
    }
    return FTB_OK;
  }

  // Window path (default when no strip height is asked for): 3x3 and 5x5 at stride 1 or 2, dilation 1.
  if (want_rows == 0 && r == s && (r == 3 || r == 5) && stride_h == stride_w && (stride_h == 1 || stride_h == 2) &&
      dil_h == 1 && dil_w == 1) {
    int threads_w = cfg && cfg->threads > 0 ? cfg->threads : 128;
    if (threads_w < 32 || threads_w > 256 || threads_w % 32) return FTB_E_BAD_CONFIG;
    const int groups_w = static_cast<int>((Q + 3) / 4);
    const long long items = static_cast<long long>(n) * c * P * groups_w;
    const long long blocks_w = (items + threads_w - 1) / threads_w;
    if (blocks_w > 0x7fffffffll) return FTB_E_TOO_LARGE;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const unsigned gb = static_cast<unsigned>(blocks_w);
    if (!multi) {
      if (r == 3 && stride_h == 1) dwconv_window_kernel<3, 1, false><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
      else if (r == 3) dwconv_window_kernel<3, 2, false><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
      else if (stride_h == 1) dwconv_window_kernel<5, 1, false><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
      else dwconv_window_kernel<5, 2, false><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
    } else {
      if (r == 3 && stride_h == 1) dwconv_window_kernel<3, 1, true><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
      else if (r == 3) dwconv_window_kernel<3, 2, true><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
      else if (stride_h == 1) dwconv_window_kernel<5, 1, true><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
      else dwconv_window_kernel<5, 2, true><<<gb, threads_w, 0, stream>>>(p, items, groups_w);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_last_cuda_error(static_cast<int>(e));
      return FTB_E_CUDA;
    }
    return FTB_OK;
  }

  const int sms = sm_count();
  int threads = cfg && cfg->threads > 0 ? cfg->threads : 256;
  if (threads < 32 || threads > 1024 || threads % 32) return FTB_E_BAD_CONFIG;
  if (threads < p.R * p.S) return FTB_E_BAD_CONFIG;
  int strip_h = cfg && cfg->tile_h > 0 ? cfg->tile_h : 0;
  if (strip_h == 0) {
    // Default: the tallest strip that still gives every SM about four CTAs.
    strip_h = p.P;
    while (strip_h > 4 && static_cast<long long>(n) * c * ((p.P + strip_h - 1) / strip_h) < 4ll * sms)
      strip_h = (strip_h + 1) / 2;
  }
  if (strip_h > p.P) strip_h = p.P;
  const size_t kDynLimit = 200 * 1024;
  auto rows_for = [&](int sh) { return (sh - 1) * stride_h + (p.R - 1) * dil_h + 1; };
  while (strip_h > 1 && static_cast<size_t>(rows_for(strip_h)) * p.tile_pitch * 4 > kDynLimit)
    strip_h = (strip_h + 1) / 2;
  p.strip_h = strip_h;
  p.strips = (p.P + strip_h - 1) / strip_h;
  p.tile_rows = rows_for(strip_h);
  const size_t smem = static_cast<size_t>(p.tile_rows) * p.tile_pitch * 4;
  if (smem > kDynLimit) return FTB_E_UNSUPPORTED;

  const bool k3s1 = (r == 3 && s == 3 && stride_h == 1 && stride_w == 1 && dil_h == 1 && dil_w == 1);
  auto kern = k3s1 ? (multi ? dwconv_kernel<true, true> : dwconv_kernel<true, false>)
                   : (multi ? dwconv_kernel<false, true> : dwconv_kernel<false, false>);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kDynLimit));
    if (e != cudaSuccess) {
      set_last_cuda_error(static_cast<int>(e));
      return FTB_E_CUDA;
    }
  }
  const long long blocks = static_cast<long long>(n) * c * p.strips;
  if (blocks > 0x7fffffffll) return FTB_E_TOO_LARGE;
  kern<<<static_cast<unsigned>(blocks), threads, smem, static_cast<cudaStream_t>(stream_v)>>>(p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return FTB_E_CUDA;
  }
  return FTB_OK;
}
}  // namespace ftb
