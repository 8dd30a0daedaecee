// Host side of the tcgen05 contraction kernel: tensor-map construction, knob
// resolution/validation and the C-ABI launchers for GEMM fp32, batched GEMM bf16,
// GEMM int8 and conv2d (implicit GEMM).
#include "ftb_host.h"
#include "ftb_umma_kernel.cuh"
#include "ftb_conv_slab_kernel.cuh"

#include <cudaTypedefs.h>
#include <cstdlib>
#include <mutex>

namespace ftb {

// ------------------------------------------------------------------ driver entry point
static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    else
      set_last_cuda_error(static_cast<int>(e));
  });
  return g_encode;
}

// rank-`rank` tiled map (128-byte swizzle unless told otherwise); strides in bytes for dims 1..rank-1.
static int make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base,
                     const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                     const uint32_t* elem_strides, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  auto fn = encode_fn();
  if (!fn) return FTB_E_CUDA;
  CUresult r = fn(map, dt, rank, const_cast<void*>(base), dims, strides_bytes, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(static_cast<int>(r));
    return FTB_E_CUDA;
  }
  return FTB_OK;
}

// ------------------------------------------------------------------ per-dtype constants
struct KindInfo {
  int kind;         // KIND_*
  int esize;        // bytes per input element
  int kblk;         // K elements per stage (128 B)
  int umma_k;       // K elements per tcgen05.mma
  uint32_t ab_fmt;  // a_format / b_format field of the instruction descriptor
  uint32_t c_fmt;   // c_format field
  CUtensorMapDataType dt;
};

static KindInfo kind_info(int kind) {
  switch (kind) {
    case KIND_BF16: return {KIND_BF16, 2, 64, 16, 1u, 1u, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16};
    case KIND_TF32: return {KIND_TF32, 4, 32, 8, 2u, 1u, CU_TENSOR_MAP_DATA_TYPE_FLOAT32};
    default: return {KIND_I8, 1, 128, 32, 1u, 2u, CU_TENSOR_MAP_DATA_TYPE_UINT8};
  }
}

// Instruction descriptor of tcgen05.mma for a dense M=128 x N=bn tile.
static uint32_t make_idesc(const KindInfo& ki, int bn, int a_mn, int b_mn, int mma_m = kTileM) {
  uint32_t d = 0;
  d |= ki.c_fmt << 4;
  d |= ki.ab_fmt << 7;
  d |= ki.ab_fmt << 10;
  d |= static_cast<uint32_t>(a_mn ? 1 : 0) << 15;
  d |= static_cast<uint32_t>(b_mn ? 1 : 0) << 16;
  d |= static_cast<uint32_t>(bn >> 3) << 17;
  d |= static_cast<uint32_t>(mma_m >> 4) << 24;
  return d;
}

// `bn` = B rows/columns staged per CTA; `epilogue_bytes` = staging of the TMA-store epilogue.
static size_t smem_needed(int bn, int stages, bool split3, size_t epilogue_bytes = 0) {
  return static_cast<size_t>(stages) * (kATileBytes + static_cast<size_t>(bn) * 128) * (split3 ? 2 : 1) +
         1024 + epilogue_bytes;
}
constexpr size_t kEpilogueStaging = 2 * kEpiBufBytes;
constexpr size_t kSmemLimit = 227 * 1024 - 2048;  // leave room for the static barriers

// N extent a single TMA box covers for an N-contiguous B operand.
static int box_mn(const KindInfo& ki) { return 128 / ki.esize; }

// Relative per-SM throughput of a (cluster, tile_n) choice on a long K loop, from
// measurement; used only to rank defaults.
static double tile_rate(int cluster, int bn, int num_kb) {
  if (num_kb <= 4) {
    // A short K loop is bound by writing the result: single CTAs with wide tiles do best
    // (measured on K = 64, M = 256, N = 3136, 64 batch entries, fp32 result).
    if (cluster == 2) return bn >= 256 ? 0.79 : bn >= 128 ? 0.63 : bn >= 64 ? 0.43 : 0.3;
    return bn >= 256 ? 1.0 : bn >= 128 ? 0.88 : bn >= 64 ? 0.7 : 0.43;
  }
  if (cluster == 2) return bn >= 512 ? 1.1 : bn >= 256 ? 1.0 : bn >= 128 ? 0.65 : bn >= 64 ? 0.35 : 0.2;
  return bn >= 256 ? 0.7 : bn >= 128 ? 0.4 : bn >= 64 ? 0.2 : 0.1;
}

// Resolves cluster / tile_n / stages and checks every knob.  `m_rows` = M of one batch
// item, `batch` items; `allow_pair` is false for conv and 3xTF32.
static int resolve_config(const ftb_config* user, const KindInfo& ki, bool split3, int b_mn, bool allow_pair,
                          long long batch, long long m_rows, long long n, int num_kb, bool f32_out,
                          int num_sms, ftb_config* out, size_t epilogue_bytes = 0, bool allow_wide = false) {
  ftb_config c;
  memset(&c, 0, sizeof(c));
  if (user) c = *user;
  if (c.cluster < 0 || c.cluster > 2) return FTB_E_BAD_CONFIG;
  if (c.cluster == 2 && !allow_pair) return FTB_E_BAD_CONFIG;
  if (c.tile_n == 512) {
    // 256 x 512 tile of a CTA pair (plain GEMMs only, no 3xTF32)
    if (c.cluster != 2 || !allow_pair || split3 || !allow_wide) return FTB_E_BAD_CONFIG;
  } else if (c.tile_n != 0 && (c.tile_n < 32 || c.tile_n > 256 || c.tile_n % 32)) {
    return FTB_E_BAD_CONFIG;
  }
  // Granularity of tile_n: one TMA box of an N-contiguous B covers box_mn columns per CTA.
  auto tile_ok = [&](int cluster, int bn) {
    const int per_cta = bn / cluster;
    if (per_cta < 16 || per_cta % 8) return false;
    if (b_mn && per_cta % box_mn(ki)) return false;
    return true;
  };
  if (c.cluster == 0 || c.tile_n == 0) {
    // Two regimes.  Many waves of tiles: rank by useful work per wave times the tile's steady-state
    // rate (big tiles win).  A problem that fits in one wave is latency-bound: its time is a fixed
    // cost plus K blocks times a per-block cost that shrinks with the tile, so the candidate that
    // spreads over the most SMs wins (ties go to the larger tile).
    double best = -1.0;
    int best_cluster = 1, best_bn = 32;
    long long best_ctas = -1;
    int wave_cluster = 0, wave_bn = 0;
    for (int cluster = 2; cluster >= 1; --cluster) {
      if (c.cluster != 0 && c.cluster != cluster) continue;
      if (cluster == 2 && (!allow_pair || num_sms < 2)) continue;
      // the 256 x 512 pair tile competes only on long K loops (its epilogue overlaps less)
      const int bn_max = (cluster == 2 && allow_wide && !split3 && num_kb > 4) ? 512 : 256;
      for (int bn = bn_max; bn >= 32; bn /= 2) {
        if (c.tile_n != 0 && c.tile_n != bn) continue;
        if (!tile_ok(cluster, bn)) continue;
        const long long tm = kTileM * cluster;
        const long long tiles = batch * ((m_rows + tm - 1) / tm) * ((n + bn - 1) / bn);
        const long long units = num_sms / cluster;
        const long long waves = (tiles + units - 1) / units;
        const double useful = static_cast<double>(batch) * m_rows * n;
        const double paid = static_cast<double>(waves) * units * tm * bn;
        const double score = useful / paid * tile_rate(cluster, bn, num_kb);
        if (score > best + 1e-9) {
          best = score;
          best_cluster = cluster;
          best_bn = bn;
        }
        if (waves == 1) {
          // SMs kept busy with real work: CTAs used times the share of their tiles inside the problem
          const long long ctas_used = static_cast<long long>(tiles * cluster * (useful / (static_cast<double>(tiles) * tm * bn)));
          if (ctas_used > best_ctas) {
            best_ctas = ctas_used;
            wave_cluster = cluster;
            wave_bn = bn;
          }
        }
      }
    }
    if (best < 0) {
      // no ranked candidate: fall back to the smallest legal single-CTA tile
      c.cluster = c.cluster ? c.cluster : 1;
      if (c.tile_n == 0) c.tile_n = b_mn && box_mn(ki) > 32 ? box_mn(ki) : 32;
    } else if (best_ctas >= 0) {
      bool best_is_single_wave;
      {
        const long long tm = kTileM * best_cluster;
        const long long tiles = batch * ((m_rows + tm - 1) / tm) * ((n + best_bn - 1) / best_bn);
        best_is_single_wave = tiles <= num_sms / best_cluster;
      }
      if (best_is_single_wave) {
        c.cluster = wave_cluster;
        c.tile_n = wave_bn;
      } else {
        c.cluster = best_cluster;
        c.tile_n = best_bn;
      }
    } else {
      c.cluster = best_cluster;
      c.tile_n = best_bn;
    }
  }
  if (!tile_ok(c.cluster, c.tile_n)) return FTB_E_BAD_CONFIG;
  const int bn_cta = c.tile_n / c.cluster;
  if (c.stages == 0) {
    c.stages = kMaxStages;
    while (c.stages > 2 && smem_needed(bn_cta, c.stages, split3, epilogue_bytes) > kSmemLimit) --c.stages;
    if (c.stages > num_kb + 1 && num_kb >= 1) c.stages = num_kb + 1 > 2 ? num_kb + 1 : 2;
    if (c.stages > kMaxStages) c.stages = kMaxStages;
  }
  if (c.stages < 2 || c.stages > kMaxStages) return FTB_E_BAD_CONFIG;
  if (smem_needed(bn_cta, c.stages, split3, epilogue_bytes) > kSmemLimit) return FTB_E_BAD_CONFIG;
  if (c.raster < 0 || c.raster > 3) return FTB_E_BAD_CONFIG;
  if (c.raster == 0) {
    // auto: a B operand much larger than what stays in L2 next to A wants grouped-M order (a wave
    // of tiles then touches a few panels of both operands instead of all of B); otherwise n-fastest
    const double b_bytes = static_cast<double>(n) * num_kb * 128.0;
    if (batch == 1 && b_bytes > 32.0 * 1024 * 1024) {
      c.raster = 3;
      if (c.group_m == 0) c.group_m = 8;
    } else {
      c.raster = 1;
    }
  }
  if (c.raster == 3 && c.group_m == 0) c.group_m = 8;
  if (c.group_m < 0) return FTB_E_BAD_CONFIG;
  if (c.split_k == 0) c.split_k = 1;
  if (c.split_k < 1 || c.split_k > 64 || c.split_k > num_kb) return FTB_E_BAD_CONFIG;
  if (c.split_k > 1 && !f32_out) return FTB_E_BAD_CONFIG;
  if (c.ctas < 0) return FTB_E_BAD_CONFIG;
  *out = c;
  return FTB_OK;
}

template <int KIND, int OUT, bool SPLIT3, bool PAIR, bool WIDE = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const StoreMaps& tc, const UmmaParams& p,
                  int ctas, cudaStream_t stream) {
  auto kern = umma_gemm_kernel<KIND, OUT, SPLIT3, PAIR, WIDE>;
  const size_t smem = smem_needed(p.b_bytes / 128, p.stages, SPLIT3, p.tma_store ? kEpilogueStaging : 0);
  // The opt-in shared-memory size is a per-device attribute of the function.
  static std::mutex mu;
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !done[dev]) {
      cudaError_t attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  static_cast<int>(kSmemLimit));
      if (attr_err != cudaSuccess) {
        set_last_cuda_error(static_cast<int>(attr_err));
        return FTB_E_CUDA;
      }
      done[dev] = true;
    }
  }
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  lc.blockDim = dim3(WIDE ? 352 : SPLIT3 ? 320 : 192, 1, 1);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  int nattr = 0;
  if (PAIR) {
    attr[nattr].id = cudaLaunchAttributeClusterDimension;
    attr[nattr].val.clusterDim.x = 2;
    attr[nattr].val.clusterDim.y = 1;
    attr[nattr].val.clusterDim.z = 1;
    ++nattr;
  }
  if (p.pdl) {
    // programmatic dependent of the kernel launched just before it on this stream
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
  }
  if (nattr) {
    lc.attrs = attr;
    lc.numAttrs = nattr;
  }
  cudaError_t e = cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p);
  count_launch();
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return FTB_E_CUDA;
  }
  return FTB_OK;
}

static int dispatch(int kind, int out, bool split3, bool pair, const CUtensorMap& ta, const CUtensorMap& tb,
                    const StoreMaps& tc, const UmmaParams& p, int ctas, cudaStream_t stream, bool wide = false) {
  if (wide) {
    if (!pair || split3) return FTB_E_BAD_CONFIG;
    if (kind == KIND_BF16 && out == OUT_BF16) return launch<KIND_BF16, OUT_BF16, false, true, true>(ta, tb, tc, p, ctas, stream);
    if (kind == KIND_BF16 && out == OUT_F32) return launch<KIND_BF16, OUT_F32, false, true, true>(ta, tb, tc, p, ctas, stream);
    if (kind == KIND_I8 && out == OUT_S32) return launch<KIND_I8, OUT_S32, false, true, true>(ta, tb, tc, p, ctas, stream);
    if (kind == KIND_TF32 && out == OUT_F32) return launch<KIND_TF32, OUT_F32, false, true, true>(ta, tb, tc, p, ctas, stream);
    return FTB_E_BAD_ARG;
  }
  if (pair) {
    if (split3) return FTB_E_BAD_CONFIG;
    if (kind == KIND_BF16 && out == OUT_BF16) return launch<KIND_BF16, OUT_BF16, false, true>(ta, tb, tc, p, ctas, stream);
    if (kind == KIND_BF16 && out == OUT_F32) return launch<KIND_BF16, OUT_F32, false, true>(ta, tb, tc, p, ctas, stream);
    if (kind == KIND_I8 && out == OUT_S32) return launch<KIND_I8, OUT_S32, false, true>(ta, tb, tc, p, ctas, stream);
    if (kind == KIND_TF32 && out == OUT_F32) return launch<KIND_TF32, OUT_F32, false, true>(ta, tb, tc, p, ctas, stream);
    return FTB_E_BAD_ARG;
  }
  if (kind == KIND_BF16 && out == OUT_BF16) return launch<KIND_BF16, OUT_BF16, false, false>(ta, tb, tc, p, ctas, stream);
  if (kind == KIND_BF16 && out == OUT_F32) return launch<KIND_BF16, OUT_F32, false, false>(ta, tb, tc, p, ctas, stream);
  if (kind == KIND_I8 && out == OUT_S32) return launch<KIND_I8, OUT_S32, false, false>(ta, tb, tc, p, ctas, stream);
  if (kind == KIND_TF32 && out == OUT_F32 && !split3) return launch<KIND_TF32, OUT_F32, false, false>(ta, tb, tc, p, ctas, stream);
  if (kind == KIND_TF32 && out == OUT_F32 && split3) return launch<KIND_TF32, OUT_F32, true, false>(ta, tb, tc, p, ctas, stream);
  return FTB_E_BAD_ARG;
}

// Fills the operand-staging fields for a plain (batched) GEMM operand of which one CTA
// stages `tile_extent` rows (K-major) or columns (MN-major).
static void operand_layout(const KindInfo& ki, int mn_major, int tile_extent, int* boxes, int* box_extent,
                           uint32_t* box_bytes, uint32_t* lbo, uint32_t* sbo, uint32_t* kadv,
                           uint32_t* layout, CUtensorMapSwizzle* swizzle) {
  *layout = 2;
  *swizzle = CU_TENSOR_MAP_SWIZZLE_128B;
  if (mn_major) {
    *box_extent = box_mn(ki);
    *boxes = tile_extent / *box_extent;
    *box_bytes = static_cast<uint32_t>(ki.kblk) * 128u;
    *lbo = *box_bytes;  // next 128-byte wide block along M/N
    *sbo = 1024;        // next group of 8 K rows
    *kadv = static_cast<uint32_t>(ki.umma_k) * 128u;
    if (ki.esize == 4) {
      // 32-bit MN-major operands exist only in the layout that swizzles 32-byte units:
      // the pattern repeats every 4 K rows.
      *layout = 1;
      *swizzle = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
      *sbo = 512;
    }
  } else {
    *box_extent = tile_extent;
    *boxes = 1;
    *box_bytes = static_cast<uint32_t>(tile_extent) * 128u;
    *lbo = 16;
    *sbo = 1024;
    *kadv = static_cast<uint32_t>(ki.umma_k * ki.esize);
  }
}

// Clears `n` floats (16-byte aligned base); the GEMM that adds its K splits into them is launched
// as a programmatic dependent and sets itself up while this runs.
__global__ void __launch_bounds__(256) zero_f32_kernel(float* __restrict__ dst, long long n) {
  grid_launch_dependents();
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long t0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  float4* d4 = reinterpret_cast<float4*>(dst);
  const long long n4 = n / 4;
  for (long long i = t0; i < n4; i += stride) d4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i = n4 * 4 + t0; i < n; i += stride) dst[i] = 0.f;
}

// Defaults for an fp32-output product that fits in one wave of CTAs.  Such a launch is not
// latency-bound but bound by what each CTA has to pull through its L2 port and by its own
// MMA chain, so wide tiles with the K loop split over otherwise idle SMs win even though the
// partial sums then meet in global memory (bulk reduce-add into a zeroed result).  Cost model
// per CTA, microseconds, constants measured on 1024^3 fp32 (single-pass and 3xTF32):
//   K blocks x max(bytes staged / 60 GB/s, 4 MMAs x passes x time of a 128 x tile_n MMA)
//   + result bytes / 35 GB/s + 2 us when the K loop is split (memset + adds) + 0.8 us for a CTA pair.
// Returns true and fills `out` when the caller left tile_n, cluster and split_k open.
static bool pick_small_f32(const ftb_config* user, const KindInfo& ki, bool split3, int b_mn, bool eligible,
                           long long batch, long long m, long long n, int num_kb, int num_sms, ftb_config* out) {
  if (!eligible) return false;
  if (user && (user->tile_n != 0 || user->cluster != 0 || user->split_k != 0)) return false;
  double best = 1e30;
  int best_cluster = 0, best_bn = 0, best_split = 0;
  for (int cluster = 1; cluster <= (split3 ? 1 : 2); ++cluster) {
    for (int bn = 32; bn <= 256; bn *= 2) {
      const int per_cta = bn / cluster;
      if (per_cta < 32 || (b_mn && per_cta % box_mn(ki))) continue;
      for (int split = 1; split <= 8; split *= 2) {
        if (split > 1 && split * 2 > num_kb) break;
        const long long ctas = batch * ((m + 128 * cluster - 1) / (128 * cluster)) * ((n + bn - 1) / bn) * split * cluster;
        if (ctas > num_sms) break;
        const int kb = (num_kb + split - 1) / split;
        const double mma_us = (bn >= 256 ? 0.140 : bn >= 128 ? 0.090 : bn >= 64 ? 0.061 : 0.050) *
                              (ki.kind == KIND_TF32 ? 1.0 : 0.5);
        const double load = kb * (16384.0 + per_cta * 128.0) / 60e3;
        const double math = kb * 4.0 * mma_us * (split3 ? 3.0 : 1.0);
        const double cost = (load > math ? load : math) + 128.0 * bn * 4.0 / 35e3 + (split > 1 ? 2.0 : 0.0) +
                            (cluster == 2 ? 0.8 : 0.0);  // a pair pays two cluster barriers
        if (cost < best) {
          best = cost;
          best_cluster = cluster;
          best_bn = bn;
          best_split = split;
        }
      }
    }
  }
  if (best_bn == 0) return false;
  memset(out, 0, sizeof(*out));
  if (user) *out = *user;
  out->cluster = best_cluster;
  out->tile_n = best_bn;
  out->split_k = best_split;
  return true;
}

int gemm_generic(int kind, int out, const void* a, const void* b, void* c, int64_t batch, int64_t m,
                 int64_t n, int64_t k, int trans_a, int trans_b, const ftb_config* user, int* status,
                 void* stream_v, void* const* extra_dst, int num_extra, const GemmExtras* extras) {
  if (!a || !b || !c) return FTB_E_BAD_ARG;
  const bool a_bcast = extras && extras->a_broadcast;
  const float* row_bias = extras ? extras->row_bias : nullptr;
  if (row_bias && out != OUT_F32) return FTB_E_BAD_ARG;
  if (num_extra < 0 || num_extra > kMaxDst - 1 || (num_extra > 0 && !extra_dst)) return FTB_E_BAD_ARG;
  for (int d = 0; d < num_extra; ++d)
    if (!extra_dst[d]) return FTB_E_BAD_ARG;
  if (batch <= 0 || m <= 0 || n <= 0 || k <= 0) return FTB_E_BAD_ARG;
  if (m > (1ll << 30) || n > (1ll << 30) || k > (1ll << 30) || batch > (1ll << 24)) return FTB_E_TOO_LARGE;
  int rc = device_ok();
  if (rc) return rc;
  const KindInfo ki = kind_info(kind);
  const bool split3 = (kind == KIND_TF32) && user && user->fp32_mode == 1;
  if (user && (user->fp32_mode < 0 || user->fp32_mode > 1)) return FTB_E_BAD_CONFIG;
  const int a_mn = trans_a ? 1 : 0;  // A given as [K,M]: M contiguous
  const int b_mn = trans_b ? 0 : 1;  // B given as [K,N]: N contiguous
  // TMA addressing rules: 16-byte aligned bases and row pitches.
  const int64_t a_pitch = (a_mn ? m : k) * ki.esize;
  const int64_t b_pitch = (b_mn ? n : k) * ki.esize;
  if ((a_pitch & 15) || (b_pitch & 15) || (reinterpret_cast<uintptr_t>(a) & 15) ||
      (reinterpret_cast<uintptr_t>(b) & 15)) {
    // Not addressable by TMA: the CUDA-core kernel takes it (one destination only).
    if (num_extra > 0 || extras) return FTB_E_UNSUPPORTED;
    if (user && ftb_validate(kind == KIND_TF32 ? 0 : kind == KIND_BF16 ? 1 : 2, user, m, n, k) != FTB_OK)
      return FTB_E_BAD_CONFIG;
    return simt_gemm(kind == KIND_BF16 ? 0 : kind == KIND_TF32 ? 1 : 2, out, a, b, c, batch, m, n, k, trans_a,
                     trans_b, stream_v);
  }

  // The staged (bulk tensor store) epilogue needs 16-byte aligned output rows and bases.
  const int out_esize = out == OUT_BF16 ? 2 : 4;
  bool store_ok = ((n * out_esize) & 15) == 0 && (reinterpret_cast<uintptr_t>(c) & 15) == 0;
  for (int d = 0; d < num_extra; ++d) store_ok = store_ok && (reinterpret_cast<uintptr_t>(extra_dst[d]) & 15) == 0;
  if (user && user->epilogue == 1) store_ok = false;  // per-thread stores asked for
  if (user && (user->epilogue < 0 || user->epilogue > 1)) return FTB_E_BAD_CONFIG;

  const int num_sms = sm_count();
  const int num_kb = static_cast<int>((k + ki.kblk - 1) / ki.kblk);
  ftb_config cfg;
  ftb_config tuned;
  if (pick_small_f32(user, ki, split3, b_mn, out == OUT_F32 && num_extra == 0, batch, m, n, num_kb, num_sms, &tuned))
    user = &tuned;
  rc = resolve_config(user, ki, split3, b_mn, !split3, batch, m, n, num_kb, out == OUT_F32, num_sms, &cfg,
                      kEpilogueStaging, true);
  if (rc) return rc;
  const bool pair = cfg.cluster == 2;
  const int tile_m = pair ? 2 * kTileM : kTileM;
  const int tiles_m = static_cast<int>((m + tile_m - 1) / tile_m);

  UmmaParams p;
  memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(m);
  p.N = static_cast<int>(n);
  p.K = static_cast<int>(k);
  p.batch = static_cast<int>(batch);
  p.bn = cfg.tile_n;
  p.stages = cfg.stages;
  p.num_kb = num_kb;
  p.tiles_m = tiles_m;
  p.tiles_n = static_cast<int>((n + p.bn - 1) / p.bn);
  p.raster = cfg.raster - 1;  // kernel: 0 n-fastest, 1 m-fastest, 2 grouped-M
  p.group_m = cfg.group_m;
  p.split_k = cfg.split_k;
  p.kblk = ki.kblk;
  const bool wide = cfg.tile_n == 512;  // one MMA covers half of the tile's columns
  p.idesc = make_idesc(ki, wide ? 256 : p.bn, a_mn, b_mn, tile_m);
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  p.pair_m = tile_m;
  p.b_rows = pair ? p.bn / 2 : p.bn;
  p.b_bytes = static_cast<uint32_t>(p.b_rows) * 128u;
  CUtensorMapSwizzle a_swz, b_swz;
  operand_layout(ki, a_mn, kTileM, &p.a_boxes, &p.a_box_mn, &p.a_box_bytes, &p.a_lbo, &p.a_sbo, &p.a_kadv,
                 &p.a_layout, &a_swz);
  operand_layout(ki, b_mn, p.b_rows, &p.b_boxes, &p.b_box_mn, &p.b_box_bytes, &p.b_lbo, &p.b_sbo, &p.b_kadv,
                 &p.b_layout, &b_swz);
  // second half of a CTA's B stage in a wide tile: 128 rows (K-major) or 128 columns (N-contiguous boxes)
  p.b_half_enc = (b_mn ? static_cast<uint32_t>(128 / p.b_box_mn) * p.b_box_bytes : 128u * 128u) >> 4;
  p.C = c;
  p.ldc = n;
  p.c_batch_stride = m * n;
  p.bias = row_bias;
  p.a_bcast = a_bcast ? 1 : 0;
  p.status = status ? status : fallback_status();
  if (!p.status) return FTB_E_CUDA;
  p.slab_cols = 128 / out_esize;
  // split-K goes through the staged epilogue as bulk fp32 reduce-adds (one destination only)
  p.tma_store = (store_ok && p.bn % p.slab_cols == 0 &&
                 (p.split_k == 1 || (out == OUT_F32 && num_extra == 0))) ? 1 : 0;
  p.diag = user ? user->reserved[0] : 0;
#ifdef FTB_PROFILE_WAITS
  // diagnostic bit 3 (with bit 2): the free-running MMAs are issued as M = 64 instructions, to see what a
  // narrower A operand costs (single-CTA tiles only; results are garbage by design)
  if (((p.diag & 32) && p.bn > 64) || ((p.diag & 64) && p.bn > 128)) return FTB_E_BAD_CONFIG;  // columns past the allocation
  if ((p.diag & 8) && !pair) p.idesc = make_idesc(ki, wide ? 256 : p.bn, a_mn, b_mn, 64);
#endif
  if (user && (user->release < 0 || user->release > 2)) return FTB_E_BAD_CONFIG;
  // (the 256 x 512 tile keeps the per-stage hand-back: its four stages are too few to give one up)
  p.release_pairs = (user && user->release == 2 && !split3 && cfg.tile_n != 512 && cfg.stages % 2 == 0 &&
                     cfg.stages >= 4) ? 1 : 0;
  p.num_dst = 1 + num_extra;
  if (num_extra > 0 && !p.tma_store) return FTB_E_UNSUPPORTED;  // several destinations only through bulk stores

  // Tensor maps: dim 0 is the contiguous one; batch is the outermost.
  CUtensorMap ta, tb;
  StoreMaps tc;
  memset(&tc, 0, sizeof(tc));
  const uint32_t ones[3] = {1, 1, 1};
  if (p.tma_store) {
    const CUtensorMapDataType odt = out == OUT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                  : out == OUT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                   : CU_TENSOR_MAP_DATA_TYPE_INT32;
    uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m), static_cast<uint64_t>(batch)};
    uint64_t strides[2] = {static_cast<uint64_t>(n) * out_esize, static_cast<uint64_t>(m) * n * out_esize};
    uint32_t box[3] = {static_cast<uint32_t>(p.slab_cols), static_cast<uint32_t>(kTileM), 1};
    for (int d = 0; d < p.num_dst; ++d) {
      rc = make_tmap(&tc.dst[d], odt, 3, d == 0 ? c : extra_dst[d - 1], dims, strides, box, ones);
      if (rc) return rc;
    }
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (a_mn) {
      dims[0] = m; dims[1] = k; dims[2] = a_bcast ? 1 : batch;
      box[0] = p.a_box_mn; box[1] = ki.kblk; box[2] = 1;
    } else {
      dims[0] = k; dims[1] = m; dims[2] = a_bcast ? 1 : batch;
      box[0] = ki.kblk; box[1] = kTileM; box[2] = 1;
    }
    strides[0] = dims[0] * ki.esize;
    strides[1] = static_cast<uint64_t>(m) * k * ki.esize;
    rc = make_tmap(&ta, ki.dt, 3, a, dims, strides, box, ones, a_swz);
    if (rc) return rc;
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (b_mn) {
      dims[0] = n; dims[1] = k; dims[2] = batch;
      box[0] = p.b_box_mn; box[1] = ki.kblk; box[2] = 1;
    } else {
      dims[0] = k; dims[1] = n; dims[2] = batch;
      box[0] = ki.kblk; box[1] = p.b_rows; box[2] = 1;
    }
    strides[0] = dims[0] * ki.esize;
    strides[1] = static_cast<uint64_t>(n) * k * ki.esize;
    rc = make_tmap(&tb, ki.dt, 3, b, dims, strides, box, ones, b_swz);
    if (rc) return rc;
  }

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.split_k > 1) {
    const long long count = static_cast<long long>(batch) * m * n;
    cudaError_t e;
    if ((reinterpret_cast<uintptr_t>(c) & 15) == 0) {
      long long blocks = (count / 4 + 255) / 256;
      if (blocks > 4ll * num_sms) blocks = 4ll * num_sms;
      if (blocks < 1) blocks = 1;
      zero_f32_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<float*>(c), count);
      count_launch();
      e = cudaGetLastError();
      p.pdl = 1;
    } else {
      e = cudaMemsetAsync(c, 0, static_cast<size_t>(count) * 4, stream);
    }
    if (e != cudaSuccess) {
      set_last_cuda_error(static_cast<int>(e));
      return FTB_E_CUDA;
    }
  }
  const long long total = static_cast<long long>(p.batch) * p.tiles_m * p.tiles_n * p.split_k;
  if (total > 0x7fffffffll) return FTB_E_TOO_LARGE;
  int ctas = cfg.ctas > 0 ? cfg.ctas : num_sms;
  if (pair) {
    if (ctas / 2 > total) ctas = static_cast<int>(total) * 2;
    ctas &= ~1;
    if (ctas < 2) ctas = 2;
  } else if (ctas > total) {
    ctas = static_cast<int>(total);
  }
  return dispatch(kind, out, split3, pair, ta, tb, tc, p, ctas, stream, wide);
}

// ------------------------------------------------------------------ conv2d as implicit GEMM
// Workspace layout: [input as N,H,W,Cp floats][weights as K, R*S*cchunks*32 floats], both regions
// 1024-byte aligned.  Cp = C rounded up to 4 (TMA pitch rule); with groups, every group's channels
// are padded to a multiple of 4 (`cgp`) and Cp = groups * cgp, so that each group starts on a
// 16-byte boundary whatever the number of channels per group.
static int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

struct ConvWs {
  int64_t cp, cgp, cchunks, in_bytes, w_bytes;
};
// Shapes that run as a 1x1 conv over their im2col form (conv_im2col_kernel).
static bool conv_small_c(int64_t c, int64_t r, int64_t s, int64_t groups) {
  return groups == 1 && c <= 8 && r * s >= 4 && r * s * c <= 1024;  // one block pass covers a pixel's row
}
static ConvWs conv_ws(int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r, int64_t s,
                      int64_t groups) {
  ConvWs ws;
  const int64_t cg = c / groups;
  ws.cgp = round_up(cg, 4);
  ws.cp = groups > 1 ? groups * ws.cgp : round_up(c, 4);
  ws.cchunks = (cg + 31) / 32;
  ws.in_bytes = round_up(n * h * w * ws.cp * 4, 1024);
  ws.w_bytes = round_up(k * r * s * ws.cchunks * 32 * 4, 1024);
  if (conv_small_c(c, r, s, groups)) {
    // room for the im2col form of a few-channel input (one row of taps x channels per output
    // pixel), bounded by one output pixel per input pixel
    const int64_t col = round_up(n * h * w * round_up(r * s * c, 32) * 4, 1024);
    if (col > ws.in_bytes) ws.in_bytes = col;
  }
  return ws;
}

// Few input channels under a filter with several taps: a 32-channel K block of the per-tap
// lowering would hold mostly padding (3 real channels in 32 for an RGB stem), so such a conv is
// run as a 1x1 conv over its im2col form instead: per output pixel one row of taps x channels,
// padded to a multiple of 32.
constexpr int kColSeg = 64;  // output pixels of one image row handled by one block

__global__ void __launch_bounds__(256)
conv_im2col_kernel(const float* __restrict__ in, const float* __restrict__ wgt, float* __restrict__ col,
                   float* __restrict__ w2, int N, int C, int H, int W, int K, int R, int S, int P, int Q, int Kp,
                   int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int segs,
                   int col_blocks) {
  grid_launch_dependents();
  const int kreal = R * S * C;
  if (static_cast<int>(blockIdx.x) < col_blocks) {
    // A block owns a segment of one output row; a thread owns one group of 4 consecutive K indices
    // (a 16-byte store) and walks the segment's pixels, so the (tap, channel) of its four entries is
    // worked out once.
    const int gpp = Kp >> 2;                    // groups per pixel
    const int ppb = 256 / gpp;                  // pixels per pass (Kp <= 1024)
    const int g = threadIdx.x % gpp, lane_px = threadIdx.x / gpp;
    const int seg = blockIdx.x % segs;
    const int oh = (blockIdx.x / segs) % P;
    const int img = blockIdx.x / (segs * P);
    int ch[4], dh[4], dw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int idx = 4 * g + j;
      const int tap = idx / C;
      ch[j] = idx < kreal ? idx - tap * C : -1;
      const int tr = tap / S;
      dh[j] = tr * dil_h - pad_h;
      dw[j] = (tap - tr * S) * dil_w - pad_w;
    }
    const float* src = in + static_cast<long long>(img) * C * H * W;
    float* dst = col + (static_cast<long long>(img) * P + oh) * Q * Kp + 4 * g;
    const int ow_end = min(Q, (seg + 1) * kColSeg);
    if (lane_px < ppb) {
      for (int ow = seg * kColSeg + lane_px; ow < ow_end; ow += ppb) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int ih = oh * stride_h + dh[j], iw = ow * stride_w + dw[j];
          v[j] = (ch[j] >= 0 && ih >= 0 && ih < H && iw >= 0 && iw < W)
                     ? __ldg(src + (static_cast<long long>(ch[j]) * H + ih) * W + iw) : 0.0f;
        }
        *reinterpret_cast<float4*>(dst + static_cast<long long>(ow) * Kp) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
  } else {
    // filter [K][C][R*S] -> [K][Kp] with the same (tap, channel) order, zero tail
    const long long total = static_cast<long long>(K) * Kp;
    const long long nb = gridDim.x - col_blocks;
    for (long long i = static_cast<long long>(blockIdx.x - col_blocks) * blockDim.x + threadIdx.x; i < total;
         i += nb * blockDim.x) {
      const int idx = static_cast<int>(i % Kp);
      const int ko = static_cast<int>(i / Kp);
      float x = 0.0f;
      if (idx < kreal) {
        const int tap = idx / C, c = idx - tap * C;
        x = wgt[(static_cast<long long>(ko) * C + c) * R * S + tap];
      }
      w2[i] = x;
    }
  }
}

// One launch: blocks [0, in_blocks) transpose NCHW -> NHWC(Cp) through a shared-memory tile of
// 32 channels x 128 pixels (16-byte loads along the pixels, 16-byte stores along the channels;
// the 129-float row pitch keeps both phases free of bank conflicts), the rest pack weights
// [K][Cg][R][S] -> [K][R][S][cchunks*32] (zero padded).
constexpr int kPreCh = 32, kPrePx = 128;

__global__ void __launch_bounds__(256)
conv_prepass_kernel(const float* __restrict__ in, const float* __restrict__ wgt, float* __restrict__ in_nhwc,
                    float* __restrict__ w_packed, int N, int C, int HW, int Cp, int K, int Cg, int RS,
                    int cchunks, int hw_tiles, int c_tiles, int in_blocks, int w_blocks, float* __restrict__ zero,
                    long long zero_n, int plane, int sub_q, int sub_row, int sub_col, int cgp) {
  __shared__ __align__(16) float tile[kPreCh][kPrePx + 1];
  // The conv kernel that follows is launched as a programmatic dependent: it may set itself up
  // (barriers, tensor memory, descriptor fetch) while this grid runs, and waits for this grid's
  // completion before it touches the workspace or the result.
  grid_launch_dependents();
  const int bid = blockIdx.x;
  if (bid >= in_blocks + w_blocks) {
    // zero the result for a conv whose partial sums meet in global memory (split reduction)
    const long long nb = gridDim.x - in_blocks - w_blocks;
    const long long t0 = static_cast<long long>(bid - in_blocks - w_blocks) * blockDim.x + threadIdx.x;
    if ((reinterpret_cast<uintptr_t>(zero) & 15) == 0) {
      float4* z4 = reinterpret_cast<float4*>(zero);
      const long long n4 = zero_n / 4;
      for (long long i = t0; i < n4; i += nb * blockDim.x) z4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (long long i = n4 * 4 + t0; i < zero_n; i += nb * blockDim.x) zero[i] = 0.f;
    } else {
      for (long long i = t0; i < zero_n; i += nb * blockDim.x) zero[i] = 0.f;
    }
  } else if (bid < in_blocks) {
    const int ct = bid % c_tiles;
    const int ht = (bid / c_tiles) % hw_tiles;
    const int img = bid / (c_tiles * hw_tiles);
    const int c0 = ct * kPreCh, p0 = ht * kPrePx;
    // `HW` counts the pixels that are copied, `plane` the pixels of one source channel plane; they
    // differ when a strided 1x1 conv keeps only every sub_row-th / sub_col-th pixel (sub_q > 0: kept
    // pixels per row), which is all such a conv reads.
    const float* src = in + static_cast<long long>(img) * C * plane;
    const bool vec = sub_q == 0 && (HW % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
    // load: thread -> (channel, 4 pixels)
    for (int i = threadIdx.x; i < kPreCh * (kPrePx / 4); i += 256) {
      const int ch = i / (kPrePx / 4), q = (i % (kPrePx / 4)) * 4;
      const int px = p0 + q;
      // Channel of the source for channel c0 + ch of the copy.  With groups (cgp > 0) the copy pads
      // every group to cgp channels: copy channel g * cgp + j is source channel g * Cg + j for
      // j < Cg and zero padding otherwise.
      int c = c0 + ch;
      if (cgp > 0) {
        const int g = c / cgp, j = c - g * cgp;
        c = (j < Cg) ? g * Cg + j : C;
      }
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < C && px < HW && sub_q > 0) {
        const float* cp_ = src + static_cast<long long>(c) * plane;
        float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (px + j < HW) t[j] = __ldg(cp_ + ((px + j) / sub_q) * sub_row + ((px + j) % sub_q) * sub_col);
        v = make_float4(t[0], t[1], t[2], t[3]);
      } else if (c < C && px < HW) {
        const float* rp = src + static_cast<long long>(c) * plane + px;
        if (vec && px + 3 < HW) {
          v = __ldg(reinterpret_cast<const float4*>(rp));
        } else {
          v.x = __ldg(rp);
          if (px + 1 < HW) v.y = __ldg(rp + 1);
          if (px + 2 < HW) v.z = __ldg(rp + 2);
          if (px + 3 < HW) v.w = __ldg(rp + 3);
        }
      }
      tile[ch][q] = v.x; tile[ch][q + 1] = v.y; tile[ch][q + 2] = v.z; tile[ch][q + 3] = v.w;
    }
    __syncthreads();
    // store: thread -> (pixel, 4 channels); Cp is a multiple of 4 and the copy is 16-byte aligned
    float* dst = in_nhwc + static_cast<long long>(img) * HW * Cp;
    for (int i = threadIdx.x; i < kPrePx * (kPreCh / 4); i += 256) {
      const int cg = (i % (kPreCh / 4)) * 4, q = i / (kPreCh / 4);
      const int c = c0 + cg, px = p0 + q;
      if (px < HW && c < Cp)
        *reinterpret_cast<float4*>(dst + static_cast<long long>(px) * Cp + c) =
            make_float4(tile[cg][q], tile[cg + 1][q], tile[cg + 2][q], tile[cg + 3][q]);
    }
  } else {
    // Filter [K][Cg][RS] -> [K][RS][cchunks*32]: a block takes, for one output channel, a run of
    // `cpp` input channels x RS taps (contiguous in the source), turns it in shared memory and
    // writes `cpp` contiguous channels per tap; both sides of the copy are coalesced.
    float* buf = &tile[0][0];
    constexpr int kBuf = kPreCh * (kPrePx + 1);
    const int cpad = cchunks * 32;
    // runs start on multiples of 4 channels so that both sides can move 16 bytes at a time
    const int cpp = RS * 4 > kBuf ? 1 : ((kBuf / RS) & ~3) < cpad ? ((kBuf / RS) & ~3) : cpad;
    const int pieces = (cpad + cpp - 1) / cpp;
    const long long kdim = static_cast<long long>(RS) * cpad;
    const long long work = static_cast<long long>(K) * pieces;
    for (long long u = bid - in_blocks; u < work; u += w_blocks) {
      const int ko = static_cast<int>(u / pieces);
      const int c0 = static_cast<int>(u % pieces) * cpp;
      const int nch = cpad - c0 < cpp ? cpad - c0 : cpp;
      if (RS <= kBuf) {
        const float* src = wgt + (static_cast<long long>(ko) * Cg + c0) * RS;
        const int real = Cg - c0 < nch ? (Cg - c0 > 0 ? Cg - c0 : 0) : nch;  // channels that exist in the source
        const int nreal = real * RS;
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
          const float4* src4 = reinterpret_cast<const float4*>(src);
          float4* buf4 = reinterpret_cast<float4*>(buf);
          for (int i = threadIdx.x; i < nreal / 4; i += blockDim.x) buf4[i] = __ldg(src4 + i);
          for (int i = (nreal & ~3) + threadIdx.x; i < nch * RS; i += blockDim.x)
            buf[i] = (i < nreal) ? __ldg(src + i) : 0.0f;
        } else {
          for (int i = threadIdx.x; i < nch * RS; i += blockDim.x) buf[i] = (i < nreal) ? __ldg(src + i) : 0.0f;
        }
        __syncthreads();
        float* dst = w_packed + ko * kdim + c0;
        if ((nch & 3) == 0 && cpp > 1) {
          const int nq = nch >> 2;
          for (int j = threadIdx.x; j < nq * RS; j += blockDim.x) {
            const int rs = j / nq, cc = (j - rs * nq) * 4;
            *reinterpret_cast<float4*>(dst + static_cast<long long>(rs) * cpad + cc) =
                make_float4(buf[cc * RS + rs], buf[(cc + 1) * RS + rs], buf[(cc + 2) * RS + rs], buf[(cc + 3) * RS + rs]);
          }
        } else {
          for (int j = threadIdx.x; j < nch * RS; j += blockDim.x) {
            const int rs = j / nch, cc = j - rs * nch;
            dst[static_cast<long long>(rs) * cpad + cc] = buf[cc * RS + rs];
          }
        }
        __syncthreads();
      } else {
        // a filter with more taps than the buffer holds: plain gather
        for (int j = threadIdx.x; j < nch * RS; j += blockDim.x) {
          const int rs = j / nch, cc = j - rs * nch;
          const int c = c0 + cc;
          w_packed[ko * kdim + static_cast<long long>(rs) * cpad + c] =
              (c < Cg) ? wgt[(static_cast<long long>(ko) * Cg + c) * RS + rs] : 0.0f;
        }
      }
    }
  }
}

// Launches the layout pass both conv kernels read from (input to channels-last, filter packed).
// `zero` (may be null): `zero_n` floats of the result to clear in the same launch.
static int conv_prepass(const float* in, const float* weight, float* in_nhwc, float* w_packed, int64_t n, int64_t c,
                        int64_t h, int64_t w, int64_t k, int64_t cg, int64_t r, int64_t s, const ConvWs& ws,
                        int num_sms, void* stream_v, float* zero = nullptr, long long zero_n = 0, int sub_q = 0,
                        int sub_p = 0, int sub_sh = 1, int sub_sw = 1, bool grouped = false, int parts = 3) {
  // parts: bit 0 = copy the input, bit 1 = pack the filter
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // sub_q > 0: keep sub_p x sub_q pixels of every plane, every sub_sh-th row and sub_sw-th column
  const int plane = static_cast<int>(h * w);
  const int HW = sub_q > 0 ? sub_p * sub_q : plane;
  const int hw_tiles = (HW + kPrePx - 1) / kPrePx, c_tiles = static_cast<int>((ws.cp + kPreCh - 1) / kPreCh);
  const int in_blocks = (parts & 1) ? static_cast<int>(n) * hw_tiles * c_tiles : 0;
  // one work unit of the filter packing = one output channel x one run of input channels
  const long long wtotal = k * r * s * ws.cchunks * 32;
  long long w_units = (wtotal + 2047) / 2048;
  if (w_units < k) w_units = k;
  int w_blocks = (parts & 2) ? static_cast<int>(w_units > 8ll * num_sms ? 8ll * num_sms : w_units) : 0;
  int z_blocks = 0;
  if (zero && zero_n > 0) {
    const long long want = (zero_n / 4 + 255) / 256;
    z_blocks = static_cast<int>(want < 1 ? 1 : want > 2 * num_sms ? 2 * num_sms : want);
  }
  if (in_blocks + w_blocks + z_blocks == 0) return FTB_OK;
  conv_prepass_kernel<<<in_blocks + w_blocks + z_blocks, 256, 0, stream>>>(
      in, weight, in_nhwc, w_packed, static_cast<int>(n), static_cast<int>(c), HW, static_cast<int>(ws.cp),
      static_cast<int>(k), static_cast<int>(cg), static_cast<int>(r * s), static_cast<int>(ws.cchunks), hw_tiles,
      c_tiles, in_blocks, w_blocks, zero, zero_n, plane, sub_q, sub_sh * static_cast<int>(w), sub_sw,
      grouped ? static_cast<int>(ws.cgp) : 0);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return FTB_E_CUDA;
  }
  return FTB_OK;
}

// Conv tiles of at most 128 output channels hand pipeline stages back two at a time unless told
// otherwise: their K block is so short (four MMAs of about a hundred cycles) that the ~80 cycles of a
// tcgen05.commit show (3-6 % on batched 64- and 128-channel layers; nothing at 256).  A stage count
// the library chose itself is made even for it.
static int conv_release_pairs(const ftb_config* user, bool split3, ftb_config* cfg) {
  const int release = user ? user->release : 0;
  if (split3 || release == 1) return 0;
  if (release == 0) {
    if (cfg->tile_n > 128) return 0;
    if ((!user || user->stages == 0) && cfg->stages >= 5 && (cfg->stages & 1)) --cfg->stages;
  }
  return (cfg->stages % 2 == 0 && cfg->stages >= 4) ? 1 : 0;
}

// One wave of conv tiles or less, knobs left open: pick tile width and reduction split together by
// what a CTA has to stage and issue (same cost model as pick_small_f32: a short tile list is
// bound by per-CTA L2 traffic and MMA chain, not by latency).  An MMA costs about the same
// whatever its width up to 128 columns, so narrow tiles only pay when they put idle SMs to work.
static bool pick_small_conv(const ftb_config* user, long long groups, long long tiles_m, int64_t kg, int num_kb,
                            bool split3, int num_sms, ftb_config* tuned) {
  if (user && (user->tile_n != 0 || user->cluster != 0 || user->split_k != 0)) return false;
  if (groups * tiles_m * ((kg + 127) / 128) > num_sms) return false;
  double best = 1e30;
  int best_bn = 0, best_split = 1;
  for (int bn = 32; bn <= 256; bn *= 2) {
    if (bn > 32 && bn >= 2 * kg) break;  // wider than the output channels: pure padding
    const long long tiles = groups * tiles_m * ((kg + bn - 1) / bn);
    if (tiles > num_sms) continue;
    for (int split = 1; split <= 32 && split <= num_kb; ++split) {
      if (num_kb % split) continue;
      if (tiles * split > num_sms) break;
      const int kb = num_kb / split;
      const double mma_us = (bn >= 256 ? 0.140 : bn >= 128 ? 0.090 : bn >= 64 ? 0.061 : 0.050) * (split3 ? 3.0 : 1.0);
      const double load = kb * (16384.0 + bn * 128.0) / 60e3;
      const double math = kb * 4.0 * mma_us;
      const double cost = (load > math ? load : math) + 128.0 * bn * 4.0 / 35e3 + (split > 1 ? 0.5 : 0.0);
      if (cost < best) {
        best = cost;
        best_bn = bn;
        best_split = split;
      }
    }
  }
  if (!best_bn) return false;
  memset(tuned, 0, sizeof(*tuned));
  if (user) *tuned = *user;
  tuned->cluster = 1;
  tuned->tile_n = best_bn;
  tuned->split_k = best_split;
  return true;
}

// Plan of the slab kernel (ftb_conv_slab_kernel.cuh) for one conv2d; `ok` is false when the
// shape or the knobs do not fit it.
struct SlabPlan {
  bool ok;
  bool pair;  // two CTAs of a cluster on two consecutive tiles (cta_group::2)
  bool gather;  // slabs built from the NCHW tensor by loader warps (no channels-last copy)
  ConvSlabParams p;
  int ctas;
  size_t smem;
  uint32_t box_w, box_h;
};

static SlabPlan plan_slab(const ftb_config* user, int64_t n, int64_t kg, int64_t P, int64_t Q, int64_t r, int64_t s,
                          int64_t cchunks, int dil_h, int dil_w, int pad_h, int pad_w, bool out_aligned,
                          int num_sms, bool cl_out = false) {
  SlabPlan sp;
  memset(&sp, 0, sizeof(sp));
  if (kg > 256) return sp;
  const int halo_w = static_cast<int>(s - 1) * dil_w, halo_h = static_cast<int>(r - 1) * dil_h;
  if (halo_w >= 64 || halo_h >= 128) return sp;
  // Bulk tensor stores of the result need 16-byte aligned rows and boxes.
  // (a channels-last result has its channels innermost: the caller has checked their pitch)
  const bool staged_ok = out_aligned && (cl_out || Q % 4 == 0);
  int tile_w = static_cast<int>(Q < 128 - halo_w ? Q : 128 - halo_w);
  if (tile_w < Q && staged_ok && !cl_out) tile_w &= ~3;
  const int slab_w = tile_w + halo_w;
  int tile_h = 128 / slab_w;
  if (tile_h > P) tile_h = static_cast<int>(P);
  if (user && user->tile_h > 0) {
    if (user->tile_h > tile_h) return sp;
    tile_h = user->tile_h;
  }
  const int slab_h = tile_h + halo_h;
  if (slab_h > 256) return sp;
  const int bn = static_cast<int>((kg + 15) / 16 * 16);
  if (user && user->tile_n != 0 && user->tile_n < kg) return sp;  // the kernel keeps all output channels in one tile
  const long long slab_rows = static_cast<long long>(slab_h) * slab_w;
  // The furthest tap reads 128 rows from its offset: past the end of what was loaded it reads
  // whatever follows in shared memory (into rows that are never stored), so the bytes after the
  // last slab must exist.
  long long reach_rows = static_cast<long long>(halo_h) * slab_w + halo_w + 128;
  if (reach_rows < slab_rows) reach_rows = slab_rows;
  const uint32_t slab_stride = static_cast<uint32_t>((slab_rows * 128 + 1023) / 1024 * 1024);
  const size_t tail = static_cast<size_t>(reach_rows * 128 > slab_stride ? reach_rows * 128 - slab_stride : 0);
  const uint32_t epi_buf = staged_ok ? static_cast<uint32_t>((32ll * tile_h * tile_w * 4 + 127) / 128 * 128) : 0u;
  const int tiles_w = static_cast<int>((Q + tile_w - 1) / tile_w);
  const int tiles_h = static_cast<int>((P + tile_h - 1) / tile_h);
  const long long tiles = n * tiles_h * tiles_w;
  if (tiles > 0x7fffffffll) return sp;
  // A CTA pair shares one MMA over two consecutive tiles and splits the filter rows between its CTAs.
  // Taken when asked for (cluster = 2) or, left open, when there are enough tiles to keep every pair
  // busy and more than 64 output channels (halving a 64-row filter tile saves little: 56.5 us single
  // against 60.3 us paired on 64 -> 64 channels at 56 x 56, batch 64; 99 against 60 us on 128 -> 128
  // at 28 x 28); it needs halves of the filter rows that are whole 8-row groups.
  const int want_cluster = user ? user->cluster : 0;
  bool pair = bn % 16 == 0 && num_sms >= 2 && want_cluster != 1 &&
              (want_cluster == 2 || (tiles >= 2ll * num_sms && bn > 64));
  const int taps = static_cast<int>(r * s);
  const size_t after_min = tail > epi_buf ? tail : epi_buf;
  if (!pair && want_cluster == 0 && bn % 16 == 0 && bn > 64 && num_sms >= 2 && tiles >= num_sms / 2 &&
      static_cast<size_t>(taps) * cchunks * bn * 128 + 2 * static_cast<size_t>(slab_stride) + after_min + 1024 > kSmemLimit) {
    // A filter that will be streamed: a pair halves the ring and the filter bytes each SM pulls from
    // L2 per tile (256 -> 256 channels at 14 x 14, batch 64: 48 us paired against 60 us single).
    pair = true;
  }
  sp.pair = pair;
  const uint32_t b_tile = static_cast<uint32_t>(pair ? bn / 2 : bn) * 128u;
  auto fits = [&](int split, int* a_stages, int* epi_bufs) {
    const int tps = (taps + split - 1) / split;
    const size_t b_bytes = static_cast<size_t>(tps) * cchunks * b_tile;
    if (b_bytes + 2 * static_cast<size_t>(slab_stride) + after_min + 1024 > kSmemLimit) return false;
    const size_t rest = kSmemLimit - 1024 - b_bytes;
    size_t st = (rest - after_min) / slab_stride;
    if (st > static_cast<size_t>(kSlabMaxStages)) st = kSlabMaxStages;
    *a_stages = static_cast<int>(st);
    *epi_bufs = epi_buf == 0 ? 0 : (rest - st * slab_stride >= 2 * static_cast<size_t>(epi_buf) ? 2 : 1);
    return true;
  };
  // The filter streamed through a ring instead of resident: stages of `group` taps' tiles (a filter
  // row where that fits, else single taps), at least two of them and two slabs.
  auto fits_streamed = [&](int* a_stages, int* epi_bufs, int* b_stages, int* b_group) {
    const int cand[][2] = {{static_cast<int>(s), 4}, {static_cast<int>(s), 3}, {1, 8}, {1, 6}, {1, 4},
                           {static_cast<int>(s), 2}, {1, 3}, {1, 2}};
    for (const auto& c : cand) {
      const int group = c[0] > taps ? taps : c[0];
      const size_t ring = static_cast<size_t>(c[1]) * group * b_tile;
      if (ring + 2 * static_cast<size_t>(slab_stride) + after_min + 1024 > kSmemLimit) continue;
      const size_t rest = kSmemLimit - 1024 - ring;
      size_t st = (rest - after_min) / slab_stride;
      if (st > static_cast<size_t>(kSlabMaxStages)) st = kSlabMaxStages;
      *a_stages = static_cast<int>(st);
      *epi_bufs = epi_buf == 0 ? 0 : (rest - st * slab_stride >= 2 * static_cast<size_t>(epi_buf) ? 2 : 1);
      *b_stages = c[1];
      *b_group = group;
      return true;
    }
    return false;
  };
  int split = 0, a_stages = 0, epi_bufs = 0, b_stages = 0, b_group = 0;
  const int algo = user ? user->algo : 0;
  const long long units_for_tiles = pair ? num_sms / 2 : num_sms;
  const long long steps_all = pair ? (tiles + 1) / 2 : tiles;
  if (algo == 5) {
    // asked for: streamed filter, every tap in one CTA
    if ((user && user->split_k > 1) || !fits_streamed(&a_stages, &epi_bufs, &b_stages, &b_group)) return sp;
    split = 1;
  } else if ((!user || user->split_k == 0) && !fits(1, &a_stages, &epi_bufs) && 2 * steps_all >= units_for_tiles &&
             fits_streamed(&a_stages, &epi_bufs, &b_stages, &b_group)) {
    // a filter that cannot stay resident, enough tiles to keep the SMs busy without splitting the taps
    split = 1;
  } else if (user && user->split_k > 0) {
    split = user->split_k;
    if (split > taps || !fits(split, &a_stages, &epi_bufs)) return sp;
  } else {
    // Splitting the taps over CTAs fills idle SMs when the tile list is short (at the price of
    // adding partial sums in global memory) and shrinks the resident filter when it would not
    // fit otherwise.
    long long want = (pair ? num_sms / 2 : num_sms) / (tiles > 0 ? (pair ? (tiles + 1) / 2 : tiles) : 1);
    if (want > 4) want = 4;
    for (int d = 1; d <= taps; ++d) {
      if ((d - 1) * ((taps + d - 1) / d) >= taps) continue;  // would leave a split without taps
      if (!fits(d, &a_stages, &epi_bufs)) continue;
      if (split == 0 || d <= want) split = d;
      if (d >= want) break;
    }
    if (split == 0 || !fits(split, &a_stages, &epi_bufs)) return sp;
  }
  const int tps = (taps + split - 1) / split;
  ConvSlabParams& p = sp.p;
  p.N = static_cast<int>(kg);
  p.bn = bn;
  p.tiles = static_cast<int>(tiles);
  p.tiles_h = tiles_h; p.tiles_w = tiles_w; p.tile_h = tile_h; p.tile_w = tile_w; p.slab_w = slab_w;
  p.R = static_cast<int>(r); p.S = static_cast<int>(s); p.cchunks = static_cast<int>(cchunks);
  p.split = split; p.taps_per_split = tps;
  p.dil_h = dil_h; p.dil_w = dil_w; p.pad_h = pad_h; p.pad_w = pad_w;
  p.P = static_cast<int>(P); p.Q = static_cast<int>(Q);
  p.a_stages = a_stages;
  p.b_stages = b_stages;
  p.b_group = b_group > 0 ? b_group : 1;
  p.epi_bufs = epi_bufs;
  p.cl_out = cl_out ? 1 : 0;
  p.epi_buf_bytes = epi_buf;
  p.slab_bytes = static_cast<uint32_t>(slab_rows * 128);
  p.slab_alloc = slab_stride;
  p.b_tile_bytes = b_tile;
  p.idesc = make_idesc(kind_info(KIND_TF32), bn, 0, 0, pair ? 2 * kTileM : kTileM);
  p.dual = bn <= 128 ? 1 : 0;  // two accumulators per tile fit tensor memory's 512 columns twice over
  const long long units_avail = pair ? num_sms / 2 : num_sms;
  const long long steps = pair ? (tiles + 1) / 2 : tiles;
  long long walkers = units_avail / split;
  if (user && user->ctas > 0) walkers = (pair ? user->ctas / 2 : user->ctas) / split;
  if (walkers > steps) walkers = steps;
  if (walkers < 1) walkers = 1;
  sp.ctas = static_cast<int>(walkers) * split * (pair ? 2 : 1);
  const size_t after = static_cast<size_t>(epi_bufs) * epi_buf > tail ? static_cast<size_t>(epi_bufs) * epi_buf : tail;
  const size_t filter_bytes = b_stages > 0 ? static_cast<size_t>(b_stages) * p.b_group * b_tile
                                           : static_cast<size_t>(tps) * cchunks * b_tile;
  sp.smem = filter_bytes + static_cast<size_t>(a_stages) * slab_stride + after + 1024;
  sp.box_w = static_cast<uint32_t>(slab_w);
  sp.box_h = static_cast<uint32_t>(slab_h);
  sp.ok = true;
  return sp;
}

static int launch_slab(const CUtensorMap& tin, const CUtensorMap& tw, const StoreMaps& tout, const SlabPlan& sp,
                       cudaStream_t stream) {
  static std::mutex mu;
  static bool done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !done[dev]) {
      cudaError_t attr_err = cudaSuccess;
      const void* kernels[8] = {reinterpret_cast<const void*>(conv_slab_kernel<false, false, false>),
                                reinterpret_cast<const void*>(conv_slab_kernel<false, true, false>),
                                reinterpret_cast<const void*>(conv_slab_kernel<true, false, false>),
                                reinterpret_cast<const void*>(conv_slab_kernel<true, true, false>),
                                reinterpret_cast<const void*>(conv_slab_kernel<false, false, true>),
                                reinterpret_cast<const void*>(conv_slab_kernel<false, true, true>),
                                reinterpret_cast<const void*>(conv_slab_kernel<true, false, true>),
                                reinterpret_cast<const void*>(conv_slab_kernel<true, true, true>)};
      for (int i = 0; i < 8 && attr_err == cudaSuccess; ++i)
        attr_err = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kSmemLimit));
      if (attr_err != cudaSuccess) {
        set_last_cuda_error(static_cast<int>(attr_err));
        return FTB_E_CUDA;
      }
      done[dev] = true;
    }
  }
  // Programmatic dependent of the layout pass launched just before it on this stream.
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.gridDim = dim3(static_cast<unsigned>(sp.ctas), 1, 1);
  lc.blockDim = dim3(sp.gather ? 480 : 224, 1, 1);
  lc.dynamicSmemBytes = sp.smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  if (sp.pair) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    lc.numAttrs = 2;
  }
  const bool streamed = sp.p.b_stages > 0;
  if (sp.pair && streamed && sp.gather) cudaLaunchKernelEx(&lc, conv_slab_kernel<true, true, true>, tin, tw, tout, sp.p);
  else if (sp.pair && streamed) cudaLaunchKernelEx(&lc, conv_slab_kernel<true, true, false>, tin, tw, tout, sp.p);
  else if (sp.pair && sp.gather) cudaLaunchKernelEx(&lc, conv_slab_kernel<true, false, true>, tin, tw, tout, sp.p);
  else if (sp.pair) cudaLaunchKernelEx(&lc, conv_slab_kernel<true, false, false>, tin, tw, tout, sp.p);
  else if (streamed && sp.gather) cudaLaunchKernelEx(&lc, conv_slab_kernel<false, true, true>, tin, tw, tout, sp.p);
  else if (streamed) cudaLaunchKernelEx(&lc, conv_slab_kernel<false, true, false>, tin, tw, tout, sp.p);
  else if (sp.gather) cudaLaunchKernelEx(&lc, conv_slab_kernel<false, false, true>, tin, tw, tout, sp.p);
  else cudaLaunchKernelEx(&lc, conv_slab_kernel<false, false, false>, tin, tw, tout, sp.p);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(static_cast<int>(e));
    return FTB_E_CUDA;
  }
  return FTB_OK;
}

int conv2d_generic(const float* in, const float* weight, const float* bias, float* out, int64_t n,
                   int64_t c, int64_t h, int64_t w, int64_t k, int64_t r, int64_t s, int stride_h,
                   int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups,
                   const ftb_config* user, void* workspace, size_t workspace_bytes, int* status,
                   void* stream_v, float* const* extra_dst, int num_extra, int filter_mode, int layout) {
  // filter_mode: 0 = pack the filter and run; 1 = pack the filter into the workspace and return;
  // 2 = the workspace already holds this filter's packing (same shape arguments and knobs)
  // layout: 0 = NCHW input and result; 1 = channels-last input [N][H][W][C] and result [N][P][Q][K]:
  // the kernels read the input where it lies (it already has the layout their tensor maps want) and
  // the layout pass only packs the filter
  if (filter_mode < 0 || filter_mode > 2 || layout < 0 || layout > 1) return FTB_E_BAD_ARG;
  const bool pack_only = filter_mode == 1;
  const bool cl = layout == 1;
  const int parts = (pack_only ? 2 : filter_mode == 2 ? 1 : 3) & (cl ? 2 : 3);
  if (!weight || (!pack_only && (!in || !out))) return FTB_E_BAD_ARG;
  if (num_extra < 0 || num_extra > kMaxDst - 1 || (num_extra > 0 && !extra_dst)) return FTB_E_BAD_ARG;
  for (int d = 0; d < num_extra; ++d)
    if (!extra_dst[d] || (reinterpret_cast<uintptr_t>(extra_dst[d]) & 15)) return FTB_E_BAD_ARG;
  // Several destinations exist only in the epilogues that leave through bulk tensor stores and
  // add nothing in global memory: the reduction is then kept inside one CTA per tile.
  ftb_config multi_cfg;
  if (user && (user->relu < 0 || user->relu > 1)) return FTB_E_BAD_CONFIG;
  const int relu = user ? user->relu : 0;
  if (num_extra > 0 || relu) {
    memset(&multi_cfg, 0, sizeof(multi_cfg));
    if (user) multi_cfg = *user;
    if (multi_cfg.split_k > 1) return num_extra > 0 ? FTB_E_UNSUPPORTED : FTB_E_BAD_CONFIG;
    if (num_extra > 0 && multi_cfg.epilogue == 1) return FTB_E_UNSUPPORTED;
    multi_cfg.split_k = 1;  // partial sums cannot be clamped, nor added into a peer's memory
    user = &multi_cfg;
  }
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || k <= 0 || r <= 0 || s <= 0 || groups <= 0) return FTB_E_BAD_ARG;
  if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0 || pad_h < 0 || pad_w < 0) return FTB_E_BAD_ARG;
  if (c % groups || k % groups) return FTB_E_BAD_ARG;
  const int64_t P = (h + 2 * pad_h - dil_h * (r - 1) - 1) / stride_h + 1;
  const int64_t Q = (w + 2 * pad_w - dil_w * (s - 1) - 1) / stride_w + 1;
  if (P <= 0 || Q <= 0) return FTB_E_BAD_ARG;
  if (n * c * h * w > (1ll << 31) || n * k * P * Q > (1ll << 31)) return FTB_E_TOO_LARGE;
  int rc = device_ok();
  if (rc) return rc;
  const int64_t cg = c / groups, kg = k / groups;
  ConvWs ws = conv_ws(n, c, h, w, k, r, s, groups);
  if (cl) {
    // Tensor maps on the caller's tensors: 16-byte aligned bases and pitches.
    if (cg % 4 || kg % 4) return FTB_E_UNSUPPORTED;
    if (!pack_only && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15)) return FTB_E_UNSUPPORTED;
    ws.cgp = cg;
    ws.cp = c;
    ws.in_bytes = 0;  // the workspace holds the packed filter only
  }
  if (!workspace || workspace_bytes < static_cast<size_t>(ws.in_bytes + ws.w_bytes)) return FTB_E_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FTB_E_WORKSPACE;
  float* in_nhwc = cl ? const_cast<float*>(in) : static_cast<float*>(workspace);
  float* w_packed = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ws.in_bytes);

  const KindInfo ki = kind_info(KIND_TF32);
  const bool split3 = user && user->fp32_mode == 1;
  if (user && (user->fp32_mode < 0 || user->fp32_mode > 1)) return FTB_E_BAD_CONFIG;
  const int num_sms = sm_count();

  const int algo = user ? user->algo : 0;
  if (algo < 0 || algo > 5) return FTB_E_BAD_CONFIG;
  const bool slab_asked = algo == 2 || algo == 5;  // 5: the slab kernel with its filter streamed
  // A 1x1 filter at stride 1 without padding is a batched GEMM on the NCHW tensors as they are:
  // out[b] (K x HW) = weight (K x C) * in[b] (C x HW), the pixels being the contiguous dimension
  // of both the B operand and the result.  No layout pass, no workspace traffic.
  {
    const bool is_gemm = !cl && r == 1 && s == 1 && stride_h == 1 && stride_w == 1 && pad_h == 0 && pad_w == 0 &&
                         groups == 1 && (h * w) % 4 == 0 && c % 4 == 0 &&
                         ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0;
    if (algo == 3 && !is_gemm && !pack_only) return FTB_E_UNSUPPORTED;
    if (algo == 3 && relu) return FTB_E_UNSUPPORTED;  // the GEMM epilogue has no clamp
    if (is_gemm && (algo == 0 || algo == 3) && !pack_only && !relu) {
      ftb_config gcfg;
      memset(&gcfg, 0, sizeof(gcfg));
      if (user) {
        gcfg = *user;
        gcfg.tile_h = 0;
        gcfg.algo = 0;
      }
      GemmExtras ex;
      ex.a_broadcast = 1;
      ex.row_bias = bias;
      return gemm_generic(KIND_TF32, OUT_F32, weight, in, out, n, k, h * w, c, 0, 0, user ? &gcfg : nullptr, status,
                          stream_v, reinterpret_cast<void* const*>(extra_dst), num_extra, &ex);
    }
  }
  // Few input channels: continue as a 1x1, stride-1, unpadded conv over the im2col form, an
  // [n][P][Q][Kp] channels-last image (written by conv_im2col_kernel where the layout pass would run).
  ConvWs wsx = ws;
  bool im2col = false;
  struct { int64_t c, h, w, r, s; int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w; } orig =
      {c, h, w, r, s, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w};
  if (!cl && (algo == 0 || algo == 4) && conv_small_c(c, r, s, groups)) {
    const int64_t kp = round_up(r * s * c, 32);
    if (round_up(n * P * Q * kp * 4, 1024) <= ws.in_bytes && n * P * Q * kp < (1ll << 31)) {
      im2col = true;
      wsx.cp = kp;
      wsx.cchunks = kp / 32;
      h = P; w = Q; r = 1; s = 1;
      stride_h = stride_w = 1; pad_h = pad_w = 0; dil_h = dil_w = 1;
    }
  }
  if (algo == 4 && !im2col) return FTB_E_UNSUPPORTED;
  // A strided 1x1 filter without padding reads only every stride-th pixel: the layout pass copies
  // just those, and what follows is a stride-1 conv over the P x Q image of kept pixels.
  int sub_sh = 1, sub_sw = 1;
  const int64_t h_in = h, w_in = w;
  if (!cl && !im2col && r == 1 && s == 1 && pad_h == 0 && pad_w == 0 && (stride_h > 1 || stride_w > 1)) {
    sub_sh = stride_h;
    sub_sw = stride_w;
    h = P;
    w = Q;
    stride_h = stride_w = 1;
  }
  const bool subsample = sub_sh > 1 || sub_sw > 1;
  // Filters with more than one tap at stride 1 go to the slab kernel when it can take them.
  SlabPlan sp;
  sp.ok = false;
  // (cluster = 2 without algo = 2 keeps meaning the per-tap lowering on CTA pairs)
  if (algo != 1 && groups == 1 && stride_h == 1 && stride_w == 1 && !split3 && (r * s > 1 || slab_asked) &&
      !(user && user->cluster == 2 && !slab_asked))
    sp = plan_slab(user, n, kg, P, Q, r, s, ws.cchunks, dil_h, dil_w, pad_h, pad_w,
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0, num_sms, cl);
  if (sp.ok && num_extra > 0 && (sp.p.epi_bufs == 0 || sp.p.split > 1)) sp.ok = false;
  if (slab_asked && !sp.ok) return FTB_E_UNSUPPORTED;
  // Left to itself the slab kernel is taken when the whole filter stays resident, or when the tile
  // list is shorter than half the SM count (where a split reduction is wanted anyway); a long tile list
  // with the taps split would add every partial sum of a large result in global memory.
  if (sp.ok && algo == 0 && sp.p.split > 1 && 2ll * sp.p.tiles > num_sms) sp.ok = false;
  if (user && (user->gather < 0 || user->gather > 2)) return FTB_E_BAD_CONFIG;
  if (sp.ok) {
    if (user) {
      rc = ftb_validate(3, user, n * P * Q, k, c * r * s);
      if (rc) return rc;
    }
    // NCHW input: the slabs are either TMA loads from a channels-last copy made by the layout pass, or
    // built from the NCHW tensor by loader warps inside the kernel (no copy: the input crosses HBM once
    // instead of three times).  Left open, the gather is taken for long tile lists whose taps are not
    // split and whose slab rows fit two warp-wide loads (64 -> 64 at 56 x 56, batch 64: 59.9 against
    // 72.8 us; 128 -> 128 at 56 x 56: 161 against 187); short lists (batch 1: 9.3 against 8.9 us) and wide
    // rows (64 -> 192 at 112 x 112, batch 8: 68.1 against 63.8) stay with the layout pass.
    const int want_gather = user ? user->gather : 0;
    sp.gather = !cl && (want_gather == 2 ||
                        (want_gather == 0 && sp.p.split == 1 && sp.p.tiles >= 2 * num_sms && sp.p.slab_w <= 64));
    rc = conv_prepass(in, weight, in_nhwc, w_packed, n, c, h, w, k, cg, r, s, ws, num_sms, stream_v,
                      (sp.p.split > 1 && !pack_only) ? out : nullptr, n * k * P * Q, 0, 0, 1, 1, false,
                      sp.gather ? (parts & ~1) : parts);
    if (rc || pack_only) return rc;
    sp.p.in_nchw = in;
    sp.p.n_imgs = static_cast<int>(n);
    sp.p.C = static_cast<int>(c);
    sp.p.H = static_cast<int>(h);
    sp.p.W = static_cast<int>(w);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    sp.p.out = out;
    sp.p.bias = bias;
    sp.p.relu = relu;
    sp.p.diag = user ? user->reserved[0] : 0;
    if (sp.p.diag & 128) sp.p.dual = 0;  // (diagnostic: one issuing thread)
    sp.p.conv_ktot = static_cast<int>(k);
    sp.p.status = status ? status : fallback_status();
    if (!sp.p.status) return FTB_E_CUDA;
    CUtensorMap tin, tw;
    memset(&tin, 0, sizeof(tin));
    if (!sp.gather) {
      uint64_t dims[4] = {static_cast<uint64_t>(ws.cp), static_cast<uint64_t>(w), static_cast<uint64_t>(h),
                          static_cast<uint64_t>(n)};
      uint64_t strides[3] = {static_cast<uint64_t>(ws.cp) * 4, static_cast<uint64_t>(w) * ws.cp * 4,
                             static_cast<uint64_t>(h) * w * ws.cp * 4};
      uint32_t box[4] = {32, sp.box_w, sp.box_h, 1};
      const uint32_t ones[4] = {1, 1, 1, 1};
      rc = make_tmap(&tin, ki.dt, 4, in_nhwc, dims, strides, box, ones);
      if (rc) return rc;
    }
    {
      const uint64_t kdim = static_cast<uint64_t>(r * s * ws.cchunks) * 32;
      uint64_t dims[3] = {kdim, static_cast<uint64_t>(kg), 1};
      uint64_t strides[2] = {kdim * 4, kdim * 4 * kg};
      uint32_t box[3] = {32, static_cast<uint32_t>(sp.pair ? sp.p.bn / 2 : sp.p.bn), 1};
      const uint32_t ones[3] = {1, 1, 1};
      rc = make_tmap(&tw, ki.dt, 3, w_packed, dims, strides, box, ones);
      if (rc) return rc;
    }
    StoreMaps tout;
    memset(&tout, 0, sizeof(tout));
    sp.p.num_dst = 1 + num_extra;
    if (sp.p.epi_bufs && cl) {
      // (channel, w, h, image) view of the channels-last result; a box is 32 channels of one output tile
      uint64_t dims[4] = {static_cast<uint64_t>(k), static_cast<uint64_t>(Q), static_cast<uint64_t>(P),
                          static_cast<uint64_t>(n)};
      uint64_t strides[3] = {static_cast<uint64_t>(k) * 4, static_cast<uint64_t>(Q) * k * 4,
                             static_cast<uint64_t>(P) * Q * k * 4};
      uint32_t box[4] = {32, static_cast<uint32_t>(sp.p.tile_w), static_cast<uint32_t>(sp.p.tile_h), 1};
      const uint32_t ones[4] = {1, 1, 1, 1};
      // A staging row is one pixel's 32 channels = 128 bytes: with the 128-byte swizzle the lanes of a warp,
      // which hold consecutive pixels, write their 16-byte chunks without bank conflicts (staging buffers
      // that start on 1024-byte boundaries).
      sp.p.cl_swz = sp.p.epi_buf_bytes % 1024 == 0 ? 1 : 0;
      for (int d = 0; d < sp.p.num_dst; ++d) {
        rc = make_tmap(&tout.dst[d], ki.dt, 4, d == 0 ? out : extra_dst[d - 1], dims, strides, box, ones,
                       sp.p.cl_swz ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
      }
    } else if (sp.p.epi_bufs) {
      // (w, h, channel, image) view of the NCHW result; a box is 32 channels of one output tile.
      uint64_t dims[4] = {static_cast<uint64_t>(Q), static_cast<uint64_t>(P), static_cast<uint64_t>(k),
                          static_cast<uint64_t>(n)};
      uint64_t strides[3] = {static_cast<uint64_t>(Q) * 4, static_cast<uint64_t>(P) * Q * 4,
                             static_cast<uint64_t>(k) * P * Q * 4};
      uint32_t box[4] = {static_cast<uint32_t>(sp.p.tile_w), static_cast<uint32_t>(sp.p.tile_h), 32, 1};
      const uint32_t ones[4] = {1, 1, 1, 1};
      for (int d = 0; d < sp.p.num_dst; ++d) {
        rc = make_tmap(&tout.dst[d], ki.dt, 4, d == 0 ? out : extra_dst[d - 1], dims, strides, box, ones,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
      }
    }
    return launch_slab(tin, tw, tout, sp, stream);
  }

  // Output tile of the implicit GEMM: tile_h x tile_w pixels (<= 128) of one image.
  int tile_w = static_cast<int>(Q < 128 ? Q : 128);
  if (tile_w * stride_w > 256) tile_w = 256 / stride_w;
  int tile_h = user && user->tile_h > 0 ? user->tile_h : 128 / tile_w;
  if (tile_h > P) tile_h = static_cast<int>(P);
  if (tile_h < 1 || tile_h * tile_w > 128 || tile_h * stride_h > 256) return FTB_E_BAD_CONFIG;
  const int tiles_w = static_cast<int>((Q + tile_w - 1) / tile_w);
  const int tiles_h = static_cast<int>((P + tile_h - 1) / tile_h);
  const int num_kb = static_cast<int>(r * s * wsx.cchunks);
  // Images of at most 64 output pixels share a tile: as many whole images as fit in its 128 rows.
  int tile_imgs = 1;
  if (tiles_h == 1 && tiles_w == 1 && tile_h * tile_w <= 64 && !(user && user->tile_h > 0)) {
    tile_imgs = 128 / (tile_h * tile_w);
    if (tile_imgs > n) tile_imgs = static_cast<int>(n);
    if (tile_imgs * tile_h * stride_h > 256) tile_imgs = 1;
  }
  const long long tiles_m = tile_imgs > 1 ? (n + tile_imgs - 1) / tile_imgs
                                          : static_cast<long long>(n) * tiles_h * tiles_w;
  ftb_config cfg;
  // The result leaves through bulk tensor stores when they can address it (16-byte aligned rows
  // and boxes) and the staging buffers fit beside the chosen pipeline depth.
  bool staged = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && Q % 4 == 0 && tile_w % 4 == 0 &&
                (P * Q * 4) % 16 == 0 && (groups == 1 || (kg * P * Q * 4) % 16 == 0);
  if (cl) staged = true;  // channels innermost: base and pitches were checked above
  if (user && user->epilogue == 1) staged = false;  // per-thread stores asked for
  if (user && (user->epilogue < 0 || user->epilogue > 1)) return FTB_E_BAD_CONFIG;
  ftb_config tuned;
  const bool conv_tuned = pick_small_conv(user, groups, tiles_m, kg, num_kb, split3, num_sms, &tuned);
  if (conv_tuned) user = &tuned;
  rc = FTB_E_BAD_CONFIG;
  if (staged)
    rc = resolve_config(user, ki, split3, 0, !split3, groups, tiles_m * kTileM, kg, num_kb, true, num_sms, &cfg,
                        kEpilogueStaging);
  if (rc) {
    staged = false;
    rc = resolve_config(user, ki, split3, 0, !split3, groups, tiles_m * kTileM, kg, num_kb, true, num_sms, &cfg);
  }
  if (rc) return rc;
  if (num_extra > 0 && !staged) return FTB_E_UNSUPPORTED;
  const bool pair = cfg.cluster == 2;
  const long long tiles_m_launch = pair ? (tiles_m + 1) / 2 : tiles_m;
  if (!conv_tuned && (!user || user->split_k == 0) && num_extra == 0 && !relu) {
    // A short tile list leaves SMs idle: split the reduction so that about all SMs get work (the
    // partial sums meet in global memory through bulk reduce-adds into the zeroed result).
    const long long tiles = groups * tiles_m_launch * ((kg + cfg.tile_n - 1) / cfg.tile_n);
    int want = static_cast<int>((num_sms / (pair ? 2 : 1)) / (tiles > 0 ? tiles : 1));
    if (want > 32) want = 32;
    int pick = 1;
    for (int d = 2; d <= want; ++d)
      if (num_kb % d == 0) pick = d;
    cfg.split_k = pick;
  }

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (im2col) {
    if (cfg.split_k > 1 && !pack_only) {
      cudaError_t e = cudaMemsetAsync(out, 0, static_cast<size_t>(n * k * P * Q) * 4, stream);
      if (e != cudaSuccess) {
        set_last_cuda_error(static_cast<int>(e));
        return FTB_E_CUDA;
      }
    }
    const int kp = static_cast<int>(wsx.cp);
    const int segs = static_cast<int>((Q + kColSeg - 1) / kColSeg);
    const long long col_blocks = (parts & 1) ? n * P * segs : 0;
    long long w_blocks = (k * kp + 255) / 256;
    if (w_blocks > 2ll * num_sms) w_blocks = 2ll * num_sms;
    if (!(parts & 2)) w_blocks = 0;
    conv_im2col_kernel<<<static_cast<unsigned>(col_blocks + w_blocks), 256, 0, stream>>>(
        in, weight, in_nhwc, w_packed, static_cast<int>(n), static_cast<int>(orig.c), static_cast<int>(orig.h),
        static_cast<int>(orig.w), static_cast<int>(k), static_cast<int>(orig.r), static_cast<int>(orig.s),
        static_cast<int>(P), static_cast<int>(Q), kp, orig.stride_h, orig.stride_w, orig.pad_h, orig.pad_w,
        orig.dil_h, orig.dil_w, segs, static_cast<int>(col_blocks));
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_last_cuda_error(static_cast<int>(e));
      return FTB_E_CUDA;
    }
  } else {
    rc = conv_prepass(in, weight, in_nhwc, w_packed, n, c, h_in, w_in, k, cg, r, s, ws, num_sms, stream_v,
                      (cfg.split_k > 1 && !pack_only) ? out : nullptr, n * k * P * Q,
                      subsample ? static_cast<int>(Q) : 0, static_cast<int>(P), sub_sh, sub_sw, groups > 1, parts);
    if (rc) return rc;
  }
  if (pack_only) return FTB_OK;
  // One launch for all groups: a tile's batch coordinate is its group, and the tensor maps of
  // the operands and of the result carry a group dimension.
  {
    UmmaParams p;
    memset(&p, 0, sizeof(p));
    p.M = static_cast<int>(tiles_m) * kTileM;
    p.N = static_cast<int>(kg);
    p.K = num_kb * ki.kblk;
    p.batch = groups;
    p.conv_groups = groups;
    p.bn = cfg.tile_n;
    p.stages = cfg.stages;
    p.num_kb = num_kb;
    p.tiles_m = static_cast<int>(tiles_m_launch);
    p.conv_tiles = static_cast<int>(tiles_m);
    p.tiles_n = static_cast<int>((kg + p.bn - 1) / p.bn);
    p.raster = cfg.raster - 1;
    p.group_m = cfg.group_m;
    p.split_k = cfg.split_k;
    p.kblk = ki.kblk;
    p.idesc = make_idesc(ki, p.bn, 0, 0, pair ? 2 * kTileM : kTileM);
    p.b_rows = pair ? p.bn / 2 : p.bn;
    p.b_bytes = static_cast<uint32_t>(p.b_rows) * 128u;
    p.a_boxes = 1;
    p.a_box_mn = kTileM;
    p.a_box_bytes = static_cast<uint32_t>(tile_imgs * tile_h * tile_w) * 128u;
    p.tile_imgs = tile_imgs;
    p.n_imgs = static_cast<int>(n);
    p.a_lbo = 16; p.a_sbo = 1024; p.a_kadv = static_cast<uint32_t>(ki.umma_k * ki.esize);
    CUtensorMapSwizzle b_swz;
    operand_layout(ki, 0, p.b_rows, &p.b_boxes, &p.b_box_mn, &p.b_box_bytes, &p.b_lbo, &p.b_sbo, &p.b_kadv,
                   &p.b_layout, &b_swz);
    p.a_layout = 2;
    p.pair_m = pair ? 2 * kTileM : kTileM;
    p.conv = 1;
    p.conv_cl = cl ? 1 : 0;
    p.slab_cols = 32;
    if (user && (user->release < 0 || user->release > 2)) return FTB_E_BAD_CONFIG;
    p.release_pairs = conv_release_pairs(user, split3, &cfg);
    p.stages = cfg.stages;
    p.pdl = 1;  // directly follows the layout pass
    p.conv_ktot = static_cast<int>(k);
    p.conv_koff = 0;
    p.relu = relu;
    p.C = out;
    p.bias = bias;
    p.P = static_cast<int>(P); p.Q = static_cast<int>(Q);
    p.tile_h = tile_h; p.tile_w = tile_w; p.tiles_h = tiles_h; p.tiles_w = tiles_w;
    p.R = static_cast<int>(r); p.S = static_cast<int>(s); p.cchunks = static_cast<int>(wsx.cchunks);
    p.stride_h = stride_h; p.stride_w = stride_w; p.pad_h = pad_h; p.pad_w = pad_w;
    p.dil_h = dil_h; p.dil_w = dil_w;
    p.status = status ? status : fallback_status();
    if (!p.status) return FTB_E_CUDA;

    CUtensorMap ta, tb;
    if (groups > 1) {
      // (c in group, group, w, h, n) view of the channels-last copy: a group's channels beyond Cg
      // (padding of the copy, or the next group) lie outside dimension 0 and read as zeros.
      uint64_t dims[5] = {static_cast<uint64_t>(cg), static_cast<uint64_t>(groups), static_cast<uint64_t>(w),
                          static_cast<uint64_t>(h), static_cast<uint64_t>(n)};
      uint64_t strides[4] = {static_cast<uint64_t>(wsx.cgp) * 4, static_cast<uint64_t>(wsx.cp) * 4,
                             static_cast<uint64_t>(w) * wsx.cp * 4, static_cast<uint64_t>(h) * w * wsx.cp * 4};
      uint32_t box[5] = {static_cast<uint32_t>(ki.kblk), 1, static_cast<uint32_t>(tile_w * stride_w),
                         static_cast<uint32_t>(tile_h * stride_h), static_cast<uint32_t>(tile_imgs)};
      uint32_t es[5] = {1, 1, static_cast<uint32_t>(stride_w), static_cast<uint32_t>(stride_h), 1};
      rc = make_tmap(&ta, ki.dt, 5, in_nhwc, dims, strides, box, es);
      if (rc) return rc;
    } else {
      // (c, w, h, n) view of the channels-last copy
      uint64_t dims[4] = {static_cast<uint64_t>(wsx.cp), static_cast<uint64_t>(w),
                          static_cast<uint64_t>(h), static_cast<uint64_t>(n)};
      uint64_t strides[3] = {static_cast<uint64_t>(wsx.cp) * 4, static_cast<uint64_t>(w) * wsx.cp * 4,
                             static_cast<uint64_t>(h) * w * wsx.cp * 4};
      uint32_t box[4] = {static_cast<uint32_t>(ki.kblk), static_cast<uint32_t>(tile_w * stride_w),
                         static_cast<uint32_t>(tile_h * stride_h), static_cast<uint32_t>(tile_imgs)};
      uint32_t es[4] = {1, static_cast<uint32_t>(stride_w), static_cast<uint32_t>(stride_h), 1};
      rc = make_tmap(&ta, ki.dt, 4, in_nhwc, dims, strides, box, es);
      if (rc) return rc;
    }
    {
      // packed filter [group][k in group][taps x channel chunks x 32]
      const uint64_t kdim = static_cast<uint64_t>(num_kb) * ki.kblk;
      uint64_t dims[3] = {kdim, static_cast<uint64_t>(kg), static_cast<uint64_t>(groups)};
      uint64_t strides[2] = {kdim * 4, kdim * 4 * kg};
      uint32_t box[3] = {static_cast<uint32_t>(ki.kblk), static_cast<uint32_t>(p.b_rows), 1};
      const uint32_t ones[3] = {1, 1, 1};
      rc = make_tmap(&tb, ki.dt, 3, w_packed, dims, strides, box, ones);
      if (rc) return rc;
    }
    const long long total = static_cast<long long>(p.batch) * p.tiles_m * p.tiles_n * p.split_k;
    if (total > 0x7fffffffll) return FTB_E_TOO_LARGE;
    int ctas = cfg.ctas > 0 ? cfg.ctas : num_sms;
    if (pair) {
      if (ctas / 2 > total) ctas = static_cast<int>(total) * 2;
      ctas &= ~1;
      if (ctas < 2) ctas = 2;
    } else if (ctas > total) {
      ctas = static_cast<int>(total);
    }
    StoreMaps tc;
    memset(&tc, 0, sizeof(tc));
    if (staged && cl) {
      // channels-last result: (k, q, p, n), or (k in group, group, q, p, n) where a box of 32
      // channels is clipped at the end of its group; the staged slab is 128-byte swizzled
      p.tma_store = 1;
      p.num_dst = 1 + num_extra;
      const int rank = groups > 1 ? 5 : 4;
      uint64_t dims[5], strides[4];
      uint32_t box[5];
      const uint32_t ones[5] = {1, 1, 1, 1, 1};
      int i = 0;
      dims[i] = static_cast<uint64_t>(kg); box[i] = 32; ++i;
      if (groups > 1) {
        strides[i - 1] = static_cast<uint64_t>(kg) * 4;
        dims[i] = static_cast<uint64_t>(groups); box[i] = 1; ++i;
      }
      strides[i - 1] = static_cast<uint64_t>(k) * 4;
      dims[i] = static_cast<uint64_t>(Q); box[i] = static_cast<uint32_t>(tile_w); ++i;
      strides[i - 1] = static_cast<uint64_t>(Q) * k * 4;
      dims[i] = static_cast<uint64_t>(P); box[i] = static_cast<uint32_t>(tile_h); ++i;
      strides[i - 1] = static_cast<uint64_t>(P) * Q * k * 4;
      dims[i] = static_cast<uint64_t>(n); box[i] = static_cast<uint32_t>(tile_imgs); ++i;
      for (int d = 0; d < p.num_dst; ++d) {
        rc = make_tmap(&tc.dst[d], ki.dt, rank, d == 0 ? out : extra_dst[d - 1], dims, strides, box, ones,
                       CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
      }
    } else if (staged && groups > 1) {
      // (w, h, channel in group, group, image) view of the NCHW result: a box of 32 channels is
      // clipped at the end of its group
      p.tma_store = 1;
      p.num_dst = 1 + num_extra;
      uint64_t dims[5] = {static_cast<uint64_t>(Q), static_cast<uint64_t>(P), static_cast<uint64_t>(kg),
                          static_cast<uint64_t>(groups), static_cast<uint64_t>(n)};
      uint64_t strides[4] = {static_cast<uint64_t>(Q) * 4, static_cast<uint64_t>(P) * Q * 4,
                             static_cast<uint64_t>(kg) * P * Q * 4, static_cast<uint64_t>(k) * P * Q * 4};
      uint32_t box[5] = {static_cast<uint32_t>(tile_w), static_cast<uint32_t>(tile_h), 32, 1,
                         static_cast<uint32_t>(tile_imgs)};
      const uint32_t ones[5] = {1, 1, 1, 1, 1};
      for (int d = 0; d < p.num_dst; ++d) {
        rc = make_tmap(&tc.dst[d], ki.dt, 5, d == 0 ? out : extra_dst[d - 1], dims, strides, box, ones,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
      }
    } else if (staged) {
      // (w, h, channel, image) view of the NCHW result
      p.tma_store = 1;
      p.num_dst = 1 + num_extra;
      uint64_t dims[4] = {static_cast<uint64_t>(Q), static_cast<uint64_t>(P), static_cast<uint64_t>(k),
                          static_cast<uint64_t>(n)};
      uint64_t strides[3] = {static_cast<uint64_t>(Q) * 4, static_cast<uint64_t>(P) * Q * 4,
                             static_cast<uint64_t>(k) * P * Q * 4};
      uint32_t box[4] = {static_cast<uint32_t>(tile_w), static_cast<uint32_t>(tile_h), 32,
                         static_cast<uint32_t>(tile_imgs)};
      const uint32_t ones[4] = {1, 1, 1, 1};
      for (int d = 0; d < p.num_dst; ++d) {
        rc = make_tmap(&tc.dst[d], ki.dt, 4, d == 0 ? out : extra_dst[d - 1], dims, strides, box, ones,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
      }
    }
    rc = dispatch(KIND_TF32, OUT_F32, split3, pair, ta, tb, tc, p, ctas, stream);
    if (rc) return rc;
  }
  return FTB_OK;
}


// ------------------------------------------------------------------ conv3d (NCDHW)
// The same implicit GEMM as the per-tap conv2d path with one more tap loop: the layout pass
// writes an [N][D][H][W][Cp] copy (its "pixels" are the D*H*W voxels) and packs the filter as
// [K][T*R*S][cchunks*32]; the tile list walks (image, output depth) pairs as its images, and the
// depth of a tap is the second coordinate of a 5-D tensor map, so that depth padding is the map's
// out-of-range fill like the padding of rows and columns.  Groups run as one launch each, on maps
// based at the group's channels.
ConvWs conv3d_ws(int64_t n, int64_t c, int64_t d, int64_t h, int64_t w, int64_t k, int64_t t, int64_t r,
                 int64_t s, int64_t groups) {
  ConvWs ws;
  const int64_t cg = c / groups;
  ws.cgp = round_up(cg, 4);
  ws.cp = groups > 1 ? groups * ws.cgp : round_up(c, 4);
  ws.cchunks = (cg + 31) / 32;
  ws.in_bytes = round_up(n * d * h * w * ws.cp * 4, 1024);
  ws.w_bytes = round_up(k * t * r * s * ws.cchunks * 32 * 4, 1024);
  return ws;
}

int conv3d_generic(const float* in, const float* weight, const float* bias, float* out, int64_t n, int64_t c,
                   int64_t d, int64_t h, int64_t w, int64_t k, int64_t t, int64_t r, int64_t s, const int* stride,
                   const int* pad, const int* dil, int groups, const ftb_config* user, void* workspace,
                   size_t workspace_bytes, int* status, void* stream_v, bool prepacked) {
  // prepacked: the workspace already holds this filter's packing (an earlier call with the same
  // shape arguments and knobs): the layout pass copies the input only
  if (!in || !weight || !out || !stride || !pad || !dil) return FTB_E_BAD_ARG;
  if (n <= 0 || c <= 0 || d <= 0 || h <= 0 || w <= 0 || k <= 0 || t <= 0 || r <= 0 || s <= 0 || groups <= 0)
    return FTB_E_BAD_ARG;
  for (int i = 0; i < 3; ++i)
    if (stride[i] <= 0 || dil[i] <= 0 || pad[i] < 0) return FTB_E_BAD_ARG;
  if (c % groups || k % groups) return FTB_E_BAD_ARG;
  const int64_t OD = (d + 2 * pad[0] - dil[0] * (t - 1) - 1) / stride[0] + 1;
  const int64_t P = (h + 2 * pad[1] - dil[1] * (r - 1) - 1) / stride[1] + 1;
  const int64_t Q = (w + 2 * pad[2] - dil[2] * (s - 1) - 1) / stride[2] + 1;
  if (OD <= 0 || P <= 0 || Q <= 0) return FTB_E_BAD_ARG;
  if (n * c * d * h * w > (1ll << 31) || n * k * OD * P * Q > (1ll << 31)) return FTB_E_TOO_LARGE;
  // A filter of one tap at stride 1 without padding is the conv2d 1x1 case on [N, C, D*H, W]
  // (a batched GEMM on the tensors as they are); same workspace size.
  if (t * r * s == 1 && stride[0] * stride[1] * stride[2] == 1 && pad[0] + pad[1] + pad[2] == 0)
    return conv2d_generic(in, weight, bias, out, n, c, d * h, w, k, 1, 1, 1, 1, 0, 0, 1, 1, groups, user, workspace,
                          workspace_bytes, status, stream_v, nullptr, 0, prepacked ? 2 : 0);
  if (user && (user->relu < 0 || user->relu > 1)) return FTB_E_BAD_CONFIG;
  if (user && (user->fp32_mode < 0 || user->fp32_mode > 1)) return FTB_E_BAD_CONFIG;
  if (user && (user->epilogue < 0 || user->epilogue > 1)) return FTB_E_BAD_CONFIG;
  const int algo3 = user ? user->algo : 0;
  if (algo3 == 3 || algo3 == 4 || algo3 < 0 || algo3 > 5) return FTB_E_UNSUPPORTED;
  const int relu = user ? user->relu : 0;
  if (relu && user->split_k > 1) return FTB_E_BAD_CONFIG;
  int rc = device_ok();
  if (rc) return rc;
  const int64_t cg = c / groups, kg = k / groups;
  const ConvWs ws = conv3d_ws(n, c, d, h, w, k, t, r, s, groups);
  if (!workspace || workspace_bytes < static_cast<size_t>(ws.in_bytes + ws.w_bytes)) return FTB_E_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return FTB_E_WORKSPACE;
  float* in_cl = static_cast<float*>(workspace);
  float* w_packed = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ws.in_bytes);
  const KindInfo ki = kind_info(KIND_TF32);
  const bool split3 = user && user->fp32_mode == 1;
  const int num_sms = sm_count();
  const int stride_h = stride[1], stride_w = stride[2];

  // Stride 1, one group: the slab kernel with a slab per (depth tap, channel chunk) and the filter
  // streamed (27 taps never stay resident).  Taken by itself when the tile list keeps the SMs busy;
  // shorter lists go to the per-tap lowering, which can split the reduction over CTAs.
  if (algo3 != 1 && groups == 1 && !split3 && kg <= 256 && stride[0] == 1 && stride_h == 1 && stride_w == 1 &&
      pad[0] <= (t - 1) * dil[0] && !(user && user->split_k > 1) && !(user && user->cluster == 2 && algo3 == 0)) {
    ftb_config scfg;
    memset(&scfg, 0, sizeof(scfg));
    if (user) scfg = *user;
    scfg.algo = 5;
    SlabPlan sp = plan_slab(&scfg, n * OD, kg, P, Q, r, s, ws.cchunks, dil[1], dil[2], pad[1], pad[2],
                            (reinterpret_cast<uintptr_t>(out) & 15) == 0, num_sms, false);
    if (sp.ok && algo3 == 0 && 2ll * sp.p.tiles < num_sms) sp.ok = false;
    if (!sp.ok && (algo3 == 2 || algo3 == 5)) return FTB_E_UNSUPPORTED;
    if (sp.ok) {
      rc = conv_prepass(in, weight, in_cl, w_packed, n, c, d * h, w, k, cg, t * r, s, ws, num_sms, stream_v, nullptr, 0,
                        0, 0, 1, 1, false, prepacked ? 1 : 3);
      if (rc) return rc;
      sp.p.out = out;
      sp.p.bias = bias;
      sp.p.relu = relu;
      sp.p.diag = 0;
      sp.p.conv_ktot = static_cast<int>(k);
      sp.p.num_dst = 1;
      sp.p.od = static_cast<int>(OD);
      sp.p.T = static_cast<int>(t);
      sp.p.pad_d = pad[0];
      sp.p.dil_d = dil[0];
      sp.p.depth = static_cast<int>(d);
      sp.p.status = status ? status : fallback_status();
      if (!sp.p.status) return FTB_E_CUDA;
      CUtensorMap tin, tw;
      {
        uint64_t dims[5] = {static_cast<uint64_t>(ws.cp), static_cast<uint64_t>(w), static_cast<uint64_t>(h),
                            static_cast<uint64_t>(d), static_cast<uint64_t>(n)};
        uint64_t strides[4] = {static_cast<uint64_t>(ws.cp) * 4, static_cast<uint64_t>(w) * ws.cp * 4,
                               static_cast<uint64_t>(h) * w * ws.cp * 4, static_cast<uint64_t>(d) * h * w * ws.cp * 4};
        uint32_t box[5] = {32, sp.box_w, sp.box_h, 1, 1};
        const uint32_t ones[5] = {1, 1, 1, 1, 1};
        rc = make_tmap(&tin, ki.dt, 5, in_cl, dims, strides, box, ones);
        if (rc) return rc;
      }
      {
        const uint64_t kdim = static_cast<uint64_t>(t * r * s * ws.cchunks) * 32;
        uint64_t dims[3] = {kdim, static_cast<uint64_t>(kg), 1};
        uint64_t strides[2] = {kdim * 4, kdim * 4 * kg};
        uint32_t box[3] = {32, static_cast<uint32_t>(sp.pair ? sp.p.bn / 2 : sp.p.bn), 1};
        const uint32_t ones[3] = {1, 1, 1};
        rc = make_tmap(&tw, ki.dt, 3, w_packed, dims, strides, box, ones);
        if (rc) return rc;
      }
      StoreMaps tout;
      memset(&tout, 0, sizeof(tout));
      if (sp.p.epi_bufs) {
        // (w, h, depth, channel, image) view of the NCDHW result; a box is 32 channels of one output tile
        uint64_t dims[5] = {static_cast<uint64_t>(Q), static_cast<uint64_t>(P), static_cast<uint64_t>(OD),
                            static_cast<uint64_t>(k), static_cast<uint64_t>(n)};
        uint64_t strides[4] = {static_cast<uint64_t>(Q) * 4, static_cast<uint64_t>(P) * Q * 4,
                               static_cast<uint64_t>(OD) * P * Q * 4, static_cast<uint64_t>(k) * OD * P * Q * 4};
        uint32_t box[5] = {static_cast<uint32_t>(sp.p.tile_w), static_cast<uint32_t>(sp.p.tile_h), 1, 32, 1};
        const uint32_t ones[5] = {1, 1, 1, 1, 1};
        rc = make_tmap(&tout.dst[0], ki.dt, 5, out, dims, strides, box, ones, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
      }
      return launch_slab(tin, tw, tout, sp, static_cast<cudaStream_t>(stream_v));
    }
  } else if (algo3 == 2 || algo3 == 5) {
    return FTB_E_UNSUPPORTED;
  }

  int tile_w = static_cast<int>(Q < 128 ? Q : 128);
  if (tile_w * stride_w > 256) tile_w = 256 / stride_w;
  int tile_h = user && user->tile_h > 0 ? user->tile_h : 128 / tile_w;
  if (tile_h > P) tile_h = static_cast<int>(P);
  if (tile_h < 1 || tile_h * tile_w > 128 || tile_h * stride_h > 256) return FTB_E_BAD_CONFIG;
  const int tiles_w = static_cast<int>((Q + tile_w - 1) / tile_w);
  const int tiles_h = static_cast<int>((P + tile_h - 1) / tile_h);
  const int num_kb = static_cast<int>(t * r * s * ws.cchunks);
  const long long tiles_m = n * OD * tiles_h * tiles_w;
  bool staged = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && Q % 4 == 0 && tile_w % 4 == 0 &&
                (P * Q * 4) % 16 == 0 && (groups == 1 || (kg * OD * P * Q * 4) % 16 == 0);
  if (user && user->epilogue == 1) staged = false;
  ftb_config cfg, tuned;
  const bool conv_tuned = !relu && pick_small_conv(user, 1, tiles_m, kg, num_kb, split3, num_sms, &tuned);
  if (conv_tuned) user = &tuned;
  rc = FTB_E_BAD_CONFIG;
  if (staged)
    rc = resolve_config(user, ki, split3, 0, !split3, 1, tiles_m * kTileM, kg, num_kb, true, num_sms, &cfg,
                        kEpilogueStaging);
  if (rc) {
    staged = false;
    rc = resolve_config(user, ki, split3, 0, !split3, 1, tiles_m * kTileM, kg, num_kb, true, num_sms, &cfg);
  }
  if (rc) return rc;
  const bool pair = cfg.cluster == 2;
  const long long tiles_m_launch = pair ? (tiles_m + 1) / 2 : tiles_m;
  if (!conv_tuned && (!user || user->split_k == 0) && !relu) {
    // a short tile list leaves SMs idle: split the reduction over CTAs (bulk reduce-adds into the
    // zeroed result)
    const long long tiles = tiles_m_launch * ((kg + cfg.tile_n - 1) / cfg.tile_n);
    int want = static_cast<int>((num_sms / (pair ? 2 : 1)) / (tiles > 0 ? tiles : 1));
    if (want > 32) want = 32;
    int pick = 1;
    for (int dv = 2; dv <= want; ++dv)
      if (num_kb % dv == 0) pick = dv;
    cfg.split_k = pick;
  }
  if (relu) cfg.split_k = 1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  rc = conv_prepass(in, weight, in_cl, w_packed, n, c, d * h, w, k, cg, t * r, s, ws, num_sms, stream_v,
                    cfg.split_k > 1 ? out : nullptr, n * k * OD * P * Q, 0, 0, 1, 1, groups > 1, prepacked ? 1 : 3);
  if (rc) return rc;

  UmmaParams p;
  memset(&p, 0, sizeof(p));
  p.M = static_cast<int>(tiles_m) * kTileM;
  p.N = static_cast<int>(kg);
  p.K = num_kb * ki.kblk;
  p.batch = 1;
  p.conv_groups = 1;
  p.bn = cfg.tile_n;
  p.stages = cfg.stages;
  p.num_kb = num_kb;
  p.tiles_m = static_cast<int>(tiles_m_launch);
  p.conv_tiles = static_cast<int>(tiles_m);
  p.tiles_n = static_cast<int>((kg + p.bn - 1) / p.bn);
  p.raster = cfg.raster - 1;
  p.group_m = cfg.group_m;
  p.split_k = cfg.split_k;
  p.kblk = ki.kblk;
  p.idesc = make_idesc(ki, p.bn, 0, 0, pair ? 2 * kTileM : kTileM);
  p.b_rows = pair ? p.bn / 2 : p.bn;
  p.b_bytes = static_cast<uint32_t>(p.b_rows) * 128u;
  p.a_boxes = 1;
  p.a_box_mn = kTileM;
  p.a_box_bytes = static_cast<uint32_t>(tile_h * tile_w) * 128u;
  p.tile_imgs = 1;
  p.n_imgs = static_cast<int>(n * OD);
  p.a_lbo = 16; p.a_sbo = 1024; p.a_kadv = static_cast<uint32_t>(ki.umma_k * ki.esize);
  CUtensorMapSwizzle b_swz;
  operand_layout(ki, 0, p.b_rows, &p.b_boxes, &p.b_box_mn, &p.b_box_bytes, &p.b_lbo, &p.b_sbo, &p.b_kadv,
                 &p.b_layout, &b_swz);
  p.a_layout = 2;
  p.pair_m = pair ? 2 * kTileM : kTileM;
  p.conv = 1;
  p.pdl = 1;
  if (user && (user->release < 0 || user->release > 2)) return FTB_E_BAD_CONFIG;
  p.release_pairs = conv_release_pairs(user, split3, &cfg);
  p.stages = cfg.stages;
  p.conv_ktot = static_cast<int>(k);
  p.relu = relu;
  p.C = out;
  p.bias = bias;
  p.P = static_cast<int>(P); p.Q = static_cast<int>(Q);
  p.tile_h = tile_h; p.tile_w = tile_w; p.tiles_h = tiles_h; p.tiles_w = tiles_w;
  p.T = static_cast<int>(t); p.R = static_cast<int>(r); p.S = static_cast<int>(s);
  p.cchunks = static_cast<int>(ws.cchunks);
  p.conv_od = static_cast<int>(OD);
  p.stride_d = stride[0]; p.stride_h = stride_h; p.stride_w = stride_w;
  p.pad_d = pad[0]; p.pad_h = pad[1]; p.pad_w = pad[2];
  p.dil_d = dil[0]; p.dil_h = dil[1]; p.dil_w = dil[2];
  p.status = status ? status : fallback_status();
  if (!p.status) return FTB_E_CUDA;
  const long long total = static_cast<long long>(p.tiles_m) * p.tiles_n * p.split_k;
  if (total > 0x7fffffffll) return FTB_E_TOO_LARGE;
  int ctas = cfg.ctas > 0 ? cfg.ctas : num_sms;
  if (pair) {
    if (ctas / 2 > total) ctas = static_cast<int>(total) * 2;
    ctas &= ~1;
    if (ctas < 2) ctas = 2;
  } else if (ctas > total) {
    ctas = static_cast<int>(total);
  }
  const uint64_t kdim = static_cast<uint64_t>(num_kb) * ki.kblk;
  for (int g = 0; g < groups; ++g) {
    p.conv_koff = static_cast<int>(g * kg);
    CUtensorMap ta, tb;
    {
      // (c of this group, w, h, d, n) view of the channels-last copy; channels beyond the group's
      // lie outside dimension 0 and read as zeros
      uint64_t dims[5] = {static_cast<uint64_t>(groups > 1 ? cg : ws.cp), static_cast<uint64_t>(w),
                          static_cast<uint64_t>(h), static_cast<uint64_t>(d), static_cast<uint64_t>(n)};
      uint64_t strides[4] = {static_cast<uint64_t>(ws.cp) * 4, static_cast<uint64_t>(w) * ws.cp * 4,
                             static_cast<uint64_t>(h) * w * ws.cp * 4, static_cast<uint64_t>(d) * h * w * ws.cp * 4};
      uint32_t box[5] = {static_cast<uint32_t>(ki.kblk), static_cast<uint32_t>(tile_w * stride_w),
                         static_cast<uint32_t>(tile_h * stride_h), 1, 1};
      uint32_t es[5] = {1, static_cast<uint32_t>(stride_w), static_cast<uint32_t>(stride_h), 1, 1};
      rc = make_tmap(&ta, ki.dt, 5, in_cl + g * ws.cgp, dims, strides, box, es);
      if (rc) return rc;
    }
    {
      uint64_t dims[3] = {kdim, static_cast<uint64_t>(kg), 1};
      uint64_t strides[2] = {kdim * 4, kdim * 4 * kg};
      uint32_t box[3] = {static_cast<uint32_t>(ki.kblk), static_cast<uint32_t>(p.b_rows), 1};
      const uint32_t ones[3] = {1, 1, 1};
      rc = make_tmap(&tb, ki.dt, 3, w_packed + static_cast<uint64_t>(g) * kg * kdim, dims, strides, box, ones);
      if (rc) return rc;
    }
    StoreMaps tc;
    memset(&tc, 0, sizeof(tc));
    if (staged) {
      // (w, h, depth, channel of this group, image) view of the NCDHW result: a box of 32 channels is
      // clipped at the end of the group
      p.tma_store = 1;
      p.num_dst = 1;
      uint64_t dims[5] = {static_cast<uint64_t>(Q), static_cast<uint64_t>(P), static_cast<uint64_t>(OD),
                          static_cast<uint64_t>(kg), static_cast<uint64_t>(n)};
      uint64_t strides[4] = {static_cast<uint64_t>(Q) * 4, static_cast<uint64_t>(P) * Q * 4,
                             static_cast<uint64_t>(OD) * P * Q * 4, static_cast<uint64_t>(k) * OD * P * Q * 4};
      uint32_t box[5] = {static_cast<uint32_t>(tile_w), static_cast<uint32_t>(tile_h), 1, 32, 1};
      const uint32_t ones[5] = {1, 1, 1, 1, 1};
      rc = make_tmap(&tc.dst[0], ki.dt, 5, out + static_cast<uint64_t>(g) * kg * OD * P * Q, dims, strides, box,
                     ones, CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc) return rc;
    }
    rc = dispatch(KIND_TF32, OUT_F32, split3, pair, ta, tb, tc, p, ctas, stream);
    if (rc) return rc;
  }
  return FTB_OK;
}

}  // namespace ftb

// ------------------------------------------------------------------ C ABI
extern "C" {

int ftb_gemm_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k, int trans_a,
                 int trans_b, const ftb_config* cfg, int* status, void* stream) {
  return ftb::gemm_generic(ftb::KIND_TF32, ftb::OUT_F32, a, b, c, 1, m, n, k, trans_a, trans_b, cfg,
                           status, stream, nullptr, 0);
}

int ftb_bgemm_f32(const float* a, const float* b, float* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                  int trans_a, int trans_b, const ftb_config* cfg, int* status, void* stream) {
  return ftb::gemm_generic(ftb::KIND_TF32, ftb::OUT_F32, a, b, c, batch, m, n, k, trans_a, trans_b, cfg,
                           status, stream, nullptr, 0);
}

int ftb_bgemm_bf16(const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                   int trans_a, int trans_b, int out_f32, const ftb_config* cfg, int* status,
                   void* stream) {
  return ftb::gemm_generic(ftb::KIND_BF16, out_f32 ? ftb::OUT_F32 : ftb::OUT_BF16, a, b, c, batch, m, n,
                           k, trans_a, trans_b, cfg, status, stream, nullptr, 0);
}

int ftb_bgemm_bf16_multi(const void* a, const void* b, void* const* c_dst, int num_dst, int64_t batch, int64_t m,
                         int64_t n, int64_t k, int trans_a, int trans_b, int out_f32, const ftb_config* cfg,
                         int* status, void* stream) {
  if (!c_dst || num_dst < 1 || num_dst > ftb::kMaxDst) return FTB_E_BAD_ARG;
  return ftb::gemm_generic(ftb::KIND_BF16, out_f32 ? ftb::OUT_F32 : ftb::OUT_BF16, a, b, c_dst[0], batch, m, n,
                           k, trans_a, trans_b, cfg, status, stream, c_dst + 1, num_dst - 1);
}

int ftb_gemm_s8(const int8_t* a, const int8_t* b, int32_t* c, int64_t m, int64_t n, int64_t k,
                int trans_a, int trans_b, const ftb_config* cfg, int* status, void* stream) {
  return ftb::gemm_generic(ftb::KIND_I8, ftb::OUT_S32, a, b, c, 1, m, n, k, trans_a, trans_b, cfg,
                           status, stream, nullptr, 0);
}

int ftb_debug_wait_profile(uint64_t* cycles, int reset) {
#ifdef FTB_PROFILE_WAITS
  if (!cycles) return FTB_E_BAD_ARG;
  unsigned long long host[ftb::PROF_SLOTS];
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(host, ftb::g_wait_cycles, sizeof(host));
  if (e == cudaSuccess && reset) {
    unsigned long long zero[ftb::PROF_SLOTS] = {0};
    e = cudaMemcpyToSymbol(ftb::g_wait_cycles, zero, sizeof(zero));
  }
  if (e != cudaSuccess) {
    ftb::set_last_cuda_error(static_cast<int>(e));
    return FTB_E_CUDA;
  }
  for (int i = 0; i < ftb::PROF_SLOTS; ++i) cycles[i] = host[i];
  return FTB_OK;
#else
  (void)cycles;
  (void)reset;
  return FTB_E_UNSUPPORTED;
#endif
}

size_t ftb_conv2d_workspace_bytes(int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                                  int64_t s, int64_t groups) {
  if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || k <= 0 || r <= 0 || s <= 0 || groups <= 0) return 0;
  const ftb::ConvWs ws = ftb::conv_ws(n, c, h, w, k, r, s, groups);
  return static_cast<size_t>(ws.in_bytes + ws.w_bytes);
}

int ftb_conv2d_nchw_f32(const float* in, const float* weight, const float* bias, float* out, int64_t n,
                        int64_t c, int64_t h, int64_t w, int64_t k, int64_t r, int64_t s, int stride_h,
                        int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups,
                        const ftb_config* cfg, void* workspace, size_t workspace_bytes, int* status,
                        void* stream) {
  return ftb::conv2d_generic(in, weight, bias, out, n, c, h, w, k, r, s, stride_h, stride_w, pad_h,
                             pad_w, dil_h, dil_w, groups, cfg, workspace, workspace_bytes, status,
                             stream, nullptr, 0, 0);
}

int ftb_conv2d_pack_filter(const float* weight, int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                           int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                           int groups, const ftb_config* cfg, void* workspace, size_t workspace_bytes,
                           void* stream) {
  return ftb::conv2d_generic(nullptr, weight, nullptr, nullptr, n, c, h, w, k, r, s, stride_h, stride_w, pad_h, pad_w,
                             dil_h, dil_w, groups, cfg, workspace, workspace_bytes, nullptr, stream, nullptr, 0, 1);
}

int ftb_conv2d_nchw_f32_prepacked(const float* in, const float* weight, const float* bias, float* out, int64_t n,
                                  int64_t c, int64_t h, int64_t w, int64_t k, int64_t r, int64_t s, int stride_h,
                                  int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups,
                                  const ftb_config* cfg, void* workspace, size_t workspace_bytes, int* status,
                                  void* stream) {
  return ftb::conv2d_generic(in, weight, bias, out, n, c, h, w, k, r, s, stride_h, stride_w, pad_h, pad_w, dil_h,
                             dil_w, groups, cfg, workspace, workspace_bytes, status, stream, nullptr, 0, 2);
}

int ftb_conv2d_nchw_f32_multi(const float* in, const float* weight, const float* bias, float* const* out_dst,
                              int num_dst, int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                              int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                              int groups, int prepacked, const ftb_config* cfg, void* workspace,
                              size_t workspace_bytes, int* status, void* stream) {
  if (!out_dst || num_dst < 1 || num_dst > ftb::kMaxDst) return FTB_E_BAD_ARG;
  return ftb::conv2d_generic(in, weight, bias, out_dst[0], n, c, h, w, k, r, s, stride_h, stride_w, pad_h,
                             pad_w, dil_h, dil_w, groups, cfg, workspace, workspace_bytes, status, stream,
                             out_dst + 1, num_dst - 1, prepacked ? 2 : 0);
}


size_t ftb_conv2d_nhwc_workspace_bytes(int64_t c, int64_t k, int64_t r, int64_t s, int64_t groups) {
  if (c <= 0 || k <= 0 || r <= 0 || s <= 0 || groups <= 0 || c % groups) return 0;
  return static_cast<size_t>(ftb::conv_ws(1, c, 1, 1, k, r, s, groups).w_bytes);
}

int ftb_conv2d_nhwc_f32(const float* in, const float* weight, const float* bias, float* out, int64_t n, int64_t c,
                        int64_t h, int64_t w, int64_t k, int64_t r, int64_t s, int stride_h, int stride_w, int pad_h,
                        int pad_w, int dil_h, int dil_w, int groups, int prepacked, const ftb_config* cfg,
                        void* workspace, size_t workspace_bytes, int* status, void* stream) {
  return ftb::conv2d_generic(in, weight, bias, out, n, c, h, w, k, r, s, stride_h, stride_w, pad_h, pad_w, dil_h,
                             dil_w, groups, cfg, workspace, workspace_bytes, status, stream, nullptr, 0,
                             prepacked ? 2 : 0, 1);
}

size_t ftb_conv3d_workspace_bytes(int64_t n, int64_t c, int64_t d, int64_t h, int64_t w, int64_t k, int64_t t,
                                  int64_t r, int64_t s, int64_t groups) {
  if (n <= 0 || c <= 0 || d <= 0 || h <= 0 || w <= 0 || k <= 0 || t <= 0 || r <= 0 || s <= 0 || groups <= 0) return 0;
  if (c % groups) return 0;
  const ftb::ConvWs ws = ftb::conv3d_ws(n, c, d, h, w, k, t, r, s, groups);
  return static_cast<size_t>(ws.in_bytes + ws.w_bytes);
}

int ftb_conv3d_ncdhw_f32(const float* in, const float* weight, const float* bias, float* out, int64_t n, int64_t c,
                         int64_t d, int64_t h, int64_t w, int64_t k, int64_t t, int64_t r, int64_t s,
                         const int32_t* stride_dhw, const int32_t* pad_dhw, const int32_t* dil_dhw, int groups,
                         int prepacked, const ftb_config* cfg, void* workspace, size_t workspace_bytes, int* status,
                         void* stream) {
  return ftb::conv3d_generic(in, weight, bias, out, n, c, d, h, w, k, t, r, s, stride_dhw, pad_dhw, dil_dhw, groups,
                             cfg, workspace, workspace_bytes, status, stream, prepacked != 0);
}

}  // extern "C"
