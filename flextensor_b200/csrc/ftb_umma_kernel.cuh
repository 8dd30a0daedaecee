// One persistent, warp-specialised tcgen05 kernel serves every dense contraction of
// the library: GEMM fp32 (TF32 or 3xTF32), batched GEMM bf16, GEMM int8 and conv2d
// lowered to an implicit GEMM.
//
//   warp 0      TMA producer     global -> 128B-swizzled shared-memory stages
//   warp 1      MMA issuer       tcgen05.mma, accumulators in TMEM (two buffers)
//   warps 2-5   epilogue         tcgen05.ld -> convert -> global stores
//   warps 6-9   split stage      only for 3xTF32: rewrites a stage as (hi, lo) pairs
//
// A CTA owns 128 accumulator rows (UMMA M = 128, one row per TMEM lane) by `bn`
// columns (UMMA N = bn), and walks the tile list with a stride of gridDim.x.  The
// two TMEM buffers let the epilogue of tile i overlap the main loop of tile i+1.
#pragma once
#include "ftb_ptx.cuh"
#include <cuda_bf16.h>

namespace ftb {

constexpr int kMaxStages = 8;
constexpr int kTileM = 128;
constexpr uint32_t kATileBytes = kTileM * 128;  // 128 rows x 128 B
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccStride = 256;            // columns between the two accumulators

enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_S32 = 2 };

struct UmmaParams {
  // problem (GEMM view)
  int M, N, K, batch;
  // tiling
  int bn, stages, num_kb, tiles_m, tiles_n, raster, group_m, split_k;
  int kblk;  // K elements held by one stage (128 B / element size)
  uint32_t idesc;
  // operand staging
  int a_mn, b_mn;          // 1 = operand is M/N-contiguous in global memory
  int a_boxes, b_boxes;    // TMA boxes per stage
  int a_box_mn, b_box_mn;  // M/N elements covered by one box (M/N-contiguous operands)
  uint32_t a_box_bytes, b_box_bytes, b_bytes;
  uint32_t a_lbo, a_sbo, b_lbo, b_sbo;
  uint32_t a_kadv, b_kadv;  // bytes added to the descriptor start per UMMA-K step
  int mma_per_kb;
  // output
  void* C;
  long long ldc, c_batch_stride;
  const float* bias;  // conv only, may be null
  // implicit-GEMM conv geometry (conv != 0)
  int conv, P, Q, tile_h, tile_w, tiles_h, tiles_w, R, S, cchunks;
  int conv_ktot, conv_koff;  // output channels of the whole conv / first channel of this group
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int* status;
};

struct TileCoord {
  int b, m, n, ks;
};

__device__ __forceinline__ TileCoord decode_tile(const UmmaParams& p, int t) {
  TileCoord c;
  c.ks = t % p.split_k;
  t /= p.split_k;
  const int per_batch = p.tiles_m * p.tiles_n;
  c.b = t / per_batch;
  const int r = t - c.b * per_batch;
  if (p.raster == 2 && p.group_m > 1) {
    const int span = p.group_m * p.tiles_n;
    const int g = r / span;
    const int first = g * p.group_m;
    const int gsz = min(p.group_m, p.tiles_m - first);
    const int q = r - g * span;
    c.m = first + q % gsz;
    c.n = q / gsz;
  } else if (p.raster == 1) {
    c.n = r / p.tiles_m;
    c.m = r - c.n * p.tiles_m;
  } else {
    c.m = r / p.tiles_n;
    c.n = r - c.m * p.tiles_n;
  }
  return c;
}

template <int KIND, int OUT, bool SPLIT3>
__global__ void __launch_bounds__(SPLIT3 ? 320 : 192, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_split[kMaxStages];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_bytes = (kATileBytes + p.b_bytes) * (SPLIT3 ? 2u : 1u);
  const uint32_t lo_off = kATileBytes + p.b_bytes;  // offset of the (Alo, Blo) pair in a stage

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_split[s]), 4);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tfull[a]), 1);
      mbar_init(smem_u32(&bar_tempty[a]), 4);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int total_tiles = p.batch * p.tiles_m * p.tiles_n * p.split_k;
  const int kb_per_split = (p.num_kb + p.split_k - 1) / p.split_k;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = decode_tile(p, t);
        const int kb0 = tc.ks * kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + kb_per_split);
        int img = 0, h0 = 0, w0 = 0;
        if (p.conv) {
          const int tw = tc.m % p.tiles_w;
          const int th = (tc.m / p.tiles_w) % p.tiles_h;
          img = tc.m / (p.tiles_w * p.tiles_h);
          h0 = th * p.tile_h * p.stride_h - p.pad_h;
          w0 = tw * p.tile_w * p.stride_w - p.pad_w;
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, &abort_flag)) {
            atomicOr(p.status, FTB_DEV_WAIT_EMPTY);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t sa = smem_base + s * stage_bytes;
          const uint32_t sb = sa + kATileBytes;
          mbar_expect_tx(full, p.a_boxes * p.a_box_bytes + p.b_boxes * p.b_box_bytes);
          if (p.conv) {
            const int cc = kb % p.cchunks;
            const int rs = kb / p.cchunks;
            const int s_ = rs % p.S, r_ = rs / p.S;
            tma_load_4d(sa, &tmap_a, full, cc * p.kblk, w0 + s_ * p.dil_w, h0 + r_ * p.dil_h, img);
          } else if (p.a_mn) {
            for (int i = 0; i < p.a_boxes; ++i)
              tma_load_3d(sa + i * p.a_box_bytes, &tmap_a, full, tc.m * kTileM + i * p.a_box_mn,
                          kb * p.kblk, tc.b);
          } else {
            tma_load_3d(sa, &tmap_a, full, kb * p.kblk, tc.m * kTileM, tc.b);
          }
          if (p.b_mn) {
            for (int i = 0; i < p.b_boxes; ++i)
              tma_load_3d(sb + i * p.b_box_bytes, &tmap_b, full, tc.n * p.bn + i * p.b_box_mn,
                          kb * p.kblk, tc.b);
          } else {
            tma_load_3d(sb, &tmap_b, full, kb * p.kblk, tc.n * p.bn, tc.b);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0;
      int local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local) {
        const TileCoord tc = decode_tile(p, t);
        const int kb0 = tc.ks * kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + kb_per_split);
        const int acc = local & 1;
        const uint32_t aph = (local >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[acc]), aph ^ 1u, &abort_flag)) {
          atomicOr(p.status, FTB_DEV_WAIT_TMEMFREE);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          const uint32_t ready = SPLIT3 ? smem_u32(&bar_split[s]) : smem_u32(&bar_full[s]);
          if (!mbar_wait(ready, ph, &abort_flag)) {
            atomicOr(p.status, SPLIT3 ? FTB_DEV_WAIT_XFORM : FTB_DEV_WAIT_FULL);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + s * stage_bytes;
          const uint32_t sb = sa + kATileBytes;
          const uint64_t da = make_smem_desc(sa, p.a_lbo, p.a_sbo);
          const uint64_t db = make_smem_desc(sb, p.b_lbo, p.b_sbo);
          for (int k = 0; k < p.mma_per_kb; ++k) {
            const uint64_t ak = da + ((static_cast<uint64_t>(k) * p.a_kadv) >> 4);
            const uint64_t bk = db + ((static_cast<uint64_t>(k) * p.b_kadv) >> 4);
            umma<KIND>(d_tmem, ak, bk, p.idesc, accumulate);
            accumulate = 1;
            if constexpr (SPLIT3) {
              const uint64_t lo = lo_off >> 4;
              umma<KIND>(d_tmem, ak + lo, bk, p.idesc, 1);  // A_lo * B_hi
              umma<KIND>(d_tmem, ak, bk + lo, p.idesc, 1);  // A_hi * B_lo
            }
          }
          tc_commit(smem_u32(&bar_empty[s]));  // frees the stage once these MMAs have read it
        }
        if (ok) tc_commit(smem_u32(&bar_tfull[acc]));
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    int local = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++local) {
      const TileCoord tc = decode_tile(p, t);
      const int acc = local & 1;
      const uint32_t aph = (local >> 1) & 1u;
      const int kb0 = tc.ks * kb_per_split;
      const bool has_work = kb0 < p.num_kb;  // a split beyond the K range contributes nothing
      const bool got = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_tfull[acc]), aph, &abort_flag));
      if (!got) {
        if (lane == 0) {
          atomicOr(p.status, FTB_DEV_WAIT_TMEMFULL);
          abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      const int row = quarter * 32 + lane;  // accumulator row owned by this thread
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccStride;
      const int n0 = tc.n * p.bn;

      // Where this thread's row goes in the output.
      bool row_ok;
      long long row_off;  // element offset of (row, column 0 of the problem)
      long long col_stride = 1;
      if (p.conv) {
        const int tw = tc.m % p.tiles_w;
        const int th = (tc.m / p.tiles_w) % p.tiles_h;
        const int img = tc.m / (p.tiles_w * p.tiles_h);
        const int oh = th * p.tile_h + row / p.tile_w;
        const int ow = tw * p.tile_w + row % p.tile_w;
        row_ok = row < p.tile_h * p.tile_w && oh < p.P && ow < p.Q;
        col_stride = static_cast<long long>(p.P) * p.Q;
        row_off = (static_cast<long long>(img) * p.conv_ktot + p.conv_koff) * col_stride +
                  static_cast<long long>(oh) * p.Q + ow;
      } else {
        const int gm = tc.m * kTileM + row;
        row_ok = gm < p.M;
        row_off = tc.b * p.c_batch_stride + static_cast<long long>(gm) * p.ldc;
      }
      row_ok = row_ok && has_work;

      for (int c = 0; c < p.bn; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c, v);
        tmem_ld_wait();
        if (c + 32 >= p.bn) {
          // Last read of this accumulator: hand it back before the stores go out.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[acc]));
        }
        if (!row_ok) continue;
        const int nbase = n0 + c;
        if (nbase >= p.N) continue;
        if (p.conv) {
          float* out = reinterpret_cast<float*>(p.C);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = nbase + j;
            if (n < p.N) {
              float x = __uint_as_float(v[j]);
              if (p.bias != nullptr && tc.ks == 0) x += p.bias[p.conv_koff + n];
              float* dst = out + row_off + n * col_stride;
              if (p.split_k > 1) atomicAdd(dst, x);
              else *dst = x;
            }
          }
        } else if constexpr (OUT == OUT_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row_off + nbase;
          const bool vec = (nbase + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          if (vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * q]),
                                                         __uint_as_float(v[j + 2 * q + 1]));
                w[q] = *reinterpret_cast<uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nbase + j < p.N) dst[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
          }
        } else {
          // fp32 and int32 results leave TMEM as raw 32-bit words.
          uint32_t* dst = reinterpret_cast<uint32_t*>(p.C) + row_off + nbase;
          if (OUT == OUT_F32 && p.split_k > 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nbase + j < p.N) atomicAdd(reinterpret_cast<float*>(dst) + j, __uint_as_float(v[j]));
          } else {
            const bool vec = (nbase + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nbase + j < p.N) dst[j] = v[j];
            }
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ 3xTF32 split stage
    if constexpr (SPLIT3) {
      const int tid = threadIdx.x - 192;  // 0..127
      uint32_t it = 0;
      bool ok = true;
      const uint32_t pair_bytes = kATileBytes + p.b_bytes;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = decode_tile(p, t);
        const int kb0 = tc.ks * kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1u;
          const bool got = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_full[s]), ph, &abort_flag));
          if (!got) {
            if (lane == 0) {
              atomicOr(p.status, FTB_DEV_WAIT_FULL);
              abort_flag = 1;
            }
            ok = false;
            break;
          }
          // x = hi + lo with hi exactly representable in TF32 (low 13 mantissa bits
          // cleared); the elementwise rewrite keeps every value at its swizzled place.
          uint8_t* base = smem_raw + (smem_base - smem_u32(smem_raw)) + s * stage_bytes;
          for (uint32_t off = tid * 16; off < pair_bytes; off += 128 * 16) {
            float4 x = *reinterpret_cast<float4*>(base + off);
            float4 hi, lo;
            hi.x = __uint_as_float(__float_as_uint(x.x) & 0xffffe000u);
            hi.y = __uint_as_float(__float_as_uint(x.y) & 0xffffe000u);
            hi.z = __uint_as_float(__float_as_uint(x.z) & 0xffffe000u);
            hi.w = __uint_as_float(__float_as_uint(x.w) & 0xffffe000u);
            lo.x = x.x - hi.x;
            lo.y = x.y - hi.y;
            lo.z = x.z - hi.z;
            lo.w = x.w - hi.w;
            *reinterpret_cast<float4*>(base + off) = hi;
            *reinterpret_cast<float4*>(base + lo_off + off) = lo;
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core reads
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_split[s]));
        }
      }
      __syncwarp();
    }
  }

  // ------------------------------------------------------------ teardown
  if (*reinterpret_cast<volatile int*>(&abort_flag)) {
    // Give copies that are still in flight time to land before shared memory is released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace ftb
