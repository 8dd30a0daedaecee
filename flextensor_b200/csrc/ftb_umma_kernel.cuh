// One persistent, warp-specialised tcgen05 kernel serves every dense contraction of
// the library: GEMM fp32 (TF32 or 3xTF32), batched GEMM bf16, GEMM int8 and conv2d
// lowered to an implicit GEMM.
//
//   warp 0      TMA producer     global -> 128B-swizzled shared-memory stages
//   warp 1      MMA issuer       tcgen05.mma, accumulators in TMEM (two buffers)
//   warps 2-5   epilogue         tcgen05.ld -> convert -> shared-memory slab -> bulk tensor stores
//                                (or per-thread global stores where bulk stores cannot address the result)
//   warps 6-9   split stage      only for 3xTF32: rewrites a stage as (hi, lo) pairs
//
// A CTA owns 128 accumulator rows (one row per TMEM lane) by `bn` columns and walks
// the tile list with a stride of the number of CTAs (or CTA pairs).  The two TMEM
// buffers let the epilogue of tile i overlap the main loop of tile i+1.
//
// PAIR = true runs two CTAs of a cluster as one tcgen05 `cta_group::2` unit on a
// 256 x bn tile: each CTA stages its own 128 rows of A and its own half of B (so every
// byte of B is fetched once per pair instead of once per CTA), the leader CTA issues
// the MMAs for both, and each CTA drains its own 128 accumulator rows.  Each CTA issues
// plain TMA loads for its own halves.
//
// WIDE = true (pairs only) doubles the tile to 256 x 512: the two TMEM accumulators then hold
// the two column halves of ONE tile instead of two tiles.  Each CTA stages 256 rows/columns of
// B per K block next to the same 128 rows of A, so a byte of A feeds twice the math (175
// instead of 131 FLOP per byte moved from L2), at the price of an epilogue that overlaps the
// next main loop only half by half.  CTA r supplies B columns [256 r, 256 r + 256) of the tile:
// accumulator half h holds tile columns [128 h, 128 h + 128) and [256 + 128 h, 256 + 128 h + 128).
//
// The producer and the MMA issuer are single threads, so their loops are latency-bound
// scalar code: everything that does not change per K block is hoisted into registers and
// the per-block work is a handful of adds (ring counters instead of div/mod, 32-bit
// descriptor halves instead of 64-bit arithmetic).
#pragma once
#include "ftb_ptx.cuh"
#include <cuda_bf16.h>

namespace ftb {

constexpr int kMaxStages = 8;
constexpr int kTileM = 128;
constexpr uint32_t kATileBytes = kTileM * 128;  // 128 rows x 128 B
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccStride = 256;            // columns between the two accumulators
constexpr int kMmaPerKb = 4;                    // a stage holds 128 B of K = 4 tcgen05.mma steps

enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_S32 = 2 };

struct UmmaParams {
  // problem (GEMM view)
  int M, N, K, batch;
  // tiling
  int bn, stages, num_kb, tiles_m, tiles_n, raster, group_m, split_k;
  int kblk;  // K elements held by one stage (128 B / element size)
  uint32_t idesc;
  // operand staging
  int a_mn, b_mn;               // 1 = operand is M/N-contiguous in global memory
  uint32_t a_layout, b_layout;  // descriptor layout type (2, or 1 for MN-major TF32)
  int pair_m;                   // rows of one tile: 128, or 256 for a CTA pair
  int b_rows;                   // B rows (K-major) or columns (MN-major) staged per CTA
  int a_boxes, b_boxes;         // TMA boxes per stage
  int a_box_mn, b_box_mn;       // M/N elements covered by one box (M/N-contiguous operands)
  uint32_t a_box_bytes, b_box_bytes, b_bytes;
  uint32_t a_lbo, a_sbo, b_lbo, b_sbo;
  uint32_t a_kadv, b_kadv;  // bytes added to the descriptor start per UMMA-K step
  uint32_t b_half_enc;      // wide tiles: descriptor offset (bytes >> 4) of the second half of a CTA's B stage
  // output
  void* C;
  long long ldc, c_batch_stride;
  const float* bias;  // conv: per output channel; GEMM (fp32 out): per row of the result; may be null
  int a_bcast;        // GEMM: every batch entry reads A of batch 0
  // implicit-GEMM conv geometry (conv != 0)
  int conv, P, Q, tile_h, tile_w, tiles_h, tiles_w, R, S, cchunks;
  int conv_ktot, conv_koff;  // output channels of the whole conv / first channel of this launch
  int conv_groups;           // > 1: the batch coordinate of a tile is its group; operands and result are
                             // addressed through tensor maps with a group dimension
  int conv_tiles;            // number of 128-pixel tiles (a CTA pair takes two consecutive ones)
  int tile_imgs;             // whole images per tile (> 1 only when an image has at most 64 output pixels)
  int n_imgs;                // images of the batch
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  // conv3d (conv_od > 0): the "images" of the tile list are (image, output depth) pairs, the filter
  // has T depth taps in front of its R x S taps, and both tensors are addressed through 5-D maps:
  // (c, w, h, d, n) for the input copy, (w, h, d, k, n) for the result.  One launch covers one group.
  int conv_od, T, stride_d, pad_d, dil_d;
  // conv_cl != 0: the result is channels-last ([N][P][Q][K]; the input then is [N][H][W][C] as the
  // caller gave it): the staged epilogue writes [pixel][32 channels] slabs like the GEMM's and stores
  // them through a (k, q, p, n) map, or (k in group, group, q, p, n) with groups.
  int conv_cl;
  int* status;
  int pdl;  // launched as a programmatic dependent: wait for the previous kernel before touching memory
  // TMA-store epilogue: tma_store != 0 stages 128-byte wide output slabs in shared memory and
  // writes each with one bulk tensor store per destination.
  int tma_store, num_dst, slab_cols;
  // 1: stages are handed back to the producer two at a time (one commit per two K blocks; needs an
  // even number of stages).  A commit costs the tensor pipe about 80 cycles, so on tiles whose K block
  // is a few hundred cycles of math the saving outweighs the slightly shorter prefetch.
  int release_pairs;
  int relu;  // conv: clamp the result at zero after the bias (never with a reduction split over CTAs)
  // diagnostic builds (-DFTB_PROFILE_WAITS) only: bit 0 = the producer signals stages without
  // loading them, bit 1 = the issuer releases stages without issuing MMAs, bit 2 = no producer at
  // all and an issuer that neither waits for stages nor releases them: MMAs back to back (results
  // are garbage; the timings tell whether the main loop is bound by the loads or by the tensor pipe)
  int diag;
};

constexpr int kMaxDst = 8;
constexpr uint32_t kEpiBufBytes = kTileM * 128;  // one staged output slab: 128 rows x 128 B

// Tensor maps of the output for the TMA-store epilogue: one per destination buffer (the
// result can be written to several buffers at once, e.g. the same slice of every rank's
// gathered output over NVLink).
struct StoreMaps {
  CUtensorMap dst[kMaxDst];
};

// Where the roles of a CTA wait (diagnostic builds only, -DFTB_PROFILE_WAITS): SM cycles spent inside
// each kind of barrier wait and each role's whole loop, summed over the CTAs of every launch into
// g_wait_cycles.  The product build compiles none of it.
enum {
  PROF_PRODUCER_EMPTY = 0,  // TMA producer waiting for a free stage
  PROF_ISSUER_FULL = 1,     // MMA issuer waiting for a stage to land
  PROF_ISSUER_TEMPTY = 2,   // MMA issuer waiting for the epilogue to hand an accumulator back
  PROF_EPI_TFULL = 3,       // epilogue (warp 2) waiting for an accumulator to complete
  PROF_PRODUCER_LOOP = 4,   // whole producer loop
  PROF_ISSUER_LOOP = 5,     // whole issuer loop
  PROF_EPI_LOOP = 6,        // whole epilogue loop of warp 2
  PROF_CTAS = 7,            // CTAs that reported
  PROF_EPI_TMEM_LD = 8,     // epilogue warp 2 (wide tiles, staged): inside the tcgen05.ld of its columns + wait
  PROF_EPI_BULK_WAIT = 9,   // same warp's leader thread waiting for a bulk store to have read its staging buffer
  PROF_EPI_STAGE = 10,      // same warp: conversion, shared-memory writes and the barriers around them
  PROF_EPI_STORE_ISSUE = 11,  // same warp's leader thread inside the bulk tensor store instructions and their commit
  PROF_EPI_VOTE = 12,       // same warp: hand-back of the accumulator, packing, and the vote of the four warps
  PROF_SLOTS = 16
};
#ifdef FTB_PROFILE_WAITS
__device__ unsigned long long g_wait_cycles[PROF_SLOTS];
#define FTB_PROF_T0(var) const long long var = clock64()
#define FTB_PROF_ADD(acc, var) (acc) += clock64() - (var)
#define FTB_PROF_FLUSH(slot, acc) atomicAdd(&g_wait_cycles[slot], static_cast<unsigned long long>(acc))
#else
#define FTB_PROF_T0(var) do { } while (0)
#define FTB_PROF_ADD(acc, var) do { } while (0)
#define FTB_PROF_FLUSH(slot, acc) do { } while (0)
#endif

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

template <int KIND, int OUT, bool SPLIT3, bool PAIR, bool WIDE = false>
__global__ void __launch_bounds__(WIDE ? 352 : SPLIT3 ? 320 : 192, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ StoreMaps tmap_c, const __grid_constant__ UmmaParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_split[kMaxStages];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  static_assert(!WIDE || (PAIR && !SPLIT3), "the 256 x 512 tile exists for CTA pairs only");
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t pair_bytes = kATileBytes + p.b_bytes;  // one (A, B) pair of a stage
  const uint32_t stage_bytes = pair_bytes * (SPLIT3 ? 2u : 1u);
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;  // 0 = leader of a pair
  const int unit = PAIR ? (blockIdx.x >> 1) : blockIdx.x;   // tile-walking unit (CTA or pair)
  const int units = PAIR ? (gridDim.x >> 1) : gridDim.x;
  const uint32_t stages = p.stages;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    // In a pair the leader's `full` barrier counts the bytes of both CTAs' loads and its
    // `tempty` barrier the epilogue warps of both.
    for (uint32_t s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), WIDE ? 2 : 1);  // a wide tile's stage is read by two issuing threads
      mbar_init(smem_u32(&bar_split[s]), 4);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tfull[a]), 1);
      // every epilogue warp that reads an accumulator reports when it is done with it: four per
      // CTA, eight where a wide tile is drained by two groups of warps
      mbar_init(smem_u32(&bar_tempty[a]), (PAIR ? 8u : 4u) * ((WIDE && p.tma_store) ? 2u : 1u));
    }
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    // the store maps too: their first use would otherwise pay the descriptor fetch in the epilogue
    if (p.tma_store)
      for (int d = 0; d < p.num_dst; ++d) prefetch_tmap(&tmap_c.dst[d]);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(&tmem_base_slot), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // peer barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  if (p.pdl) grid_dependency_wait();  // everything above overlapped the previous kernel's tail

  const int total_tiles = p.batch * p.tiles_m * p.tiles_n * p.split_k;
  const int num_kb = p.num_kb;
  const int kb_per_split = (num_kb + p.split_k - 1) / p.split_k;
  const uint32_t full0 = smem_u32(&bar_full[0]);
  const uint32_t empty0 = smem_u32(&bar_empty[0]);
  const uint32_t split0 = smem_u32(&bar_split[0]);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int kblk = p.kblk;
      const int a_boxes = p.a_boxes, b_boxes = p.b_boxes;
      const int a_box_mn = p.a_box_mn, b_box_mn = p.b_box_mn;
      const uint32_t a_box_bytes = p.a_box_bytes, b_box_bytes = p.b_box_bytes;
      const uint32_t tx = a_boxes * a_box_bytes + b_boxes * b_box_bytes;
      const bool a_mn = p.a_mn != 0, b_mn = p.b_mn != 0, conv = p.conv != 0;
      const bool grouped = conv && p.conv_groups > 1;  // grouped conv: a tile's batch coordinate is its group
      const bool conv3d = conv && p.conv_od > 0;       // (c, w, h, d, n) input map
      const bool release_pairs = p.release_pairs != 0;
      // In a pair every completion is reported to the leader's barrier.
      const uint32_t full_sig0 = PAIR ? map_to_cta(full0, 0) : full0;
      uint32_t s = 0, ph = 0, sa = smem_base;
      bool ok = true;
      long long prof_wait = 0;
      FTB_PROF_T0(prof_loop0);
      for (int t = unit; t < total_tiles && ok; t += units) {
        const TileCoord tc = decode_tile(p, t);
        const int kb0 = tc.ks * kb_per_split;
        const int kb1 = min(num_kb, kb0 + kb_per_split);
        const int m0 = tc.m * p.pair_m + static_cast<int>(cta_rank) * kTileM;
        const int n0 = tc.n * p.bn + static_cast<int>(cta_rank) * p.b_rows;
        const int ab = p.a_bcast ? 0 : tc.b;  // batch coordinate of A
        // conv: walking (r, s, channel chunk) with counters instead of div/mod per block
        int img = 0, h0 = 0, w0 = 0, cc = 0, ts = 0, tr = 0, td = 0, d0 = 0;
        if (conv) {
          // this CTA's 128-pixel tile; one past the end (odd tile count in a pair) lands outside
          // the tensor and loads zeros
          const int mt = PAIR ? tc.m * 2 + static_cast<int>(cta_rank) : tc.m;
          const int tw = mt % p.tiles_w;
          const int th = (mt / p.tiles_w) % p.tiles_h;
          img = mt / (p.tiles_w * p.tiles_h) * p.tile_imgs;  // first image of the tile
          h0 = th * p.tile_h * p.stride_h - p.pad_h;
          w0 = tw * p.tile_w * p.stride_w - p.pad_w;
          cc = kb0 % p.cchunks;
          const int rs = kb0 / p.cchunks;
          ts = rs % p.S;
          tr = rs / p.S;
          if (conv3d) {
            td = tr / p.R;
            tr -= td * p.R;
            const int n_img = img / p.conv_od;
            d0 = (img - n_img * p.conv_od) * p.stride_d - p.pad_d;
            img = n_img;
          }
        }
        int kc = kb0 * kblk;  // K coordinate of the block
        for (int kb = kb0; kb < kb1; ++kb, kc += kblk) {
          FTB_PROF_T0(prof_w0);
#ifdef FTB_PROFILE_WAITS
          if (p.diag & 4) {
            // diagnostic bit 6: this thread issues the same free-running MMAs as the issuer, into
            // columns 128.. of tensor memory (tiles of at most 128 columns): do two issuing threads
            // get twice the instruction rate of one?
            if constexpr (!PAIR && !WIDE && !SPLIT3) {
              if (p.diag & 64) {
                const uint32_t xa_hi = smem_desc_hi(p.a_lbo, p.a_sbo, p.a_layout);
                const uint32_t xb_hi = smem_desc_hi(p.b_lbo, p.b_sbo, p.b_layout);
                const uint32_t xa = smem_desc_lo(smem_base, p.a_lbo);
                const uint32_t xb = xa + (kATileBytes >> 4) + smem_desc_lo(0, p.b_lbo) - smem_desc_lo(0, p.a_lbo);
#pragma unroll
                for (int k = 0; k < kMmaPerKb; ++k)
                  umma<KIND, false>(tmem_base + 128u, xa + k * (p.a_kadv >> 4), xa_hi, xb + k * (p.b_kadv >> 4), xb_hi,
                                    p.idesc, 1u);
              }
            }
            continue;
          }
#endif
          if ((!release_pairs || (s & 1u) == 0) &&
              !mbar_wait(empty0 + 8 * (release_pairs ? (s >> 1) : s), ph ^ 1u, &abort_flag)) {
            atomicOr(p.status, FTB_DEV_WAIT_EMPTY);
            abort_flag = 1;
            ok = false;
            break;
          }
          FTB_PROF_ADD(prof_wait, prof_w0);
          const uint32_t sb = sa + kATileBytes;
          const uint32_t full = full_sig0 + 8 * s;
#ifdef FTB_PROFILE_WAITS
          if (p.diag & 4) continue;
          if (p.diag & 1) {
            if (cta_rank == 0) mbar_arrive(full0 + 8 * s);
            sa += stage_bytes;
            if (++s == stages) {
              s = 0;
              ph ^= 1u;
              sa = smem_base;
            }
            continue;
          }
#endif
          if constexpr (PAIR) {
            // The leader arms the phase for the two equal halves.  (Bytes of the peer may be
            // reported before that; the phase still cannot complete until the leader's
            // own arrival.)
            if (cta_rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * tx);
            if (conv) {
              if (conv3d)
                tma_load_5d_pair(sa, &tmap_a, full, cc * kblk, w0 + ts * p.dil_w, h0 + tr * p.dil_h,
                                 d0 + td * p.dil_d, img);
              else if (grouped)
                tma_load_5d_pair(sa, &tmap_a, full, cc * kblk, tc.b, w0 + ts * p.dil_w, h0 + tr * p.dil_h, img);
              else tma_load_4d_pair(sa, &tmap_a, full, cc * kblk, w0 + ts * p.dil_w, h0 + tr * p.dil_h, img);
              if (++cc == p.cchunks) {
                cc = 0;
                if (++ts == p.S) {
                  ts = 0;
                  if (++tr == p.R) {
                    tr = 0;
                    ++td;
                  }
                }
              }
            } else if (a_mn) {
              for (int i = 0; i < a_boxes; ++i)
                tma_load_3d_pair(sa + i * a_box_bytes, &tmap_a, full, m0 + i * a_box_mn, kc, ab);
            } else {
              tma_load_3d_pair(sa, &tmap_a, full, kc, m0, ab);
            }
            if (b_mn) {
              for (int i = 0; i < b_boxes; ++i)
                tma_load_3d_pair(sb + i * b_box_bytes, &tmap_b, full, n0 + i * b_box_mn, kc, tc.b);
            } else {
              tma_load_3d_pair(sb, &tmap_b, full, kc, n0, tc.b);
            }
          } else {
            mbar_expect_tx(full, tx);
            if (conv) {
              if (conv3d)
                tma_load_5d(sa, &tmap_a, full, cc * kblk, w0 + ts * p.dil_w, h0 + tr * p.dil_h, d0 + td * p.dil_d, img);
              else if (grouped)
                tma_load_5d(sa, &tmap_a, full, cc * kblk, tc.b, w0 + ts * p.dil_w, h0 + tr * p.dil_h, img);
              else tma_load_4d(sa, &tmap_a, full, cc * kblk, w0 + ts * p.dil_w, h0 + tr * p.dil_h, img);
              if (++cc == p.cchunks) {
                cc = 0;
                if (++ts == p.S) {
                  ts = 0;
                  if (++tr == p.R) {
                    tr = 0;
                    ++td;
                  }
                }
              }
            } else if (a_mn) {
              for (int i = 0; i < a_boxes; ++i)
                tma_load_3d(sa + i * a_box_bytes, &tmap_a, full, m0 + i * a_box_mn, kc, ab);
            } else {
              tma_load_3d(sa, &tmap_a, full, kc, m0, ab);
            }
            if (b_mn) {
              for (int i = 0; i < b_boxes; ++i)
                tma_load_3d(sb + i * b_box_bytes, &tmap_b, full, n0 + i * b_box_mn, kc, tc.b);
            } else {
              tma_load_3d(sb, &tmap_b, full, kc, n0, tc.b);
            }
          }
          sa += stage_bytes;
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
            sa = smem_base;
          }
        }
      }
#ifdef FTB_PROFILE_WAITS
      if ((p.diag & 68) == 68 && !PAIR && !WIDE && !SPLIT3) {
        // this thread's own MMAs are complete before the kernel gives tensor memory back
        tc_commit(empty0);
        mbar_wait(empty0, 0, &abort_flag);
      }
#endif
      long long prof_loop = 0;
      FTB_PROF_ADD(prof_loop, prof_loop0);
      FTB_PROF_FLUSH(PROF_PRODUCER_EMPTY, prof_wait);
      FTB_PROF_FLUSH(PROF_PRODUCER_LOOP, prof_loop);
      FTB_PROF_FLUSH(PROF_CTAS, 1);
      (void)prof_wait; (void)prof_loop;
    }
    __syncwarp();
  } else if (warp == 1 || (WIDE && warp == 10)) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only in a pair)
    // A wide tile has TWO issuing threads, one per accumulator half (warps 1 and 10).  Measured: one
    // thread gets a tcgen05.mma out about every 137 cycles whatever its shape, and a second thread
    // issuing at the same time gets as many again in the same time, so a single thread keeps the
    // tensor pipe (128 cycles of math per 256-column MMA) at most 93 % busy.  Both threads read every
    // stage (its `empty` barrier counts two commits); each owns one half's accumulator, waits for it
    // and reports it complete by itself, so the second half trails the first by however long the
    // epilogue held it back and the halves' drains do not fall together.
    const uint32_t wide_half = (WIDE && warp == 10) ? 1u : 0u;
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc = p.idesc;
      const uint32_t a_hi = smem_desc_hi(p.a_lbo, p.a_sbo, p.a_layout);
      const uint32_t b_hi = smem_desc_hi(p.b_lbo, p.b_sbo, p.b_layout);
      const uint32_t a_lo0 = smem_desc_lo(smem_base, p.a_lbo);
      const uint32_t b_off = kATileBytes >> 4;
      const uint32_t b_lbo_delta = smem_desc_lo(0, p.b_lbo) - smem_desc_lo(0, p.a_lbo);
      const uint32_t a_k = p.a_kadv >> 4, b_k = p.b_kadv >> 4;
      const uint32_t stage_enc = stage_bytes >> 4;
      const uint32_t lo_enc = pair_bytes >> 4;  // (A_lo, B_lo) pair of a 3xTF32 stage
      const uint32_t ready0 = SPLIT3 ? split0 : full0;
      // Barriers the commits arrive on; in a pair both CTAs' copies are signalled.
      const uint32_t tfull0 = smem_u32(&bar_tfull[0]);
      uint32_t s = 0, ph = 0, a_lo = a_lo0;
      int local = 0;
      bool ok = true;
      long long prof_full = 0, prof_tempty = 0;
      FTB_PROF_T0(prof_loop0);
      // The issuer is one in-order thread feeding a shallow MMA queue: every cycle it spends between
      // two MMAs on something else shows up as an idle tensor pipe (measured: about 80 cycles per
      // barrier wait, about 80 per commit).  So it asks about the NEXT stage before it issues the
      // MMAs of the current one; the probe's latency then runs under the MMA issue.
      uint32_t ready = 0;
      const bool release_pairs = p.release_pairs != 0;
      for (int t = unit; t < total_tiles && ok; t += units, ++local) {
        const int ks = (p.split_k > 1) ? (t % p.split_k) : 0;
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(num_kb, kb0 + kb_per_split);
        // Plain tiles alternate between the two accumulators; a wide tile owns both (one per half).
        const uint32_t acc = WIDE ? wide_half : (local & 1);
        const uint32_t aph = WIDE ? (local & 1u) : ((local >> 1) & 1u);
        FTB_PROF_T0(prof_t0);
        if (!mbar_wait(smem_u32(&bar_tempty[acc]), aph ^ 1u, &abort_flag)) {
          atomicOr(p.status, FTB_DEV_WAIT_TMEMFREE);
          abort_flag = 1;
          break;
        }
        FTB_PROF_ADD(prof_tempty, prof_t0);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          FTB_PROF_T0(prof_f0);
#ifdef FTB_PROFILE_WAITS
          if (!(p.diag & 4))
#endif
          if (!ready && !mbar_wait(ready0 + 8 * s, ph, &abort_flag)) {
            atomicOr(p.status, SPLIT3 ? FTB_DEV_WAIT_XFORM : FTB_DEV_WAIT_FULL);
            abort_flag = 1;
            ok = false;
            break;
          }
          FTB_PROF_ADD(prof_full, prof_f0);
          tc_fence_after();
          {
            // has the next stage of the ring landed already?  (answer used in the next iteration)
            const uint32_t sn = (s + 1 == stages) ? 0u : s + 1;
            ready = mbar_test_wait(ready0 + 8 * sn, sn == 0 ? (ph ^ 1u) : ph);
          }
          const uint32_t b_lo = a_lo + b_off + b_lbo_delta;
#ifdef FTB_PROFILE_WAITS
          if (!WIDE && (p.diag & 2) && kb > kb0 && kb + 1 < kb1) {
            if constexpr (PAIR) tc_commit_pair_both(empty0 + 8 * s);
            else tc_commit(empty0 + 8 * s);
            a_lo += stage_enc;
            if (++s == stages) {
              s = 0;
              ph ^= 1u;
              a_lo = a_lo0;
            }
            continue;
          }
#endif
          if constexpr (WIDE) {
            const uint32_t b_half = b_lo + wide_half * p.b_half_enc;  // this thread's 256 columns of B
#pragma unroll
            for (int k = 0; k < kMmaPerKb; ++k)
              umma<KIND, PAIR>(d_tmem, a_lo + k * a_k, a_hi, b_half + k * b_k, b_hi, idesc, k > 0 ? 1u : accumulate);
            tc_commit_pair_both(empty0 + 8 * s);
            accumulate = 1;
            a_lo += stage_enc;
            if (++s == stages) {
              s = 0;
              ph ^= 1u;
              a_lo = a_lo0;
            }
            continue;
          } else {
#pragma unroll
            for (int k = 0; k < kMmaPerKb; ++k) {
              const uint32_t ak = a_lo + k * a_k;
              const uint32_t bk = b_lo + k * b_k;
#ifdef FTB_PROFILE_WAITS
              // diagnostic bits 4 and 5: consecutive MMAs go to two (four, tiles of at most 64 columns)
              // different accumulators, so that no MMA adds to the result of the one before it
              const uint32_t d_k = (p.diag & 32) ? d_tmem + 64u * k
                                   : (p.diag & 16) ? tmem_base + ((acc ^ (k & 1u)) * kAccStride) : d_tmem;
              umma<KIND, PAIR>(d_k, ak, a_hi, bk, b_hi, idesc, accumulate);
#else
              umma<KIND, PAIR>(d_tmem, ak, a_hi, bk, b_hi, idesc, accumulate);
#endif
              accumulate = 1;
              if constexpr (SPLIT3) {
                umma<KIND, PAIR>(d_tmem, ak + lo_enc, a_hi, bk, b_hi, idesc, 1);  // A_lo * B_hi
                umma<KIND, PAIR>(d_tmem, ak, a_hi, bk + lo_enc, b_hi, idesc, 1);  // A_hi * B_lo
              }
            }
          }
          // Free the stage (in both CTAs of a pair) once these MMAs have read it.
#ifdef FTB_PROFILE_WAITS
          if (p.diag & 4) continue;
#endif
          if (!release_pairs) {
            if constexpr (PAIR) tc_commit_pair_both(empty0 + 8 * s);
            else tc_commit(empty0 + 8 * s);
          } else if (s & 1u) {
            // stages s - 1 and s go back together
            if constexpr (PAIR) tc_commit_pair_both(empty0 + 8 * (s >> 1));
            else tc_commit(empty0 + 8 * (s >> 1));
          }
          a_lo += stage_enc;
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
            a_lo = a_lo0;
          }
        }
        if (ok) {
          if constexpr (PAIR) {
            tc_commit_pair_both(tfull0 + 8 * acc);
          } else {
            tc_commit(tfull0 + 8 * acc);
          }
        }
      }
      long long prof_loop = 0;
      FTB_PROF_ADD(prof_loop, prof_loop0);
      if (wide_half == 0) {
        FTB_PROF_FLUSH(PROF_ISSUER_FULL, prof_full);
        FTB_PROF_FLUSH(PROF_ISSUER_TEMPTY, prof_tempty);
        FTB_PROF_FLUSH(PROF_ISSUER_LOOP, prof_loop);
      }
      (void)prof_full; (void)prof_tempty; (void)prof_loop;
    }
    __syncwarp();
  } else if (warp < 6 || (WIDE && p.tma_store != 0 && warp < 10)) {
    // ------------------------------------------------------------ epilogue
    // A wide tile's staged epilogue runs on two groups of four warps (2-5 and 6-9): both read the
    // same accumulator half, each takes every other slab through its own staging buffer, so a half
    // is drained, and handed back to the MMA issuer, in half the time.
    const int grp = (WIDE && warp >= 6) ? 1 : 0;
    const int bar_sync_id = 1 + 2 * grp, bar_vote_id = 2 + 2 * grp;
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const int row = quarter * 32 + lane;  // accumulator row owned by this thread
    const int bn = WIDE ? 256 : p.bn, N = p.N;  // accumulator columns drained per pass
    const uint32_t tempty_sig0 =
        PAIR ? map_to_cta(smem_u32(&bar_tempty[0]), 0) : smem_u32(&bar_tempty[0]);
    const uint32_t epi_base = smem_base + stages * stage_bytes;  // two output slabs after the stages
    uint32_t slab_seq = 0;
    int local = 0;
    bool alive = true;
    long long prof_tfull = 0, prof_ld = 0, prof_bulk = 0, prof_stage = 0, prof_issue = 0, prof_vote = 0;
    FTB_PROF_T0(prof_loop0);
    for (int t = unit; t < total_tiles && alive; t += units, ++local) {
      const TileCoord tc = decode_tile(p, t);
     // a wide tile is drained in two passes, one per accumulator half
#pragma unroll 1
     for (int half = 0; half < (WIDE ? 2 : 1); ++half) {
      const uint32_t acc = WIDE ? static_cast<uint32_t>(half) : (local & 1);
      const uint32_t aph = WIDE ? (local & 1u) : ((local >> 1) & 1u);
      const bool has_work = tc.ks * kb_per_split < num_kb;  // a split past the K range adds nothing
      FTB_PROF_T0(prof_e0);
      bool got = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_tfull[acc]), aph, &abort_flag));
      FTB_PROF_ADD(prof_tfull, prof_e0);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccStride;
      // A wide tile's accumulator half is wanted back by the MMA issuer as soon as possible (the
      // next tile cannot start before it is free), so a warp first pulls all of its group's 128
      // columns of the half into registers (every other slab: two slabs of 64 columns for a 16-bit
      // result, four of 32 for a 32-bit one) and hands the accumulator back - before the warps
      // agree on anything - and only then converts, stages and stores, under the next tile's main loop.
      uint32_t wide_v[WIDE ? 4 : 1][32];
      if constexpr (WIDE) {
        if (p.tma_store && got) {
          tc_fence_after();
          FTB_PROF_T0(prof_l0);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int col = (OUT == OUT_BF16) ? grp * 64 + (q >> 1) * 128 + (q & 1) * 32 : grp * 32 + q * 64;
            tmem_ld_32x32(taddr + col, wide_v[q]);
          }
          tmem_ld_wait();
          FTB_PROF_ADD(prof_ld, prof_l0);
          prof_vote -= clock64();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_sig0 + 8 * acc);
          if constexpr (OUT == OUT_BF16) {
            // a 16-bit result is rounded and packed right away: half the registers to carry
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(wide_v[q][2 * j]),
                                                          __uint_as_float(wide_v[q][2 * j + 1]));
                wide_v[q][j] = *reinterpret_cast<uint32_t*>(&h2);
              }
          }
        }
      }
      // The staged epilogue synchronises the four warps with each other: they must agree.
      if (p.tma_store) got = named_barrier_all(bar_vote_id, 128, got);
#ifdef FTB_PROFILE_WAITS
      if (WIDE && p.tma_store && prof_vote < 0) prof_vote += clock64();
#endif
      if (!got) {
        if (lane == 0) {
          atomicOr(p.status, FTB_DEV_WAIT_TMEMFULL);
          abort_flag = 1;
        }
        alive = false;
        break;
      }
      tc_fence_after();
      const int n0 = tc.n * p.bn;
      // problem column of accumulator column c (a slab of 32 or 64 columns never straddles the
      // boundary between the two CTAs' parts of a wide tile)
      auto ncol = [&](int c) { return WIDE ? n0 + ((c & 128) << 1) + half * 128 + (c & 127) : n0 + c; };

      // Where this thread's row goes in the output.
      bool row_ok;
      long long row_off;  // element offset of (row, column 0 of the problem)
      long long col_stride = 1;
      int conv_mt = 0, conv_tw = 0, conv_th = 0, conv_img = 0, conv_dep = 0;
      // first output channel of this tile's group (grouped conv: group = batch coordinate)
      const int koff = p.conv ? p.conv_koff + tc.b * N : 0;
      if (p.conv) {
        const int mt = PAIR ? tc.m * 2 + static_cast<int>(cta_rank) : tc.m;
        const int tw = mt % p.tiles_w;
        const int th = (mt / p.tiles_w) % p.tiles_h;
        // several small images per tile: rows are [image][pixel of the image]
        const int px_per_img = p.tile_h * p.tile_w;
        const int img_l = p.tile_imgs > 1 ? row / px_per_img : 0;
        const int rr = p.tile_imgs > 1 ? row - img_l * px_per_img : row;
        const int img0 = mt / (p.tiles_w * p.tiles_h) * p.tile_imgs;
        const int img = img0 + img_l;
        conv_mt = mt; conv_tw = tw; conv_th = th; conv_img = img0;
        const int oh = th * p.tile_h + rr / p.tile_w;
        const int ow = tw * p.tile_w + rr % p.tile_w;
        row_ok = mt < p.conv_tiles && row < p.tile_imgs * px_per_img && img < p.n_imgs && oh < p.P && ow < p.Q;
        col_stride = static_cast<long long>(p.P) * p.Q;
        if (p.conv_od > 0) {
          // conv3d: image index = (image, output depth); a channel of the result is od planes
          conv_img = img0 / p.conv_od;
          conv_dep = img0 - conv_img * p.conv_od;
          row_off = static_cast<long long>(conv_dep) * col_stride + static_cast<long long>(oh) * p.Q + ow;
          col_stride *= p.conv_od;
          row_off += (static_cast<long long>(conv_img) * p.conv_ktot + koff) * col_stride;
        } else if (p.conv_cl) {
          row_off = ((static_cast<long long>(img) * p.P + oh) * p.Q + ow) * p.conv_ktot + koff;
          col_stride = 1;
        } else {
          row_off = (static_cast<long long>(img) * p.conv_ktot + koff) * col_stride +
                    static_cast<long long>(oh) * p.Q + ow;
        }
      } else {
        const int gm = tc.m * p.pair_m + static_cast<int>(cta_rank) * kTileM + row;
        row_ok = gm < p.M;
        row_off = tc.b * p.c_batch_stride + static_cast<long long>(gm) * p.ldc;
      }
      row_ok = row_ok && has_work;

      if (p.conv && !p.conv_cl && p.tma_store) {
        // ---- conv, staged: TMEM -> registers -> [channel][tile_h][tile_w] in shared memory -> one
        // bulk tensor store (fp32 reduce-add under split-K) per 32 output channels.  Lanes hold
        // consecutive pixels, so the shared-memory writes of a channel are conflict-free and global
        // memory sees whole rows of every channel plane of the NCHW result.
        const bool leader = (warp == 2 && lane == 0);
        const int px_img = p.tile_h * p.tile_w;
        const bool in_tile = row < p.tile_imgs * px_img;
        const uint32_t ch_stride = static_cast<uint32_t>(px_img) * 4u;
        // staging is [image of the tile][channel][pixel]: the box of the store is (w, h, 32 channels, images)
        const uint32_t row_byte = p.tile_imgs > 1
            ? static_cast<uint32_t>(row / px_img) * 32u * ch_stride + static_cast<uint32_t>(row % px_img) * 4u
            : static_cast<uint32_t>(row) * 4u;
        const bool add_bias = p.bias != nullptr && tc.ks == 0;
        const bool tile_ok = has_work && conv_mt < p.conv_tiles;
        for (int c = 0; c < bn; c += 32, ++slab_seq) {
          const uint32_t buf = epi_base + (slab_seq & 1u) * kEpiBufBytes;
          if (leader) bulk_wait_group_read<1>();
          named_barrier_sync(1, 128);
          uint32_t v[32];
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
          if (c + 32 >= bn) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(tempty_sig0 + 8 * acc);
              else mbar_arrive(tempty_sig0 + 8 * acc);
            }
          }
          if (in_tile) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = __uint_as_float(v[j]);
              if (add_bias && n0 + c + j < N) x += p.bias[koff + n0 + c + j];
              if (p.relu) x = fmaxf(x, 0.0f);
              st_shared_f32(buf + static_cast<uint32_t>(j) * ch_stride + row_byte, x);
            }
          }
          fence_proxy_async_smem();
          named_barrier_sync(1, 128);
          if (leader) {
            if (tile_ok && n0 + c < N) {
              if (p.conv_od > 0) {
                // conv3d: (w, h, depth, channel, image)
                if (p.split_k > 1)
                  tma_reduce_add_5d(&tmap_c.dst[0], buf, conv_tw * p.tile_w, conv_th * p.tile_h, conv_dep, n0 + c, conv_img);
                else
                  for (int d = 0; d < p.num_dst; ++d)
                    tma_store_5d(&tmap_c.dst[d], buf, conv_tw * p.tile_w, conv_th * p.tile_h, conv_dep, n0 + c, conv_img);
              } else if (p.conv_groups > 1) {
                if (p.split_k > 1)
                  tma_reduce_add_5d(&tmap_c.dst[0], buf, conv_tw * p.tile_w, conv_th * p.tile_h, n0 + c, tc.b, conv_img);
                else
                  for (int d = 0; d < p.num_dst; ++d)
                    tma_store_5d(&tmap_c.dst[d], buf, conv_tw * p.tile_w, conv_th * p.tile_h, n0 + c, tc.b, conv_img);
              } else if (p.split_k > 1) {
                tma_reduce_add_4d(&tmap_c.dst[0], buf, conv_tw * p.tile_w, conv_th * p.tile_h, n0 + c, conv_img);
              } else {
                for (int d = 0; d < p.num_dst; ++d)
                  tma_store_4d(&tmap_c.dst[d], buf, conv_tw * p.tile_w, conv_th * p.tile_h, n0 + c, conv_img);
              }
            }
            bulk_commit_group();
          }
        }
        continue;
      }
      if (p.tma_store) {
        // ---- staged epilogue: TMEM -> registers -> swizzled shared slab -> bulk tensor store(s)
        const int slab_cols = p.slab_cols;  // 64 for bf16 output, 32 for 32-bit output
        const bool leader = (warp == (grp ? 6 : 2) && lane == 0);
        const int m0 = tc.m * p.pair_m + static_cast<int>(cta_rank) * kTileM;
        const uint32_t swz = static_cast<uint32_t>(row & 7);
        const int c_step = WIDE ? 2 * slab_cols : slab_cols;
        if constexpr (WIDE) {
          // the accumulator columns are already in registers (wide_v) and the accumulator handed back
          auto& v = wide_v;
          float bias = 0.0f;
          if constexpr (OUT == OUT_F32) {
            if (p.bias != nullptr && tc.ks == 0 && m0 + row < p.M) bias = p.bias[m0 + row];
          }
          const uint32_t buf = epi_base + static_cast<uint32_t>(grp) * kEpiBufBytes;
          const uint32_t row_addr = buf + static_cast<uint32_t>(row) * 128u;
          constexpr int kSlabs = (OUT == OUT_BF16) ? 2 : 4;
#pragma unroll
          for (int i = 0; i < kSlabs; ++i) {
            const int c = grp * slab_cols + i * c_step;
            // the store that used this group's buffer before must have finished reading it
            FTB_PROF_T0(prof_b0);
            if (leader) bulk_wait_group_read<0>();
            FTB_PROF_ADD(prof_bulk, prof_b0);
            FTB_PROF_T0(prof_s0);
            named_barrier_sync(bar_sync_id, 128);
            if constexpr (OUT == OUT_BF16) {
              // v[2 * i + part][0..15] hold 32 columns as packed pairs
#pragma unroll
              for (int part = 0; part < 2; ++part) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const uint32_t chunk = static_cast<uint32_t>(part * 4 + j);
                  st_shared_v4(row_addr + ((chunk ^ swz) << 4), v[2 * i + part][4 * j], v[2 * i + part][4 * j + 1],
                               v[2 * i + part][4 * j + 2], v[2 * i + part][4 * j + 3]);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  w[q] = v[i][4 * j + q];
                  if constexpr (OUT == OUT_F32) w[q] = __float_as_uint(__uint_as_float(w[q]) + bias);
                }
                st_shared_v4(row_addr + ((static_cast<uint32_t>(j) ^ swz) << 4), w[0], w[1], w[2], w[3]);
              }
            }
            fence_proxy_async_smem();  // the slab must be visible to the bulk-copy engine
            named_barrier_sync(bar_sync_id, 128);
            FTB_PROF_ADD(prof_stage, prof_s0);
            FTB_PROF_T0(prof_i0);
            if (leader) {
              if (has_work && ncol(c) < N) {
                if (p.split_k > 1) {
                  tma_reduce_add_3d(&tmap_c.dst[0], buf, ncol(c), m0, tc.b);
                } else {
                  for (int d = 0; d < p.num_dst; ++d) tma_store_3d(&tmap_c.dst[d], buf, ncol(c), m0, tc.b);
                }
              }
              bulk_commit_group();
            }
            FTB_PROF_ADD(prof_issue, prof_i0);
          }
          slab_seq += kSlabs;
        } else
        for (int c = grp * slab_cols; c < bn; c += c_step, ++slab_seq) {
          // plain tiles alternate between the two buffers; a group of a wide tile owns one
          const uint32_t buf = epi_base + (WIDE ? static_cast<uint32_t>(grp) : (slab_seq & 1u)) * kEpiBufBytes;
          // The store that used this buffer before must have finished reading it.
          if (leader) {
            if constexpr (WIDE) bulk_wait_group_read<0>();
            else bulk_wait_group_read<1>();
          }
          named_barrier_sync(bar_sync_id, 128);
          const uint32_t row_addr = buf + static_cast<uint32_t>(row) * 128u;
          if constexpr (OUT == OUT_BF16) {
            // both 32-column loads are in flight before the one wait
            uint32_t v[2][32];
            tmem_ld_32x32(taddr + c, v[0]);
            tmem_ld_32x32(taddr + c + 32, v[1]);
            tmem_ld_wait();
#pragma unroll
            for (int part = 0; part < 2; ++part) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[part][j * 8 + 2 * q]),
                                                            __uint_as_float(v[part][j * 8 + 2 * q + 1]));
                  w[q] = *reinterpret_cast<uint32_t*>(&h2);
                }
                const uint32_t chunk = static_cast<uint32_t>(part * 4 + j);
                st_shared_v4(row_addr + ((chunk ^ swz) << 4), w[0], w[1], w[2], w[3]);
              }
            }
          } else {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c, v);
            tmem_ld_wait();
            if constexpr (OUT == OUT_F32) {
              if (p.conv_cl) {
                // channels-last conv: the bias belongs to the column (output channel)
                if (p.bias != nullptr && tc.ks == 0) {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (n0 + c + j < N) v[j] = __float_as_uint(__uint_as_float(v[j]) + p.bias[koff + n0 + c + j]);
                }
                if (p.relu) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(fmaxf(__uint_as_float(v[j]), 0.0f));
                }
              } else if (p.bias != nullptr && tc.ks == 0 && m0 + row < p.M) {
                const float bias = p.bias[m0 + row];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + bias);
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_shared_v4(row_addr + ((static_cast<uint32_t>(j) ^ swz) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2],
                           v[4 * j + 3]);
          }
          if (c + c_step >= bn) {
            // Last read of this accumulator (by this group): hand it back to the MMA issuer.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(tempty_sig0 + 8 * acc);
              else mbar_arrive(tempty_sig0 + 8 * acc);
            }
          }
          fence_proxy_async_smem();  // the slab must be visible to the bulk-copy engine
          named_barrier_sync(bar_sync_id, 128);
          if (leader) {
            if (p.conv_cl) {
              // the slab's rows are the tile's pixels in (image, row, column) order: the box of the store
              if (has_work && conv_mt < p.conv_tiles && n0 + c < N) {
                const int x = conv_tw * p.tile_w, y = conv_th * p.tile_h;
                if (p.conv_groups > 1) {
                  if (p.split_k > 1)
                    tma_reduce_add_5d(&tmap_c.dst[0], buf, n0 + c, tc.b, x, y, conv_img);
                  else
                    for (int d = 0; d < p.num_dst; ++d) tma_store_5d(&tmap_c.dst[d], buf, n0 + c, tc.b, x, y, conv_img);
                } else if (p.split_k > 1) {
                  tma_reduce_add_4d(&tmap_c.dst[0], buf, n0 + c, x, y, conv_img);
                } else {
                  for (int d = 0; d < p.num_dst; ++d) tma_store_4d(&tmap_c.dst[d], buf, n0 + c, x, y, conv_img);
                }
              }
            } else if (has_work && ncol(c) < N) {
              if (p.split_k > 1) {
                // partial sums of the K splits meet in global memory (fp32 result, one destination)
                tma_reduce_add_3d(&tmap_c.dst[0], buf, ncol(c), m0, tc.b);
              } else {
                for (int d = 0; d < p.num_dst; ++d) tma_store_3d(&tmap_c.dst[d], buf, ncol(c), m0, tc.b);
              }
            }
            bulk_commit_group();
          }
        }
        continue;
      }

      for (int c = 0; c < bn; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c, v);
        tmem_ld_wait();
        if (c + 32 >= bn) {
          // Last read of this accumulator: hand it back before the stores go out.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(tempty_sig0 + 8 * acc);
            else mbar_arrive(tempty_sig0 + 8 * acc);
          }
        }
        if (!row_ok) continue;
        const int nbase = ncol(c);
        if (nbase >= N) continue;
        if (p.conv) {
          float* out = reinterpret_cast<float*>(p.C);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = nbase + j;
            if (n < N) {
              float x = __uint_as_float(v[j]);
              if (p.bias != nullptr && tc.ks == 0) x += p.bias[koff + n];
              if (p.relu) x = fmaxf(x, 0.0f);
              float* dst = out + row_off + n * col_stride;
              if (p.split_k > 1) atomicAdd(dst, x);
              else *dst = x;
            }
          }
        } else if constexpr (OUT == OUT_BF16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row_off + nbase;
          const bool vec = (nbase + 32 <= N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
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
              if (nbase + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
          }
        } else {
          // fp32 and int32 results leave TMEM as raw 32-bit words.
          uint32_t* dst = reinterpret_cast<uint32_t*>(p.C) + row_off + nbase;
          if constexpr (OUT == OUT_F32) {
            if (p.bias != nullptr && tc.ks == 0) {
              const float bias = p.bias[tc.m * p.pair_m + static_cast<int>(cta_rank) * kTileM + row];
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + bias);
            }
          }
          if (OUT == OUT_F32 && p.split_k > 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nbase + j < N) atomicAdd(reinterpret_cast<float*>(dst) + j, __uint_as_float(v[j]));
          } else {
            const bool vec = (nbase + 32 <= N) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
            if (vec) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nbase + j < N) dst[j] = v[j];
            }
          }
        }
      }
     }
    }
    if (warp == 2 && lane == 0) {
      long long prof_loop = 0;
      FTB_PROF_ADD(prof_loop, prof_loop0);
      FTB_PROF_FLUSH(PROF_EPI_TFULL, prof_tfull);
      FTB_PROF_FLUSH(PROF_EPI_LOOP, prof_loop);
      FTB_PROF_FLUSH(PROF_EPI_TMEM_LD, prof_ld);
      FTB_PROF_FLUSH(PROF_EPI_BULK_WAIT, prof_bulk);
      FTB_PROF_FLUSH(PROF_EPI_STAGE, prof_stage);
      FTB_PROF_FLUSH(PROF_EPI_STORE_ISSUE, prof_issue);
      FTB_PROF_FLUSH(PROF_EPI_VOTE, prof_vote);
      (void)prof_loop;
    }
    (void)prof_tfull; (void)prof_ld; (void)prof_bulk; (void)prof_stage; (void)prof_issue; (void)prof_vote;
    // Shared memory must outlive the bulk stores' reads of it.  Their global writes are part of
    // this grid's memory operations and are complete when the grid is; only stores into a peer
    // GPU's memory (several destinations) are waited for in full before the CTA exits.
    if (p.tma_store && lane == 0 && (warp == 2 || (WIDE && warp == 6))) {
      if (p.num_dst > 1) bulk_wait_group<0>();
      else bulk_wait_group_read<0>();
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ 3xTF32 split stage
    if constexpr (SPLIT3) {
      const int tid = threadIdx.x - 192;  // 0..127
      uint32_t s = 0, ph = 0;
      bool ok = true;
      uint8_t* const stage0 = smem_raw + (smem_base - smem_u32(smem_raw));
      for (int t = unit; t < total_tiles && ok; t += units) {
        const int ks = (p.split_k > 1) ? (t % p.split_k) : 0;
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(num_kb, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          const bool got = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, ph, &abort_flag));
          if (!got) {
            if (lane == 0) {
              atomicOr(p.status, FTB_DEV_WAIT_FULL);
              abort_flag = 1;
            }
            ok = false;
            break;
          }
          // x = hi + lo.  The tensor core reads an fp32 operand as TF32 by dropping the low 13
          // mantissa bits, so the stage as it landed already serves as `hi`; only
          // lo = x - (x with those bits cleared), which is exact in fp32, has to be written.  The
          // rewrite is elementwise, so every value keeps its swizzled place.
          uint8_t* base = stage0 + s * stage_bytes;
          for (uint32_t off = tid * 16; off < pair_bytes; off += 128 * 16) {
            const float4 x = *reinterpret_cast<const float4*>(base + off);
            float4 lo;
            lo.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xffffe000u);
            lo.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xffffe000u);
            lo.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xffffe000u);
            lo.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xffffe000u);
            *reinterpret_cast<float4*>(base + pair_bytes + off) = lo;
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core reads
          __syncwarp();
          if (lane == 0) mbar_arrive(split0 + 8 * s);
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
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
  if constexpr (PAIR) cluster_sync_all();  // the peer's shared memory and TMEM stay alive until both are done
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace ftb
