// conv2d (stride 1) on the tensor cores with the input staged once per channel chunk and
// the filter held in shared memory for the whole kernel - or, when it does not fit, passed through
// a ring of shared-memory stages (STREAM).  Also stride-1 conv3d (one slab per depth tap and
// channel chunk, STREAM only) and channels-last results.
//
// The implicit-GEMM lowering in ftb_umma_kernel.cuh fetches one shifted copy of the input
// tile per filter tap, so an R x S filter reads the same pixels R*S times from L2.  Here a
// CTA loads, per chunk of 32 input channels, ONE slab of (tile_h + halo) x (tile_w + halo)
// pixels (channels-last, 128 B per pixel, 128-byte swizzled by the TMA unit).  Because
// successive pixels are successive 128-byte rows of the slab, the A operand of tap (r, s)
// is the same slab read from a row offset of r*dil_h*slab_w + s*dil_w: only the start
// address of the shared-memory descriptor moves.  Accumulator row m then stands for the
// pixel (m / slab_w, m % slab_w) of the tile; rows with m % slab_w >= tile_w are junk
// (they mix the end of one image row with the start of the next) and are never stored.
//
// The filter (this CTA's taps x channel chunks x bn output channels) is loaded once and
// stays resident, so the steady-state traffic of a tile is the slab alone.
//
//   warp 0      TMA producer     filter once, then one slab per (tile, channel chunk)
//   warp 1      MMA issuer       taps x 4 tcgen05.mma per slab, accumulators in TMEM
//   warps 2-5   epilogue         tcgen05.ld -> [channel][pixel] staging -> bulk tensor stores of NCHW rows
//                                (bulk reduce-adds when the taps are split; per-thread stores where bulk
//                                stores cannot address the rows)
//
// CTAs with the same blockIdx.x % split share a subset of the taps and walk the tile list
// with a stride of gridDim.x / split.
//
// STREAM = true: the filter is not resident.  The producer follows every slab with that channel
// chunk's filter tiles, b_group taps per ring stage, and the issuer hands a stage back (one
// tcgen05.commit) after its taps' MMAs.  A CTA then re-reads the filter from L2 for every tile -
// a few KB per tap - instead of splitting the taps over CTAs, whose partial sums would have to be
// added in global memory.
//
// PAIR = true runs two CTAs of a cluster as one tcgen05 `cta_group::2` unit on two consecutive
// tiles (M = 256): each CTA stages the slab of its own tile and HALF of the filter's output
// channels, the leader issues one MMA for both.  A 128 x 64 TF32 MMA is 32 cycles of math but
// reads 6 KB of operands from shared memory and costs the single issuing thread about as long to
// issue; the 256 x 64 form does twice the math per instruction and reads 5 KB per SM.
#pragma once
#include "ftb_umma_kernel.cuh"

namespace ftb {

constexpr int kSlabMaxStages = 4;
constexpr int kSlabMaxBStages = 8;

struct ConvSlabParams {
  int N;        // output channels of this launch
  int bn;       // accumulator columns (>= N, multiple of 16)
  int tiles;    // output tiles: images x tiles_h x tiles_w
  int tiles_h, tiles_w, tile_h, tile_w, slab_w;
  int R, S, cchunks, split, taps_per_split;
  int dil_h, dil_w, pad_h, pad_w, P, Q;
  int conv_ktot;  // output channels of the whole tensor
  int a_stages;
  // staged epilogue: epi_bufs (0 = off, 1 or 2) buffers of 32 channels x tile pixels after the slabs
  int epi_bufs;
  int relu;     // clamp the result at zero after the bias (never with split taps)
  int diag;     // diagnostic builds (-DFTB_PROFILE_WAITS) only, results are garbage: 1 = every tap reads the
                // slab from offset 0, 2 = tap offsets rounded down to a multiple of eight pixel rows (the
                // 1024-byte period of the swizzle); timing either against the real kernel shows what the
                // taps' odd start addresses cost
  int num_dst;  // destinations of the staged epilogue (1..kMaxDst): the same box goes to each of them
  // Streamed filter (b_stages > 0): a filter too large to stay resident is not split over CTAs (whose
  // partial sums would meet in global memory) but passed through a ring of b_stages stages, each
  // holding the b_group consecutive taps' tiles of one channel chunk; a CTA then re-reads the filter
  // from L2 for every tile, which is far less than re-reading the input once per tap.
  int b_stages, b_group;
  // conv3d at stride 1 (od > 0, streamed filter only): the tile list walks (image, output depth) pairs,
  // the filter has T depth taps in front of its R x S taps, and every (depth tap, channel chunk) pair
  // gets a slab of its own, from input plane `output depth - pad_d + depth tap * dil_d` (planes outside
  // the input read as zeros); input map (c, w, h, d, n), result map (w, h, d, k, n).
  int od, T, pad_d, dil_d, depth;
  // GATHER instantiations: no channels-last copy of the input exists; eight loader warps build every
  // slab from the NCHW tensor `in_nchw` [n_imgs][C][H][W] themselves (coalesced 32-byte reads along
  // the rows, conflict-free 4-byte writes into the swizzled slab), zero-filling the padding.
  const float* in_nchw;
  int n_imgs, C, H, W;
  // Two issuing threads (accumulators of at most 128 columns).  One thread gets a tcgen05.mma out about
  // every 137 cycles whatever its shape (measured), which leaves a 64-column TF32 MMA's tensor pipe three
  // quarters idle; a second thread issuing at the same time gets as many again.  The taps of every slab are
  // dealt to the two threads alternately, each adds its taps into an accumulator of its own (128 columns
  // apart) and the epilogue adds the two.  Used by a CTA whose share of the taps is at least two.
  int dual;
  int cl_swz;   // channels-last staging rows are written in the 128-byte swizzle of their store map
  int cl_out;   // the result is channels-last [N][P][Q][K]: staged as [pixel][32 channels], stored through a
                // (k, q, p, n) map
  uint32_t epi_buf_bytes;
  uint32_t slab_bytes;   // bytes one slab load delivers
  uint32_t slab_alloc;   // bytes reserved per slab stage (covers the furthest tap's 128 rows)
  uint32_t b_tile_bytes; // bn x 128 B
  uint32_t idesc;
  float* out;
  const float* bias;
  int* status;
};

// 32 columns of a tile's accumulator; with two issuing threads (`other` = the distance to the second
// thread's accumulator, else 0) the sum of the two partial accumulators.
__device__ __forceinline__ void slab_acc_ld(uint32_t taddr, uint32_t other, uint32_t (&v)[32]) {
  tmem_ld_32x32(taddr, v);
  if (other) {
    uint32_t w[32];
    tmem_ld_32x32(taddr + other, w);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
  } else {
    tmem_ld_wait();
  }
}

template <bool PAIR, bool STREAM, bool GATHER>
__global__ void __launch_bounds__(GATHER ? 480 : 224, 1)
conv_slab_kernel(const __grid_constant__ CUtensorMap tmap_in, const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ StoreMaps tmap_out,
                 const __grid_constant__ ConvSlabParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_afull[kSlabMaxStages];
  __shared__ __align__(8) uint64_t bar_aempty[kSlabMaxStages];
  __shared__ __align__(8) uint64_t bar_bfull;
  __shared__ __align__(8) uint64_t bar_bsfull[kSlabMaxBStages];
  __shared__ __align__(8) uint64_t bar_bsempty[kSlabMaxBStages];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_stages = p.a_stages;

  // a tile-walking unit is a CTA, or a CTA pair that takes two consecutive tiles at a time
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int unit = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int units = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int ks = unit % p.split;
  const int walker = unit / p.split;
  const int walkers = units / p.split;
  const int steps = PAIR ? (p.tiles + 1) / 2 : p.tiles;  // positions of the tile list a unit walks over
  const int taps = p.R * p.S;
  const int tap0 = ks * p.taps_per_split;
  const int tap1 = min(taps, tap0 + p.taps_per_split);
  const int ntaps = tap1 - tap0;
  const bool dual = p.dual != 0 && ntaps >= 2;
  constexpr int kIssuer2Warp = GATHER ? 14 : 6;   // the last warp of the CTA
  constexpr uint32_t kDualCols = 128;             // columns between the two threads' accumulators
  // filter (or the ring its tiles stream through) first, slabs after it
  constexpr bool streamed = STREAM;  // p.b_stages > 0
  const uint32_t b_stage_bytes = static_cast<uint32_t>(p.b_group) * p.b_tile_bytes;
  const uint32_t b_base = smem_base;
  const uint32_t a_base = smem_base + (streamed ? static_cast<uint32_t>(p.b_stages) * b_stage_bytes
                                                : static_cast<uint32_t>(p.taps_per_split * p.cchunks) * p.b_tile_bytes);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (uint32_t s = 0; s < a_stages; ++s) {
      // a slab is complete when its TMA bytes have landed, or when every loader warp (of both CTAs
      // of a pair) has written its part
      mbar_init(smem_u32(&bar_afull[s]), GATHER ? (PAIR ? 16u : 8u) : 1u);
      mbar_init(smem_u32(&bar_aempty[s]), dual ? 2 : 1);  // one commit per issuing thread
    }
    mbar_init(smem_u32(&bar_bfull), 1);
    for (int s = 0; s < p.b_stages; ++s) {
      mbar_init(smem_u32(&bar_bsfull[s]), 1);
      mbar_init(smem_u32(&bar_bsempty[s]), dual ? 2 : 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tfull[a]), dual ? 2 : 1);
      mbar_init(smem_u32(&bar_tempty[a]), PAIR ? 8 : 4);  // the leader's copy counts both CTAs' epilogue warps
    }
    fence_mbar_init();
    fence_proxy_async_smem();
    if constexpr (!GATHER) prefetch_tmap(&tmap_in);
    prefetch_tmap(&tmap_w);
    if (p.epi_bufs)
      for (int d = 0; d < p.num_dst; ++d) prefetch_tmap(&tmap_out.dst[d]);
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
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  // Launched as a programmatic dependent of the layout pass: everything above overlapped its tail.
  grid_dependency_wait();
  const uint32_t afull0 = smem_u32(&bar_afull[0]);
  const uint32_t aempty0 = smem_u32(&bar_aempty[0]);
  const uint32_t bfull = smem_u32(&bar_bfull);
  const uint32_t bsfull0 = smem_u32(&bar_bsfull[0]);
  const uint32_t bsempty0 = smem_u32(&bar_bsempty[0]);
  const int tiles_per_img = p.tiles_h * p.tiles_w;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && ntaps > 0) {
      // In a pair every completion is reported to the leader's barriers, which the leader arms for
      // the bytes of both CTAs; each CTA stages its own tile's slab and its own half of the filter rows.
      const uint32_t bfull_sig = PAIR ? map_to_cta(bfull, 0) : bfull;
      const uint32_t afull_sig0 = PAIR ? map_to_cta(afull0, 0) : afull0;
      const uint32_t b_bytes_all = static_cast<uint32_t>(ntaps * p.cchunks) * p.b_tile_bytes;
      const uint32_t bsfull_sig0 = PAIR ? map_to_cta(bsfull0, 0) : bsfull0;
      const int n0_half = static_cast<int>(cta_rank) * (p.bn / 2);
      uint32_t bs = 0, bph = 0;
      if (!streamed) {
        if (cta_rank == 0) mbar_expect_tx(bfull, PAIR ? 2u * b_bytes_all : b_bytes_all);
        uint32_t dst = b_base;
        int kc = tap0 * p.cchunks * 32;  // the packed filter is [k_out][tap][chunk][32]
        const int n0 = static_cast<int>(cta_rank) * (p.bn / 2);
        for (int i = 0; i < ntaps * p.cchunks; ++i, dst += p.b_tile_bytes, kc += 32) {
          if constexpr (PAIR) tma_load_3d_pair(dst, &tmap_w, bfull_sig, kc, n0, 0);
          else tma_load_3d(dst, &tmap_w, bfull, kc, 0, 0);
        }
      }
      uint32_t s = 0, ph = 0, sa = a_base;
      bool ok = true;
      long long prof_wait = 0;
      FTB_PROF_T0(prof_loop0);
      for (int tp = walker; tp < steps && ok; tp += walkers) {
        // a tile index past the end (odd tile count in a pair) addresses an image outside the
        // tensor: its loads deliver zeros and its result is never stored
        const int t = PAIR ? 2 * tp + static_cast<int>(cta_rank) : tp;
        const int img = t / tiles_per_img;
        const int rem = t - img * tiles_per_img;
        const int th = rem / p.tiles_w, tw = rem - th * p.tiles_w;
        const int h0 = th * p.tile_h - p.pad_h, w0 = tw * p.tile_w - p.pad_w;
        // conv3d: `img` counts (image, output depth) pairs
        const int img_n = p.od > 0 ? img / p.od : img;
        const int d0 = p.od > 0 ? (img - img_n * p.od) - p.pad_d : 0;
        const int depth_taps = STREAM && p.od > 0 ? p.T : 1;
        bool any_plane = false;
        for (int td = 0; td < depth_taps && ok; ++td) {
        const int dz = d0 + td * p.dil_d;
        if (depth_taps > 1) {
          // a single CTA skips depth taps that fall into the padding (a pair shares its MMAs between
          // two tiles that may lie in different planes, so it loads zeros instead); the last tap is
          // taken if nothing else was, so that the accumulator is always written
          const bool inside = dz >= 0 && dz < p.depth;
          if (!PAIR && !inside && !(td + 1 == depth_taps && !any_plane)) continue;
          any_plane = true;
        }
        const int tap_base = tap0 + td * (p.R * p.S);
        for (int cc = 0; cc < p.cchunks && ok; ++cc) {
          if constexpr (!GATHER) {
          FTB_PROF_T0(prof_w0);
          if (!mbar_wait(aempty0 + 8 * s, ph ^ 1u, &abort_flag)) {
            atomicOr(p.status, FTB_DEV_WAIT_EMPTY);
            abort_flag = 1;
            ok = false;
            break;
          }
          FTB_PROF_ADD(prof_wait, prof_w0);
          if constexpr (PAIR) {
            if (cta_rank == 0) mbar_expect_tx(afull0 + 8 * s, 2u * p.slab_bytes);
            if (p.od > 0) tma_load_5d_pair(sa, &tmap_in, afull_sig0 + 8 * s, cc * 32, w0, h0, dz, img_n);
            else tma_load_4d_pair(sa, &tmap_in, afull_sig0 + 8 * s, cc * 32, w0, h0, img);
          } else {
            mbar_expect_tx(afull0 + 8 * s, p.slab_bytes);
            if (p.od > 0) tma_load_5d(sa, &tmap_in, afull0 + 8 * s, cc * 32, w0, h0, dz, img_n);
            else tma_load_4d(sa, &tmap_in, afull0 + 8 * s, cc * 32, w0, h0, img);
          }
          sa += p.slab_alloc;
          if (++s == a_stages) {
            s = 0;
            ph ^= 1u;
            sa = a_base;
          }
          }
          if (streamed) {
            // this chunk's filter tiles, b_group taps per stage, in the order the issuer takes them
            for (int g0 = 0; g0 < ntaps && ok; g0 += p.b_group) {
              const int nt = min(p.b_group, ntaps - g0);
              if (!mbar_wait(bsempty0 + 8 * bs, bph ^ 1u, &abort_flag)) {
                atomicOr(p.status, FTB_DEV_WAIT_EMPTY);
                abort_flag = 1;
                ok = false;
                break;
              }
              const uint32_t bytes = static_cast<uint32_t>(nt) * p.b_tile_bytes;
              uint32_t dst = b_base + bs * b_stage_bytes;
              int kc = ((tap_base + g0) * p.cchunks + cc) * 32;  // the packed filter is [k_out][tap][chunk][32]
              if constexpr (PAIR) {
                if (cta_rank == 0) mbar_expect_tx(bsfull0 + 8 * bs, 2u * bytes);
                for (int j = 0; j < nt; ++j, dst += p.b_tile_bytes, kc += p.cchunks * 32)
                  tma_load_3d_pair(dst, &tmap_w, bsfull_sig0 + 8 * bs, kc, n0_half, 0);
              } else {
                mbar_expect_tx(bsfull0 + 8 * bs, bytes);
                for (int j = 0; j < nt; ++j, dst += p.b_tile_bytes, kc += p.cchunks * 32)
                  tma_load_3d(dst, &tmap_w, bsfull0 + 8 * bs, kc, 0, 0);
              }
              if (++bs == static_cast<uint32_t>(p.b_stages)) {
                bs = 0;
                bph ^= 1u;
              }
            }
          }
        }
        }
      }
      long long prof_loop = 0;
      FTB_PROF_ADD(prof_loop, prof_loop0);
      FTB_PROF_FLUSH(PROF_PRODUCER_EMPTY, prof_wait);
      FTB_PROF_FLUSH(PROF_PRODUCER_LOOP, prof_loop);
      FTB_PROF_FLUSH(PROF_CTAS, 1);
      (void)prof_wait; (void)prof_loop;
    }
    __syncwarp();
  } else if (warp == 1 || warp == kIssuer2Warp) {
    // ------------------------------------------------------------ MMA issuer(s)
    const uint32_t me = (warp == 1) ? 0u : 1u;  // this thread takes the taps of this parity when there are two
    if (lane == 0 && ntaps > 0 && cta_rank == 0 && (me == 0 || dual)) {
      const uint32_t idesc = p.idesc;
      const uint32_t hi = smem_desc_hi(16, 1024, 2);
      const uint32_t b_tile_enc = p.b_tile_bytes >> 4;
      const uint32_t slab_enc = p.slab_alloc >> 4;
      const uint32_t a_lo0 = smem_desc_lo(a_base, 16);
      const uint32_t b_lo0 = smem_desc_lo(b_base, 16);
      // first tap of this CTA as (row, column) of the filter
      const int tr0 = tap0 / p.S, ts0 = tap0 - tr0 * p.S;
      uint32_t s = 0, ph = 0, a_lo = a_lo0;
      uint32_t bs = 0, bph = 0;
      const uint32_t b_stage_enc = b_stage_bytes >> 4;
      int local = 0;
      bool ok = streamed || mbar_wait(bfull, 0, &abort_flag);
      if (!ok) {
        atomicOr(p.status, FTB_DEV_WAIT_FULL);
        abort_flag = 1;
      }
      long long prof_full = 0, prof_tempty = 0;
      FTB_PROF_T0(prof_iloop0);
      for (int tp = walker; tp < steps && ok; tp += walkers, ++local) {
        const uint32_t acc = local & 1;
        const uint32_t aph = (local >> 1) & 1u;
        FTB_PROF_T0(prof_t0);
        if (!mbar_wait(smem_u32(&bar_tempty[acc]), aph ^ 1u, &abort_flag)) {
          atomicOr(p.status, FTB_DEV_WAIT_TMEMFREE);
          abort_flag = 1;
          break;
        }
        FTB_PROF_ADD(prof_tempty, prof_t0);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride + me * kDualCols;
        uint32_t accumulate = 0;
        // conv3d: the same walk over depth taps as the producer's (skips included)
        const int depth_taps = STREAM && p.od > 0 ? p.T : 1;
        int d0 = 0;
        if (depth_taps > 1 && !PAIR) {
          const int img = tp / tiles_per_img;
          d0 = img % p.od - p.pad_d;
        }
        bool any_plane = false;
        for (int td = 0; td < depth_taps && ok; ++td) {
        if (depth_taps > 1) {
          const int dz = d0 + td * p.dil_d;
          const bool inside = dz >= 0 && dz < p.depth;
          if (!PAIR && !inside && !(td + 1 == depth_taps && !any_plane)) continue;
          any_plane = true;
        }
        for (int cc = 0; cc < p.cchunks; ++cc) {
          FTB_PROF_T0(prof_f0);
          if (!mbar_wait(afull0 + 8 * s, ph, &abort_flag)) {
            atomicOr(p.status, FTB_DEV_WAIT_FULL);
            abort_flag = 1;
            ok = false;
            break;
          }
          FTB_PROF_ADD(prof_full, prof_f0);
          tc_fence_after();
          int tr = tr0, ts = ts0;
          if constexpr (STREAM) {
            for (int g0 = 0; g0 < ntaps && ok; g0 += p.b_group) {
              // the next stage of the filter ring: b_group taps' tiles of this channel chunk
              if (!mbar_wait(bsfull0 + 8 * bs, bph, &abort_flag)) {
                atomicOr(p.status, FTB_DEV_WAIT_FULL);
                abort_flag = 1;
                ok = false;
                break;
              }
              tc_fence_after();
              uint32_t b_lo = b_lo0 + bs * b_stage_enc;
              const int nt = min(p.b_group, ntaps - g0);
              for (int j = 0; j < nt; ++j) {
                const uint32_t ta_lo = a_lo + static_cast<uint32_t>(tr * p.dil_h * p.slab_w + ts * p.dil_w) * 8u;
                if (!dual || (static_cast<uint32_t>(g0 + j) & 1u) == me) {
#pragma unroll
                  for (int k = 0; k < kMmaPerKb; ++k) {
                    umma<KIND_TF32, PAIR>(d_tmem, ta_lo + 2u * k, hi, b_lo + 2u * k, hi, idesc, accumulate);
                    accumulate = 1;
                  }
                }
                b_lo += b_tile_enc;
                if (++ts == p.S) {
                  ts = 0;
                  ++tr;
                }
              }
              // hand the ring stage back once these MMAs have read it
              if constexpr (PAIR) tc_commit_pair_both(bsempty0 + 8 * bs);
              else tc_commit(bsempty0 + 8 * bs);
              if (++bs == static_cast<uint32_t>(p.b_stages)) {
                bs = 0;
                bph ^= 1u;
              }
            }
            if (!ok) break;
          } else {
          uint32_t b_lo = b_lo0 + static_cast<uint32_t>(cc) * b_tile_enc;
          for (int tap = 0; tap < ntaps; ++tap) {
            // The slab is read from `off` pixel rows in.  The tensor core applies the 128-byte
            // swizzle to the absolute shared-memory address, exactly as the TMA unit did when it
            // wrote the slab, so a start address that is not a multiple of the 1024-byte swizzle
            // period needs nothing else in the descriptor (its base-offset field stays 0; measured:
            // setting it to the row phase gives wrong sums).
            uint32_t off = static_cast<uint32_t>(tr * p.dil_h * p.slab_w + ts * p.dil_w);
#ifdef FTB_PROFILE_WAITS
            if (p.diag & 1) off = 0;
            if (p.diag & 2) off &= ~7u;
#endif
            const uint32_t ta_lo = a_lo + off * 8u;
            if (!dual || (static_cast<uint32_t>(tap) & 1u) == me) {
#pragma unroll
              for (int k = 0; k < kMmaPerKb; ++k) {
                umma<KIND_TF32, PAIR>(d_tmem, ta_lo + 2u * k, hi, b_lo + 2u * k, hi, idesc, accumulate);
                accumulate = 1;
              }
            }
            b_lo += static_cast<uint32_t>(p.cchunks) * b_tile_enc;
            if (++ts == p.S) {
              ts = 0;
              ++tr;
            }
          }
          }
          if constexpr (PAIR) tc_commit_pair_both(aempty0 + 8 * s);
          else tc_commit(aempty0 + 8 * s);
          a_lo += slab_enc;
          if (++s == a_stages) {
            s = 0;
            ph ^= 1u;
            a_lo = a_lo0;
          }
        }
        }
        if (ok) {
          if constexpr (PAIR) tc_commit_pair_both(smem_u32(&bar_tfull[acc]));
          else tc_commit(smem_u32(&bar_tfull[acc]));
        }
      }
      long long prof_iloop = 0;
      FTB_PROF_ADD(prof_iloop, prof_iloop0);
      if (me == 0) {
        FTB_PROF_FLUSH(PROF_ISSUER_FULL, prof_full);
        FTB_PROF_FLUSH(PROF_ISSUER_TEMPTY, prof_tempty);
        FTB_PROF_FLUSH(PROF_ISSUER_LOOP, prof_iloop);
      }
      (void)prof_full; (void)prof_tempty; (void)prof_iloop;
    }
    __syncwarp();
  } else if (GATHER && warp >= 6 && warp < 14) {
    // ------------------------------------------------------------ slab loader (NCHW input)
    // 256 threads build the slab of every (tile, channel chunk): warp g takes the channels 4 g .. 4 g + 3
    // of the chunk, its lanes 32 consecutive slab pixels, so that a warp-wide load is one 128-byte line
    // of a channel plane (minus what falls into the padding).  The writes into the swizzled slab (16-byte
    // chunk index = (channel / 4) ^ (pixel & 7)) collide four ways, which is nothing beside the loads'
    // latency; sixteen loads are in flight per thread.
    if (ntaps > 0) {
      const int lt = static_cast<int>(threadIdx.x) - 192;
      const int g = lt >> 5;
      const int slab_h = p.tile_h + (p.R - 1) * p.dil_h;
      const int plane = p.H * p.W;
      const uint32_t afull_sig0 = PAIR ? map_to_cta(afull0, 0) : afull0;
      uint32_t s = 0, ph = 0, sa = a_base;
      bool ok = true;
      for (int tp = walker; tp < steps && ok; tp += walkers) {
        const int t = PAIR ? 2 * tp + static_cast<int>(cta_rank) : tp;
        const int img = t / tiles_per_img;
        const int rem = t - img * tiles_per_img;
        const int th = rem / p.tiles_w, tw = rem - th * p.tiles_w;
        const int h0 = th * p.tile_h - p.pad_h, w0 = tw * p.tile_w - p.pad_w;
        const bool img_ok = img < p.n_imgs;
        for (int cc = 0; cc < p.cchunks && ok; ++cc) {
          if (lane == 0) ok = mbar_wait(aempty0 + 8 * s, ph ^ 1u, &abort_flag);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) {
            if (lane == 0) {
              atomicOr(p.status, FTB_DEV_WAIT_EMPTY);
              abort_flag = 1;
            }
            break;
          }
          const int ch0 = cc * 32 + 4 * g;
          const float* src = p.in_nchw + (static_cast<long long>(img) * p.C + ch0) * static_cast<long long>(plane);
          // rows of the slab in groups of kRows, a lane per slab column: the row tests are uniform over
          // the warp and the address arithmetic is a few instructions per 4 * kRows loads (the loader is
          // bound by instruction issue as much as by latency: a version that worked out row and column
          // per pixel was half as fast)
          constexpr int kRows = 4;
          const bool c1 = ch0 + 1 < p.C, c2 = ch0 + 2 < p.C, c3 = ch0 + 3 < p.C;
          const bool c0 = img_ok && ch0 < p.C;
          for (int sr0 = 0; sr0 < slab_h; sr0 += kRows) {
            for (int sc = lane; sc < p.slab_w; sc += 32) {
              const int w = w0 + sc;
              const bool col_ok = c0 && w >= 0 && w < p.W;
              float v[kRows][4];
#pragma unroll
              for (int r = 0; r < kRows; ++r) {
                const int h = h0 + sr0 + r;
                const bool inside = col_ok && sr0 + r < slab_h && h >= 0 && h < p.H;
                const float* at = src + h * p.W + w;
                v[r][0] = inside ? __ldg(at) : 0.0f;
                v[r][1] = (inside && c1) ? __ldg(at + plane) : 0.0f;
                v[r][2] = (inside && c2) ? __ldg(at + 2 * plane) : 0.0f;
                v[r][3] = (inside && c3) ? __ldg(at + 3 * plane) : 0.0f;
              }
#pragma unroll
              for (int r = 0; r < kRows; ++r) {
                if (sr0 + r < slab_h) {
                  const uint32_t px = static_cast<uint32_t>((sr0 + r) * p.slab_w + sc);
                  st_shared_v4(sa + px * 128u + ((static_cast<uint32_t>(g) ^ (px & 7u)) << 4), __float_as_uint(v[r][0]),
                               __float_as_uint(v[r][1]), __float_as_uint(v[r][2]), __float_as_uint(v[r][3]));
                }
              }
            }
          }
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster_release(afull_sig0 + 8 * s);
            else mbar_arrive(afull0 + 8 * s);
          }
          sa += p.slab_alloc;
          if (++s == a_stages) {
            s = 0;
            ph ^= 1u;
            sa = a_base;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int prow = row / p.slab_w, pcol = row - prow * p.slab_w;
    const bool in_tile = prow < p.tile_h && pcol < p.tile_w;
    const long long plane = static_cast<long long>(p.P) * p.Q;
    int local = 0;
    uint32_t epi_seq = 0;
    const uint32_t epi_base = a_base + a_stages * p.slab_alloc;
    const uint32_t tempty_sig0 = PAIR ? map_to_cta(smem_u32(&bar_tempty[0]), 0) : smem_u32(&bar_tempty[0]);
    long long prof_tfull = 0;
    FTB_PROF_T0(prof_eloop0);
    if (ntaps > 0) {
      for (int tp = walker; tp < steps; tp += walkers, ++local) {
        const int t = PAIR ? 2 * tp + static_cast<int>(cta_rank) : tp;
        const bool tile_valid = t < p.tiles;
        const uint32_t acc = local & 1;
        const uint32_t aph = (local >> 1) & 1u;
        FTB_PROF_T0(prof_e0);
        bool got = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_tfull[acc]), aph, &abort_flag));
        FTB_PROF_ADD(prof_tfull, prof_e0);
        // The staged epilogue synchronises the four warps with each other: they must agree.
        if (p.epi_bufs) got = named_barrier_all(2, 128, got);
        if (!got) {
          if (lane == 0) {
            atomicOr(p.status, FTB_DEV_WAIT_TMEMFULL);
            abort_flag = 1;
          }
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccStride;
        const int img = t / tiles_per_img;
        const int rem = t - img * tiles_per_img;
        const int th = rem / p.tiles_w, tw = rem - th * p.tiles_w;
        // conv3d: `img` counts (image, output depth) pairs
        const int img_n = p.od > 0 ? img / p.od : img;
        const int img_d = p.od > 0 ? img - img_n * p.od : 0;
        if (p.epi_bufs && p.cl_out) {
          // ---- channels-last result: TMEM -> registers -> [tile_h][tile_w][32 channels] in shared memory
          // (a lane writes its pixel's 128 bytes) -> one bulk tensor store per 32 output channels
          const bool leader = (warp == 2 && lane == 0);
          const uint32_t px_row = static_cast<uint32_t>(prow * p.tile_w + pcol) * 128u;
          const uint32_t px_swz = p.cl_swz ? (static_cast<uint32_t>(prow * p.tile_w + pcol) & 7u) : 0u;
          for (int c = 0; c < p.bn; c += 32, ++epi_seq) {
            const uint32_t buf = epi_base + (p.epi_bufs == 2 ? (epi_seq & 1u) : 0u) * p.epi_buf_bytes;
            // the accumulator columns come into registers (and the accumulator goes back) while the previous
            // bulk store is still reading the staging buffer
            uint32_t v[32];
            slab_acc_ld(taddr + c, dual ? kDualCols : 0u, v);
            if (c + 32 >= p.bn) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(tempty_sig0 + 8 * acc);
                else mbar_arrive(tempty_sig0 + 8 * acc);
              }
            }
            if (leader) {
              if (p.epi_bufs == 2) bulk_wait_group_read<1>();
              else bulk_wait_group_read<0>();
            }
            named_barrier_sync(1, 128);
            if (in_tile) {
              const bool add_bias = p.bias != nullptr && ks == 0;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float x = __uint_as_float(v[j]);
                if (add_bias && c + j < p.N) x += p.bias[c + j];
                if (p.relu) x = fmaxf(x, 0.0f);
                v[j] = __float_as_uint(x);
              }
              // (the lanes' 128-byte pitch would make these stores collide on their banks: chunk j of pixel
              // px goes to position j ^ (px & 7), which the swizzled store map undoes)
#pragma unroll
              for (int j = 0; j < 8; ++j)
                st_shared_v4(buf + px_row + ((static_cast<uint32_t>(j) ^ px_swz) << 4), v[4 * j], v[4 * j + 1],
                             v[4 * j + 2], v[4 * j + 3]);
            }
            fence_proxy_async_smem();
            named_barrier_sync(1, 128);
            if (leader) {
              if (c < p.N && tile_valid) {
                if (p.split > 1) {
                  tma_reduce_add_4d(&tmap_out.dst[0], buf, c, tw * p.tile_w, th * p.tile_h, img);
                } else {
                  for (int d = 0; d < p.num_dst; ++d)
                    tma_store_4d(&tmap_out.dst[d], buf, c, tw * p.tile_w, th * p.tile_h, img);
                }
              }
              bulk_commit_group();
            }
          }
          continue;
        }
        if (p.epi_bufs) {
          // ---- TMEM -> registers -> [channel][tile_h][tile_w] in shared memory -> one bulk tensor
          // store (or fp32 reduce-add when the taps are split) per 32 output channels.  Lanes hold
          // consecutive pixels, so the shared-memory writes of one channel are conflict-free and
          // global memory sees whole rows of every channel plane.
          const bool leader = (warp == 2 && lane == 0);
          const uint32_t px_off = static_cast<uint32_t>(prow * p.tile_w + pcol) * 4u;
          const uint32_t ch_stride = static_cast<uint32_t>(p.tile_h * p.tile_w) * 4u;
          for (int c = 0; c < p.bn; c += 32, ++epi_seq) {
            const uint32_t buf = epi_base + (p.epi_bufs == 2 ? (epi_seq & 1u) : 0u) * p.epi_buf_bytes;
            // the accumulator columns come into registers (and the accumulator goes back) while the previous
            // bulk store is still reading the staging buffer
            uint32_t v[32];
            slab_acc_ld(taddr + c, dual ? kDualCols : 0u, v);
            if (c + 32 >= p.bn) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(tempty_sig0 + 8 * acc);
                else mbar_arrive(tempty_sig0 + 8 * acc);
              }
            }
            if (leader) {
              if (p.epi_bufs == 2) bulk_wait_group_read<1>();
              else bulk_wait_group_read<0>();
            }
            named_barrier_sync(1, 128);
            if (in_tile) {
              const bool add_bias = p.bias != nullptr && ks == 0;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float x = __uint_as_float(v[j]);
                if (add_bias && c + j < p.N) x += p.bias[c + j];
                if (p.relu) x = fmaxf(x, 0.0f);
                st_shared_f32(buf + static_cast<uint32_t>(j) * ch_stride + px_off, x);
              }
            }
            fence_proxy_async_smem();
            named_barrier_sync(1, 128);
            if (leader) {
              if (c < p.N && tile_valid) {
                if (p.od > 0) {
                  // conv3d: (w, h, depth, channel, image)
                  for (int d = 0; d < p.num_dst; ++d)
                    tma_store_5d(&tmap_out.dst[d], buf, tw * p.tile_w, th * p.tile_h, img_d, c, img_n);
                } else if (p.split > 1) {
                  tma_reduce_add_4d(&tmap_out.dst[0], buf, tw * p.tile_w, th * p.tile_h, c, img);
                } else {
                  // every destination gets the same box: this GPU's result and, in a batch-sharded
                  // run, the same images of every peer's gathered output (stores over NVLink)
                  for (int d = 0; d < p.num_dst; ++d)
                    tma_store_4d(&tmap_out.dst[d], buf, tw * p.tile_w, th * p.tile_h, c, img);
                }
              }
              bulk_commit_group();
            }
          }
          continue;
        }
        const int oh = th * p.tile_h + prow, ow = tw * p.tile_w + pcol;
        const bool row_ok = in_tile && oh < p.P && ow < p.Q && tile_valid;
        const long long ch_stride = p.cl_out ? 1 : (p.od > 0 ? plane * p.od : plane);
        float* dst0 = p.cl_out ? p.out + (static_cast<long long>(img) * plane + static_cast<long long>(oh) * p.Q + ow) * p.conv_ktot
                      : p.od > 0 ? p.out + (static_cast<long long>(img_n) * p.conv_ktot * p.od + img_d) * plane +
                                       static_cast<long long>(oh) * p.Q + ow
                                 : p.out + static_cast<long long>(img) * p.conv_ktot * plane + static_cast<long long>(oh) * p.Q + ow;
        for (int c = 0; c < p.bn; c += 32) {
          uint32_t v[32];
          slab_acc_ld(taddr + c, dual ? kDualCols : 0u, v);
          if (c + 32 >= p.bn) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(tempty_sig0 + 8 * acc);
              else mbar_arrive(tempty_sig0 + 8 * acc);
            }
          }
          if (!row_ok) continue;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = c + j;
            if (n < p.N) {
              float x = __uint_as_float(v[j]);
              if (p.bias != nullptr && ks == 0) x += p.bias[n];
              if (p.relu) x = fmaxf(x, 0.0f);
              float* dst = dst0 + n * ch_stride;
              if (p.split > 1) atomicAdd(dst, x);
              else *dst = x;
            }
          }
        }
      }
    }
    if (warp == 2 && lane == 0) {
      long long prof_eloop = 0;
      FTB_PROF_ADD(prof_eloop, prof_eloop0);
      FTB_PROF_FLUSH(PROF_EPI_TFULL, prof_tfull);
      FTB_PROF_FLUSH(PROF_EPI_LOOP, prof_eloop);
      (void)prof_eloop;
    }
    (void)prof_tfull;
    // Shared memory must outlive the bulk stores' reads of it; their global writes are complete
    // when the grid is - except stores into a peer GPU's memory, which are waited for in full.
    if (p.epi_bufs && warp == 2 && lane == 0) {
      if (p.num_dst > 1) bulk_wait_group<0>();
      else bulk_wait_group_read<0>();
    }
    __syncwarp();
  }

  // ------------------------------------------------------------ teardown
  if (*reinterpret_cast<volatile int*>(&abort_flag)) {
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
