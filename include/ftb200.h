/*
 * ftb200 - C ABI of the B200 (sm_100a) kernel backend that stands where FlexTensor's
 * TVM-built CUDA modules stood.
 *
 * The reference has no C boundary of its own: its boundary is the callable returned by
 * `tvm.build(s, bufs, target)` (README.md:153-158, flextensor/optimize/common.py:34-48,
 * flextensor/measure.py:87-110), called destination-passing with the arrays of `bufs`
 * in order, output last.  Each launcher below is what that callable binds to for one
 * operator of flextensor/nn/ops.py; the operator it replaces is cited beside it.
 *
 * Conventions
 *   - every pointer is a device pointer owned by the caller; the library allocates no
 *     device memory at run time (its image holds two `__device__` status words and the fixed
 *     FTB_NOALLOC_SCRATCH_BYTES array of ftb_conv2d_nchw_f32_noalloc, resident on every GPU
 *     that loads it);
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it;
 *   - return value: 0 on success, a negative FTB_E_* code otherwise; nothing throws,
 *     exits or prints;
 *   - `status` is a device int (may be NULL): kernels OR a non-zero FTB_DEV_* bit into it
 *     when a bounded in-kernel wait ran out; read it after synchronising the stream;
 *   - `cfg` may be NULL: every knob then takes its default (0 means "default" per field).
 */
#ifndef FTB200_H_
#define FTB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FTB_VERSION 100

enum ftb_error {
  FTB_OK = 0,
  FTB_E_BAD_ARG = -1,     /* null pointer, non-positive extent, unknown enum value      */
  FTB_E_UNSUPPORTED = -2, /* shape the kernels cannot take (e.g. conv groups that break 16-byte alignment) */
  FTB_E_BAD_CONFIG = -3,  /* knob outside its range or over the shared-memory budget    */
  FTB_E_WORKSPACE = -4,   /* workspace missing or too small                             */
  FTB_E_CUDA = -5,        /* a CUDA runtime/driver call failed; see ftb_last_cuda_error */
  FTB_E_NO_DEVICE = -6,   /* current device is not compute capability 10.x              */
  FTB_E_TOO_LARGE = -7    /* size beyond a stated maximum of the entry point            */
};

/* Knobs of the kernels: the config space the scheduler searches
 * (replaces the split/fuse/reorder/unroll factors of flextensor/templates/cuda.py:390-661). */
typedef struct ftb_config {
  int32_t tile_n;    /* accumulator columns per tile: 32, 64, 128 or 256; 512 with cluster 2 (GEMMs) */
  int32_t stages;    /* shared-memory pipeline depth, 2..8                                */
  int32_t raster;    /* tile order: 0 auto, 1 n-fastest, 2 m-fastest, 3 grouped-M         */
  int32_t group_m;   /* group height for raster 3                                         */
  int32_t split_k;   /* K splits accumulated with atomics (fp32 outputs only)             */
  int32_t fp32_mode; /* fp32 inputs: 0 = single-pass TF32, 1 = 3xTF32 (fp32-grade)        */
  int32_t ctas;      /* persistent CTAs (default: one per SM)                             */
  int32_t tile_h;    /* conv2d: output rows per tile; depthwise: output rows per strip    */
  int32_t threads;   /* depthwise: threads per CTA                                        */
  int32_t cluster;   /* 1 = one CTA per 128-row tile, 2 = CTA pair on a 256-row tile       */
  int32_t algo;      /* conv2d: 0 auto; 1 one shifted input tile per filter tap; 2 one input slab per
                        channel chunk shared by all taps, filter resident in shared memory (stride 1,
                        groups 1, <= 256 output channels, single-pass TF32); 3 batched GEMM on the
                        NCHW tensors as they are (1x1 filter, stride 1, no padding, groups 1); 4 a 1x1
                        conv over the im2col form of the input (at most 8 input channels, groups 1); 5 the
                        slab kernel of 2 with the filter streamed through a ring of shared-memory stages
                        instead of resident (what 0 and 2 pick by themselves for a filter that does not
                        fit and a tile list long enough to keep the SMs busy)                            */
  int32_t epilogue;  /* 0 = bulk tensor stores from shared memory wherever they can address the result
                        (default); 1 = per-thread global stores everywhere (same bits; for diagnosis)   */
  int32_t release;   /* 1 = a pipeline stage goes back to the loader after every K block; 2 = stages go back
                        two at a time (half the tcgen05.commit count; needs an even number of stages >= 4,
                        ignored otherwise, for 3xTF32 and for tile_n = 512); 0 = 1 for GEMMs, and for the
                        per-tap conv kernels 2 on tiles of at most 128 output channels, else 1           */
  int32_t relu;      /* conv2d and depthwise: 1 = clamp the result at zero after the bias (the conv + bias +
                        ReLU chain of a network as one kernel); not a search knob                       */
  int32_t gather;    /* conv2d on NCHW tensors, slab kernel: 1 = the layout pass writes a channels-last copy and
                        the slabs are TMA loads; 2 = eight loader warps of the kernel build the slabs from the
                        NCHW tensor themselves (no copy: the input crosses HBM once); 0 = 2 for long tile lists
                        with unsplit taps and slab rows of at most 64 pixels, else 1                          */
  int32_t reserved[1];
} ftb_config;

int ftb_version(void);
const char* ftb_strerror(int code);
/* Last CUDA error code seen by a launcher of this process (cudaError_t / CUresult value). */
int ftb_last_cuda_error(void);
/* 0 when the current device can run the kernels (compute capability 10.x). */
int ftb_device_check(void);
/* Checks a knob set against the limits of an operator without launching:
 * op = 0 gemm_f32, 1 bgemm_bf16, 2 gemm_s8, 3 conv2d, 4 depthwise
 * (host-side counterpart of flextensor/scheduler.py:58-76 verify_code). */
int ftb_validate(int op, const ftb_config* cfg, int64_t m, int64_t n, int64_t k);
/* Number of kernels this library has launched in this process (all entry points). */
int64_t ftb_launch_count(void);

/* Self-test of the failure path (no counterpart in the reference): launches one thread that waits,
 * with the same bounded wait every kernel uses, on a barrier nothing completes.  After about two
 * seconds the wait gives up, ORs FTB_DEV bit 1 into *status and the kernel ends normally; the
 * context stays usable.  Lets a host verify that a stuck pipeline surfaces as a status, not a hang. */
int ftb_selftest_bounded_wait(int* status, void* stream);

/* Diagnostic builds only (library compiled with -DFTB_PROFILE_WAITS; the product build returns
 * FTB_E_UNSUPPORTED): synchronises the device and copies out sixteen counters of SM cycles, summed
 * over the CTAs of every tensor-core GEMM launch since the last reset - [0] producer waiting for a
 * free stage, [1] MMA issuer waiting for a stage to land, [2] MMA issuer waiting for a free
 * accumulator, [3] epilogue waiting for a finished accumulator, [4] [5] [6] the whole loops of the
 * producer, the issuer and the first epilogue warp, [7] CTAs that reported, [8] [9] [10] first
 * epilogue warp of a 256 x 512 tile: inside its tcgen05.ld, waiting for a bulk store to release
 * its staging buffer, converting and staging, [11] issuing bulk stores, [12] handing the
 * accumulator back, packing and voting ([13]-[15] unused).  Tells which hand-off
 * of the pipeline a kernel is waiting on; no counterpart in the reference. */
int ftb_debug_wait_profile(uint64_t* cycles, int reset);

/* GEMM entry points: operands whose row pitch or base address is not a multiple of 16 bytes cannot
 * be read by TMA; such calls are served by a CUDA-core kernel (correct, roughly 10x slower; plain
 * fp32 arithmetic for fp32 inputs).  Everything else runs on the tcgen05 kernel. */

/* C[M,N] = op(A) . op(B), fp32 in/out, TF32 tensor cores (flextensor/nn/ops.py:1074-1108 gemm).
 * trans_a = 0: A is [M,K] row-major, 1: A is [K,M]; trans_b = 0: B is [K,N], 1: B is [N,K]. */
int ftb_gemm_f32(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                 int trans_a, int trans_b, const ftb_config* cfg, int* status, void* stream);

/* C[b,M,N] = op(A[b]) . op(B[b]) in fp32 (flextensor/nn/ops.py:1111-1158 batch_gemm as the
 * reference defines it: fp32 placeholders). */
int ftb_bgemm_f32(const float* a, const float* b, float* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                  int trans_a, int trans_b, const ftb_config* cfg, int* status, void* stream);

/* C[b,M,N] = op(A[b]) . op(B[b]); bf16 inputs, fp32 accumulate, output bf16 (out_f32 = 0) or
 * fp32 (out_f32 = 1) (flextensor/nn/ops.py:1111-1158 batch_gemm, extended to bf16). */
int ftb_bgemm_bf16(const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n,
                   int64_t k, int trans_a, int trans_b, int out_f32, const ftb_config* cfg,
                   int* status, void* stream);

/* The same, with the result written to `num_dst` (1..8) buffers at once: c_dst is a host array of
 * device pointers, each to a [batch,M,N] buffer that may live on this GPU or be a mapped buffer
 * of a peer GPU.  Used by the batch-sharded path to place a rank's slice of the output directly
 * in every rank's gathered buffer (an all-gather fused into the GEMM epilogue as bulk tensor
 * stores over NVLink).  Needs N*elem_size % 16 == 0
 * and 16-byte aligned destinations; no counterpart in the reference (it is single-device). */
int ftb_bgemm_bf16_multi(const void* a, const void* b, void* const* c_dst, int num_dst, int64_t batch,
                         int64_t m, int64_t n, int64_t k, int trans_a, int trans_b, int out_f32,
                         const ftb_config* cfg, int* status, void* stream);

/* C[M,N] (int32) = op(A) . op(B), int8 inputs, exact int32 accumulation
 * (contract of flextensor/test/test_tvm/legacy/gemm_int8.py:15-21,143-148; trans_b = 1 is its
 * B[N,K] layout, trans_b = 0 the numpy `A @ B` layout). */
int ftb_gemm_s8(const int8_t* a, const int8_t* b, int32_t* c, int64_t m, int64_t n, int64_t k,
                int trans_a, int trans_b, const ftb_config* cfg, int* status, void* stream);

/* out[N,K,P,Q] = conv2d(in[N,C,H,W], w[K,C/groups,R,S]) (+ bias[K]), cross-correlation with
 * zero padding folded into the loads (flextensor/nn/ops.py:83-117 zero_pad2d + :419-479
 * conv2d_nchw).  `workspace` holds the channels-last copy of the input and the packed
 * weights; its size comes from ftb_conv2d_workspace_bytes. */
size_t ftb_conv2d_workspace_bytes(int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                                  int64_t s, int64_t groups);
int ftb_conv2d_nchw_f32(const float* in, const float* weight, const float* bias, float* out,
                        int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r, int64_t s,
                        int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                        int groups, const ftb_config* cfg, void* workspace, size_t workspace_bytes,
                        int* status, void* stream);

/* Filter packing taken off the per-call path (weights are constant per task: the reference
 * binds them as a placeholder of the task, flextensor/task.py:74-78).  ftb_conv2d_pack_filter writes the
 * packed form of `weight` into the filter region of `workspace` and returns; after it,
 * ftb_conv2d_nchw_f32_prepacked runs the conv with the SAME shape arguments, knobs and workspace
 * and only lays out the input.  `weight` is still passed (1x1 filters that run as a GEMM on the
 * NCHW tensors read it as it is).  The caller re-packs when the weights change. */
int ftb_conv2d_pack_filter(const float* weight, int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                           int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                           int groups, const ftb_config* cfg, void* workspace, size_t workspace_bytes,
                           void* stream);
int ftb_conv2d_nchw_f32_prepacked(const float* in, const float* weight, const float* bias, float* out, int64_t n,
                                  int64_t c, int64_t h, int64_t w, int64_t k, int64_t r, int64_t s, int stride_h,
                                  int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int groups,
                                  const ftb_config* cfg, void* workspace, size_t workspace_bytes, int* status,
                                  void* stream);

/* The same, with the result written to `num_dst` (1..8) buffers at once: c_dst-style host array of
 * device pointers to [N,K,P,Q] buffers, this GPU's or a peer GPU's mapped memory (16-byte
 * aligned).  The batch-sharded path places a rank's images in every rank's gathered output this
 * way (bulk tensor stores over NVLink from the conv epilogue).  Only the epilogues that leave
 * through bulk stores can do it: output rows of a multiple of 16 bytes, no reduction split over
 * CTAs; anything else returns FTB_E_UNSUPPORTED and the caller copies the result itself.
 * `prepacked` != 0: the workspace already holds the filter's packing (see above).  No
 * counterpart in the reference (it is single-device). */
int ftb_conv2d_nchw_f32_multi(const float* in, const float* weight, const float* bias, float* const* out_dst,
                              int num_dst, int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                              int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
                              int groups, int prepacked, const ftb_config* cfg, void* workspace,
                              size_t workspace_bytes, int* status, void* stream);

/* The same convolution on channels-last tensors: in[N,H,W,C], out[N,P,Q,K] (+ bias[K]); the filter keeps the
 * reference's [K,C/groups,R,S] layout.  This is the B200 form of the layout rewrite the reference applies to
 * conv2d tasks (flextensor/scheduler.py:825-862 Rewriter, NCHW -> NCHWc for the CPU): the tensor-core kernels
 * want the channels innermost, so a caller that keeps its activations channels-last skips the layout pass of
 * ftb_conv2d_nchw_f32 altogether - the tensor maps sit on `in` and `out` themselves.  Needs channels per group
 * (in and out) that are multiples of 4 and 16-byte aligned tensors, else FTB_E_UNSUPPORTED.  `workspace`
 * (256-byte aligned, ftb_conv2d_nhwc_workspace_bytes) holds the packed filter only; `prepacked` != 0: it
 * already holds this filter's packing from an earlier call with the same shape arguments and knobs.  Knobs
 * as for conv2d; `algo` 3 and 4 do not apply. */
size_t ftb_conv2d_nhwc_workspace_bytes(int64_t c, int64_t k, int64_t r, int64_t s, int64_t groups);
int ftb_conv2d_nhwc_f32(const float* in, const float* weight, const float* bias, float* out, int64_t n, int64_t c,
                        int64_t h, int64_t w, int64_t k, int64_t r, int64_t s, int stride_h, int stride_w, int pad_h,
                        int pad_w, int dil_h, int dil_w, int groups, int prepacked, const ftb_config* cfg,
                        void* workspace, size_t workspace_bytes, int* status, void* stream);

/* out[N,K,OD,P,Q] = conv3d(in[N,C,D,H,W], w[K,C/groups,T,R,S]) (+ bias[K]), cross-correlation with
 * zero padding folded into the loads (flextensor/nn/ops.py:157-189 zero_pad3d + :689-751
 * conv3d_ncdhw).  stride_dhw / pad_dhw / dil_dhw point at three host ints each (depth, height,
 * width).  The same implicit-GEMM kernel as conv2d with a third tap loop; groups run as one launch
 * each.  Knobs as for conv2d; `algo` 0, 1 or 5 (5: at stride 1 and one group, the slab kernel with one input
 * slab per depth tap and channel chunk and the filter streamed; 0 picks it for long tile lists).  `workspace` as for conv2d, sized by
 * ftb_conv3d_workspace_bytes; `prepacked` != 0: it already holds this filter's packing from an earlier call
 * with the same shape arguments and knobs (weights are constant per task), only the input is laid out. */
size_t ftb_conv3d_workspace_bytes(int64_t n, int64_t c, int64_t d, int64_t h, int64_t w, int64_t k, int64_t t,
                                  int64_t r, int64_t s, int64_t groups);
int ftb_conv3d_ncdhw_f32(const float* in, const float* weight, const float* bias, float* out, int64_t n, int64_t c,
                         int64_t d, int64_t h, int64_t w, int64_t k, int64_t t, int64_t r, int64_t s,
                         const int32_t* stride_dhw, const int32_t* pad_dhw, const int32_t* dil_dhw, int groups,
                         int prepacked, const ftb_config* cfg, void* workspace, size_t workspace_bytes, int* status,
                         void* stream);

/* conv2d without a caller workspace - no counterpart in the reference.
 *
 * For callers that cannot allocate device memory: code that receives its input and output
 * buffers from another runtime and has no allocator of its own, or a serving loop that bans
 * allocation after start-up (cudaMalloc synchronises the device and may fail when memory is
 * tight).  Same computation and arguments as ftb_conv2d_nchw_f32 minus the workspace: the
 * channels-last copy of the input and the packed weights go into a fixed array of
 * FTB_NOALLOC_SCRATCH_BYTES that the library keeps in device global memory (every GPU that loads
 * the library holds it until the process exits).  The call allocates and frees nothing.
 *
 *   - a shape whose workspace (ftb_conv2d_workspace_bytes) exceeds FTB_NOALLOC_SCRATCH_BYTES is
 *     refused with FTB_E_TOO_LARGE;
 *   - the first call on a device looks up the array's device address (once per device, with that
 *     device current); make that first call before starting any stream capture;
 *   - all calls share the one array and it keeps what the last call wrote; nothing in it needs
 *     clearing (each call rewrites every byte it later reads), but two calls that overlap in time
 *     on the same GPU - different streams, or different threads - race on it: serialise them. */
#define FTB_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
int ftb_conv2d_nchw_f32_noalloc(const float* in, const float* weight, const float* bias, float* out,
                                int64_t n, int64_t c, int64_t h, int64_t w, int64_t k, int64_t r,
                                int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h,
                                int dil_w, int groups, const ftb_config* cfg, int* status, void* stream);

/* out[N,C*f,P,Q] = depthwise conv of in[N,C,H,W] with w[C,f,R,S] (+ bias[C*f])
 * (flextensor/nn/ops.py:622-678 depthwise_conv2d_nchw; note the [C,f,R,S] weight layout). */
int ftb_dwconv2d_nchw_f32(const float* in, const float* weight, const float* bias, float* out,
                          int64_t n, int64_t c, int64_t h, int64_t w, int64_t factor, int64_t r,
                          int64_t s, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h,
                          int dil_w, const ftb_config* cfg, int* status, void* stream);

/* The same, with the result written to `num_dst` (1..8) buffers at once (all [N,C*f,P,Q], equally
 * aligned): this GPU's memory or a peer GPU's mapped buffer.  The batch-sharded path places a
 * rank's images directly in every rank's gathered output this way (plain stores over NVLink, no
 * collective); no counterpart in the reference (it is single-device). */
int ftb_dwconv2d_nchw_f32_multi(const float* in, const float* weight, const float* bias, float* const* out_dst,
                                int num_dst, int64_t n, int64_t c, int64_t h, int64_t w, int64_t factor,
                                int64_t r, int64_t s, int stride_h, int stride_w, int pad_h, int pad_w,
                                int dil_h, int dil_w, const ftb_config* cfg, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FTB200_H_ */
