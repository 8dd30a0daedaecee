/* TEST INFRASTRUCTURE - plain-C restatement of the reference's operators and of the loop
 * nest its llvm template produces.  Not part of the product path: used by tests as a second
 * checker and by bench.py as the timed CPU baseline.
 *
 * Part 1 (fto_*_naive): the index expressions of flextensor/nn/ops.py of pku-liang/FlexTensor,
 * one loop per axis, the reduction innermost, exactly as a default te.create_schedule would
 * run them (this is the parity reference of flextensor/optimize/common.py:63-82):
 *   zero_pad2d ops.py:83-117, conv2d_nchw :419-479, depthwise_conv2d_nchw :622-678,
 *   gemm :1074-1108, batch_gemm :1111-1158, int8 GEMM test/test_tvm/legacy/gemm_int8.py:15-21.
 *
 * Part 2 (fto_*_tiled): the loop structure flextensor/templates/cpu.py:316-518
 * (cpu_schedule_simple) emits for a config: the outermost spatial parts fused and run
 * `parallel` (:370-387), a write-cache block per inner tile (:320,408), the reduce loops
 * placed above the innermost spatial tile (:477-493), the innermost spatial axis vectorised
 * (:388-405,498-505).  Tile factors are arguments, the way split factors are knobs there.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline int64_t out_size(int64_t size, int64_t kernel, int64_t stride, int64_t pad, int64_t dil) {
  return (size + 2 * pad - dil * (kernel - 1) - 1) / stride + 1;
}

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

int fto_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Number of OpenMP threads the tiled nests use from now on (launchers such as torchrun export
 * OMP_NUM_THREADS=1; the timed CPU baseline asks for every core it is allowed to run on). */
void fto_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------ part 1: naive */

/* C[i,j] = sum_k opA(i,k) * opB(k,j); double accumulation when acc64 != 0. */
void fto_gemm_f32_naive(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int ta,
                        int tb, int acc64) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      double accd = 0.0;
      float accf = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        const float a = ta ? A[k * M + i] : A[i * K + k];
        const float b = tb ? B[j * K + k] : B[k * N + j];
        if (acc64) accd += (double)a * (double)b;
        else accf += a * b;
      }
      C[i * N + j] = acc64 ? (float)accd : accf;
    }
}

/* bf16 inputs (bit patterns), fp32 accumulate of exact products, bf16 or fp32 output. */
void fto_bgemm_bf16_naive(const uint16_t* A, const uint16_t* B, void* C, int64_t batch, int64_t M, int64_t N,
                          int64_t K, int ta, int tb, int out_f32) {
  for (int64_t b = 0; b < batch; ++b) {
    const uint16_t* Ab = A + b * M * K;
    const uint16_t* Bb = B + b * K * N;
    for (int64_t i = 0; i < M; ++i)
      for (int64_t j = 0; j < N; ++j) {
        double acc = 0.0; /* products of bf16 are exact in double; the sum is the fp32-accumulate truth */
        for (int64_t k = 0; k < K; ++k) {
          const float a = bf16_to_f32(ta ? Ab[k * M + i] : Ab[i * K + k]);
          const float bb = bf16_to_f32(tb ? Bb[j * K + k] : Bb[k * N + j]);
          acc += (double)a * (double)bb;
        }
        if (out_f32) ((float*)C)[(b * M + i) * N + j] = (float)acc;
        else ((uint16_t*)C)[(b * M + i) * N + j] = f32_to_bf16((float)acc);
      }
  }
}

void fto_gemm_s8_naive(const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K, int ta,
                       int tb) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      int32_t acc = 0;
      for (int64_t k = 0; k < K; ++k) {
        const int32_t a = ta ? A[k * M + i] : A[i * K + k];
        const int32_t b = tb ? B[j * K + k] : B[k * N + j];
        acc += a * b;
      }
      C[i * N + j] = acc;
    }
}

/* Explicit padded tensor, then the conv lambda; returns 0, or -1 when allocation fails. */
int fto_conv2d_nchw_f32_naive(const float* in, const float* w, const float* bias, float* out, int64_t N,
                              int64_t C, int64_t H, int64_t W, int64_t K, int64_t R, int64_t S, int64_t sh,
                              int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw, int64_t groups,
                              int acc64) {
  const int64_t HP = H + 2 * ph, WP = W + 2 * pw;
  const int64_t P = out_size(H, R, sh, ph, dh), Q = out_size(W, S, sw, pw, dw);
  const int64_t Cg = C / groups, Kg = K / groups;
  float* pad = (float*)calloc((size_t)(N * C * HP * WP), sizeof(float));
  if (!pad) return -1;
  for (int64_t b = 0; b < N; ++b)
    for (int64_t c = 0; c < C; ++c)
      for (int64_t h = 0; h < HP; ++h)
        for (int64_t x = 0; x < WP; ++x)
          if (h >= ph && h < H + ph && x >= pw && x < W + pw)
            pad[((b * C + c) * HP + h) * WP + x] = in[((b * C + c) * H + (h - ph)) * W + (x - pw)];
  for (int64_t b = 0; b < N; ++b)
    for (int64_t k = 0; k < K; ++k)
      for (int64_t h = 0; h < P; ++h)
        for (int64_t x = 0; x < Q; ++x) {
          double accd = 0.0;
          float accf = 0.0f;
          for (int64_t rc = 0; rc < Cg; ++rc)
            for (int64_t rw = 0; rw < S; ++rw)
              for (int64_t rh = 0; rh < R; ++rh) {
                const float a = pad[((b * C + (k / Kg) * Cg + rc) * HP + h * sh + rh * dh) * WP + x * sw + rw * dw];
                const float ww = w[((k * Cg + rc) * R + rh) * S + rw];
                if (acc64) accd += (double)a * (double)ww;
                else accf += a * ww;
              }
          float v = acc64 ? (float)accd : accf;
          if (bias) v = acc64 ? (float)(accd + (double)bias[k]) : v + bias[k];
          out[((b * K + k) * P + h) * Q + x] = v;
        }
  free(pad);
  return 0;
}

int fto_dwconv2d_nchw_f32_naive(const float* in, const float* w, const float* bias, float* out, int64_t N,
                                int64_t C, int64_t H, int64_t W, int64_t F, int64_t R, int64_t S, int64_t sh,
                                int64_t sw, int64_t ph, int64_t pw, int64_t dh, int64_t dw, int acc64) {
  const int64_t HP = H + 2 * ph, WP = W + 2 * pw;
  const int64_t P = out_size(H, R, sh, ph, dh), Q = out_size(W, S, sw, pw, dw);
  float* pad = (float*)calloc((size_t)(N * C * HP * WP), sizeof(float));
  if (!pad) return -1;
  for (int64_t b = 0; b < N; ++b)
    for (int64_t c = 0; c < C; ++c)
      for (int64_t h = 0; h < H; ++h)
        memcpy(pad + ((b * C + c) * HP + h + ph) * WP + pw, in + ((b * C + c) * H + h) * W, (size_t)W * 4);
  const int64_t CO = C * F;
  for (int64_t b = 0; b < N; ++b)
    for (int64_t c = 0; c < CO; ++c)
      for (int64_t h = 0; h < P; ++h)
        for (int64_t x = 0; x < Q; ++x) {
          double accd = 0.0;
          float accf = 0.0f;
          for (int64_t rw = 0; rw < S; ++rw)
            for (int64_t rh = 0; rh < R; ++rh) {
              const float a = pad[((b * C + c / F) * HP + h * sh + rh * dh) * WP + x * sw + rw * dw];
              const float ww = w[(((c / F) * F + c % F) * R + rh) * S + rw];
              if (acc64) accd += (double)a * (double)ww;
              else accf += a * ww;
            }
          float v = acc64 ? (float)accd : accf;
          if (bias) v = acc64 ? (float)(accd + (double)bias[c]) : v + bias[c];
          out[((b * CO + c) * P + h) * Q + x] = v;
        }
  free(pad);
  return 0;
}

/* ------------------------------------------------------------------ part 2: llvm-template loop nests */

/* GEMM C = A[M,K] . B[K,N] (row-major).  Outer (i, j) tiles fused and parallel; per tile a
 * write-cache block acc[ti][tj]; k split in blocks of tk hoisted above the (ii, jj) tile; jj
 * vectorised.  ti <= 16, tj <= 64. */
void fto_gemm_f32_tiled(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int ti, int tj,
                        int tk) {
  const int64_t mt = (M + ti - 1) / ti, nt = (N + tj - 1) / tj;
#pragma omp parallel for schedule(static)
  for (int64_t tile = 0; tile < mt * nt; ++tile) {
    const int64_t i0 = (tile / nt) * ti, j0 = (tile % nt) * tj;
    const int il = (int)(M - i0 < ti ? M - i0 : ti), jl = (int)(N - j0 < tj ? N - j0 : tj);
    float acc[16][64];
    for (int ii = 0; ii < il; ++ii)
      for (int jj = 0; jj < jl; ++jj) acc[ii][jj] = 0.0f;
    for (int64_t k0 = 0; k0 < K; k0 += tk) {
      const int64_t k1 = k0 + tk < K ? k0 + tk : K;
      for (int64_t k = k0; k < k1; ++k)
        for (int ii = 0; ii < il; ++ii) {
          const float a = A[(i0 + ii) * K + k];
          const float* brow = B + k * N + j0;
#pragma omp simd
          for (int jj = 0; jj < jl; ++jj) acc[ii][jj] += a * brow[jj];
        }
    }
    for (int ii = 0; ii < il; ++ii)
      for (int jj = 0; jj < jl; ++jj) C[(i0 + ii) * N + j0 + jj] = acc[ii][jj];
  }
}

/* The same nest for bf16 storage with fp32 accumulation, one batch item after another. */
void fto_bgemm_bf16_tiled(const uint16_t* A, const uint16_t* B, uint16_t* C, int64_t batch, int64_t M, int64_t N,
                          int64_t K, int ti, int tj, int tk) {
  const int64_t mt = (M + ti - 1) / ti, nt = (N + tj - 1) / tj;
#pragma omp parallel for schedule(static)
  for (int64_t tile = 0; tile < batch * mt * nt; ++tile) {
    const int64_t b = tile / (mt * nt), r = tile % (mt * nt);
    const int64_t i0 = (r / nt) * ti, j0 = (r % nt) * tj;
    const uint16_t* Ab = A + b * M * K;
    const uint16_t* Bb = B + b * K * N;
    const int il = (int)(M - i0 < ti ? M - i0 : ti), jl = (int)(N - j0 < tj ? N - j0 : tj);
    float acc[16][64];
    for (int ii = 0; ii < il; ++ii)
      for (int jj = 0; jj < jl; ++jj) acc[ii][jj] = 0.0f;
    for (int64_t k0 = 0; k0 < K; k0 += tk) {
      const int64_t k1 = k0 + tk < K ? k0 + tk : K;
      for (int64_t k = k0; k < k1; ++k)
        for (int ii = 0; ii < il; ++ii) {
          const float a = bf16_to_f32(Ab[(i0 + ii) * K + k]);
          const uint16_t* brow = Bb + k * N + j0;
#pragma omp simd
          for (int jj = 0; jj < jl; ++jj) acc[ii][jj] += a * bf16_to_f32(brow[jj]);
        }
    }
    for (int ii = 0; ii < il; ++ii)
      for (int jj = 0; jj < jl; ++jj) C[(b * M + i0 + ii) * N + j0 + jj] = f32_to_bf16(acc[ii][jj]);
  }
}

void fto_gemm_s8_tiled(const int8_t* A, const int8_t* B, int32_t* C, int64_t M, int64_t N, int64_t K, int ti,
                       int tj, int tk) {
  const int64_t mt = (M + ti - 1) / ti, nt = (N + tj - 1) / tj;
#pragma omp parallel for schedule(static)
  for (int64_t tile = 0; tile < mt * nt; ++tile) {
    const int64_t i0 = (tile / nt) * ti, j0 = (tile % nt) * tj;
    const int il = (int)(M - i0 < ti ? M - i0 : ti), jl = (int)(N - j0 < tj ? N - j0 : tj);
    int32_t acc[16][64];
    for (int ii = 0; ii < il; ++ii)
      for (int jj = 0; jj < jl; ++jj) acc[ii][jj] = 0;
    for (int64_t k0 = 0; k0 < K; k0 += tk) {
      const int64_t k1 = k0 + tk < K ? k0 + tk : K;
      for (int64_t k = k0; k < k1; ++k)
        for (int ii = 0; ii < il; ++ii) {
          const int32_t a = A[(i0 + ii) * K + k];
          const int8_t* brow = B + k * N + j0;
#pragma omp simd
          for (int jj = 0; jj < jl; ++jj) acc[ii][jj] += a * (int32_t)brow[jj];
        }
    }
    for (int ii = 0; ii < il; ++ii)
      for (int jj = 0; jj < jl; ++jj) C[(i0 + ii) * N + j0 + jj] = acc[ii][jj];
  }
}

/* conv2d NCHW, groups = 1: (b, k-block, h) fused and parallel; write cache acc[tk][Q]; reduce
 * (rc, rh, rw) above the innermost spatial tile; w vectorised.  Padding read through a
 * bounds test (the pad op inlined, as `force_inline` does in the reference).  tk <= 8, Q <= 512. */
int fto_conv2d_nchw_f32_tiled(const float* in, const float* w, float* out, int64_t N, int64_t C, int64_t H,
                              int64_t W, int64_t K, int64_t R, int64_t S, int64_t sh, int64_t sw, int64_t ph,
                              int64_t pw, int64_t dh, int64_t dw, int tk) {
  const int64_t P = out_size(H, R, sh, ph, dh), Q = out_size(W, S, sw, pw, dw);
  if (Q > 512 || tk > 8 || tk < 1) return -1;
  const int64_t kt = (K + tk - 1) / tk;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < N * kt * P; ++t) {
    const int64_t b = t / (kt * P), k0 = ((t / P) % kt) * tk, h = t % P;
    const int kl = (int)(K - k0 < tk ? K - k0 : tk);
    float acc[8][512];
    for (int kk = 0; kk < kl; ++kk)
      for (int64_t x = 0; x < Q; ++x) acc[kk][x] = 0.0f;
    for (int64_t rc = 0; rc < C; ++rc)
      for (int64_t rh = 0; rh < R; ++rh) {
        const int64_t ih = h * sh + rh * dh - ph;
        if (ih < 0 || ih >= H) continue;
        const float* irow = in + ((b * C + rc) * H + ih) * W;
        for (int64_t rw = 0; rw < S; ++rw) {
          const int64_t off = rw * dw - pw;
          /* output columns whose tap lies inside the row */
          int64_t x_lo = off < 0 ? (-off + sw - 1) / sw : 0;
          int64_t x_hi = (W - 1 - off) / sw + 1;
          if (x_hi > Q) x_hi = Q;
          for (int kk = 0; kk < kl; ++kk) {
            const float ww = w[(((k0 + kk) * C + rc) * R + rh) * S + rw];
            float* arow = acc[kk];
#pragma omp simd
            for (int64_t x = x_lo; x < x_hi; ++x) arow[x] += irow[x * sw + off] * ww;
          }
        }
      }
    for (int kk = 0; kk < kl; ++kk)
      memcpy(out + ((b * K + k0 + kk) * P + h) * Q, acc[kk], (size_t)Q * 4);
  }
  return 0;
}

/* depthwise conv2d NCHW: (b, c_out, h-block) fused and parallel, w vectorised. */
int fto_dwconv2d_nchw_f32_tiled(const float* in, const float* w, float* out, int64_t N, int64_t C, int64_t H,
                                int64_t W, int64_t F, int64_t R, int64_t S, int64_t sh, int64_t sw, int64_t ph,
                                int64_t pw, int64_t dh, int64_t dw, int th) {
  const int64_t P = out_size(H, R, sh, ph, dh), Q = out_size(W, S, sw, pw, dw);
  if (Q > 512 || th < 1) return -1;
  const int64_t CO = C * F, ht = (P + th - 1) / th;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < N * CO * ht; ++t) {
    const int64_t b = t / (CO * ht), c = (t / ht) % CO, h0 = (t % ht) * th;
    const float* wk = w + c * R * S; /* [c//F][c%F] flattens to c */
    for (int64_t h = h0; h < h0 + th && h < P; ++h) {
      float acc[512];
      for (int64_t x = 0; x < Q; ++x) acc[x] = 0.0f;
      for (int64_t rh = 0; rh < R; ++rh) {
        const int64_t ih = h * sh + rh * dh - ph;
        if (ih < 0 || ih >= H) continue;
        const float* irow = in + ((b * C + c / F) * H + ih) * W;
        for (int64_t rw = 0; rw < S; ++rw) {
          const int64_t off = rw * dw - pw;
          int64_t x_lo = off < 0 ? (-off + sw - 1) / sw : 0;
          int64_t x_hi = (W - 1 - off) / sw + 1;
          if (x_hi > Q) x_hi = Q;
          const float ww = wk[rh * S + rw];
#pragma omp simd
          for (int64_t x = x_lo; x < x_hi; ++x) acc[x] += irow[x * sw + off] * ww;
        }
      }
      memcpy(out + ((b * CO + c) * P + h) * Q, acc, (size_t)Q * 4);
    }
  }
  return 0;
}
