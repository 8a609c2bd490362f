/*
 * apnn_oracle.c -- CPU restatement of APNN-TC's host-side verification loops.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the
 * test-suite, the smoke entry and the benchmark's cpu_baseline / reference arm
 * may load it; the product library never does and has no CPU fallback.
 *
 * Paths cited below are relative to the APNN-TC project root;
 * LIB = APNN-TC-lib/bmmaTensorCoreGemm/src.
 *
 * Parity status
 *   pinned   : rand stream, fill order, GEMM/conv accumulators, low-bit pack,
 *              2x2 average pool + pack, Bit_compression plane layout.  These are
 *              compared in the test-suite against the reference's own host
 *              functions compiled unmodified into oracle/_ref/ and against
 *              fixtures generated from them.
 *   unpinned : signed (+-1) weight correction, threshold requantisation, max
 *              pooling, batch dimension, stride, 1x1 filters, w1a3 GEMM.  The
 *              reference has no host loop for these; they are defined here as
 *              integer functions of the pinned accumulator.
 *
 * Layouts (all words are uint32, K or C fastest, planes outermost)
 *   GEMM : W[wb][M][K/32], X[xb][N][K/32], D[M][N] int32
 *   conv : X[xb][B][H+2p][W+2p][CIN/32], Wt[wb][COUT][R][R][CIN/32],
 *          Out[B][Ho][Wo][COUT] int32, packed Out[ob][B][Ho][Wo][COUT/32]
 *   packed words hold 32 consecutive channels, lowest channel in bit 31.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------- */
/* glibc rand(), default seed.  The reference fills every operand with rand()
 * and never calls srand (LIB/71_bmmaTensorCoreGemm.cu:313,323), so its inputs
 * are the default-seed stream of glibc's additive-feedback generator
 * (degree 31, separation 3, seeded through the Lehmer minimal standard
 * generator; first output 0x6b8b4567).  Restated here so the stream does not
 * depend on process-wide libc state. */
typedef struct {
  uint32_t r[34];
  int pos; /* index of the oldest element (i-34) in the ring */
} apnn_rand_t;

void apnn_oracle_srand(apnn_rand_t *s, uint32_t seed) {
  int32_t init[34];
  if (seed == 0) seed = 1;
  init[0] = (int32_t)seed;
  for (int i = 1; i < 31; i++) {
    int32_t hi = init[i - 1] / 127773, lo = init[i - 1] % 127773;
    int32_t w = 16807 * lo - 2836 * hi;
    if (w < 0) w += 2147483647;
    init[i] = w;
  }
  for (int i = 31; i < 34; i++) init[i] = init[i - 31];
  for (int i = 0; i < 34; i++) s->r[i] = (uint32_t)init[i];
  s->pos = 0;
  /* discard the first 310 values */
  for (int i = 34; i < 344; i++) {
    uint32_t v = s->r[(s->pos + 3) % 34] + s->r[(s->pos + 31) % 34];
    s->r[s->pos] = v;
    s->pos = (s->pos + 1) % 34;
  }
}

uint32_t apnn_oracle_rand(apnn_rand_t *s) {
  /* ring holds values i-34 .. i-1 starting at pos; new = r[i-31] + r[i-3] */
  uint32_t v = s->r[(s->pos + 3) % 34] + s->r[(s->pos + 31) % 34];
  s->r[s->pos] = v;
  s->pos = (s->pos + 1) % 34;
  return v >> 1;
}

void apnn_oracle_rand_words(uint32_t seed, uint32_t *out, long n) {
  apnn_rand_t s;
  apnn_oracle_srand(&s, seed);
  for (long i = 0; i < n; i++) out[i] = apnn_oracle_rand(&s);
}

/* init_matrices of the GEMM programs: W planes first, then X planes, one
 * rand() per 32-bit word (LIB/71_bmmaTensorCoreGemm.cu:305-327). */
void apnn_oracle_fill_gemm(uint32_t *W, uint32_t *X, int M, int N, int K,
                           int wbits, int xbits, uint32_t seed) {
  apnn_rand_t s;
  apnn_oracle_srand(&s, seed);
  long kw = K / 32;
  for (int b = 0; b < wbits; b++)
    for (int i = 0; i < M; i++)
      for (long j = 0; j < kw; j++) W[((long)b * M + i) * kw + j] = apnn_oracle_rand(&s);
  for (int b = 0; b < xbits; b++)
    for (int i = 0; i < N; i++)
      for (long j = 0; j < kw; j++) X[((long)b * N + i) * kw + j] = apnn_oracle_rand(&s);
}

/* init_matrices of the conv programs: X first, halo ring included, then the
 * filter (LIB/67_bmmaTensorCoreGemm.cu:324-350).  One image, 3x3. */
void apnn_oracle_fill_conv(uint32_t *X, uint32_t *Wt, int H, int Wd, int CIN,
                           int COUT, int xbits, int wbits, uint32_t seed) {
  apnn_rand_t s;
  apnn_oracle_srand(&s, seed);
  long cw = CIN / 32;
  long nx = (long)(H + 2) * (Wd + 2) * cw;
  for (int b = 0; b < xbits; b++)
    for (long i = 0; i < nx; i++) X[b * nx + i] = apnn_oracle_rand(&s);
  long nw = (long)COUT * 9 * cw;
  for (int b = 0; b < wbits; b++)
    for (long i = 0; i < nw; i++) Wt[b * nw + i] = apnn_oracle_rand(&s);
}

/* ------------------------------------------------------------------------- */
/* GEMM accumulators.  compute_ref, bit by bit as the reference writes it
 * (LIB/71_bmmaTensorCoreGemm.cu:350-376): for every plane pair and every bit
 * of every word, tmp += 2^xb * 2^wb * x_bit * w_bit.  Rows [m0, m1) only, so a
 * caller can time a bounded sample or split rows over threads. */
void apnn_oracle_gemm_bitserial_rows(const uint32_t *W, const uint32_t *X, int32_t *D,
                                     int M, int N, int K, int wbits, int xbits,
                                     int m0, int m1) {
  long kw = K / 32;
  for (int m = m0; m < m1; m++) {
    for (int n = 0; n < N; n++) {
      int32_t tmp = 0;
      for (int xb = 0; xb < xbits; xb++) {
        int xmul = 1 << xb;
        for (int wb = 0; wb < wbits; wb++) {
          int wmul = 1 << wb;
          for (long kt = 0; kt < kw; kt++) {
            uint32_t w = W[((long)wb * M + m) * kw + kt];
            uint32_t x = X[((long)xb * N + n) * kw + kt];
            for (int k = 0; k < 32; k++) {
              int xv = (int)((x >> k) & 1u);
              int wv = (int)((w >> k) & 1u);
              tmp += xmul * wmul * xv * wv;
            }
          }
        }
      }
      D[(long)m * N + n] = tmp;
    }
  }
}

void apnn_oracle_gemm_bitserial(const uint32_t *W, const uint32_t *X, int32_t *D,
                                int M, int N, int K, int wbits, int xbits) {
  apnn_oracle_gemm_bitserial_rows(W, X, D, M, N, K, wbits, xbits, 0, M);
}

/* The same quantity with one popcount per word pair.  Used for shapes the
 * bit-serial loop cannot finish; the test-suite proves the two equal on every
 * small shape first.  Callers thread it by giving each thread a row range. */
void apnn_oracle_gemm_popc_rows(const uint32_t *W, const uint32_t *X, int32_t *D,
                                int M, int N, int K, int wbits, int xbits,
                                int m0, int m1) {
  long kw = K / 32;
  for (int m = m0; m < m1; m++) {
    for (int n = 0; n < N; n++) {
      int32_t tmp = 0;
      for (int xb = 0; xb < xbits; xb++)
        for (int wb = 0; wb < wbits; wb++) {
          const uint32_t *wr = W + ((long)wb * M + m) * kw;
          const uint32_t *xr = X + ((long)xb * N + n) * kw;
          int32_t c = 0;
          for (long kt = 0; kt < kw; kt++) c += __builtin_popcount(wr[kt] & xr[kt]);
          tmp += c << (xb + wb);
        }
      D[(long)m * N + n] = tmp;
    }
  }
}

void apnn_oracle_gemm_popc(const uint32_t *W, const uint32_t *X, int32_t *D,
                           int M, int N, int K, int wbits, int xbits) {
  apnn_oracle_gemm_popc_rows(W, X, D, M, N, K, wbits, xbits, 0, M);
}

/* Row sums S[r] = sum_b 2^b popcount(P[b][r][:]) -- the term the +-1 weight
 * reading needs: sum_k (2w-1) x = 2 acc - S_x.  Unpinned (project-defined). */
void apnn_oracle_row_sums(const uint32_t *P, int32_t *S, int rows, int K, int bits) {
  long kw = K / 32;
  for (int r = 0; r < rows; r++) {
    int32_t t = 0;
    for (int b = 0; b < bits; b++) {
      int32_t c = 0;
      for (long kt = 0; kt < kw; kt++) c += __builtin_popcount(P[((long)b * rows + r) * kw + kt]);
      t += c << b;
    }
    S[r] = t;
  }
}

/* ------------------------------------------------------------------------- */
/* Convolution accumulators.  compute_ref of the conv programs
 * (LIB/67_bmmaTensorCoreGemm.cu:375-410) is the case B=1, R=3, stride=1 of
 * this loop: a valid correlation over an input that already carries its halo,
 * K ordered (i, j, c).  Batch, stride and R=1 are project extensions
 * (unpinned); each image carries its own halo of p=(R-1)/2 pixels and output
 * (ho, wo) reads the window whose top-left haloed coordinate is
 * (ho*stride, wo*stride), i.e. symmetric padding p. */
void apnn_oracle_conv_bitserial(const uint32_t *Wt, const uint32_t *X, int32_t *Out,
                                int B, int H, int Wd, int CIN, int COUT, int R,
                                int stride, int wbits, int xbits) {
  int p = (R - 1) / 2;
  int Hp = H + 2 * p, Wp = Wd + 2 * p;
  int Ho = (H - 1) / stride + 1, Wo = (Wd - 1) / stride + 1;
  long cw = CIN / 32;
  long xplane = (long)B * Hp * Wp * cw;
  long wplane = (long)COUT * R * R * cw;
  for (int co = 0; co < COUT; co++)
    for (int b = 0; b < B; b++)
      for (int m = 0; m < Ho; m++)
        for (int n = 0; n < Wo; n++) {
          int32_t tmp = 0;
          for (int xb = 0; xb < xbits; xb++) {
            int xmul = 1 << xb;
            for (int wb = 0; wb < wbits; wb++) {
              int wmul = 1 << wb;
              for (int i = 0; i < R; i++)
                for (int j = 0; j < R; j++)
                  for (long kt = 0; kt < cw; kt++) {
                    uint32_t x = X[xb * xplane +
                                   (((long)b * Hp + (m * stride + i)) * Wp + (n * stride + j)) * cw + kt];
                    uint32_t w = Wt[wb * wplane + (((long)co * R + i) * R + j) * cw + kt];
                    for (int k = 0; k < 32; k++) {
                      int xv = (int)((x >> k) & 1u);
                      int wv = (int)((w >> k) & 1u);
                      tmp += xmul * wmul * xv * wv;
                    }
                  }
            }
          }
          Out[(((long)b * Ho + m) * Wo + n) * COUT + co] = tmp;
        }
}

/* Word-popcount form of the same loop, output channels [co0, co1) only so
 * callers can thread it. */
void apnn_oracle_conv_popc_range(const uint32_t *Wt, const uint32_t *X, int32_t *Out,
                                 int B, int H, int Wd, int CIN, int COUT, int R,
                                 int stride, int wbits, int xbits, int co0, int co1) {
  int p = (R - 1) / 2;
  int Hp = H + 2 * p, Wp = Wd + 2 * p;
  int Ho = (H - 1) / stride + 1, Wo = (Wd - 1) / stride + 1;
  long cw = CIN / 32;
  long xplane = (long)B * Hp * Wp * cw;
  long wplane = (long)COUT * R * R * cw;
  for (int co = co0; co < co1; co++)
    for (int b = 0; b < B; b++)
      for (int m = 0; m < Ho; m++)
        for (int n = 0; n < Wo; n++) {
          int32_t tmp = 0;
          for (int xb = 0; xb < xbits; xb++)
            for (int wb = 0; wb < wbits; wb++) {
              int32_t c = 0;
              for (int i = 0; i < R; i++)
                for (int j = 0; j < R; j++) {
                  const uint32_t *xr = X + xb * xplane +
                      (((long)b * Hp + (m * stride + i)) * Wp + (n * stride + j)) * cw;
                  const uint32_t *wr = Wt + wb * wplane + (((long)co * R + i) * R + j) * cw;
                  for (long kt = 0; kt < cw; kt++) c += __builtin_popcount(xr[kt] & wr[kt]);
                }
              tmp += c << (xb + wb);
            }
          Out[(((long)b * Ho + m) * Wo + n) * COUT + co] = tmp;
        }
}

/* Window sums of the activations, S[b][ho][wo] = sum over the RxRxCIN window of
 * the activation value; halo pixels are part of the stored tensor (zeros when
 * the caller padded with zeros).  Unpinned. */
void apnn_oracle_conv_window_sums(const uint32_t *X, int32_t *S, int B, int H, int Wd,
                                  int CIN, int R, int stride, int xbits) {
  int p = (R - 1) / 2;
  int Hp = H + 2 * p, Wp = Wd + 2 * p;
  int Ho = (H - 1) / stride + 1, Wo = (Wd - 1) / stride + 1;
  long cw = CIN / 32;
  long xplane = (long)B * Hp * Wp * cw;
  for (int b = 0; b < B; b++)
    for (int m = 0; m < Ho; m++)
      for (int n = 0; n < Wo; n++) {
        int32_t t = 0;
        for (int xb = 0; xb < xbits; xb++) {
          int32_t c = 0;
          for (int i = 0; i < R; i++)
            for (int j = 0; j < R; j++) {
              const uint32_t *xr = X + xb * xplane +
                  (((long)b * Hp + (m * stride + i)) * Wp + (n * stride + j)) * cw;
              for (long kt = 0; kt < cw; kt++) c += __builtin_popcount(xr[kt]);
            }
          t += c << xb;
        }
        S[((long)b * Ho + m) * Wo + n] = t;
      }
}

/* ------------------------------------------------------------------------- */
/* Epilogue pieces.  All operate on a [rows][C] int32 matrix. */

/* v = 2*acc - S[row] (sign_axis 0) or 2*acc - S[col] (sign_axis 1).  Unpinned. */
void apnn_oracle_signed_correct(int32_t *V, const int32_t *S, long rows, int C, int sign_axis) {
  for (long r = 0; r < rows; r++)
    for (int c = 0; c < C; c++)
      V[r * C + c] = 2 * V[r * C + c] - (sign_axis == 0 ? S[r] : S[c]);
}

/* 2x2 pooling over [B][H][W][C].  mode 1: (a+b+c+d)/4 with C's truncating
 * division, exactly as compute_ref_pack_pool writes it
 * (LIB/68_bmmaTensorCoreGemm.cu:522-535).  mode 2: maximum (unpinned). */
void apnn_oracle_pool2x2(const int32_t *In, int32_t *Out, int B, int H, int Wd, int C, int mode) {
  int Hh = H / 2, Wh = Wd / 2;
  for (int b = 0; b < B; b++)
    for (int m = 0; m < Hh; m++)
      for (int n = 0; n < Wh; n++)
        for (int c = 0; c < C; c++) {
          int32_t v1 = In[(((long)b * H + 2 * m) * Wd + 2 * n) * C + c];
          int32_t v2 = In[(((long)b * H + 2 * m) * Wd + 2 * n + 1) * C + c];
          int32_t v3 = In[(((long)b * H + 2 * m + 1) * Wd + 2 * n) * C + c];
          int32_t v4 = In[(((long)b * H + 2 * m + 1) * Wd + 2 * n + 1) * C + c];
          int32_t o;
          if (mode == 1) {
            o = (v1 + v2 + v3 + v4) / 4;
          } else {
            o = v1;
            if (v2 > o) o = v2;
            if (v3 > o) o = v3;
            if (v4 > o) o = v4;
          }
          Out[(((long)b * Hh + m) * Wh + n) * C + c] = o;
        }
}

/* Level of one value.  mode 1: the low out_bits bits of v -- what every fused
 * reference kernel and compute_ref_pack do (LIB/66_bmmaTensorCoreGemm.cuh:390-407,
 * LIB/67_bmmaTensorCoreGemm.cu:456-477).  mode 2: number of per-channel
 * thresholds T[c][0..2^ob-2] (ascending) that v reaches (unpinned). */
static inline uint32_t level_of(int32_t v, int c, int out_bits, int mode, const int32_t *T) {
  if (mode == 1) return (uint32_t)v & ((1u << out_bits) - 1u);
  int nl = (1 << out_bits) - 1;
  uint32_t l = 0;
  for (int j = 0; j < nl; j++) l += (v >= T[(long)c * nl + j]) ? 1u : 0u;
  return l;
}

void apnn_oracle_levels(const int32_t *V, int32_t *L, long rows, int C, int out_bits,
                        int mode, const int32_t *T) {
  for (long r = 0; r < rows; r++)
    for (int c = 0; c < C; c++) L[r * C + c] = (int32_t)level_of(V[r * C + c], c, out_bits, mode, T);
}

/* Plane split + pack along the channel axis: Out[ob][rows][C/32], the first of
 * every 32 channels lands in bit 31 (the shift-left-then-or loop of
 * LIB/66_bmmaTensorCoreGemm.cuh:393-402; the kernels get the same word with
 * __brev(__ballot_sync)). */
void apnn_oracle_requant_pack(const int32_t *V, uint32_t *Out, long rows, int C,
                              int out_bits, int mode, const int32_t *T) {
  long cw = C / 32;
  for (long r = 0; r < rows; r++)
    for (long ct = 0; ct < cw; ct++) {
      uint32_t val[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int c = 0; c < 32; c++) {
        int ch = (int)(ct * 32 + c);
        uint32_t l = level_of(V[r * C + ch], ch, out_bits, mode, T);
        for (int b = 0; b < out_bits; b++) val[b] = (val[b] << 1) | ((l >> b) & 1u);
      }
      for (int b = 0; b < out_bits; b++) Out[((long)b * rows + r) * cw + ct] = val[b];
    }
}

/* compute_ref_pack for the GEMM (LIB/66_bmmaTensorCoreGemm.cuh:356-408) and the
 * conv (LIB/67_bmmaTensorCoreGemm.cu:412-478), and compute_ref_pack_pool
 * (LIB/68_bmmaTensorCoreGemm.cu:484-565), composed from the pieces above with
 * heap storage for the int32 intermediate (the reference keeps it on the
 * stack). */
void apnn_oracle_gemm_pack(const uint32_t *W, const uint32_t *X, uint32_t *Out, int M, int N,
                           int K, int wbits, int xbits, int out_bits) {
  int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)M * N);
  apnn_oracle_gemm_bitserial(W, X, acc, M, N, K, wbits, xbits);
  apnn_oracle_requant_pack(acc, Out, M, N, out_bits, 1, 0);
  free(acc);
}

void apnn_oracle_conv_pack(const uint32_t *Wt, const uint32_t *X, uint32_t *Out, int H, int Wd,
                           int CIN, int COUT, int wbits, int xbits, int out_bits, int pool) {
  int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)H * Wd * COUT);
  apnn_oracle_conv_bitserial(Wt, X, acc, 1, H, Wd, CIN, COUT, 3, 1, wbits, xbits);
  if (pool) {
    int32_t *pl = (int32_t *)malloc(sizeof(int32_t) * (size_t)(H / 2) * (Wd / 2) * COUT);
    apnn_oracle_pool2x2(acc, pl, 1, H, Wd, COUT, 1);
    apnn_oracle_requant_pack(pl, Out, (long)(H / 2) * (Wd / 2), COUT, out_bits, 1, 0);
    free(pl);
  } else {
    apnn_oracle_requant_pack(acc, Out, (long)H * Wd, COUT, out_bits, 1, 0);
  }
  free(acc);
}

/* ------------------------------------------------------------------------- */
/* Packers of the network layer (APNN-TC-nn/src/kernel.cuh). */

/* Quantize_val (APNN-TC-nn/src/kernel.cuh:29-44): clip to [-10, 10], map
 * affinely onto 2^bits steps, round to nearest even (the commented
 * __float2uint_rn store).  The top of the range would give 2^bits; it is
 * clamped to the largest level so the result fits `bits` bits (project
 * choice; the reference never stores the value). */
void apnn_oracle_quantize(const float *in, uint32_t *lv, long n, int bits) {
  for (long i = 0; i < n; i++) {
    float x = in[i];
    if (x < -10.0f) x = -10.0f;
    if (x > 10.0f) x = 10.0f;
    float q = (x - (-10.0f)) * (float)(1 << bits) * 1.0f / (float)(10 - (-10));
    /* round half to even, as cvt.rni does */
    float f = __builtin_floorf(q);
    float d = q - f;
    uint32_t u = (uint32_t)f;
    if (d > 0.5f || (d == 0.5f && (u & 1u))) u += 1;
    if (u > (1u << bits) - 1u) u = (1u << bits) - 1u;
    lv[i] = u;
  }
}

/* Bit_compression (APNN-TC-nn/src/kernel.cuh:46-77): levels[rows][C] (one
 * uint32 per element) -> planes[b][rows][PAD128(C)/32], channel c of a row in
 * bit 31-(c%32) of word c/32.  Channels beyond C are zero here (the reference
 * leaves those words unwritten). */
void apnn_oracle_bit_compress(const uint32_t *lv, uint32_t *planes, long rows, int C, int bits) {
  long cw = ((C + 127) / 128) * 4;
  memset(planes, 0, sizeof(uint32_t) * (size_t)bits * rows * cw);
  for (int b = 0; b < bits; b++)
    for (long r = 0; r < rows; r++)
      for (int c = 0; c < C; c++)
        if ((lv[r * C + c] >> b) & 1u) planes[((long)b * rows + r) * cw + c / 32] |= 1u << (31 - (c % 32));
}

/* Inverse of the plane layout, for tests: planes -> integer levels. */
void apnn_oracle_bit_expand(const uint32_t *planes, int32_t *lv, long rows, int Cpad, int bits) {
  long cw = Cpad / 32;
  for (long r = 0; r < rows; r++)
    for (int c = 0; c < Cpad; c++) {
      int32_t v = 0;
      for (int b = 0; b < bits; b++)
        v |= (int32_t)((planes[((long)b * rows + r) * cw + c / 32] >> (31 - (c % 32))) & 1u) << b;
      lv[r * Cpad + c] = v;
    }
}

/* Batch-norm + clip/round quantiser folded to integer thresholds (unpinned).
 * y = scale[c]*(v-mu)/sigma + bias[c]; the quantiser above maps y to level
 * >= j exactly when y >= (j-0.5)*20/2^bits - 10, so with scale > 0
 * T[c][j-1] = ceil(mu + sigma*((j-0.5)*20/2^bits - 10 - bias[c])/scale[c]).
 * Computed in double; the table, not this formula, is what the kernels and
 * apnn_oracle_requant_pack share. */
void apnn_oracle_fold_bn(const float *scale, const float *bias, double mu, double sigma,
                         int C, int out_bits, int32_t *T) {
  int nl = (1 << out_bits) - 1;
  for (int c = 0; c < C; c++)
    for (int j = 1; j <= nl; j++) {
      double edge = (j - 0.5) * 20.0 / (double)(1 << out_bits) - 10.0;
      double t = mu + sigma * (edge - (double)bias[c]) / (double)scale[c];
      double ct = __builtin_ceil(t);
      if (ct > 2147483647.0) ct = 2147483647.0;
      if (ct < -2147483648.0) ct = -2147483648.0;
      T[(long)c * nl + (j - 1)] = (int32_t)ct;
    }
}

/* First-layer re-layout (project-defined, unpinned): Quantize_val on every element, then each
 * output pixel's RxRxC window laid along the channel axis, k = (i*R + j)*C + c, zeros outside
 * the image and up to PAD128(R*R*C).  planes[bits][B][Ho][Wo][Kp/32], element k in bit 31-k%32. */
void apnn_oracle_quantize_im2col(const float *img, uint32_t *planes, int B, int H, int Wd, int C,
                                 int R, int stride, int bits) {
  int pad = (R - 1) / 2;
  int Ho = (H - 1) / stride + 1, Wo = (Wd - 1) / stride + 1;
  long kw = ((long)R * R * C + 127) / 128 * 4;
  long pixels = (long)B * Ho * Wo;
  memset(planes, 0, sizeof(uint32_t) * (size_t)bits * pixels * kw);
  for (int b = 0; b < B; b++)
    for (int ho = 0; ho < Ho; ho++)
      for (int wo = 0; wo < Wo; wo++) {
        long pix = ((long)b * Ho + ho) * Wo + wo;
        for (int i = 0; i < R; i++)
          for (int j = 0; j < R; j++) {
            int hi = ho * stride + i - pad, wi = wo * stride + j - pad;
            if (hi < 0 || hi >= H || wi < 0 || wi >= Wd) continue;
            for (int c = 0; c < C; c++) {
              uint32_t lv;
              apnn_oracle_quantize(img + (((long)b * H + hi) * Wd + wi) * C + c, &lv, 1, bits);
              long k = ((long)i * R + j) * C + c;
              for (int p = 0; p < bits; p++)
                if ((lv >> p) & 1u) planes[((long)p * pixels + pix) * kw + k / 32] |= 1u << (31 - (k % 32));
            }
          }
      }
}
