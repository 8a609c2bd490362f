/*
 * apnn_b200.h -- C ABI of the B200 (sm_100a) arbitrary-precision GEMM / convolution
 * library.  Plain pointers and sizes only; every device pointer is memory the
 * caller allocated (cudaMalloc or equivalent) and still owns, as in the reference,
 * where kernels allocate nothing.  Every entry point returns a status code and
 * never aborts.  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *
 * Reference interfaces cited below are paths inside the APNN-TC project;
 * LIB = APNN-TC-lib/bmmaTensorCoreGemm/src, NN = APNN-TC-nn/src.
 *
 * Tensor layouts (identical to the reference, uint32 words, planes outermost,
 * K / channel fastest, 16-byte aligned):
 *   GEMM  W[wbits][M][K/32]   X[xbits][N][K/32]   D[M][N] int32
 *         D = sum_wb sum_xb 2^(wb+xb) popcount(W[wb][m] & X[xb][n])
 *         packed D[out_bits][M][N/32], column n in bit 31-(n%32)
 *   conv  X[xbits][B][H+2p][W+2p][CIN/32] (halo of p=(R-1)/2 pixels stored with
 *         every image), Wt[wbits][COUT][R][R][CIN/32],
 *         Out[B][Ho][Wo][COUT] int32 or packed Out[out_bits][B][Ho][Wo][COUT/32]
 */
#ifndef APNN_B200_H
#define APNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum apnn_status {
  APNN_OK = 0,
  APNN_ERR_INVALID_ARG = 1, /* null pointer, non-positive size, bad enum */
  APNN_ERR_UNSUPPORTED = 2, /* bit-width pair or shape rule not supported */
  APNN_ERR_ALIGNMENT = 3,   /* pointer not 16-byte aligned / K not a multiple of 128 */
  APNN_ERR_WORKSPACE = 4,   /* workspace missing or too small for the chosen algorithm */
  APNN_ERR_CUDA = 5,        /* a CUDA call failed; see apnn_last_cuda_error() */
  APNN_ERR_NO_DEVICE = 6,   /* no sm_100 device available */
  APNN_ERR_TIMEOUT = 7      /* a bounded device-side wait expired; the output is incomplete */
} apnn_status;

/* What the fused epilogue writes. */
enum {
  APNN_OUT_INT32 = 0,     /* int32 value per output element */
  APNN_OUT_LOWBITS = 1,   /* low out_bits bits of the value, plane-split and packed (the
                             reference's fused kernels) */
  APNN_OUT_THRESHOLDS = 2, /* level = number of per-channel int32 thresholds the value reaches
                              (batch-norm + quantiser folded on the host), packed */
  APNN_OUT_FLOAT = 3      /* float per output element: float(value) * affine_scale[c] + affine_bias[c], the
                             multiply and the add rounded separately (no fused multiply-add) -- the output
                             layer's batch-norm affine, Out128Layer of NN/kernel.cuh:397-447, whose
                             (K - 2*popc) is the +-1 dot product `value`.  apnn_gemm_i8, apnn_conv2d_i8 and
                             apnn_requantize_i32 only */
};
/* Which operand's bits mean -1/+1 instead of 0/1 (that operand must be 1-bit). */
enum { APNN_SIGN_NONE = 0, APNN_SIGN_W = 1, APNN_SIGN_X = 2 };
/* 2x2 pooling applied to the int32 value before requantisation (conv only). */
enum { APNN_POOL_NONE = 0, APNN_POOL_AVG2 = 1, APNN_POOL_MAX2 = 2 };
/* Contraction path. */
enum {
  APNN_ALGO_AUTO = 0,    /* TCGEN05 when a large enough workspace is given and the problem is
                            big enough to fill the device, else IMMA */
  APNN_ALGO_BMMA = 1,    /* 1-bit and-popcount mma.sync per plane pair (emulated on sm_100a;
                            kept as the measured comparison), no workspace */
  APNN_ALGO_IMMA = 2,    /* planes spread to u8 in registers, mma.sync m16n8k32, no workspace */
  APNN_ALGO_TCGEN05 = 3, /* planes expanded to int8 in the workspace, TMA-fed tcgen05 kind::i8
                            with TMEM accumulators */
  APNN_ALGO_TCGEN05_PAIR = 4 /* GEMM only: the same on CTA pairs (cta_group::2, 256x256 tiles,
                                each SM stages half of both operands); same workspace */
};

typedef struct apnn_epilogue {
  uint32_t struct_size;      /* sizeof(apnn_epilogue), as APNN_EPILOGUE_INIT sets it: a caller compiled against
                                another layout of this structure is refused with APNN_ERR_INVALID_ARG instead of
                                being misread */
  int32_t out_mode;          /* APNN_OUT_* */
  int32_t out_bits;          /* 1..8 for the packed modes */
  int32_t signed_operand;    /* APNN_SIGN_*: value = 2*acc - (sum of the other operand's row) */
  int32_t pool;              /* APNN_POOL_* (conv only; H and W even) */
  int32_t out_halo;          /* conv only: write the output inside a zeroed ring of this many
                                pixels, so it can feed the next conv directly */
  int32_t in_halo;           /* conv only: the stored input carries a ring of in_halo pixels;
                                0 means exactly (R-1)/2.  Lets a 1x1 shortcut read a tensor
                                that was written with the ring a 3x3 consumer needs. */
  const int32_t *thresholds; /* device, [channels][2^out_bits - 1] ascending; channel = n
                                (GEMM) or output channel (conv) */
  const int32_t *residual_in; /* optional, device, dense int32 [rows][channels] (rows = M, or
                                 B*Ho*Wo after pooling, no ring): added to the value before
                                 requantisation -- the residual injection of a ResNet block
                                 (semantics of NN/kernel.cuh:779-831) */
  int32_t *residual_out;      /* optional, same shape: receives the int32 value (after the
                                 residual add) next to the requantised output, i.e. the
                                 "save_residual" output of NN/param.h:943-945 */
  int32_t n_peer_out;         /* GEMM on the tcgen05 CTA-pair kernel only: number of extra
                                 destinations in peer_out (0..7) */
  int32_t out_i8;             /* apnn_conv2d_i8 / apnn_gemm_i8 only, with a quantising out_mode: 1 =
                                 write one byte per output element (the level), rows of `channels`
                                 bytes in the byte order of apnn_expand_planes and the same ring
                                 as the packed output, instead of packed planes -- the next
                                 layer's int8 operand without an expand pass.  No reference
                                 counterpart. */
  void *peer_out[7];          /* every output tile is also stored, in D's layout, to these
                                 addresses -- peer-mapped memory of other GPUs (NVLink): with D and
                                 peer_out[] pointing at this rank's slot of a [ranks][M][N/ranks]
                                 buffer on every GPU, the N-sharded GEMM leaves the gathered
                                 result everywhere without a separate all-gather.  The caller
                                 synchronises the ranks before reading.  No reference counterpart
                                 (the reference is single-GPU). */
  int32_t residual_i16;       /* apnn_conv2d_i8 / apnn_gemm_i8 only: bit 0 = residual_in holds int16,
                                 bit 1 = residual_out holds int16, instead of int32 (half the traffic
                                 of the residual tensors, which bound the second convolution of a
                                 ResNet block).  The caller guarantees the values fit (|value| <=
                                 (2^xbits - 1) * K plus the bound of the added residual); stores
                                 saturate.  No reference counterpart. */
  const float *affine_scale;  /* APNN_OUT_FLOAT: device, [channels] */
  const float *affine_bias;   /* APNN_OUT_FLOAT: device, [channels] */
} apnn_epilogue;
/* Initialiser that zeroes every field and records the structure's size: apnn_epilogue e = APNN_EPILOGUE_INIT; */
#define APNN_EPILOGUE_INIT {(uint32_t)sizeof(apnn_epilogue)}

const char *apnn_status_string(apnn_status s);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char *apnn_last_cuda_error(void);
int apnn_version(void);

/* ---- GEMM ----------------------------------------------------------------------
 * apnn_gemm replaces the int32-output kernels
 *   apmm_w1a2 (LIB/71_bmmaTensorCoreGemm.cu:80), apmm_w2a2 (LIB/72_...cu:80),
 *   apmm_w1a4 (LIB/78_...cu:80) and the w1a3 binary the README runs,
 * launched there as <<<SMs, 256, 65536>>>(W, X, D, M, N, K, wb, xb).
 * Supported (wbits, xbits): (1,2) (1,3) (1,4) (2,2) and their transposes.
 * Rules: K % 128 == 0; W, X, D 16-byte aligned; M, N >= 1 (ragged edges handled). */
apnn_status apnn_gemm(void *stream, int wbits, int xbits, const void *W, const void *X,
                      int32_t *D, int M, int N, int K);

/* apnn_gemm_ex adds the fused epilogue and the algorithm / workspace choice; with
 * APNN_OUT_LOWBITS it replaces apmm_w1a2_decompose (LIB/66_bmmaTensorCoreGemm.cuh:81-280)
 * and apmm_w2a2_decompose (LIB/73_bmmaTensorCoreGemm.cuh:81-297), which FC_new_global /
 * Output_new_global call (NN/kernel.cuh:299-318).  Packed modes need N % 32 == 0.
 * epi == NULL means int32 output.  workspace may be NULL for every algorithm but APNN_ALGO_TCGEN05.
 * With a workspace (APNN_ALGO_TCGEN05, or AUTO) every pair of widths from {1, 2, 3, 4, 8} runs --
 * the reference's w4a4 / w1a8 / w2a8 programs (LIB/83, 77, 76_bmmaTensorCoreGemm.cu) included:
 * on the int8 path a level of up to 8 bits is one byte whatever its width.  apnn_conv2d_ex
 * follows the same rule. */
apnn_status apnn_gemm_ex(void *stream, int algo, int wbits, int xbits, const void *W,
                         const void *X, void *D, int M, int N, int K,
                         const apnn_epilogue *epi, void *workspace, size_t workspace_bytes);

/* Bytes of device workspace `algo` needs for this problem (0 unless APNN_ALGO_TCGEN05). */
size_t apnn_gemm_workspace_bytes(int algo, int wbits, int xbits, int M, int N, int K);

/* The tcgen05 kernel bounds every barrier wait (2 s) and raises a flag in the workspace
 * instead of hanging.  This call synchronises `stream` and returns APNN_ERR_TIMEOUT if the
 * last APNN_ALGO_TCGEN05 GEMM that used this workspace with these sizes gave up, APNN_OK
 * otherwise.  No counterpart in the reference (its kernels have no waits). */
apnn_status apnn_gemm_check(void *stream, const void *workspace, int M, int N, int K);

/* The two stages of APNN_ALGO_TCGEN05 as entry points of their own, so that a static
 * operand (the weights of a layer) is expanded once and reused.  No counterpart in the
 * reference, whose kernels read the planes directly.
 * apnn_expand_planes: planes[bits][rows][K/32] -> out_i8[rows][K] (32-byte aligned, as is any
 *   workspace), one byte per element,
 *   value = sum_p bit_p << p, or -1/+1 for a 1-bit operand with is_signed != 0.  The byte
 *   order inside each group of 32 k is a fixed permutation shared by both operands.
 * apnn_gemm_i8: D = W8 * X8^T over operands produced by apnn_expand_planes, same epilogue;
 *   problems with at least as many 256x256 tiles as SM pairs run on CTA pairs (cta_group::2)
 *   (signed_operand must be APNN_SIGN_NONE: the sign is in the bytes; pass w_signed /
 *   x_signed to say which operand holds -1/+1).  status_flag: 4 bytes of device memory,
 *   written 0 at launch and non-zero if a bounded wait expires. */
apnn_status apnn_expand_planes(void *stream, const void *planes, void *out_i8, long rows, int K,
                               int bits, int is_signed);
/* Both operands of a GEMM in one launch (what apnn_gemm_ex does internally). */
apnn_status apnn_expand_planes_pair(void *stream, const void *planes_w, void *w_i8, long rows_w,
                                    int wbits, int w_signed, const void *planes_x, void *x_i8,
                                    long rows_x, int xbits, int x_signed, int K);
apnn_status apnn_gemm_i8(void *stream, const void *W8, const void *X8, void *D, int M, int N, int K,
                         int w_signed, int x_signed, const apnn_epilogue *epi, int *status_flag);
/* apnn_gemm_w8: the layer form of apmm_w1a2 and its siblings (LIB/71_bmmaTensorCoreGemm.cu:80, 72, 78) for
 * callers short of device memory: static weights as the int8 rows apnn_expand_planes made once, activations
 * straight from their packed planes X[xbits][N][K/32] as the producing layer (or apnn_bit_compress) left
 * them.  The CTA-pair kernel's own warps spread the bits into its shared-memory stages, so no expand pass
 * runs and the activations never exist as int8 rows in HBM (no workspace beyond the status flag).  The price
 * is speed: at 8192^3 w1a2 0.45 ms per call against 0.31 ms for apnn_expand_planes + apnn_gemm_i8.
 * xbits in 1..4 (x_signed only with xbits == 1); every M and N (ragged edges handled).  Epilogue as
 * apnn_gemm_i8 without out_i8, residual_i16 and APNN_OUT_FLOAT.  With APNN_XPLANES=1 in the environment
 * apnn_gemm_ex takes this route for X whenever it runs the CTA-pair kernel. */
apnn_status apnn_gemm_w8(void *stream, const void *W8, int xbits, const void *X, void *D, int M, int N, int K,
                         int w_signed, int x_signed, const apnn_epilogue *epi, int *status_flag);

/* ---- operands of at most two bits on the 4-bit floating-point tensor path ----------
 * No counterpart in the reference.  tcgen05.mma kind::mxf4 multiplies e2m1 operands (4-bit floats: 0, 0.5, 1,
 * 1.5, 2, 3, 4, 6 and their negatives) at twice the int8 rate and accumulates in fp32.  The levels 0..3 of a
 * one- or two-plane operand and the -1 / +1 of a signed one-plane operand are e2m1 values; with every block scale
 * factor set to 1 all products and partial sums are small integers, exact in fp32 while |sum| < 2^24.  So for
 * wbits, xbits <= 2 the contraction of apmm_w1a2 / apmm_w2a2 (LIB/71_, 72_bmmaTensorCoreGemm.cu:80) runs there
 * bit for bit (tests compare with the oracle and with the int8 path, sums up to 786432 included).
 * apnn_expand_planes_fp4: planes[bits][rows][K/32] -> out_fp4[rows][K/2], two elements per byte (bits 1 or 2;
 *   is_signed only with bits == 1), K % 256 == 0, a fixed permutation inside each group of 32 k.
 * apnn_gemm_fp4: D = W4 * X4^T over such operands on CTA pairs (256 x 224 tiles), epilogue as apnn_gemm_i8
 *   without out_i8, residual_i16 and APNN_OUT_FLOAT; K % 256 == 0 and 9 * K < 2^24, else APNN_ERR_UNSUPPORTED.
 * apnn_gemm_ex / apnn_gemm_host take this path by themselves when the widths allow and the problem is large
 * enough for CTA pairs (APNN_FP4=0 in the environment keeps int8). */
apnn_status apnn_expand_planes_fp4(void *stream, const void *planes, void *out_fp4, long rows, int K,
                                   int bits, int is_signed);
apnn_status apnn_gemm_fp4(void *stream, const void *W4, const void *X4, void *D, int M, int N, int K,
                          const apnn_epilogue *epi, int *status_flag);

/* A tcgen05 GEMM that allocates nothing and needs no workspace argument.  No counterpart
 * in the reference.  It exists for callers that cannot cudaMalloc a workspace: code running
 * inside a host application whose own memory pool already owns the device's memory, or a
 * latency-critical loop that cannot afford the device-wide synchronisation of cudaMalloc /
 * cudaFree and has no spare buffer to pass.  The int8 images of W and X are written to a
 * fixed array inside the library image (APNN_STATIC_SCRATCH_BYTES of device memory on every
 * GPU that loads the library, held until the process exits).
 *   - Limit: align256(M*K) + align256(N*K) <= APNN_STATIC_SCRATCH_BYTES (e.g. 2048x2048x8192,
 *     4096x4096x4096); anything larger returns APNN_ERR_WORKSPACE and launches nothing.
 *   - All calls on a device share the one array: calls whose kernels may overlap on the GPU
 *     race on it, so keep them on one stream or order them with events.  The array is not
 *     cleared between calls and does not need to be; the status flag (4 bytes of caller
 *     device memory, 0 = completed, non-zero = a bounded wait expired) is reset by each call.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress) and caches it; make that first call outside stream capture.
 * Arguments and results are those of apnn_gemm_ex (wbits, xbits in 1..4, same epilogue). */
#define APNN_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
apnn_status apnn_gemm_static_scratch(void *stream, int wbits, int xbits, const void *W, const void *X,
                                     void *D, int M, int N, int K, const apnn_epilogue *epi,
                                     int *status_flag);

/* ---- convolution ---------------------------------------------------------------
 * Implicit-GEMM RxR convolution, R odd in 1..11, stride in 1..4, symmetric padding (R-1)/2
 * carried by the input.  With B = 1, R = 3, stride = 1:
 *   epi NULL / APNN_OUT_INT32      -> compute_conv_imma (LIB/51_...cu:58 w1a2, LIB/48_...cu:58
 *                                     w2a2, LIB/53_...cu:58 w1a4, LIB/59_...cu:58 w1a3)
 *   APNN_OUT_LOWBITS               -> APConv_w1a2_pack (LIB/67_bmmaTensorCoreGemm.cu:58),
 *                                     APConv_w2a2_pack (LIB/70_...cu:58)
 *   APNN_OUT_LOWBITS + POOL_AVG2   -> APConv_w1a2_pack_pool (LIB/68_...cu:58),
 *                                     APConv_w2a2_pack_pool (LIB/69_...cuh:59)
 * which Conv_new_global calls (NN/kernel.cuh:285-289).
 * Rules: CIN % 128 == 0; packed modes need COUT % 32 == 0; pooling needs even Ho, Wo. */
apnn_status apnn_conv2d(void *stream, int wbits, int xbits, const void *Wt, const void *X,
                        void *Out, int B, int H, int W, int CIN, int COUT, int R, int stride,
                        const apnn_epilogue *epi);

/* apnn_conv2d_ex adds the algorithm / workspace choice.  APNN_ALGO_TCGEN05 (stride 1 or 2, any supported R)
 * expands activations and filter to int8 in the workspace and runs the implicit GEMM on
 * tcgen05 kind::i8, each A tile a 4-D TMA box of output pixels; APNN_ALGO_AUTO picks it when
 * the workspace is large enough and the contraction is at least ~2 GFLOP, else the
 * warp-level kernel.  apnn_conv2d_check is apnn_gemm_check for this workspace layout.
 * apnn_conv2d_i8 runs on operands already expanded by apnn_expand_planes: X8[B][H+2h][W+2h][CIN]
 * (h = epi->in_halo, or (R-1)/2 when that is 0)
 * and W8[COUT][R*R*CIN] (expand the filter once per model, the activations once per layer). */
apnn_status apnn_conv2d_ex(void *stream, int algo, int wbits, int xbits, const void *Wt, const void *X,
                           void *Out, int B, int H, int W, int CIN, int COUT, int R, int stride,
                           const apnn_epilogue *epi, void *workspace, size_t workspace_bytes);
size_t apnn_conv2d_workspace_bytes(int algo, int B, int H, int W, int CIN, int COUT, int R);
apnn_status apnn_conv2d_check(void *stream, const void *workspace, int B, int H, int W, int CIN, int COUT,
                              int R);
/* w_signed: bit 0 = the filter bytes are signed (-1/+1 weights), bit 1 = the activation bytes are signed
 * (the centred 8-bit first layer, APNN_QUANT_CENTRED below). */
apnn_status apnn_conv2d_i8(void *stream, const void *W8, const void *X8, void *Out, int B, int H, int W,
                           int CIN, int COUT, int R, int stride, int w_signed,
                           const apnn_epilogue *epi, int *status_flag);

/* The quantising part of the epilogue on its own: int32 values[rows][N] -> levels (out_mode
 * APNN_OUT_LOWBITS or APNN_OUT_THRESHOLDS with epi->thresholds [N][2^out_bits - 1]) -> packed
 * planes [out_bits][rows][N/32], or int8 rows [rows][N] when epi->out_i8 is set; with APNN_OUT_FLOAT
 * -> float[rows][N] = float(value) * affine_scale[n] + affine_bias[n].  It follows a
 * GEMM whose int32 result was produced by split-K (apnn_gemm_i8 splits K over idle SMs when a
 * problem has few tiles and a long K, which needs the int32 output).  N % 32 == 0; pooling,
 * residuals and sign correction are not taken here.  Semantics of `val & 3` / thresholds as in
 * the fused epilogue (LIB/66_bmmaTensorCoreGemm.cuh:263-268). */
apnn_status apnn_requantize_i32(void *stream, const int32_t *values, void *out, long rows, int N,
                                const apnn_epilogue *epi);

/* 2x2 maximum over int8 rows (levels as apnn_conv2d_i8 writes them with out_i8): in
 * [B][H+2*in_halo][W+2*in_halo][C] -> out [B][H/2+2*out_halo][W/2+2*out_halo][C], ring untouched.
 * For threshold outputs with ascending thresholds the maximum of the levels is the level of the
 * maximum, so an unpooled convolution followed by this pass equals APNN_POOL_MAX2 in the
 * epilogue; it lets pooled stride-1 layers run on the flat convolution.  C % 16 == 0, H and W
 * even, both pointers 16-byte aligned.  Pooling semantics: NN/kernel.cuh:856-859 (OR of
 * binarised outputs = maximum of 1-bit levels). */
apnn_status apnn_maxpool2x2_i8(void *stream, const void *in_i8, void *out_i8, int B, int H, int W, int C,
                               int in_halo, int out_halo);

/* ---- packers -------------------------------------------------------------------
 * apnn_bit_compress replaces Bit_compression (NN/kernel.cuh:46-77): one uint32 level per
 * element, levels[rows][C] -> planes[bits][rows][PAD128(C)/32], channel c in bit 31-(c%32);
 * channels C..PAD128(C)-1 are written as zero.
 * apnn_quantize_pack fuses Quantize_val (NN/kernel.cuh:29-44: clip to [-10,10], affine to
 * 2^bits steps, round to nearest even, clamped to 2^bits-1) in front of it, replacing the
 * kernel pair images_quantization launches (NN/kernel.cuh:129-161). */
apnn_status apnn_bit_compress(void *stream, const uint32_t *levels, uint32_t *planes, long rows,
                              int C, int bits);
apnn_status apnn_quantize_pack(void *stream, const float *values, uint32_t *planes, long rows,
                               int C, int bits);
/* First-layer variant of the pair above: quantises a float NHWC image [B][H][W][C] and lays
 * every output pixel's RxRxC window (symmetric padding (R-1)/2, given stride) out along the
 * channel axis: planes[bits][B][Ho][Wo][PAD128(R*R*C)/32], element k = (i*R + j)*C + c, zero
 * where the window leaves the image.  A first layer (3 channels, 7x7 or 11x11 filter:
 * NN/alexnet.cu:43-45, NN/resnet18.cu:40-42) then runs as a 1x1 convolution over R*R*C channels
 * with the filter rows in the same k order, instead of over C padded to 128. */
apnn_status apnn_quantize_im2col(void *stream, const float *images, uint32_t *planes, int B, int H,
                                 int W, int C, int R, int stride, int bits);

/* The same first-layer gather written straight as the int8 operand of apnn_conv2d_i8 (a 1x1
 * convolution over kp "channels"): out_i8[B*Ho*Wo][kp], one quantised level per byte in the
 * byte order of apnn_expand_planes, zero beyond R*R*C.  kp: a multiple of 64, >= R*R*C.
 * Replaces images_quantization + Bit_compression + the expand pass for the first layer
 * (NN/kernel.cuh:129-161); no counterpart of the window gather in the reference. */
/* bits may carry APNN_QUANT_CENTRED (with 8 bits only): every level is stored as level - 128 in a signed byte,
 * elements outside the image stay 0 -- the image at 8-bit precision with zero meaning zero, as the
 * reference's full-precision first layer skips out-of-frame pixels (InConv128Layer, NN/kernel.cuh:583-682:
 * float image x +-1 filter).  With +-1 filter bytes the int32 accumulator is exact and equals 12.8 x the
 * reference's float sum of the quantised image.  Run the convolution with bit 1 of w_signed set. */
#define APNN_QUANT_CENTRED 0x100
apnn_status apnn_quantize_im2col_i8(void *stream, const float *images, void *out_i8, int B, int H,
                                    int W, int C, int R, int stride, int bits, int kp);

/* The first-layer gather as whole words: out_i8[B*Ho*Wo][kp] with an output pixel's row made of
 * R segments of seg = 4*ceil(R*C/4) bytes in plain byte order (byte p of the row is k = p):
 * segment i, byte t < R*C = the level of input element (row ho*stride - pad + i, column
 * wo*stride - pad + t/C, channel t%C), zero outside the image; every other byte is zero.  The
 * filter row for apnn_conv2d_i8 is laid out the same way, k = i*seg + j*C + c.  kp: a multiple
 * of 64, >= R*seg.  Returns APNN_ERR_UNSUPPORTED for rows it does not cover (W*C not a multiple
 * of 4, Wo*kp/16 > 2048): use apnn_quantize_im2col_i8 there.  No counterpart in the reference. */
apnn_status apnn_quantize_window_rows_i8(void *stream, const float *images, void *out_i8, int B,
                                         int H, int W, int C, int R, int stride, int bits, int kp);

/* A strided first layer without the window copy: the image regrouped into stride x stride pixel blocks.
 * out_i8[B][H/stride + 2*halo][W/stride + 2*halo][cpad]: block (hb, wb) is one "pixel" of cpad bytes, byte
 * (di*stride + dj)*C + c = the level of image pixel (stride*hb + di, stride*wb + dj), channel c (plain order,
 * byte p is channel p), the remaining bytes 0; the ring of halo blocks is not written (zero it once).  The RxR
 * stride-s convolution (padding p = (R-1)/2) of the image equals the stride-1 convolution of this tensor with
 * R' = 2*ceil(p/s) + 1 taps a side and in_halo = ceil(p/s), whose filter holds the weight of image tap
 * (ti, tj, c), ti = s*(bi - ceil(p/s)) + di + p, at block tap (bi, bj), channel (di*s + dj)*C + c, and 0
 * where ti or tj falls outside 0..R-1 -- run it with apnn_conv2d_i8 like any other layer.  The quantised image
 * is written once (cpad bytes per block) instead of once per window.  bits as in apnn_quantize_im2col_i8
 * (APNN_QUANT_CENTRED included).  stride 2..4, H and W multiples of it, stride*C a multiple of 4,
 * stride*stride*C <= cpad, cpad a multiple of 16; APNN_ERR_UNSUPPORTED otherwise.  No counterpart in the
 * reference, whose first layer reads the float image directly (NN/kernel.cuh:583-682). */
apnn_status apnn_quantize_blocks_i8(void *stream, const float *images, void *out_i8, int B, int H, int W,
                                    int C, int stride, int bits, int halo, int cpad);

/* ---- measurement aid ------------------------------------------------------------
 * Launches an operand-resident issue loop of one contraction instruction on every SM and
 * returns the operations one launch performs; the caller times the launch with events to
 * get the device's peak for that path (the roofline denominator).  kind 0: tcgen05.mma
 * kind::i8 (128x256x32, operands fixed in shared memory), 1: mma.sync m16n8k32 u8,
 * 2: mma.sync m16n8k256 b1 and.popc (bit operations), 3 / 4: kind 0 with N = 128 / 64,
 * 5: tcgen05.mma kind::mxf4 (128x224x64, e2m1 operands, unit scale factors).
 * scratch_flag: 4 bytes of device
 * memory.  No counterpart in the reference. */
apnn_status apnn_probe_peak(void *stream, int kind, int iters, int *scratch_flag,
                            double *ops_per_launch);

/* ---- host-buffer front end -----------------------------------------------------
 * For callers that hold operands in host memory (the reference's main() programs:
 * malloc + cudaMemcpy around every launch, LIB/71_bmmaTensorCoreGemm.cu:498-571).
 * A handle owns a stream and a grow-only device arena; apnn_gemm_host copies W and X
 * in, runs apnn_gemm_ex, copies D out and synchronises. */
typedef struct apnn_handle_s *apnn_handle;
apnn_status apnn_create(apnn_handle *h, int device);
apnn_status apnn_destroy(apnn_handle h);
apnn_status apnn_gemm_host(apnn_handle h, int algo, int wbits, int xbits, const void *W_host,
                           const void *X_host, void *D_host, int M, int N, int K,
                           const apnn_epilogue *epi_host_thresholds);
apnn_status apnn_conv2d_host(apnn_handle h, int wbits, int xbits, const void *Wt_host,
                             const void *X_host, void *Out_host, int B, int H, int W, int CIN,
                             int COUT, int R, int stride, const apnn_epilogue *epi_host_thresholds);

#ifdef __cplusplus
}
#endif
#endif /* APNN_B200_H */
