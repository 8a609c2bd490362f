/*
 * apnn_b200_shims.h -- host functions carrying the reference's kernel names and argument
 * lists, forwarding to the C ABI in apnn_b200.h.  A reference program replaces its kernel
 * body with this header and turns `kernel<<<SMs, 256, 65536>>>(args)` into `kernel(args)`.
 * Paths cited are inside the APNN-TC project; LIB = APNN-TC-lib/bmmaTensorCoreGemm/src.
 * Like the reference (checkKernelErrors, LIB/71_bmmaTensorCoreGemm.cu:65-75), a failure
 * prints a message and aborts.
 */
#ifndef APNN_B200_SHIMS_H
#define APNN_B200_SHIMS_H

#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "apnn_b200.h"

#define APNN_SHIM_CHECK(expr)                                                                  \
  do {                                                                                         \
    apnn_status s_ = (expr);                                                                   \
    if (s_ != APNN_OK) {                                                                       \
      printf("Line %d: '%s' failed: %s %s\n", __LINE__, #expr, apnn_status_string(s_),         \
             apnn_last_cuda_error());                                                          \
      abort();                                                                                 \
    }                                                                                          \
  } while (0)

/* LIB/71_bmmaTensorCoreGemm.cu:80, LIB/72_...cu:80, LIB/78_...cu:80 (and the w1a3 binary) */
inline void apmm(const int4* W, const int4* X, int* D, int M_GLOBAL, int N_GLOBAL, int K_GLOBAL, int wb, int xb,
                 cudaStream_t stream = 0) {
  APNN_SHIM_CHECK(apnn_gemm(stream, wb, xb, W, X, D, M_GLOBAL, N_GLOBAL, K_GLOBAL));
}
inline void apmm_w1a2(const int4* W, const int4* X, int* D, int M, int N, int K, int wb = 1, int xb = 2,
                      cudaStream_t s = 0) { apmm(W, X, D, M, N, K, wb, xb, s); }
inline void apmm_w1a3(const int4* W, const int4* X, int* D, int M, int N, int K, int wb = 1, int xb = 3,
                      cudaStream_t s = 0) { apmm(W, X, D, M, N, K, wb, xb, s); }
inline void apmm_w1a4(const int4* W, const int4* X, int* D, int M, int N, int K, int wb = 1, int xb = 4,
                      cudaStream_t s = 0) { apmm(W, X, D, M, N, K, wb, xb, s); }
inline void apmm_w2a2(const int4* W, const int4* X, int* D, int M, int N, int K, int wb = 2, int xb = 2,
                      cudaStream_t s = 0) { apmm(W, X, D, M, N, K, wb, xb, s); }

/* The reference's fused kernels keep the low bits of the accumulator: the epilogue descriptor for that,
 * every field named (nothing here depends on the order of the structure's members). */
inline apnn_epilogue apnn_shim_lowbits(int out_bits, int pool) {
  apnn_epilogue e = APNN_EPILOGUE_INIT;
  e.out_mode = APNN_OUT_LOWBITS;
  e.out_bits = out_bits;
  e.signed_operand = APNN_SIGN_NONE;
  e.pool = pool;
  return e;
}

/* LIB/66_bmmaTensorCoreGemm.cuh:81, LIB/73_...cuh:81: accumulator & 3, plane-split, packed along N */
inline void apmm_decompose(const int4* W, const int4* X, int* D, int M, int N, int K, int wb, int xb, int out_bits,
                           cudaStream_t s = 0) {
  apnn_epilogue e = apnn_shim_lowbits(out_bits, APNN_POOL_NONE);
  APNN_SHIM_CHECK(apnn_gemm_ex(s, APNN_ALGO_AUTO, wb, xb, W, X, D, M, N, K, &e, nullptr, 0));
}
inline void apmm_w1a2_decompose(const int4* W, const int4* X, int* D, int M, int N, int K, int wb = 1, int xb = 2,
                                cudaStream_t s = 0) { apmm_decompose(W, X, D, M, N, K, wb, xb, 2, s); }
inline void apmm_w2a2_decompose(const int4* W, const int4* X, int* D, int M, int N, int K, int wb = 2, int xb = 2,
                                cudaStream_t s = 0) { apmm_decompose(W, X, D, M, N, K, wb, xb, 2, s); }

/* LIB/51_...cu:58 (w1a2), LIB/48_...cu:58 (w2a2), LIB/53_...cu:58 (w1a4), LIB/59_...cu:58 (w1a3):
 * int32 3x3 conv over one pre-haloed image */
inline void compute_conv_imma(const int4* W, const int4* X, int* Output, int Height, int Width, int CIN, int COUT,
                              int wb, int xb, cudaStream_t s = 0) {
  APNN_SHIM_CHECK(apnn_conv2d(s, wb, xb, W, X, Output, 1, Height, Width, CIN, COUT, 3, 1, nullptr));
}

/* LIB/67_...cu:58, LIB/68_...cu:58, LIB/70_...cu:58, LIB/69_...cuh:59 */
inline void APConv_pack(const int4* W, const int4* X, int* Output, int Height, int Width, int CIN, int COUT, int wb,
                        int xb, int pool, cudaStream_t s = 0) {
  apnn_epilogue e = apnn_shim_lowbits(2, pool ? APNN_POOL_AVG2 : APNN_POOL_NONE);
  APNN_SHIM_CHECK(apnn_conv2d(s, wb, xb, W, X, Output, 1, Height, Width, CIN, COUT, 3, 1, &e));
}
inline void APConv_w1a2_pack(const int4* W, const int4* X, int* O, int H, int Wd, int CIN, int COUT,
                             cudaStream_t s = 0) { APConv_pack(W, X, O, H, Wd, CIN, COUT, 1, 2, 0, s); }
inline void APConv_w1a2_pack_pool(const int4* W, const int4* X, int* O, int H, int Wd, int CIN, int COUT,
                                  cudaStream_t s = 0) { APConv_pack(W, X, O, H, Wd, CIN, COUT, 1, 2, 1, s); }
inline void APConv_w2a2_pack(const int4* W, const int4* X, int* O, int H, int Wd, int CIN, int COUT,
                             cudaStream_t s = 0) { APConv_pack(W, X, O, H, Wd, CIN, COUT, 2, 2, 0, s); }
inline void APConv_w2a2_pack_pool(const int4* W, const int4* X, int* O, int H, int Wd, int CIN, int COUT,
                                  cudaStream_t s = 0) { APConv_pack(W, X, O, H, Wd, CIN, COUT, 2, 2, 1, s); }

/* ---- layer boundary: quantise + pack (paths inside APNN-TC-nn/src) ------------------------
 * uin32 is the reference's name for a 32-bit word (utility.h).  Layouts as Bit_compression
 * writes them (kernel.cuh:46-77): [bit][rows][PAD128(C)/32], channel c in bit 31 - c%32. */
#ifndef APNN_SHIM_UIN32
#define APNN_SHIM_UIN32
typedef unsigned int uin32;
#endif
inline int apnn_shim_pad128(int c) { return (c + 127) / 128 * 128; }
inline int apnn_shim_pad8(int c) { return (c + 7) / 8 * 8; }

#define APNN_SHIM_CUDA(expr)                                                                   \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess) {                                                                   \
      printf("Line %d: '%s' failed: %s\n", __LINE__, #expr, cudaGetErrorString(e_));           \
      abort();                                                                                 \
    }                                                                                          \
  } while (0)

/* kernel.cuh:129-161: host float NHWC images -> newly allocated device bit planes (the caller
 * frees them); Quantize_val + Bit_compression in one launch.  The reference's Quantize_val never
 * stores its result (kernel.cuh:42); this one does. */
inline uin32* images_quantization(float* images, int batch, int image_width, int image_height, int image_channel,
                                  int bit = 2, cudaStream_t s = 0) {
  const long rows = (long)batch * image_height * image_width;
  float* images_gpu = nullptr;
  uin32* bit_images_gpu = nullptr;
  APNN_SHIM_CUDA(cudaMalloc(&images_gpu, rows * image_channel * sizeof(float)));
  APNN_SHIM_CUDA(cudaMalloc(&bit_images_gpu, (size_t)bit * rows * apnn_shim_pad128(image_channel) / 8));
  APNN_SHIM_CUDA(cudaMemcpyAsync(images_gpu, images, rows * image_channel * sizeof(float), cudaMemcpyHostToDevice, s));
  APNN_SHIM_CHECK(apnn_quantize_pack(s, images_gpu, bit_images_gpu, rows, image_channel, bit));
  APNN_SHIM_CUDA(cudaStreamSynchronize(s));
  APNN_SHIM_CUDA(cudaFree(images_gpu));
  return bit_images_gpu;
}

/* kernel.cuh:164-197: device float filter [O][Fh][Fw][C] -> planes [bit][O*Fh*Fw][PAD128(C)/32].
 * The reference assigns the new buffer to a by-value pointer (kernel.cuh:186), so its caller never
 * sees it; here the pointer is passed by reference. */
inline void filter_quantization(uin32*& bit_filter_gpu, float* filter_gpu, int out_channel, int filter_width,
                                int filter_height, int in_channel, int bit, cudaStream_t s = 0) {
  const long rows = (long)out_channel * filter_height * filter_width;
  APNN_SHIM_CUDA(cudaMalloc(&bit_filter_gpu, (size_t)bit * rows * apnn_shim_pad128(in_channel) / 8));
  APNN_SHIM_CHECK(apnn_quantize_pack(s, filter_gpu, bit_filter_gpu, rows, in_channel, bit));
  APNN_SHIM_CUDA(cudaStreamSynchronize(s));
}

/* kernel.cuh:200-237: device float weights [out][in] -> caller-allocated planes [bit][out][PAD128(in)/32] */
inline void weight_quantization(uin32* bit_weight_gpu, float* weight_gpu, int in_channel, int out_channel, int bit,
                                cudaStream_t s = 0) {
  APNN_SHIM_CHECK(apnn_quantize_pack(s, weight_gpu, bit_weight_gpu, out_channel, in_channel, bit));
  APNN_SHIM_CUDA(cudaStreamSynchronize(s));
}

/* kernel.cuh:239-282: as above, and -- like the reference (kernel.cuh:279) -- it frees the float
 * input.  The reference's Bit_compression_fc_hidden writes every plane to the same words
 * (kernel.cuh:122); this one keeps the planes apart as weight_quantization does. */
inline void weight_quantization_fc_hidden(uin32* bit_weight_gpu, float* weight_gpu, int in_channel, int out_channel,
                                          int bit, cudaStream_t s = 0) {
  weight_quantization(bit_weight_gpu, weight_gpu, in_channel, out_channel, bit, s);
  APNN_SHIM_CUDA(cudaFree(weight_gpu));
}

/* ---- layer launches (kernel.cuh:285-318) ---------------------------------------------------
 * The reference's __global__ wrappers read a device-resident layer struct; these host
 * functions take the host copy of the same struct (any type with the reference's field
 * names: Conv128LayerParam / Fc128LayerParam / Out128LayerParam of param.h) and pass the
 * arguments the reference passes: the batch folded into the height for the convolution
 * (kernel.cuh:287-288), and for the fully connected layers the activations as the first
 * (1-bit) operand and the weights as the second (2-bit) one (kernel.cuh:299-318).  The
 * reference gives the GEMM STEP counts where sizes are meant (8*STEP8(h), STEP8(w),
 * STEP128(k)); the sizes are passed here: PAD8(batch) rows, weight_width columns rounded up
 * to 32, PAD128(input_width) deep. */
template <class ConvParam>
inline void Conv_new_global(const ConvParam* p, cudaStream_t s = 0) {
  APConv_w1a2_pack((const int4*)p->filter_gpu, (const int4*)p->input_gpu, (int*)p->output_gpu,
                   apnn_shim_pad8(p->batch) * p->input_height, p->input_width, p->input_channels, p->output_channels, s);
}
template <class FcParam>
inline void FC_new_global(const FcParam* p, cudaStream_t s = 0) {
  apmm_w1a2_decompose((const int4*)p->input_gpu, (const int4*)p->weight_gpu, (int*)p->output_gpu,
                      apnn_shim_pad8(p->input_height), (p->weight_width + 31) / 32 * 32, apnn_shim_pad128(p->input_width),
                      1, 2, s);
}
template <class OutParam>
inline void Output_new_global(const OutParam* p, cudaStream_t s = 0) {
  FC_new_global(p, s);
}

#endif /* APNN_B200_SHIMS_H */
