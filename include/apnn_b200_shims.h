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

/* LIB/66_bmmaTensorCoreGemm.cuh:81, LIB/73_...cuh:81: accumulator & 3, plane-split, packed along N */
inline void apmm_decompose(const int4* W, const int4* X, int* D, int M, int N, int K, int wb, int xb, int out_bits,
                           cudaStream_t s = 0) {
  apnn_epilogue e = {APNN_OUT_LOWBITS, out_bits, APNN_SIGN_NONE, APNN_POOL_NONE, 0, 0, nullptr};
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
  apnn_epilogue e = {APNN_OUT_LOWBITS, 2, APNN_SIGN_NONE, pool ? APNN_POOL_AVG2 : APNN_POOL_NONE, 0, 0, nullptr};
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

#endif /* APNN_B200_SHIMS_H */
