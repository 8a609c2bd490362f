// tcgen05 kind::i8 GEMM path: planes -> int8 rows in a caller workspace, then a TMA-fed,
// TMEM-accumulating GEMM.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>
#include "../../include/apnn_b200.h"

namespace apnn {
size_t tc5_workspace_bytes(int M, int N, int K);
// True when the problem is large enough for this path to beat the warp-level core.
bool tc5_worthwhile(int M, int N, int K);
apnn_status tc5_gemm(cudaStream_t s, int wbits, int xbits, const uint32_t* W, const uint32_t* X, void* D, int M,
                     int N, int K, const apnn_epilogue* epi, void* workspace, int pair = 0);
// The two stages of tc5_gemm on their own: planes -> int8 rows (rows x K bytes), and the
// int8 GEMM over already expanded operands (static weights are expanded once).
apnn_status tc5_expand(cudaStream_t s, const uint32_t* planes, uint8_t* out, long long rows, int K, int bits,
                       bool is_signed);
apnn_status tc5_expand2(cudaStream_t s, const uint32_t* pa, uint8_t* oa, long long rows_a, int bits_a, bool signed_a,
                        const uint32_t* pb, uint8_t* ob, long long rows_b, int bits_b, bool signed_b, int K);
apnn_status tc5_gemm_i8(cudaStream_t s, const uint8_t* A8, const uint8_t* B8, void* D, int M, int N, int K,
                        bool a_signed, bool b_signed, const apnn_epilogue* epi, int* status_flag);
// Convolution on the same kernel (implicit GEMM over 4-D TMA boxes of output pixels):
// R odd up to 11, stride 1 or 2, CIN % 128 == 0; H, W are the input extent.  workspace holds the int8 activations (halo
// included), the int8 filter and the status flag.
size_t tc5_conv_workspace_bytes(int B, int H, int W, int CIN, int COUT, int R);
bool tc5_conv_supported(int H, int W, int R, int stride, int pool);
apnn_status tc5_conv(cudaStream_t s, int wbits, int xbits, const uint32_t* Wt, const uint32_t* X, void* Out, int B,
                     int H, int W, int CIN, int COUT, int R, int stride, const apnn_epilogue* epi, void* workspace);
apnn_status tc5_conv_i8(cudaStream_t s, const uint8_t* X8, const uint8_t* W8, void* Out, int B, int H, int W,
                        int CIN, int COUT, int R, int stride, bool w_signed, const apnn_epilogue* epi, int* status_flag,
                        bool x_signed = false);
int tc5_conv_read_error_flag(cudaStream_t s, const void* workspace, int B, int H, int W, int CIN, int COUT, int R);
// The same GEMM on CTA pairs (cta_group::2, 256 x 256 tiles); worthwhile once there are at
// least as many pair tiles as SM pairs.
bool tc5_pair_worthwhile(int M, int N, int K);
apnn_status tc5_gemm_i8_pair(cudaStream_t s, const uint8_t* A8, const uint8_t* B8, void* D, int M, int N, int K,
                             bool a_signed, bool b_signed, const apnn_epilogue* epi, int* status_flag,
                             const uint32_t* xplanes = nullptr, int xbits = 0);
apnn_status tc5_expand_fp4(cudaStream_t s, const uint32_t* planes, uint8_t* out, long long rows, int K, int bits,
                           bool is_signed);
apnn_status tc5_gemm_fp4_pair(cudaStream_t s, const uint8_t* A4, const uint8_t* B4, void* D, int M, int N, int K,
                              const apnn_epilogue* epi, int* status_flag);
// The flat convolution on CTA pairs (256 positions x 256 channels per pair): stride 1, no pooling,
// CIN % 128 == 0, COUT % 256 == 0, thresholds -> int8 rows, no residuals.  H, W: input extent.
bool tc5_conv_pair_applies(int B, int H, int W, int CIN, int COUT, int R, int stride, const apnn_epilogue* epi);
apnn_status tc5_conv_i8_pair(cudaStream_t s, const uint8_t* X8, const uint8_t* W8, void* Out, int B, int H, int W,
                             int CIN, int COUT, int R, bool w_signed, const apnn_epilogue* epi, int* status_flag);
// Where the status flag lives inside a GEMM / convolution workspace.
int* tc5_flag_slot(void* workspace, int M, int N, int K);
int* tc5_conv_flag_slot(void* workspace, int B, int H, int W, int CIN, int COUT, int R);
// Flag raised by a bounded wait (0 = ran to completion); synchronises the stream.
int tc5_read_error_flag(cudaStream_t s, const void* workspace, int M, int N, int K);
}  // namespace apnn
