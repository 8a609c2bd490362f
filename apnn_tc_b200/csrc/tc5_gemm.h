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
                     int N, int K, const apnn_epilogue* epi, void* workspace);
// The two stages of tc5_gemm on their own: planes -> int8 rows (rows x K bytes), and the
// int8 GEMM over already expanded operands (static weights are expanded once).
apnn_status tc5_expand(cudaStream_t s, const uint32_t* planes, uint8_t* out, long long rows, int K, int bits,
                       bool is_signed);
apnn_status tc5_gemm_i8(cudaStream_t s, const uint8_t* A8, const uint8_t* B8, void* D, int M, int N, int K,
                        bool a_signed, bool b_signed, const apnn_epilogue* epi, int* status_flag);
// Flag raised by a bounded wait (0 = ran to completion); synchronises the stream.
int tc5_read_error_flag(cudaStream_t s, const void* workspace, int M, int N, int K);
}  // namespace apnn
