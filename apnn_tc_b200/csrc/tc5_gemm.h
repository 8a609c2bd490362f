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
// Flag raised by a bounded wait (0 = ran to completion); synchronises the stream.
int tc5_read_error_flag(cudaStream_t s, const void* workspace, int M, int N, int K);
}  // namespace apnn
