// Helpers shared by the translation units behind the C ABI.
#pragma once
#include <cuda_runtime.h>
#include "../../include/apnn_b200.h"

namespace apnn {
// Records the CUDA error text for apnn_last_cuda_error() and returns APNN_ERR_CUDA.
apnn_status cuda_fail(cudaError_t e, const char* where);
int device_sm_count();
// Validates an epilogue descriptor; wbits/xbits are the widths of the W and X arguments.
apnn_status check_epilogue(const apnn_epilogue* e, int channels, bool is_conv, int wbits, int xbits,
                           bool i8_rows_ok = false);
}  // namespace apnn
