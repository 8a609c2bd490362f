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
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device); safe to call from several threads.
cudaError_t ensure_max_smem(const void* kernel, int bytes);
// Address of the driver's cuTensorMapEncodeTiled (null if unavailable); looked up once, thread-safe.
void* tensor_map_encoder();
// Launch attribute for programmatic dependent launch: writes it to attrs[0] and returns 1, or
// returns 0 when APNN_PDL=0 is set in the environment (read once).  Only for kernels that execute
// griddepcontrol.wait before touching anything an earlier kernel of the stream produces.
int pdl_attribute(cudaLaunchAttribute* attrs);
}  // namespace apnn
