// Warp-level core kernels for operand widths A = 4 bit, B = 1 bit.
#include "core_inst.cuh"
namespace apnn {
template cudaError_t launch_pair<4, 1>(int, const CoreParams&, cudaStream_t, int);
}
