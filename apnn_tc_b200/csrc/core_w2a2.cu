// Warp-level core kernels for operand widths A = 2 bit, B = 2 bit.
#include "core_inst.cuh"
namespace apnn {
template cudaError_t launch_pair<2, 2>(int, const CoreParams&, cudaStream_t, int);
}
