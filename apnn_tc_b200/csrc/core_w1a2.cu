// Warp-level core kernels for operand widths A = 1 bit, B = 2 bit.
#include "core_inst.cuh"
namespace apnn {
template cudaError_t launch_pair<1, 2>(int, const CoreParams&, cudaStream_t, int);
}
