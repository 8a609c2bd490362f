// Warp-level core kernels for operand widths A = 1 bit, B = 4 bit.
#include "core_inst.cuh"
namespace apnn {
template cudaError_t launch_pair<1, 4>(int, const CoreParams&, cudaStream_t, int);
}
