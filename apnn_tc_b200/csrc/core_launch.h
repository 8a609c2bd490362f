// Host-side entry of the warp-level plane contraction core.
#pragma once
#include <cuda_runtime.h>
#include "apnn_device.cuh"

namespace apnn {

enum { TILE_AUTO = -1, TILE_BIG = 0, TILE_SMALL = 1 };
enum { CORE_U8 = 0, CORE_B1 = 1 };  // same values as KIND_U8 / KIND_B1

// True when a kernel is instantiated for this (A bits, B bits) pair.
bool core_supports(int abits, int bbits);
// Tile class that fills the device best for this problem.
int core_pick_tile(const CoreParams& p, int sm_count);
// Launches one contraction; p.M counts A rows (GEMM rows or conv output pixels).
cudaError_t launch_core(int kind, int abits, int bbits, const CoreParams& p, cudaStream_t s, int tile_class);

}  // namespace apnn
