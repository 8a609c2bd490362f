// Tile configurations of the warp-level core and the per-pair launcher that the
// core_wXaY.cu translation units instantiate (one bit-width pair each, so they build in
// parallel).
#pragma once
#include "core_launch.h"
#include "plane_core.cuh"

namespace apnn {

// tile classes
//   big   : 128 x 128 outputs, 8 warps (2 x 4), each warp 64 x 32
//   small :  64 x  32 outputs, 2 x 1 warps of 32 x 32 times two K groups (4 warps): spreads tiny
//            problems over many SMs and halves a warp's serial chain of K steps
//   b1    : 128 x 64 outputs, 8 warps (4 x 2); one accumulator set per weight class, so the
//            warp tile shrinks to 32 x 32
template <int KIND, int AB, int BB>
using BigCfg = CoreCfg<KIND, AB, BB, 4, 4, 2, 4, ((AB * 128 + BB * 128) * 64 * 4 <= 160 * 1024 ? 4 : 3)>;
template <int KIND, int AB, int BB>
using SmallCfg = CoreCfg<KIND, AB, BB, 2, 4, 2, 1, 4, 2>;   // four groups measured no faster than two
template <int AB, int BB>
using B1Cfg = CoreCfg<KIND_B1, AB, BB, 2, 4, 4, 2, 4>;

template <class Cfg>
cudaError_t launch_cfg(const CoreParams& p, cudaStream_t stream) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 16 || !attr_set[dev]) {
    e = cudaFuncSetAttribute(plane_core_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev < 16) attr_set[dev] = true;
  }
  long long tiles_m = ((long long)p.M + Cfg::BM - 1) / Cfg::BM;  // pooled rows are laid out 4 per window
  long long tiles_n = ((long long)p.N + Cfg::BN - 1) / Cfg::BN;
  long long grid = tiles_m * tiles_n;
  if (grid <= 0 || grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  plane_core_kernel<Cfg><<<(unsigned)grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError();
}

template <int AB, int BB>
cudaError_t launch_pair(int kind, const CoreParams& p, cudaStream_t s, int tile_class) {
  if (kind == KIND_B1) return launch_cfg<B1Cfg<AB, BB>>(p, s);
  if (tile_class == TILE_BIG) return launch_cfg<BigCfg<KIND_U8, AB, BB>>(p, s);
  return launch_cfg<SmallCfg<KIND_U8, AB, BB>>(p, s);
}

}  // namespace apnn
