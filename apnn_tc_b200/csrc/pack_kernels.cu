// Layer-boundary packers: one value per element in, bit planes out.
//
// A warp converts 128 consecutive channels of one row per step: every lane fetches four
// elements with one 128-bit load (512 contiguous bytes per warp), builds its 4-bit slice
// of each plane, the eight lanes that share an output word OR their slices together with
// three shuffles, and one lane per word stores it.  Channel c lands in bit 31-(c%32) of
// word c/32, planes outermost, rows padded with zero channels to a multiple of 128.
#include "../../include/apnn_b200.h"
#include "api_internal.h"

namespace apnn {

namespace {

__device__ __forceinline__ uint32_t quantize_level(float x, float steps, uint32_t maxlv) {
  // clip to [-10, 10]; ((x + 10) * 2^bits) / 20 without contraction; round to nearest even
  x = fminf(fmaxf(x, -10.0f), 10.0f);
  float qf = __fdiv_rn(__fmul_rn(__fadd_rn(x, 10.0f), steps), 20.0f);
  uint32_t u = __float2uint_rn(qf);
  return u > maxlv ? maxlv : u;
}

template <bool FROM_FLOAT>
__global__ void __launch_bounds__(256) pack_planes_kernel(const void* __restrict__ in, uint32_t* __restrict__ planes,
                                                          long long rows, int C, int bits) {
  const int lane = threadIdx.x & 31;
  const int groups = (C + 127) >> 7;           // 128-channel groups per row
  const int cw = groups * 4;                    // words per row per plane
  const long long tasks = rows * groups;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  const bool vec_ok = (C & 3) == 0;

  for (long long task = warp0; task < tasks; task += nwarps) {
    const long long row = task / groups;
    const int grp = (int)(task - row * groups);
    const int c0 = grp * 128 + lane * 4;
    uint32_t e[4] = {0u, 0u, 0u, 0u};
    const long long base = row * C + c0;
    if (vec_ok && c0 + 3 < C) {
      if (FROM_FLOAT) {
        float4 v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(in) + base));
        e[0] = quantize_level(v.x, steps, maxlv);
        e[1] = quantize_level(v.y, steps, maxlv);
        e[2] = quantize_level(v.z, steps, maxlv);
        e[3] = quantize_level(v.w, steps, maxlv);
      } else {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(in) + base));
        e[0] = v.x; e[1] = v.y; e[2] = v.z; e[3] = v.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (c0 + j < C) {
          if (FROM_FLOAT) e[j] = quantize_level(__ldg(reinterpret_cast<const float*>(in) + base + j), steps, maxlv);
          else e[j] = __ldg(reinterpret_cast<const uint32_t*>(in) + base + j);
        }
    }
    const int sub = lane & 7;
    for (int b = 0; b < bits; b++) {
      uint32_t nib = (((e[0] >> b) & 1u) << 3) | (((e[1] >> b) & 1u) << 2) | (((e[2] >> b) & 1u) << 1) |
                     ((e[3] >> b) & 1u);
      uint32_t word = nib << (28 - 4 * sub);
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 2);
      word |= __shfl_xor_sync(0xffffffffu, word, 4);
      if (sub == (b & 7)) planes[((long long)b * rows + row) * cw + grp * 4 + (lane >> 3)] = word;
    }
  }
}

template <bool FROM_FLOAT>
apnn_status launch_pack(void* stream, const void* in, uint32_t* planes, long rows, int C, int bits) {
  if (!in || !planes) return APNN_ERR_INVALID_ARG;
  if (rows <= 0 || C <= 0 || bits < 1 || bits > 8) return APNN_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(in) & 15u) || (reinterpret_cast<uintptr_t>(planes) & 15u)) return APNN_ERR_ALIGNMENT;
  long long tasks = (long long)rows * ((C + 127) / 128);
  long long blocks = (tasks + 7) / 8;
  long long cap = (long long)device_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  pack_planes_kernel<FROM_FLOAT><<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, planes, rows,
                                                                                                     C, bits);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pack_planes launch");
  return APNN_OK;
}

}  // namespace
}  // namespace apnn

extern "C" {

apnn_status apnn_bit_compress(void* stream, const uint32_t* levels, uint32_t* planes, long rows, int C, int bits) {
  return apnn::launch_pack<false>(stream, levels, planes, rows, C, bits);
}

apnn_status apnn_quantize_pack(void* stream, const float* values, uint32_t* planes, long rows, int C, int bits) {
  return apnn::launch_pack<true>(stream, values, planes, rows, C, bits);
}

}  // extern "C"
