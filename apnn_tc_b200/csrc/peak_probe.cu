// Measurement aid: operand-resident issue loops that give the roofline denominators for
// the three contraction paths on the device at hand (no global-memory traffic in the loop).
//   kind 0: tcgen05.mma kind::i8, M=128 N=256 K=32, operands fixed in shared memory,
//           two TMEM accumulators, one CTA per SM
//   kind 3, 4: the same with N=128 and N=64 (narrow tiles of the convolution path)
//   kind 5: tcgen05.mma kind::mxf4 (e2m1 operands, unit ue8m0 scale factors in TMEM), M=128 N=224 K=64
//   kind 1: mma.sync m16n8k32 u8, register operands
//   kind 2: mma.sync m16n8k256 b1 and.popc, register operands
#include <cuda.h>

#include "../../include/apnn_b200.h"
#include "api_internal.h"
#include "apnn_device.cuh"

namespace apnn {
namespace {

constexpr unsigned long long PROBE_WAIT_NS = 2000000000ull;

template <int PN, bool MX = false>   // MMA width N: 256, 128 or 64 (224 for MX)
__global__ void __launch_bounds__(128, 1) probe_tcgen05_i8(int iters, int* flag) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  // A: 128 rows x 128 B, B: 256 rows x 128 B (one swizzle row of K each), then barrier + slot
  const uint32_t bar = base + 128 * 128 + 256 * 128;
  const uint32_t slot = bar + 8;
  for (uint32_t i = threadIdx.x; i < (128 * 128 + 256 * 128) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem_raw + (base - raw))[i] = MX ? 0x22222222u : 0x01010101u;   // ones either way
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(slot));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem_raw + (slot - raw));
  if (MX) {
    // scale factors: 32 columns of every lane behind the two accumulators, every byte 0x7F (ue8m0 1.0)
    const uint32_t t0 = tmem + ((uint32_t)((threadIdx.x >> 5) * 32) << 16) + 2 * PN;
#pragma unroll
    for (int i = 0; i < 4; i++)
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(t0 + 8 * i), "r"(0x7F7F7F7Fu)
                   : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  if (threadIdx.x == 0) {
    auto desc = [](uint32_t a) {
      return (uint64_t)((a & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)64 << 32) | ((uint64_t)1 << 46) |
             ((uint64_t)2 << 61);
    };
    const uint64_t ad = desc(base), bd = desc(base + 128 * 128);
    const uint32_t idesc = MX ? ((1u << 7) | (1u << 10) | ((uint32_t)(PN >> 3) << 17) | (1u << 23) | (8u << 24))
                              : ((2u << 4) | ((uint32_t)(PN >> 3) << 17) | (8u << 24));
    for (int it = 0; it < iters; it++) {
      const uint32_t d = tmem + (it & 1) * PN;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        if (MX)
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d),
              "l"(ad + 2u * k), "l"(bd + 2u * k), "r"(idesc), "r"(tmem + 2 * PN), "r"(tmem + 2 * PN + 16),
              "r"((uint32_t)(it > 1 || k > 0))
              : "memory");
        else
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
              "l"(ad + 2u * k), "l"(bd + 2u * k), "r"(idesc), "r"((uint32_t)(it > 1 || k > 0))
              : "memory");
      }
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    unsigned long long t0 = 0;
    bool done = false;
    for (uint32_t spin = 0; !done; spin++) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.b32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(bar)
          : "memory");
      done = ok != 0;
      if (!done && (spin & 255u) == 255u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > PROBE_WAIT_NS) { atomicExch(flag, 1); break; }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem));
  }
}

template <int KIND>
__global__ void __launch_bounds__(512) probe_mma_sync(int iters, int* sink) {
  int c[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) c[i][j] = 0;
  const uint32_t a0 = threadIdx.x * 2654435761u, a1 = a0 ^ 0x9e3779b9u, a2 = a0 * 3u, a3 = a1 * 5u;
  const uint32_t b0 = a0 + 17u, b1 = a1 + 29u;
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      if (KIND == 1) mma_u8(c[i], a0 & 0x03030303u, a1 & 0x03030303u, a2 & 0x03030303u, a3 & 0x03030303u,
                            b0 & 0x01010101u, b1 & 0x01010101u);
      else mma_b1(c[i], a0, a1, a2, a3, b0, b1);
    }
  }
  int s = 0;
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) s += c[i][j];
  if (s == 0x12345678) sink[0] = s;
}

}  // namespace
}  // namespace apnn

extern "C" apnn_status apnn_probe_peak(void* stream, int kind, int iters, int* scratch_flag, double* ops_per_launch) {
  using namespace apnn;
  if (!scratch_flag || !ops_per_launch || iters <= 0 || kind < 0 || kind > 5) return APNN_ERR_INVALID_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int sms = device_sm_count();
  cudaError_t e = cudaMemsetAsync(scratch_flag, 0, sizeof(int), s);
  if (e != cudaSuccess) return cuda_fail(e, "probe flag reset");
  if (kind == 0 || kind == 3 || kind == 4 || kind == 5) {
    const int smem = 128 * 128 + 256 * 128 + 1024 + 64;
    const int pn = kind == 0 ? 256 : kind == 3 ? 128 : kind == 4 ? 64 : 224;
    auto kern = kind == 0 ? probe_tcgen05_i8<256> : kind == 3 ? probe_tcgen05_i8<128> : kind == 4 ? probe_tcgen05_i8<64>
                                                                                                   : probe_tcgen05_i8<224, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail(e, "probe smem attribute");
    kern<<<sms, 128, smem, s>>>(iters, scratch_flag);
    *ops_per_launch = (double)sms * iters * 4.0 * 2.0 * 128 * pn * (kind == 5 ? 64 : 32);
  } else if (kind == 1) {
    probe_mma_sync<1><<<sms * 2, 512, 0, s>>>(iters, scratch_flag);
    *ops_per_launch = (double)sms * 2 * 16 * iters * 8.0 * 2.0 * 16 * 8 * 32;
  } else {
    probe_mma_sync<2><<<sms * 2, 512, 0, s>>>(iters, scratch_flag);
    *ops_per_launch = (double)sms * 2 * 16 * iters * 8.0 * 2.0 * 16 * 8 * 256;
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "probe launch");
  return APNN_OK;
}
