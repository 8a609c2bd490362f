// Device-side helpers shared by the kernels: PTX wrappers and the parameter block
// of the plane contraction core.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace apnn {

// Values mirror include/apnn_b200.h.
enum { OUT_INT32 = 0, OUT_LOWBITS = 1, OUT_THRESHOLDS = 2, OUT_FLOAT = 3 };
enum { SIGN_NONE = 0, SIGN_A = 1, SIGN_B = 2 };  // which core operand holds -1/+1 bits
enum { POOL_NONE = 0, POOL_AVG2 = 1, POOL_MAX2 = 2 };

// One problem for the contraction core: out[m][n] = sum_k a(m,k) * b(n,k), where
// a(m,k) = sum_p 2^p Aplane[p][m][k] and likewise b.  GEMM: A = W, B = X.
// Convolution: A = activations gathered per output pixel (implicit im2col),
// B = filter rows (one per output channel), K ordered (tap_i, tap_j, channel).
struct CoreParams {
  const uint32_t* A;
  const uint32_t* B;
  long long a_plane_words;  // words between consecutive bit planes of A
  long long b_plane_words;
  int M;                    // rows of A processed (GEMM rows, conv output pixels, or pooled windows * 4)
  int N;                    // rows of B = output channels
  int kchunks;              // K / 128
  int a_row_words;          // GEMM: K/32
  int b_row_words;          // K/32
  // convolution gather (is_conv != 0)
  int is_conv;
  int Ho, Wo;               // conv output size before pooling
  int Hp, Wp;               // stored input size including halo
  int cin_words;            // CIN / 32
  int cin_chunks;           // CIN / 128
  int R, stride;
  int in_off;               // stored ring width minus (R-1)/2: extra offset of pixel (0,0)
  // epilogue
  void* out;
  const int32_t* thresholds;
  int out_mode, out_bits, sign, pool;
  int out_h, out_w, out_halo;   // conv: output spatial size after pooling, ring width
  long long out_plane_words;    // packed: words between output bit planes
  const int32_t* residual_in;   // optional dense int32 [rows][N] added before requantisation
  int32_t* residual_out;        // optional dense int32 [rows][N]: the value after the add
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy global -> shared; bytes beyond src_bytes are zero-filled.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// D(16x8, s32) += A(16x32, u8) * B(32x8, u8)
__device__ __forceinline__ void mma_u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D(16x8, s32) += popcount(A(16x256, b1) & B(256x8, b1))
__device__ __forceinline__ void mma_b1(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k256.row.col.s32.b1.b1.s32.and.popc {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace apnn
