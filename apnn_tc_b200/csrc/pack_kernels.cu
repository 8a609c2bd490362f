// Layer-boundary packers: one value per element in, bit planes out.
//
// A warp converts 128 consecutive channels of one row per step: every lane fetches four
// elements with one 128-bit load (512 contiguous bytes per warp), builds its 4-bit slice
// of each plane, the eight lanes that share an output word OR their slices together with
// three shuffles, and one lane per word stores it.  Channel c lands in bit 31-(c%32) of
// word c/32, planes outermost, rows padded with zero channels to a multiple of 128.
#include <cstring>

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

// 8 bits: (t * 256) / 20 with t = x + 10 equals rint-for-rint the single product t * 12.8f for every float t
// in [0, 20] -- checked exhaustively over all 1 101 004 801 of them (oracle/check_quantise8.c) -- so the
// division is not needed.
__device__ __forceinline__ uint32_t quantize_level8(float x) {
  x = fminf(fmaxf(x, -10.0f), 10.0f);
  const uint32_t u = __float2uint_rn(__fmul_rn(__fadd_rn(x, 10.0f), 12.8f));
  return u > 255u ? 255u : u;
}

// The quantiser is a non-decreasing function of x (every float operation in it is), so
// level(x) = #{ j : x >= first_x[j] } with first_x[j] the smallest float that reaches level j+1.
// For up to 3 bits the kernels compare against those 2^bits - 1 floats (found once on the host
// by bisection over the float ordering, with the same float arithmetic) instead of dividing.
struct QuantSteps {
  float first_x[7];
  int n;   // 2^bits - 1, or 0: use the arithmetic form
};
template <int NSTEPS>
__device__ __forceinline__ uint32_t quantize_by_steps(float x, const QuantSteps& qs) {
  uint32_t lv = 0;
#pragma unroll
  for (int j = 0; j < NSTEPS; j++) lv += x >= qs.first_x[j] ? 1u : 0u;
  return lv;
}
// Four elements at once -> their levels in the four bytes of a word.
__device__ __forceinline__ uint32_t quantize4_by_steps(const float4& f, const QuantSteps& qs) {
  if (qs.n == 3)
    return quantize_by_steps<3>(f.x, qs) | (quantize_by_steps<3>(f.y, qs) << 8) | (quantize_by_steps<3>(f.z, qs) << 16) |
           (quantize_by_steps<3>(f.w, qs) << 24);
  if (qs.n == 1)
    return quantize_by_steps<1>(f.x, qs) | (quantize_by_steps<1>(f.y, qs) << 8) | (quantize_by_steps<1>(f.z, qs) << 16) |
           (quantize_by_steps<1>(f.w, qs) << 24);
  return quantize_by_steps<7>(f.x, qs) | (quantize_by_steps<7>(f.y, qs) << 8) | (quantize_by_steps<7>(f.z, qs) << 16) |
         (quantize_by_steps<7>(f.w, qs) << 24);
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

// Rows of at most 32 channels (the 3-channel image of a first layer): one thread per row
// builds the single non-zero word of every plane and stores the row's four words at once.
template <bool FROM_FLOAT>
__global__ void __launch_bounds__(256) pack_narrow_rows_kernel(const void* __restrict__ in,
                                                               uint32_t* __restrict__ planes, long long rows, int C,
                                                               int bits) {
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  for (long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x; row < rows;
       row += (long long)gridDim.x * blockDim.x) {
    uint32_t word[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    for (int c = 0; c < C; c++) {
      uint32_t lv;
      if (FROM_FLOAT) lv = quantize_level(__ldg(reinterpret_cast<const float*>(in) + row * C + c), steps, maxlv);
      else lv = __ldg(reinterpret_cast<const uint32_t*>(in) + row * C + c);
#pragma unroll
      for (int b = 0; b < 8; b++) word[b] |= ((lv >> b) & 1u) << (31 - c);
    }
#pragma unroll
    for (int b = 0; b < 8; b++)
      if (b < bits) reinterpret_cast<uint4*>(planes)[(long long)b * rows + row] = make_uint4(word[b], 0u, 0u, 0u);
  }
}

// First-layer re-layout: quantise a float NHWC image and gather every output pixel's R x R x C
// window into channels, k = (i*R + j)*C + c, zero outside the image and beyond R*R*C up to the
// next multiple of 128.  The convolution then becomes a 1x1 convolution over R*R*C "channels"
// instead of one over C padded to 128 (42x less contraction work for a 3-channel image).
// One thread builds one 32-k word of every plane of one output pixel.
__global__ void __launch_bounds__(256) quantize_im2col_kernel(const float* __restrict__ img,
                                                              uint32_t* __restrict__ planes, int B, int H, int W,
                                                              int C, int R, int stride, int bits, int Ho, int Wo,
                                                              int kwords) {
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  const int pad = (R - 1) / 2;
  const int kreal = R * R * C;
  const long long pixels = (long long)B * Ho * Wo;
  const long long total = pixels * kwords;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const long long pix = t / kwords;
    const int w = (int)(t - pix * kwords);
    const int wo = (int)(pix % Wo);
    const long long t2 = pix / Wo;
    const int ho = (int)(t2 % Ho);
    const int b = (int)(t2 / Ho);
    uint32_t word[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    int k = w * 32;
    if (k < kreal) {
      // walk (tap row i, tap column j, channel c) incrementally: two divisions per word, none per element
      int tap = k / C, c = k - tap * C;
      int i = tap / R, j = tap - i * R;
      const int hbase = ho * stride - pad, wbase = wo * stride - pad;
      const float* ib = img + (long long)b * H * W * C;
      for (int e = 0; e < 32 && k < kreal; e++, k++) {
        const int hi = hbase + i, wi = wbase + j;
        if (hi >= 0 && hi < H && wi >= 0 && wi < W) {
          const uint32_t lv = quantize_level(__ldg(ib + ((long long)hi * W + wi) * C + c), steps, maxlv);
#pragma unroll
          for (int p = 0; p < 8; p++) word[p] |= ((lv >> p) & 1u) << (31 - e);
        }
        if (++c == C) {
          c = 0;
          if (++j == R) { j = 0; ++i; }
        }
      }
    }
#pragma unroll
    for (int p = 0; p < 8; p++)
      if (p < bits) planes[(long long)p * total + t] = word[p];
  }
}

template <bool FROM_FLOAT>
apnn_status launch_pack(void* stream, const void* in, uint32_t* planes, long rows, int C, int bits) {
  if (!in || !planes) return APNN_ERR_INVALID_ARG;
  if (rows <= 0 || C <= 0 || bits < 1 || bits > 8) return APNN_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(in) & 15u) || (reinterpret_cast<uintptr_t>(planes) & 15u)) return APNN_ERR_ALIGNMENT;
  long long cap = (long long)device_sm_count() * 8;
  if (C <= 32) {
    long long nb = (rows + 255) / 256;
    if (nb > cap) nb = cap;
    pack_narrow_rows_kernel<FROM_FLOAT><<<(unsigned)nb, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, planes, rows,
                                                                                                        C, bits);
    cudaError_t e0 = cudaGetLastError();
    if (e0 != cudaSuccess) return cuda_fail(e0, "pack_narrow_rows launch");
    return APNN_OK;
  }
  long long tasks = (long long)rows * ((C + 127) / 128);
  long long blocks = (tasks + 7) / 8;
  if (blocks > cap) blocks = cap;
  pack_planes_kernel<FROM_FLOAT><<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, planes, rows,
                                                                                                     C, bits);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pack_planes launch");
  return APNN_OK;
}

}  // namespace
// The same re-layout with each image element quantised once per output row instead of once per
// window it falls in: a CTA owns the output rows (b, ho) it walks; it loads the R input rows
// that row needs with coalesced 16-byte loads, quantises them into shared memory as one byte
// per element (zero bytes for the padding ring), and then every thread assembles 32-k words
// from contiguous runs of R*C bytes.  Output words of one row are contiguous in every plane.
template <int BITS>   // plane count, or 0 to take it from the argument
__global__ void __launch_bounds__(256) quantize_im2col_rows_kernel(const float* __restrict__ img,
                                                                   uint32_t* __restrict__ planes, int B, int H,
                                                                   int W, int C, int R, int stride, int bits,
                                                                   int Ho, int Wo, int kwords, int rowlen) {
  extern __shared__ __align__(16) unsigned char lv_s[];   // [R][rowlen]
  if (BITS) bits = BITS;
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  const int pad = (R - 1) / 2;
  const int kreal = R * R * C, tapw = R * C, wc = W * C;
  const long long plane_words = (long long)B * Ho * Wo * kwords;
  const bool vec = (wc & 3) == 0;
  for (int orow = blockIdx.x; orow < B * Ho; orow += gridDim.x) {
    const int b = orow / Ho, ho = orow - b * Ho;
    const int hbase = ho * stride - pad;
    __syncthreads();   // the previous row's readers are done
    // zero the left / right padding bytes of every staged row
    for (int t = threadIdx.x; t < R * 2 * pad * C; t += blockDim.x) {
      const int i = t / (2 * pad * C), o = t - i * (2 * pad * C);
      lv_s[i * rowlen + (o < pad * C ? o : wc + o)] = 0;
    }
    for (int i = 0; i < R; i++) {
      const int hi = hbase + i;
      unsigned char* dst = lv_s + i * rowlen + pad * C;
      if (hi < 0 || hi >= H) {
        for (int t = threadIdx.x; t < wc; t += blockDim.x) dst[t] = 0;
      } else {
        const float* src = img + ((long long)b * H + hi) * wc;
        if (vec) {
          for (int t = threadIdx.x; t < wc / 4; t += blockDim.x) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(src) + t);
            dst[4 * t] = (unsigned char)quantize_level(f.x, steps, maxlv);
            dst[4 * t + 1] = (unsigned char)quantize_level(f.y, steps, maxlv);
            dst[4 * t + 2] = (unsigned char)quantize_level(f.z, steps, maxlv);
            dst[4 * t + 3] = (unsigned char)quantize_level(f.w, steps, maxlv);
          }
        } else {
          for (int t = threadIdx.x; t < wc; t += blockDim.x)
            dst[t] = (unsigned char)quantize_level(__ldg(src + t), steps, maxlv);
        }
      }
    }
    __syncthreads();
    const long long out0 = (long long)orow * Wo * kwords;
    for (int t = threadIdx.x; t < Wo * kwords; t += blockDim.x) {
      const int wo = t / kwords, w = t - wo * kwords;
      uint32_t word[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      int k = w * 32;
      if (k < kreal) {
        int i = k / tapw, off = k - i * tapw;
        const unsigned char* rowp = lv_s + i * rowlen + wo * stride * C;
        for (int e = 0; e < 32 && k < kreal; e++, k++) {
          const uint32_t lv = rowp[off];
#pragma unroll
          for (int pl = 0; pl < 8; pl++)
            if (pl < bits) word[pl] |= ((lv >> pl) & 1u) << (31 - e);
          if (++off == tapw) { off = 0; rowp += rowlen; }
        }
      }
#pragma unroll
      for (int pl = 0; pl < 8; pl++)
        if (pl < bits) planes[(long long)pl * plane_words + out0 + t] = word[pl];
    }
  }
}


// First layer straight to the int8 operand of the tcgen05 path: the same window gather as
// quantize_im2col_rows_kernel, but every output pixel becomes a row of kp bytes, one level per
// byte in the byte order apnn_expand_planes produces (within each group of 32 k, element e sits
// at byte 4*((31-e)&7) + ((31-e)>>3)), zero beyond R*R*C.  No packed planes, no expand pass.
__global__ void __launch_bounds__(256) quantize_im2col_i8_kernel(const float* __restrict__ img,
                                                                 uint8_t* __restrict__ out, int B, int H, int W,
                                                                 int C, int R, int stride, int bits, int Ho, int Wo,
                                                                 int kp, int rowlen, int lpad, uint32_t xormask) {
  // xormask: 0, or 0x80808080 for the centred 8-bit form (level - 128 as a signed byte) -- applied to
  // elements inside the image only, so that padding stays the byte 0
  extern __shared__ __align__(16) unsigned char lv_s[];   // [R][rowlen], image columns start at byte lpad
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  const int pad = (R - 1) / 2;
  const int kreal = R * R * C, tapw = R * C, wc = W * C;
  const int groups = kp / 32;
  const bool vec = (wc & 3) == 0;
  const int quads = wc >> 2;
  for (int orow = blockIdx.x; orow < B * Ho; orow += gridDim.x) {
    const int b = orow / Ho, ho = orow - b * Ho;
    const int hbase = ho * stride - pad;
    __syncthreads();   // the previous row's readers are done
    // padding bytes left and right of the image columns
    for (int t = threadIdx.x; t < R * (rowlen - wc); t += blockDim.x) {
      const int i = t / (rowlen - wc), o = t - i * (rowlen - wc);
      lv_s[i * rowlen + (o < lpad ? o : wc + o)] = 0;
    }
    if (vec) {
      // all R rows in one flat loop: every thread's loads are independent and in flight together
      for (int t = threadIdx.x; t < R * quads; t += blockDim.x) {
        const int i = t / quads, q = t - i * quads;
        const int hi = hbase + i;
        uint32_t packed = 0u;
        if (hi >= 0 && hi < H) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(img + ((long long)b * H + hi) * wc) + q);
          packed = (quantize_level(f.x, steps, maxlv) | (quantize_level(f.y, steps, maxlv) << 8) |
                    (quantize_level(f.z, steps, maxlv) << 16) | (quantize_level(f.w, steps, maxlv) << 24)) ^ xormask;
        }
        *reinterpret_cast<uint32_t*>(lv_s + i * rowlen + lpad + 4 * q) = packed;
      }
    } else {
      for (int t = threadIdx.x; t < R * wc; t += blockDim.x) {
        const int i = t / wc, q = t - i * wc;
        const int hi = hbase + i;
        lv_s[i * rowlen + lpad + q] =
            (hi >= 0 && hi < H) ? (unsigned char)(quantize_level(__ldg(img + ((long long)b * H + hi) * wc + q), steps, maxlv) ^ (xormask & 0xffu)) : 0;
      }
    }
    __syncthreads();
    uint8_t* orow_out = out + (long long)orow * Wo * kp;
    for (int t = threadIdx.x; t < Wo * groups; t += blockDim.x) {
      const int wo = t / groups, w = t - wo * groups;
      uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      int k = w * 32;
      if (k < kreal) {
        int i = k / tapw, off = k - i * tapw;
        const unsigned char* rowp = lv_s + i * rowlen + (lpad - pad * C) + wo * stride * C;
#pragma unroll
        for (int e = 0; e < 32; e++) {
          if (k + e < kreal) {
            r[(31 - e) & 7] |= (uint32_t)rowp[off] << (8 * ((31 - e) >> 3));
            if (++off == tapw) { off = 0; rowp += rowlen; }
          }
        }
      }
      asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(orow_out + (long long)t * 32), "r"(r[0]),
                   "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                   : "memory");
    }
  }
}

// The same gather when one pass of the block covers an output row (Wo * kp/32 <= blockDim.x):
// a thread keeps its (pixel, 32-byte group) for the whole kernel, so the 32 shared-memory
// offsets of its elements are computed once and the per-row work is 32 byte loads, 32
// shift-ORs and one 32-byte store, with no index arithmetic or branches.
template <int TPT, int NQ>   // 32-byte groups per thread; 16-byte input quads per thread and row
__global__ void __launch_bounds__(512) quantize_im2col_i8_fixed_kernel(const float* __restrict__ img,
                                                                       uint8_t* __restrict__ out, int B, int H, int W,
                                                                       int C, int R, int stride, int bits, int Ho,
                                                                       int Wo, int kp, int rowlen, int lpad,
                                                                       const QuantSteps qs) {
  extern __shared__ __align__(16) unsigned char lv_s[];   // [R][rowlen], image columns start at byte lpad
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  const int pad = (R - 1) / 2;
  const int kreal = R * R * C, tapw = R * C, wc = W * C;
  const int groups = kp / 32;
  const int quads = wc >> 2;
  const int T = blockDim.x;
  // this thread's tasks (task = threadIdx.x + j * blockDim.x) and the offsets of their 32 elements,
  // two 16-bit offsets per register (byte 0 of the buffer, always padding, for k >= R*R*C)
  uint32_t src[TPT][16];
#pragma unroll
  for (int j = 0; j < TPT; j++) {
    const int task = threadIdx.x + j * T;
    const bool worker = task < Wo * groups;
    const int wo = task / groups, w = task - wo * groups;
    int k = w * 32;
    int i = k / tapw, off = k - i * tapw;
#pragma unroll
    for (int e = 0; e < 32; e++) {
      const uint32_t o = (worker && k + e < kreal) ? (uint32_t)(i * rowlen + (lpad - pad * C) + wo * stride * C + off) : 0u;
      if (e & 1) src[j][e >> 1] |= o << 16;
      else src[j][e >> 1] = o;
      if (++off == tapw) { off = 0; i++; }
    }
  }
  for (int t = threadIdx.x; t < R * (rowlen - wc); t += T) {
    const int i = t / (rowlen - wc), o = t - i * (rowlen - wc);
    lv_s[i * rowlen + (o < lpad ? o : wc + o)] = 0;
  }
  // the R input rows of an output row pass through registers: fetched while the previous row
  // is assembled, quantised into shared memory afterwards (R * W*C/4 <= NQ * blockDim.x)
  float4 nxt[NQ];
  // which input element quad each of this thread's slots carries: fixed for the kernel
  int tap_row[NQ], img_off[NQ], smem_off[NQ];
#pragma unroll
  for (int u = 0; u < NQ; u++) {
    const int t = threadIdx.x + u * T;
    const int i = t / quads, q = t - i * quads;
    tap_row[u] = t < R * quads ? i : -1000000;      // never inside the image
    img_off[u] = i * wc + 4 * q;
    smem_off[u] = i * rowlen + lpad + 4 * q;
  }
  auto fetch = [&](int orow) {
    const int b = orow / Ho, ho = orow - b * Ho;
    const int hbase = ho * stride - pad;
    const float* first = img + ((long long)b * H + hbase) * wc;
#pragma unroll
    for (int u = 0; u < NQ; u++) {
      const int hi = hbase + tap_row[u];
      nxt[u] = make_float4(-100.f, -100.f, -100.f, -100.f);   // clips to level 0: rows outside the image
      if (hi >= 0 && hi < H) nxt[u] = __ldg(reinterpret_cast<const float4*>(first + img_off[u]));
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int u = 0; u < NQ; u++) {
      if (tap_row[u] >= 0) {
        const float4 f = nxt[u];
        uint32_t packed;
        if (qs.n)
          packed = quantize4_by_steps(f, qs);
        else
          packed = quantize_level(f.x, steps, maxlv) | (quantize_level(f.y, steps, maxlv) << 8) |
                   (quantize_level(f.z, steps, maxlv) << 16) | (quantize_level(f.w, steps, maxlv) << 24);
        *reinterpret_cast<uint32_t*>(lv_s + smem_off[u]) = packed;
      }
    }
  };
  int orow = blockIdx.x;
  if (orow < B * Ho) fetch(orow);
  for (; orow < B * Ho; orow += gridDim.x) {
    __syncthreads();   // the previous row's readers are done
    stash();
    __syncthreads();
    if (orow + (int)gridDim.x < B * Ho) fetch(orow + gridDim.x);
#pragma unroll
    for (int j = 0; j < TPT; j++) {
      const int task = threadIdx.x + j * T;
      if (task < Wo * groups) {
        uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
        for (int e = 0; e < 32; e++) {
          const uint32_t o = (e & 1) ? (src[j][e >> 1] >> 16) : (src[j][e >> 1] & 0xffffu);
          r[(31 - e) & 7] |= (uint32_t)lv_s[o] << (8 * ((31 - e) >> 3));
        }
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(out + ((long long)orow * Wo * groups + task) * 32),
                     "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                     : "memory");
      }
    }
  }
}

// First layer as whole words: an output pixel's row is R segments of `seg` bytes (R*C rounded up
// to a multiple of 4), segment i holding the R*C levels of filter row i in their order along the
// staged image row, then zeros.  A thread owns TPT 16-byte pieces of the output row for the
// whole kernel: four 32-bit words, each two aligned shared-memory words funnel-shifted by the
// window's byte offset (the last word of a segment masked to its real bytes), then one 16-byte
// store.  Against the byte-wise gather above this is about 16 instead of 50 instructions per
// 16 output bytes; the quantise phase is the same.
// G consecutive output rows of an image share one pass: they need R + (G-1)*stride input rows
// instead of G*R, so every image element is quantised fewer times (7x7 stride 4, G = 3: 5 rows
// per output row instead of 7; 11x11 stride 4: 6.3 instead of 11).
template <int TPT, int NQ, int G>
__global__ void __launch_bounds__(512) quantize_window_rows_i8_kernel(const float* __restrict__ img,
                                                                      uint8_t* __restrict__ out, int B, int H, int W,
                                                                      int C, int R, int stride, int bits, int Ho,
                                                                      int Wo, int kp, int seg, int rowlen, int lpad,
                                                                      const QuantSteps qs, uint32_t xormask,
                                                                      float outside) {
  // xormask: 0, or 0x80808080 for the centred 8-bit form (level - 128 as a signed byte).  outside: the value
  // rows outside the image are read as -- one that quantises to the byte 0 after the xor: -100 (level 0), or
  // 0.0 in the centred form (level 128)
  extern __shared__ __align__(16) unsigned char lv_s[];   // [R + (G-1)*stride][rowlen], image columns start at byte lpad >= 8
  const uint32_t* lv32 = reinterpret_cast<const uint32_t*>(lv_s);
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  const int pad = (R - 1) / 2;
  const int wc = W * C;
  const int pieces = kp / 16, segw = seg / 4;
  const int quads = wc >> 2;
  const int T = blockDim.x;
  const int rows_in = R + (G - 1) * stride;           // staged input rows per pass
  const int groups_per_image = (Ho + G - 1) / G;
  const int ngroups = B * groups_per_image;
  const uint32_t lastmask = 0xffffffffu >> (8 * (seg - R * C));   // the real bytes of a segment's last word
  // word indices of a piece's four words, 16 bits each (0: the zero words at the start of the
  // buffer, for k beyond the R segments), and the funnel shift of its pixel
  uint32_t idx01[TPT], idx23[TPT], shift[TPT];
#pragma unroll
  for (int j = 0; j < TPT; j++) {
    const int task = threadIdx.x + j * T;
    const bool worker = task < Wo * pieces;
    const int wo = task / pieces, c = task - wo * pieces;
    const int a0 = lpad - pad * C + wo * stride * C;   // byte of the window's first element in a staged row
    shift[j] = worker ? 8u * (uint32_t)(a0 & 3) : 0u;   // bits 8..11: word u is the last of its segment
    uint32_t w4[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int wd = 4 * c + u, i = wd / segw, t = wd - i * segw;
      w4[u] = (worker && i < R) ? (uint32_t)((i * rowlen + (a0 & ~3)) / 4 + t) : 0u;
      if (t == segw - 1) shift[j] |= 256u << u;
    }
    idx01[j] = w4[0] | (w4[1] << 16);
    idx23[j] = w4[2] | (w4[3] << 16);
  }
  for (int t = threadIdx.x; t < rows_in * (rowlen - wc); t += T) {
    const int i = t / (rowlen - wc), o = t - i * (rowlen - wc);
    lv_s[i * rowlen + (o < lpad ? o : wc + o)] = 0;
  }
  float4 nxt[NQ];
  int tap_row[NQ], img_off[NQ], smem_off[NQ];
#pragma unroll
  for (int u = 0; u < NQ; u++) {
    const int t = threadIdx.x + u * T;
    const int i = t / quads, q = t - i * quads;
    tap_row[u] = t < rows_in * quads ? i : -1000000;      // never inside the image
    img_off[u] = i * wc + 4 * q;
    smem_off[u] = i * rowlen + lpad + 4 * q;
  }
  auto fetch = [&](int group) {
    const int b = group / groups_per_image, ho = (group - b * groups_per_image) * G;
    const int hbase = ho * stride - pad;
    const float* first = img + ((long long)b * H + hbase) * wc;
#pragma unroll
    for (int u = 0; u < NQ; u++) {
      const int hi = hbase + tap_row[u];
      nxt[u] = make_float4(outside, outside, outside, outside);   // rows outside the image: the byte 0
      if (hi >= 0 && hi < H) nxt[u] = __ldg(reinterpret_cast<const float4*>(first + img_off[u]));
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int u = 0; u < NQ; u++) {
      if (tap_row[u] >= 0) {
        const float4 f = nxt[u];
        uint32_t packed;
        if (qs.n)
          packed = quantize4_by_steps(f, qs);
        else if (bits == 8)
          packed = quantize_level8(f.x) | (quantize_level8(f.y) << 8) | (quantize_level8(f.z) << 16) |
                   (quantize_level8(f.w) << 24);
        else
          packed = quantize_level(f.x, steps, maxlv) | (quantize_level(f.y, steps, maxlv) << 8) |
                   (quantize_level(f.z, steps, maxlv) << 16) | (quantize_level(f.w, steps, maxlv) << 24);
        *reinterpret_cast<uint32_t*>(lv_s + smem_off[u]) = packed ^ xormask;
      }
    }
  };
  int group = blockIdx.x;
  if (group < ngroups) fetch(group);
  for (; group < ngroups; group += gridDim.x) {
    __syncthreads();   // the previous pass's readers are done
    stash();
    __syncthreads();
    if (group + (int)gridDim.x < ngroups) fetch(group + gridDim.x);
    const int b = group / groups_per_image, ho0 = (group - b * groups_per_image) * G;
#pragma unroll
    for (int g = 0; g < G; g++) {
      if (ho0 + g >= Ho) break;
      // output row ho0 + g reads the staged rows from g*stride on; word 0 of every staged row is padding
      const uint32_t* rows32 = lv32 + g * stride * (rowlen >> 2);
      uint4* orow_out = reinterpret_cast<uint4*>(out + ((long long)b * Ho + ho0 + g) * Wo * kp);
#pragma unroll
      for (int j = 0; j < TPT; j++) {
        const int task = threadIdx.x + j * T;
        if (task < Wo * pieces) {
          const uint32_t i0 = idx01[j] & 0xffffu, i1 = idx01[j] >> 16, i2 = idx23[j] & 0xffffu, i3 = idx23[j] >> 16;
          uint4 v;
          v.x = __funnelshift_r(rows32[i0], rows32[i0 + 1], shift[j]) & ((shift[j] & 0x100u) ? lastmask : 0xffffffffu);
          v.y = __funnelshift_r(rows32[i1], rows32[i1 + 1], shift[j]) & ((shift[j] & 0x200u) ? lastmask : 0xffffffffu);
          v.z = __funnelshift_r(rows32[i2], rows32[i2 + 1], shift[j]) & ((shift[j] & 0x400u) ? lastmask : 0xffffffffu);
          v.w = __funnelshift_r(rows32[i3], rows32[i3 + 1], shift[j]) & ((shift[j] & 0x800u) ? lastmask : 0xffffffffu);
          orow_out[task] = v;
        }
      }
    }
  }
}

// Host restatement of quantize_level with the same IEEE single-precision operations.
static uint32_t quantize_level_host(float x, int bits) {
  volatile float a = x < -10.0f ? -10.0f : (x > 10.0f ? 10.0f : x);   // NaN never reaches here
  volatile float s1 = a + 10.0f;
  volatile float s2 = s1 * (float)(1 << bits);
  volatile float q = s2 / 20.0f;
  const uint32_t u = (uint32_t)nearbyintf(q);   // round to nearest even, as __float2uint_rn
  const uint32_t maxlv = (1u << bits) - 1u;
  return u > maxlv ? maxlv : u;
}
static QuantSteps make_quant_steps(int bits) {
  static QuantSteps cache[4];   // per bit width; a race would only recompute the same values
  if (bits <= 3 && cache[bits].n) return cache[bits];
  QuantSteps qs;
  memset(&qs, 0, sizeof(qs));
  if (bits > 3) return qs;
  qs.n = (1 << bits) - 1;
  for (int j = 0; j < qs.n; j++) {
    // bisection over the ordered floats of [-10, 10]: smallest x with level >= j + 1
    float lo = -10.0f, hi = 10.0f;   // level(lo) = 0 < j + 1 <= level(hi) = 2^bits - 1
    while (nextafterf(lo, hi) < hi) {
      const float mid = lo + (hi - lo) * 0.5f;
      const float m = (mid <= lo) ? nextafterf(lo, hi) : (mid >= hi ? nextafterf(hi, lo) : mid);
      if (quantize_level_host(m, bits) >= (uint32_t)(j + 1)) hi = m;
      else lo = m;
    }
    qs.first_x[j] = hi;
  }
  cache[bits] = qs;
  return qs;
}

// 2x2 maximum over int8 NHWC rows: a thread owns 16 channels of one output pixel.
__global__ void __launch_bounds__(256) maxpool2x2_i8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                                            int B, int Ho, int Wo, int C, int ih, int oh) {
  const int cv = C >> 4;   // 16-byte vectors per pixel
  const long long total = (long long)B * Ho * Wo * cv;
  const int Wi = 2 * Wo + 2 * ih, Hi = 2 * Ho + 2 * ih, Wq = Wo + 2 * oh, Hq = Ho + 2 * oh;
  asm volatile("griddepcontrol.wait;" ::: "memory");   // launched as a programmatic dependent of the producing layer
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(t % cv);
    long long pix = t / cv;
    const int wo = (int)(pix % Wo);
    pix /= Wo;
    const int ho = (int)(pix % Ho);
    const int b = (int)(pix / Ho);
    const uint4* src = reinterpret_cast<const uint4*>(in + (((long long)b * Hi + 2 * ho + ih) * Wi + 2 * wo + ih) * C) + v;
    const uint4 a = __ldg(src), c = __ldg(src + cv);
    const uint4 d = __ldg(src + (long long)Wi * cv), e = __ldg(src + (long long)Wi * cv + cv);
    uint4 m;
    m.x = __vmaxu4(__vmaxu4(a.x, c.x), __vmaxu4(d.x, e.x));
    m.y = __vmaxu4(__vmaxu4(a.y, c.y), __vmaxu4(d.y, e.y));
    m.z = __vmaxu4(__vmaxu4(a.z, c.z), __vmaxu4(d.z, e.z));
    m.w = __vmaxu4(__vmaxu4(a.w, c.w), __vmaxu4(d.w, e.w));
    reinterpret_cast<uint4*>(out + (((long long)b * Hq + ho + oh) * Wq + wo + oh) * C)[v] = m;
  }
}

// First layer with a stride: the image regrouped into stride x stride pixel blocks ("space to depth").  Block
// (hb, wb) of image b becomes one pixel of cpad bytes, byte (di*stride + dj)*C + c = level of pixel
// (stride*hb + di, stride*wb + dj), channel c; bytes from stride*stride*C on are 0.  The strided RxR convolution of
// the image is then a stride-1 convolution with 2*ceil(pad/stride)+1 taps a side over these pixels (taps the filter
// does not reach carry weight 0), which the flat tcgen05 convolution runs like any other layer -- and the quantised
// image is written once (cpad bytes per block) instead of once per window (R*R*C bytes per output pixel).
// A thread owns 16 bytes of a block (one aligned store; a warp writes 512 contiguous bytes): four groups of four
// bytes, each group four consecutive floats of one image row because stride*C is a multiple of 4.
__global__ void __launch_bounds__(256) quantize_blocks_i8_kernel(const float* __restrict__ img, uint8_t* __restrict__ out,
                                                                 int B, int H, int W, int C, int stride, int bits,
                                                                 int halo, int cpad, const QuantSteps qs, uint32_t xormask) {
  const int Hb = H / stride, Wb = W / stride;
  const int seg = stride * C;                 // floats (and bytes) of a block row; a multiple of 4
  const int used = stride * seg;              // bytes of a block that hold levels
  const int chunks = cpad >> 4;
  const float steps = (float)(1 << bits);
  const uint32_t maxlv = (1u << bits) - 1u;
  const long long row_pitch = (long long)(Wb + 2 * halo) * cpad;
  // one row of blocks per (blockIdx.y, blockIdx.z) = (hb, b): no 64-bit index arithmetic per thread
  const int hb = (int)blockIdx.y, b = (int)blockIdx.z;
  for (int t = (int)(blockIdx.x * blockDim.x + threadIdx.x); t < Wb * chunks; t += (int)(gridDim.x * blockDim.x)) {
    const int wb = t / chunks, j = t - wb * chunks;
    const float* blk = img + (((long long)b * H + (long long)hb * stride) * W + (long long)wb * stride) * C;
    uint32_t w4[4];
#pragma unroll
    for (int g = 0; g < 4; g++) {
      const int k = 16 * j + 4 * g;   // first byte of the group inside the block
      w4[g] = 0u;
      if (k < used) {
        const int row = k / seg, off = k - row * seg;
        const float4 f = __ldg(reinterpret_cast<const float4*>(blk + (long long)row * W * C + off));
        uint32_t packed;
        if (qs.n)
          packed = quantize4_by_steps(f, qs);
        else if (bits == 8)
          packed = quantize_level8(f.x) | (quantize_level8(f.y) << 8) | (quantize_level8(f.z) << 16) | (quantize_level8(f.w) << 24);
        else
          packed = quantize_level(f.x, steps, maxlv) | (quantize_level(f.y, steps, maxlv) << 8) |
                   (quantize_level(f.z, steps, maxlv) << 16) | (quantize_level(f.w, steps, maxlv) << 24);
        w4[g] = packed ^ xormask;
      }
    }
    uint8_t* dst = out + ((long long)b * (Hb + 2 * halo) + hb + halo) * row_pitch + (long long)(wb + halo) * cpad + 16 * j;
    *reinterpret_cast<uint4*>(dst) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
}

// int32 values [rows][N] -> levels (low bits, or count of per-channel thresholds reached) ->
// packed planes [bits][rows][N/32] or int8 rows [rows][N] in the operand byte order.
// A warp owns one 32-column group and walks rows: a lane keeps its column's thresholds in
// registers, loads are 128 contiguous bytes per row, planes are packed by ballot.
__global__ void __launch_bounds__(256) requantize_i32_kernel(const int32_t* __restrict__ acc, void* __restrict__ out,
                                                             long long rows, int N, int out_mode, int out_bits,
                                                             const int32_t* __restrict__ thresholds, int out_i8,
                                                             const float* __restrict__ affine_scale,
                                                             const float* __restrict__ affine_bias) {
  const int groups = N >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t nl = (1u << out_bits) - 1u;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int row_lanes = warps / groups > 0 ? warps / groups : 1;   // warps that share a column group, striding rows
  const int pos = 4 * ((31 - lane) & 7) + ((31 - lane) >> 3);      // byte of element `lane` in the operand order
  const int g = warp % groups, r0 = warp / groups;
  if (r0 >= row_lanes) return;   // surplus warps of the last block (the whole warp leaves together)
  asm volatile("griddepcontrol.wait;" ::: "memory");   // launched as a programmatic dependent of the producing GEMM
  {
    int32_t thr[7];
#pragma unroll
    for (int k = 0; k < 7; k++)
      thr[k] = (out_mode == APNN_OUT_THRESHOLDS && (uint32_t)k < nl && nl <= 7) ? __ldg(thresholds + (long long)(g * 32 + lane) * nl + k)
                                                                               : 0x7fffffff;
    // four rows per trip, their loads issued together: a trip is one dependent load -> compare -> store chain, and
    // with one row in flight per warp the kernel ran at a fifth of the memory rate
    constexpr int U = 4;
    if (out_mode == APNN_OUT_FLOAT) {
      // the output layer's affine: float(value) * scale[c] + bias[c], multiply and add rounded separately
      const float sc = __ldg(affine_scale + g * 32 + lane), bi = __ldg(affine_bias + g * 32 + lane);
      for (long long row = r0; row < rows; row += (long long)U * row_lanes) {
        int x[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const long long rr = row + (long long)u * row_lanes;
          x[u] = rr < rows ? __ldg(acc + rr * N + g * 32 + lane) : 0;
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          const long long rr = row + (long long)u * row_lanes;
          if (rr < rows) reinterpret_cast<float*>(out)[rr * N + g * 32 + lane] = __fadd_rn(__fmul_rn((float)x[u], sc), bi);
        }
      }
      return;
    }
    for (long long row = r0; row < rows; row += (long long)U * row_lanes) {
      int xs[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const long long rr = row + (long long)u * row_lanes;
        xs[u] = rr < rows ? __ldg(acc + rr * N + g * 32 + lane) : 0;
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const long long rr = row + (long long)u * row_lanes;
        if (rr >= rows) break;   // uniform over the warp
        const int x = xs[u];
        uint32_t lv;
        if (out_mode != APNN_OUT_THRESHOLDS) {
          lv = (uint32_t)x & nl;
        } else if (nl <= 7) {
          lv = 0;
#pragma unroll
          for (int k = 0; k < 7; k++) lv += x >= thr[k] ? 1u : 0u;
        } else {
          lv = 0;
          const int32_t* T = thresholds + (long long)(g * 32 + lane) * nl;
          for (uint32_t k = 0; k < nl; k++) lv += x >= __ldg(T + k) ? 1u : 0u;
        }
        if (out_i8) {
          reinterpret_cast<uint8_t*>(out)[rr * N + g * 32 + pos] = (uint8_t)lv;
        } else {
          for (int b = 0; b < out_bits; b++) {
            const uint32_t word = __brev(__ballot_sync(0xffffffffu, (lv >> b) & 1u));
            if (lane == 0) reinterpret_cast<uint32_t*>(out)[(long long)b * rows * groups + rr * groups + g] = word;
          }
        }
      }
    }
  }
}

}  // namespace apnn

extern "C" {

apnn_status apnn_bit_compress(void* stream, const uint32_t* levels, uint32_t* planes, long rows, int C, int bits) {
  return apnn::launch_pack<false>(stream, levels, planes, rows, C, bits);
}

apnn_status apnn_quantize_pack(void* stream, const float* values, uint32_t* planes, long rows, int C, int bits) {
  return apnn::launch_pack<true>(stream, values, planes, rows, C, bits);
}

apnn_status apnn_quantize_im2col(void* stream, const float* images, uint32_t* planes, int B, int H, int W, int C,
                                 int R, int stride, int bits) {
  using namespace apnn;
  if (!images || !planes) return APNN_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || bits < 1 || bits > 8) return APNN_ERR_INVALID_ARG;
  if (R < 1 || R > 11 || (R & 1) == 0 || stride < 1 || stride > 4) return APNN_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(images) & 15u) || (reinterpret_cast<uintptr_t>(planes) & 15u)) return APNN_ERR_ALIGNMENT;
  const int Ho = (H - 1) / stride + 1, Wo = (W - 1) / stride + 1;
  const int kwords = (R * R * C + 127) / 128 * 4;
  const long long total = (long long)B * Ho * Wo * kwords;
  const int pad = (R - 1) / 2;
  const int rowlen = ((W + 2 * pad) * C + 15) / 16 * 16;
  const size_t smem = (size_t)R * rowlen;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (smem <= 48 * 1024) {
    // one CTA per output row, as many resident rows as the device holds at once
    long long nb = (long long)B * Ho, cap = (long long)device_sm_count() * 8;
    if (nb > cap) nb = cap;
    auto kern = bits == 1 ? quantize_im2col_rows_kernel<1> : bits == 2 ? quantize_im2col_rows_kernel<2>
              : bits == 3 ? quantize_im2col_rows_kernel<3> : bits == 4 ? quantize_im2col_rows_kernel<4>
                                                           : quantize_im2col_rows_kernel<0>;
    kern<<<(unsigned)nb, 256, smem, s>>>(images, planes, B, H, W, C, R, stride, bits, Ho, Wo, kwords, rowlen);
  } else {
    long long nb = (total + 255) / 256, cap = (long long)device_sm_count() * 16;
    if (nb > cap) nb = cap;
    quantize_im2col_kernel<<<(unsigned)nb, 256, 0, s>>>(images, planes, B, H, W, C, R, stride, bits, Ho, Wo, kwords);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "quantize_im2col launch");
  return APNN_OK;
}

apnn_status apnn_quantize_im2col_i8(void* stream, const float* images, void* out_i8, int B, int H, int W, int C,
                                    int R, int stride, int bits, int kp) {
  using namespace apnn;
  if (!images || !out_i8) return APNN_ERR_INVALID_ARG;
  const bool centred = (bits & APNN_QUANT_CENTRED) != 0;
  bits &= ~APNN_QUANT_CENTRED;
  if (centred && bits != 8) return APNN_ERR_INVALID_ARG;
  const uint32_t xormask = centred ? 0x80808080u : 0u;
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || bits < 1 || bits > 8) return APNN_ERR_INVALID_ARG;
  if (R < 1 || R > 11 || (R & 1) == 0 || stride < 1 || stride > 4) return APNN_ERR_UNSUPPORTED;
  if (kp < R * R * C || kp % 64 != 0) return APNN_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(images) & 15u) || (reinterpret_cast<uintptr_t>(out_i8) & 31u)) return APNN_ERR_ALIGNMENT;
  const int Ho = (H - 1) / stride + 1, Wo = (W - 1) / stride + 1;
  const int pad = (R - 1) / 2;
  const int lpad = pad * C < 4 ? 4 : (pad * C + 3) / 4 * 4;   // image columns start on a 4-byte boundary; byte 0 is always padding
  const int rowlen = (lpad + W * C + pad * C + 15) / 16 * 16;
  const size_t smem = (size_t)R * rowlen;
  if (smem > 48 * 1024) return APNN_ERR_UNSUPPORTED;   // rows of this width: use apnn_quantize_im2col + apnn_expand_planes
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int tasks = Wo * (kp / 32), wc = W * C;
  const int tpt = tasks <= 512 ? 1 : 2;
  const int per_thread = (tasks + tpt - 1) / tpt;
  const int threads = per_thread < 128 ? 128 : (per_thread + 31) / 32 * 32;
  const int quads_per_row = R * (wc >> 2);
  const int nq = quads_per_row <= 4 * threads ? 4 : 8;
  // two tasks per thread or eight quads per thread measured slower than the generic kernel (register
  // pressure halves the resident blocks): the fixed-task kernel takes rows of at most 512 groups
  if (!centred && (wc & 3) == 0 && tasks <= 512 && nq == 4 && (size_t)R * rowlen < 65536) {
    long long nb = (long long)B * Ho, cap = (long long)device_sm_count() * (2048 / threads);
    if (nb > cap) nb = cap;
    auto kern = tpt == 1 ? (nq == 4 ? quantize_im2col_i8_fixed_kernel<1, 4> : quantize_im2col_i8_fixed_kernel<1, 8>)
                         : (nq == 4 ? quantize_im2col_i8_fixed_kernel<2, 4> : quantize_im2col_i8_fixed_kernel<2, 8>);
    kern<<<(unsigned)nb, threads, smem, st>>>(images, reinterpret_cast<uint8_t*>(out_i8), B, H, W, C, R, stride, bits, Ho, Wo,
                                              kp, rowlen, lpad, make_quant_steps(bits));
  } else {
    long long nb = (long long)B * Ho, cap = (long long)device_sm_count() * 8;
    if (nb > cap) nb = cap;
    quantize_im2col_i8_kernel<<<(unsigned)nb, 256, smem, st>>>(images, reinterpret_cast<uint8_t*>(out_i8), B, H, W, C, R,
                                                              stride, bits, Ho, Wo, kp, rowlen, lpad, xormask);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "quantize_im2col_i8 launch");
  return APNN_OK;
}

apnn_status apnn_quantize_window_rows_i8(void* stream, const float* images, void* out_i8, int B, int H, int W, int C,
                                         int R, int stride, int bits, int kp) {
  using namespace apnn;
  if (!images || !out_i8) return APNN_ERR_INVALID_ARG;
  const bool centred = (bits & APNN_QUANT_CENTRED) != 0;
  bits &= ~APNN_QUANT_CENTRED;
  if (centred && bits != 8) return APNN_ERR_INVALID_ARG;
  const uint32_t xormask = centred ? 0x80808080u : 0u;
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || bits < 1 || bits > 8) return APNN_ERR_INVALID_ARG;
  if (R < 1 || R > 11 || (R & 1) == 0 || stride < 1 || stride > 4) return APNN_ERR_UNSUPPORTED;
  const int seg = (R * C + 3) / 4 * 4;
  if (kp < R * seg || kp % 64 != 0) return APNN_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(images) & 15u) || (reinterpret_cast<uintptr_t>(out_i8) & 15u)) return APNN_ERR_ALIGNMENT;
  const int Ho = (H - 1) / stride + 1, Wo = (W - 1) / stride + 1;
  const int pad = (R - 1) / 2, wc = W * C;
  const int lpad = pad * C < 8 ? 8 : (pad * C + 3) / 4 * 4;   // words 0 and 1 of the buffer are always zero
  const int rowlen = (lpad + wc + pad * C + 8 + 15) / 16 * 16;
  const int tasks = Wo * (kp / 16);
  const int tpt = tasks <= 512 ? 1 : (tasks <= 1024 ? 2 : 4);
  int threads = ((tasks + tpt - 1) / tpt + 31) / 32 * 32;
  if (threads < 128) threads = 128;
  // Output rows per pass: G rows stage R + (G-1)*stride input rows.  Four quads per thread keep
  // two blocks resident per SM (64 registers); eight quads (about 120 registers, one block) pay
  // only where sharing saves at least 40 % of the quantisation (11x11 filters).
  const int quads = wc >> 2;
  auto threads_for = [&](int g, int per_thread) { return (((R + (g - 1) * stride) * quads + per_thread - 1) / per_thread + 31) / 32 * 32; };
  auto fits = [&](int g) { return (size_t)(R + (g - 1) * stride) * rowlen <= 48 * 1024 && Ho >= g; };
  int G = 1, nq = 4;
  if (fits(3) && threads_for(3, 4) <= 512) G = 3;
  else if (fits(2) && threads_for(2, 4) <= 512) G = 2;
  else if (fits(3) && threads_for(3, 8) <= 512 && 10 * (R + 2 * stride) <= 6 * 3 * R) { G = 3; nq = 8; }
  else if (threads_for(1, 4) > 512) nq = 8;
  if (threads < threads_for(G, nq) && threads_for(G, nq) <= 512) threads = threads_for(G, nq);
  const int rows_in = R + (G - 1) * stride, quads_all = rows_in * quads;
  const size_t smem = (size_t)rows_in * rowlen;
  // rows the fixed per-thread tasks do not cover: use apnn_quantize_im2col_i8
  if ((wc & 3) || smem > 48 * 1024 || tasks > 4 * 512 || quads_all > nq * threads) return APNN_ERR_UNSUPPORTED;
  const int groups = B * ((Ho + G - 1) / G);
  long long nb = groups, cap = (long long)device_sm_count() * (2048 / threads);
  if (nb > cap) nb = cap;
#define APNN_WINDOW_KERNEL(TPT_) \
  (G == 3 ? (nq == 4 ? quantize_window_rows_i8_kernel<TPT_, 4, 3> : quantize_window_rows_i8_kernel<TPT_, 8, 3>) \
   : G == 2 ? quantize_window_rows_i8_kernel<TPT_, 4, 2>                                                           \
            : (nq == 4 ? quantize_window_rows_i8_kernel<TPT_, 4, 1> : quantize_window_rows_i8_kernel<TPT_, 8, 1>))
  auto kern = tpt == 1 ? APNN_WINDOW_KERNEL(1) : tpt == 2 ? APNN_WINDOW_KERNEL(2) : APNN_WINDOW_KERNEL(4);
#undef APNN_WINDOW_KERNEL
  kern<<<(unsigned)nb, threads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      images, reinterpret_cast<uint8_t*>(out_i8), B, H, W, C, R, stride, bits, Ho, Wo, kp, seg, rowlen, lpad,
      make_quant_steps(bits), xormask, centred ? 0.0f : -100.0f);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "quantize_window_rows_i8 launch");
  return APNN_OK;
}

apnn_status apnn_quantize_blocks_i8(void* stream, const float* images, void* out_i8, int B, int H, int W, int C, int stride,
                                    int bits, int halo, int cpad) {
  using namespace apnn;
  if (!images || !out_i8) return APNN_ERR_INVALID_ARG;
  const bool centred = (bits & APNN_QUANT_CENTRED) != 0;
  bits &= ~APNN_QUANT_CENTRED;
  if (centred && bits != 8) return APNN_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || bits < 1 || bits > 8 || halo < 0 || halo > 8) return APNN_ERR_INVALID_ARG;
  if (stride < 2 || stride > 4 || H % stride || W % stride || (stride * C) % 4 || stride * stride * C > cpad || cpad % 16)
    return APNN_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(images) & 15u) || (reinterpret_cast<uintptr_t>(out_i8) & 15u)) return APNN_ERR_ALIGNMENT;
  const int per_row = (W / stride) * (cpad / 16);
  if (H / stride > 65535 || B > 65535) return APNN_ERR_UNSUPPORTED;
  const dim3 grid((unsigned)((per_row + 255) / 256), (unsigned)(H / stride), (unsigned)B);
  quantize_blocks_i8_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      images, reinterpret_cast<uint8_t*>(out_i8), B, H, W, C, stride, bits, halo, cpad, make_quant_steps(bits),
      centred ? 0x80808080u : 0u);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "quantize_blocks_i8 launch");
  return APNN_OK;
}

apnn_status apnn_maxpool2x2_i8(void* stream, const void* in_i8, void* out_i8, int B, int H, int W, int C, int in_halo,
                               int out_halo) {
  using namespace apnn;
  if (!in_i8 || !out_i8 || B <= 0 || H <= 0 || W <= 0 || C <= 0) return APNN_ERR_INVALID_ARG;
  if (in_halo < 0 || in_halo > 8 || out_halo < 0 || out_halo > 8) return APNN_ERR_INVALID_ARG;
  if ((H & 1) || (W & 1)) return APNN_ERR_UNSUPPORTED;
  if (C % 16 != 0 || (reinterpret_cast<uintptr_t>(in_i8) & 15u) || (reinterpret_cast<uintptr_t>(out_i8) & 15u))
    return APNN_ERR_ALIGNMENT;
  const long long total = (long long)B * (H / 2) * (W / 2) * (C / 16);
  long long nb = (total + 255) / 256, cap = (long long)device_sm_count() * 32;
  if (nb > cap) nb = cap;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)nb, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)pdl_attribute(attr);
  cudaError_t e = cudaLaunchKernelEx(&cfg, maxpool2x2_i8_kernel, reinterpret_cast<const uint8_t*>(in_i8),
                                     reinterpret_cast<uint8_t*>(out_i8), B, H / 2, W / 2, C, in_halo, out_halo);
  if (e != cudaSuccess) return cuda_fail(e, "maxpool2x2_i8 launch");
  return APNN_OK;
}

apnn_status apnn_requantize_i32(void* stream, const int32_t* values, void* out, long rows, int N, const apnn_epilogue* epi) {
  using namespace apnn;
  if (!values || !out || !epi || rows <= 0 || N <= 0) return APNN_ERR_INVALID_ARG;
  if (epi->struct_size != sizeof(apnn_epilogue)) return APNN_ERR_INVALID_ARG;
  const bool to_float = epi->out_mode == APNN_OUT_FLOAT;
  if (epi->out_mode != APNN_OUT_LOWBITS && epi->out_mode != APNN_OUT_THRESHOLDS && !to_float) return APNN_ERR_INVALID_ARG;
  if (to_float && (!epi->affine_scale || !epi->affine_bias || epi->out_i8)) return APNN_ERR_INVALID_ARG;
  if (!to_float && (epi->out_bits < 1 || epi->out_bits > 8 || (epi->out_mode == APNN_OUT_THRESHOLDS && !epi->thresholds)))
    return APNN_ERR_INVALID_ARG;
  if (epi->pool != APNN_POOL_NONE || epi->residual_in || epi->residual_out || epi->signed_operand != APNN_SIGN_NONE ||
      epi->n_peer_out != 0)
    return APNN_ERR_UNSUPPORTED;
  if (N % 32 != 0) return APNN_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(values) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return APNN_ERR_ALIGNMENT;
  // every column group gets the same number of warps; more of them when there are many rows
  const int groups = N / 32;
  long long per_group = (rows + 7) / 8;   // at least 8 rows per warp, fewer warps only when the device is full
  const long long cap = (long long)device_sm_count() * 64 / groups;
  if (per_group > cap) per_group = cap;
  if (per_group < 1) per_group = 1;
  const long long warps = per_group * groups;
  const unsigned nb = (unsigned)((warps + 7) / 8);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(nb, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)pdl_attribute(attr);
  cudaError_t e = cudaLaunchKernelEx(&cfg, requantize_i32_kernel, values, out, (long long)rows, N, (int)epi->out_mode,
                                     (int)epi->out_bits, epi->thresholds, (int)epi->out_i8, epi->affine_scale,
                                     epi->affine_bias);
  if (e != cudaSuccess) return cuda_fail(e, "requantize_i32 launch");
  return APNN_OK;
}

}  // extern "C"
