// tcgen05 path for large GEMMs and 3x3 / 1x1 stride-1 convolutions.
//
// Step 1 (expand_planes_kernel): every operand is rewritten once from bit planes to one
// int8 per element, value = sum_p bit_p << p (or -1/+1 for a signed 1-bit operand), rows of
// K bytes in the caller's workspace.  Within each group of 32 k the byte order is the
// "spread" order (bit q+8j of the word -> byte 4q+j); both operands use it, so the dot
// product is unchanged.
//
// Step 2 (tc5_gemm_kernel): persistent, warp-specialised int8 GEMM.  One CTA per SM walks
// over 128 x 256 output tiles.  Warp 0 streams K blocks of 128 bytes per row with TMA
// (128-byte swizzle) through a 4-stage shared-memory ring; warp 1 issues tcgen05.mma
// kind::i8 (M=128, N=256, K=32) from shared-memory descriptors into one of two 256-column
// TMEM accumulators; warps 2-5 drain the other accumulator with tcgen05.ld and run the
// epilogue (int32 stores, or requantise + bit-plane pack: a thread owns one row and 32
// consecutive columns, i.e. exactly one output word per plane).  No cluster, no multicast.
//
// Convolution reuses the same kernel as an implicit GEMM: the activations are expanded to
// int8 NHWC (halo included), and the A tile of a K block is one 4-D TMA box -- 128 bytes of
// channels x (bw x bh x bb) output pixels -- fetched at the halo offset of the filter tap,
// which lands in shared memory as the same 128-byte-swizzled row block a GEMM tile would.
// K runs over (tap_i, tap_j, 128-channel block), matching the filter rows' K order.  A
// 2x2 pooling window lies inside one warp (the box is at most 16 pixels wide), so the
// epilogue pools with three lane shuffles before requantising.
//
// Every mbarrier wait is bounded: on expiry the kernel raises a flag in global memory,
// stops issuing work, and falls through to the common tear-down (TMEM is released).
#include <cuda.h>

#include <cstring>

#include "api_internal.h"
#include "apnn_device.cuh"
#include "tc5_common.cuh"
#include "tc5_gemm.h"

namespace apnn {

namespace {

using tc5::BM;
using tc5::BK;

constexpr int A_STAGE_BYTES = BM * BK;
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 6;

// Tile width N is 256 (4 stages of 48 KiB) when that still fills the device, else 128
// (6 stages of 32 KiB): twice as many tiles for mid-sized problems.
template <int BN>
struct TileCfg {
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int B_STAGE_BYTES = BN * BK;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  // each epilogue warp keeps the tile's thresholds as one 16-byte entry per column
  static constexpr int THR_BYTES_PER_WARP = BN * 16;
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + 4 * THR_BYTES_PER_WARP;
  static constexpr int TMEM_COLS = 2 * BN;
};
constexpr int GROUP_M = 16;  // tiles are walked in bands of 16 row-tiles for L2 reuse

// ------------------------------------------------------------------ expand kernel
struct ExpandJob {
  const uint32_t* planes;
  uint8_t* out;
  long long total;  // rows * K/32 words per plane
  int bits;
  int is_signed;
};

// One 32-k word of every plane -> 32 bytes.  Two words per thread per trip so their loads overlap.
template <int BITS>
__device__ __forceinline__ void expand_words(const ExpandJob& j, long long first, long long step) {
  for (long long i = first; i < j.total; i += 2 * step) {
    const long long i2 = i + step;
    const bool two = i2 < j.total;
    uint32_t w[2][BITS];
#pragma unroll
    for (int p = 0; p < BITS; p++) {
      w[0][p] = __ldg(j.planes + p * j.total + i);
      w[1][p] = two ? __ldg(j.planes + p * j.total + i2) : 0u;
    }
#pragma unroll
    for (int u = 0; u < 2; u++) {
      if (u == 1 && !two) break;
      uint32_t r[8];
#pragma unroll
      for (int q = 0; q < 8; q++) {
        uint32_t v = 0;
#pragma unroll
        for (int p = 0; p < BITS; p++) {
          uint32_t s = (q >= p) ? (w[u][p] >> (q - p)) : (w[u][p] << (p - q));
          v |= s & (0x01010101u << p);
        }
        // signed 1-bit operand: bit 1 -> +1 (0x01), bit 0 -> -1 (0xFF)
        r[q] = (BITS == 1 && j.is_signed) ? (0xFFFFFFFFu ^ (v * 0xFEu)) : v;
      }
      // one 32-byte store per word: a warp writes 1 KiB of whole sectors per instruction
      uint8_t* dst = j.out + (u == 0 ? i : i2) * 32;
      asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                   "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                   : "memory");
    }
  }
}

// Blocks [0, blocks_a) work on job a, the rest on job b (one launch for both GEMM operands).
__global__ void __launch_bounds__(256) expand_planes_kernel(const ExpandJob a, const ExpandJob b, int blocks_a) {
  const bool first = (int)blockIdx.x < blocks_a;
  const ExpandJob& j = first ? a : b;
  const long long nblk = first ? blocks_a : (long long)gridDim.x - blocks_a;
  const long long blk = first ? blockIdx.x : blockIdx.x - blocks_a;
  const long long i0 = blk * blockDim.x + threadIdx.x;
  const long long step = nblk * blockDim.x;
  switch (j.bits) {
    case 1: expand_words<1>(j, i0, step); break;
    case 2: expand_words<2>(j, i0, step); break;
    case 3: expand_words<3>(j, i0, step); break;
    case 4: expand_words<4>(j, i0, step); break;
    default: expand_words<8>(j, i0, step); break;
  }
}

using namespace tc5;

struct Tc5Params {
  void* out;
  const int32_t* thresholds;
  int M, N, kblocks;
  int tiles_m, tiles_n;
  int out_mode, out_bits;
  uint32_t idesc;
  long long out_plane_words;
  int* error_flag;
  // convolution (is_conv != 0): an A tile is a box of bw x bh x bb output pixels
  int is_conv;
  int bw, bh, bb;
  int tiles_w, tiles_h;  // boxes per image along w and h
  int Bn, Ho, Wo;        // batch and conv output extent (before pooling)
  int cblocks, R;        // CIN / 128, filter size
  int in_off;            // stored ring width minus (R-1)/2
  int stride;            // conv stride (1 or 2)
  int pool, out_h, out_w, out_halo;
  uint32_t a_box_bytes;  // bytes one A box deposits
  const int32_t* residual_in;  // optional dense int32 [rows][N], added before requantisation
  int32_t* residual_out;       // optional dense int32 [rows][N], the value after the add
};

// Output row (units of N channels) and validity of tile row r; for pooled outputs only the
// top-left pixel of a window is a writer.
struct RowDst {
  long long row;    // output row, ring included
  long long dense;  // output row without the ring (index of the residual tensors)
  bool valid;
};
__device__ __forceinline__ RowDst row_destination(const Tc5Params& p, int tm, int r) {
  RowDst d;
  if (!p.is_conv) {
    d.row = (long long)tm * BM + r;
    d.dense = d.row;
    d.valid = d.row < p.M;
    return d;
  }
  const int tw = tm % p.tiles_w;
  const int t2 = tm / p.tiles_w;
  const int th = t2 % p.tiles_h;
  const int bg = t2 / p.tiles_h;
  const int wi = r % p.bw;
  const int r2 = r / p.bw;
  const int hi = r2 % p.bh;
  const int bi = r2 / p.bh;
  const int b = bg * p.bb + bi, ho = th * p.bh + hi, wo = tw * p.bw + wi;
  d.valid = bi < p.bb && b < p.Bn && ho < p.Ho && wo < p.Wo;
  int oh = ho, ow = wo;
  if (p.pool != POOL_NONE) {
    d.valid = d.valid && ((hi | wi) & 1) == 0;
    oh = ho >> 1;
    ow = wo >> 1;
  }
  const int hh = p.out_halo;
  d.row = ((long long)b * (p.out_h + 2 * hh) + oh + hh) * (p.out_w + 2 * hh) + ow + hh;
  d.dense = ((long long)b * p.out_h + oh) * p.out_w + ow;
  return d;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band = GROUP_M * tiles_n;
  const int g = tile / band;
  const int first = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first);
  const int r = tile - g * band;
  tm = first + r % rows;
  tn = r / rows;
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
tc5_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Tc5Params p) {
  using Cfg = TileCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then the TMEM pointer
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  uint8_t* thr_stage = smem_raw + (bars + 256u - raw);  // 4 x THR_BYTES_PER_WARP

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) *p.error_flag = 0;  // only ever raised after a 2 s wait, long after this store
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                 "r"(Cfg::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        int w0 = 0, h0 = 0, b0 = 0;
        if (p.is_conv) {
          w0 = (tm % p.tiles_w) * p.bw;
          const int t2 = tm / p.tiles_w;
          h0 = (t2 % p.tiles_h) * p.bh;
          b0 = (t2 / p.tiles_h) * p.bb;
        }
        int tap = 0, cb = 0;  // conv: K block = (filter tap, 128-channel block)
        for (int kb = 0; kb < p.kblocks; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) { ok = false; break; }
          const uint32_t sa = base + s * STAGE_BYTES;
          if (!p.is_conv) {
            mbar_expect_tx(full_bar(s), STAGE_BYTES);
            tma_load_2d(sa, &map_a, kb * BK, tm * BM, full_bar(s));
          } else {
            mbar_expect_tx(full_bar(s), p.a_box_bytes + Cfg::B_STAGE_BYTES);
            const int ti = tap / p.R, tj = tap - ti * p.R;
            tma_load_4d(sa, &map_a, cb * BK, w0 * p.stride + tj + p.in_off, h0 * p.stride + ti + p.in_off, b0, full_bar(s));
            if (++cb == p.cblocks) { cb = 0; tap++; }
          }
          tma_load_2d(sa + A_STAGE_BYTES, &map_b, kb * BK, tn * BN, full_bar(s));
        }
      }
      if (!ok) atomicExch(p.error_flag, 1);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t tl = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tl++) {
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.kblocks; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(full_bar(s), ph)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * STAGE_BYTES;
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + A_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 32; k++) {
            // advancing 32 bytes along K inside the swizzle row = +2 in 16-byte units
            tc_mma_i8(d_tmem, adesc + 2u * k, bdesc + 2u * k, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(empty_bar(s));  // frees the stage when these MMAs have read it
        }
        if (ok) tc_commit(tfull_bar(acc));  // accumulator complete
      }
      if (!ok) atomicExch(p.error_flag, 2);
    }
  } else {
    // ---------------- epilogue warps (2..5) ----------------
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 belong to this warp
    uint32_t tl = 0;
    bool ok = true;
    const int nl = (1 << p.out_bits) - 1;
    // thresholds of up to 2-bit outputs are staged per tile in this warp's shared-memory
    // slice, one int4 per column (unused slots = INT_MAX), so a value costs one broadcast
    // 16-byte load instead of nl global loads
    const bool thr_staged = p.out_mode == OUT_THRESHOLDS && nl <= 3;
    int4* thr_s = reinterpret_cast<int4*>(thr_stage + (warp - 2) * Cfg::THR_BYTES_PER_WARP);
    int staged_tn = -1;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tl++) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      if (thr_staged && tn != staged_tn) {
        __syncwarp();
        for (int cidx = lane; cidx < BN; cidx += 32) {
          const int col = tn * BN + cidx;
          int4 t4 = make_int4(0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff);
          if (col < p.N) {
            const int32_t* T = p.thresholds + (long long)col * nl;
            t4.x = __ldg(T);
            if (nl > 1) { t4.y = __ldg(T + 1); t4.z = __ldg(T + 2); }
          }
          thr_s[cidx] = t4;
        }
        __syncwarp();
        staged_tn = tn;
      }
      const uint32_t acc = tl & 1u;
      const uint32_t aph = (tl >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), aph)) { ok = false; break; }
      tc_fence_after();
      const RowDst dst = row_destination(p, tm, quarter * 32 + lane);
      const long long row = dst.row;
      const bool row_ok = dst.valid;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        tmem_ld_wait();
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) continue;  // uniform over the warp
        if (p.pool != POOL_NONE) {
          // the four pixels of a window are lanes l, l^1 (next column) and l^bw, l^bw^1 (next row)
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const int a0 = (int)v[j];
            const int a1 = __shfl_xor_sync(0xffffffffu, a0, 1);
            const int a2 = __shfl_xor_sync(0xffffffffu, a0, p.bw);
            const int a3 = __shfl_xor_sync(0xffffffffu, a1, p.bw);
            v[j] = (uint32_t)(p.pool == POOL_AVG2 ? (a0 + a1 + a2 + a3) / 4 : max(max(a0, a1), max(a2, a3)));
          }
        }
        if (!row_ok) continue;
        if (p.residual_in != nullptr || p.residual_out != nullptr) {
          const long long at = dst.dense * (long long)p.N + col0;
          if ((p.N & 3) == 0 && col0 + 32 <= p.N) {
            // this thread's 32 columns are 128 contiguous bytes: 16-byte accesses
            if (p.residual_in != nullptr) {
              const int4* R4 = reinterpret_cast<const int4*>(p.residual_in + at);
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const int4 r = __ldg(R4 + j);
                v[4 * j] += (uint32_t)r.x; v[4 * j + 1] += (uint32_t)r.y;
                v[4 * j + 2] += (uint32_t)r.z; v[4 * j + 3] += (uint32_t)r.w;
              }
            }
            if (p.residual_out != nullptr) {
              uint4* O4 = reinterpret_cast<uint4*>(p.residual_out + at);
#pragma unroll
              for (int j = 0; j < 8; j++) O4[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < p.N) {
                if (p.residual_in != nullptr) v[j] = (uint32_t)((int)v[j] + __ldg(p.residual_in + at + j));
                if (p.residual_out != nullptr) p.residual_out[at + j] = (int32_t)v[j];
              }
          }
        }
        if (p.out_mode == OUT_INT32) {
          int32_t* D = reinterpret_cast<int32_t*>(p.out) + row * p.N + col0;
          if ((p.N & 3) == 0 && col0 + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 8; j++)
              reinterpret_cast<uint4*>(D)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < p.N) D[j] = (int32_t)v[j];
          }
        } else {
          // packed modes need N % 32 == 0, so this word is whole
          uint32_t lv[32];
          if (p.out_mode == OUT_LOWBITS) {
#pragma unroll
            for (int j = 0; j < 32; j++) lv[j] = v[j] & (uint32_t)nl;
          } else if (thr_staged) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const int4 t4 = thr_s[c * 32 + j];
              const int x = (int)v[j];
              lv[j] = (x >= t4.x ? 1u : 0u) + (x >= t4.y ? 1u : 0u) + (x >= t4.z ? 1u : 0u);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const int32_t* T = p.thresholds + (long long)(col0 + j) * nl;
              uint32_t l = 0;
              for (int t = 0; t < nl; t++) l += ((int32_t)v[j] >= __ldg(T + t)) ? 1u : 0u;
              lv[j] = l;
            }
          }
          uint32_t* O = reinterpret_cast<uint32_t*>(p.out);
          for (int b = 0; b < p.out_bits; b++) {
            uint32_t word = 0;
#pragma unroll
            for (int j = 0; j < 32; j++) word |= ((lv[j] >> b) & 1u) << (31 - j);
            O[b * p.out_plane_words + row * (p.N >> 5) + (col0 >> 5)] = word;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (!ok && lane == 0) atomicExch(p.error_flag, 3);
  }

  // ---------------- tear-down ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS));
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// rows x K bytes, row-major; box = box_rows x 128 bytes, 128-byte swizzle, zero fill outside
bool make_operand_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// int8 NHWC activations [B][Hp][Wp][CIN]; box = 128 channels x bw x bh x bb pixels
// With a traversal stride s the box spans bw*s x bh*s stored pixels and picks every s-th one.
bool make_activation_map(CUtensorMap* map, const void* base, int B, int Hp, int Wp, int CIN, int bw, int bh, int bb,
                         int stride) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)CIN, (cuuint64_t)Wp, (cuuint64_t)Hp, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)CIN, (cuuint64_t)Wp * CIN, (cuuint64_t)Hp * Wp * CIN};
  cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)(bw * stride), (cuuint32_t)(bh * stride), (cuuint32_t)bb};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <int BN>
cudaError_t launch_tc5(cudaStream_t s, const CUtensorMap& map_a, const CUtensorMap& map_b, const Tc5Params& p,
                       int grid) {
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 16 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(tc5_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TileCfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev < 16) attr_set[dev] = true;
  }
  tc5_gemm_kernel<BN><<<grid, THREADS, TileCfg<BN>::SMEM_BYTES, s>>>(map_a, map_b, p);
  return cudaGetLastError();
}

// Tile width: 256 unless that leaves the device under-filled and 128 does better.
int pick_bn(long long tiles_m, int N, int sms) {
  long long t256 = tiles_m * ((N + 255) / 256), t128 = tiles_m * ((N + 127) / 128);
  if (t256 >= sms) return 256;
  // waves needed with each width, in units of a 256-wide tile's work
  double w256 = (double)((t256 + sms - 1) / sms);
  double w128 = 0.5 * (double)((t128 + sms - 1) / sms);
  return w128 < w256 ? 128 : 256;
}

uint32_t make_idesc(bool a_signed, bool b_signed, int bn) {
  // D = s32, A/B = u8 or s8, both K-major, N = bn, M = 128
  return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

}  // namespace

size_t tc5_workspace_bytes(int M, int N, int K) {
  // int8 copies of both operands + a 256-byte slot for the kernel's error flag
  return align_up((size_t)M * K, 256) + align_up((size_t)N * K, 256) + 256;
}

bool tc5_worthwhile(int M, int N, int K) {
  long long tiles = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
  return tiles >= 64 && K >= 1024;
}

namespace {
int expand_blocks(long long total, int sms) {
  long long want = (total + 511) / 512, cap = (long long)sms * 16;
  long long b = want < cap ? want : cap;
  return (int)(b < 1 ? 1 : b);
}
ExpandJob make_job(const uint32_t* planes, uint8_t* out, long long rows, int K, int bits, bool is_signed) {
  ExpandJob j;
  j.planes = planes;
  j.out = out;
  j.total = rows * (K / 32);
  j.bits = (bits >= 5 && bits <= 8) ? 8 : bits;
  j.is_signed = is_signed ? 1 : 0;
  return j;
}
// planes of 5..7 bits run through the 8-plane code path and therefore need 8 readable planes;
// the ABI only admits 1..4 and 8
}  // namespace

apnn_status tc5_expand(cudaStream_t s, const uint32_t* planes, uint8_t* out, long long rows, int K, int bits,
                       bool is_signed) {
  const int sms = device_sm_count();
  ExpandJob a = make_job(planes, out, rows, K, bits, is_signed);
  const int blocks = expand_blocks(a.total, sms);
  expand_planes_kernel<<<blocks, 256, 0, s>>>(a, a, blocks);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "expand_planes launch");
  return APNN_OK;
}

// Both operands of a GEMM in one launch.
apnn_status tc5_expand2(cudaStream_t s, const uint32_t* pa, uint8_t* oa, long long rows_a, int bits_a, bool signed_a,
                        const uint32_t* pb, uint8_t* ob, long long rows_b, int bits_b, bool signed_b, int K) {
  const int sms = device_sm_count();
  ExpandJob a = make_job(pa, oa, rows_a, K, bits_a, signed_a);
  ExpandJob b = make_job(pb, ob, rows_b, K, bits_b, signed_b);
  const int ba = expand_blocks(a.total, sms), bb = expand_blocks(b.total, sms);
  expand_planes_kernel<<<ba + bb, 256, 0, s>>>(a, b, ba);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "expand_planes launch");
  return APNN_OK;
}

apnn_status tc5_gemm_i8(cudaStream_t s, const uint8_t* A8, const uint8_t* B8, void* D, int M, int N, int K,
                        bool a_signed, bool b_signed, const apnn_epilogue* epi, int* status_flag) {
  if (tc5_pair_worthwhile(M, N, K) || (epi && epi->n_peer_out > 0))
    return tc5_gemm_i8_pair(s, A8, B8, D, M, N, K, a_signed, b_signed, epi, status_flag);
  cudaError_t e;
  const int sms = device_sm_count();
  Tc5Params p;
  memset(&p, 0, sizeof(p));
  p.tiles_m = (M + BM - 1) / BM;
  const int bn = pick_bn(p.tiles_m, N, sms);
  CUtensorMap map_a, map_b;
  if (!make_operand_map(&map_a, A8, M, K, BM) || !make_operand_map(&map_b, B8, N, K, bn)) {
    return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  }
  p.out = D;
  p.thresholds = epi ? epi->thresholds : nullptr;
  p.M = M;
  p.N = N;
  p.kblocks = K / BK;
  p.tiles_n = (N + bn - 1) / bn;
  p.out_mode = epi ? epi->out_mode : APNN_OUT_INT32;
  p.out_bits = epi ? epi->out_bits : 0;
  p.out_plane_words = (long long)M * (N / 32);
  p.error_flag = status_flag;
  p.residual_in = epi ? epi->residual_in : nullptr;
  p.residual_out = epi ? epi->residual_out : nullptr;
  p.idesc = make_idesc(a_signed, b_signed, bn);
  long long tiles = (long long)p.tiles_m * p.tiles_n;
  int grid = (int)(tiles < sms ? tiles : sms);
  e = bn == 256 ? launch_tc5<256>(s, map_a, map_b, p, grid) : launch_tc5<128>(s, map_a, map_b, p, grid);
  if (e != cudaSuccess) return cuda_fail(e, "tc5_gemm launch");
  return APNN_OK;
}

apnn_status tc5_gemm(cudaStream_t s, int wbits, int xbits, const uint32_t* W, const uint32_t* X, void* D, int M,
                     int N, int K, const apnn_epilogue* epi, void* workspace, int pair) {
  uint8_t* wa = reinterpret_cast<uint8_t*>(workspace);
  uint8_t* wb = wa + align_up((size_t)M * K, 256);
  int* err = reinterpret_cast<int*>(wb + align_up((size_t)N * K, 256));
  const int sign = epi ? epi->signed_operand : APNN_SIGN_NONE;
  apnn_status st = tc5_expand2(s, W, wa, M, wbits, sign == APNN_SIGN_W, X, wb, N, xbits, sign == APNN_SIGN_X, K);
  if (st != APNN_OK) return st;
  if (pair) return tc5_gemm_i8_pair(s, wa, wb, D, M, N, K, sign == APNN_SIGN_W, sign == APNN_SIGN_X, epi, err);
  return tc5_gemm_i8(s, wa, wb, D, M, N, K, sign == APNN_SIGN_W, sign == APNN_SIGN_X, epi, err);
}

// ------------------------------------------------------------------ convolution
// Pixel box of an A tile: bw x bh (x bb whole images when an image is smaller than a tile),
// at most 128 pixels, chosen for the fewest wasted MMA rows.  With pooling the box is a
// power of two wide (<= 16) and even high, so a 2x2 window never straddles warps.
bool tc5_conv_box(int Ho, int Wo, int pool, int* bw_out, int* bh_out, int* bb_out) {
  double best = -1.0;
  for (int bw = 1; bw <= 128 && bw <= Wo; bw++) {
    if (pool && !(bw == 2 || bw == 4 || bw == 8 || bw == 16)) continue;
    int bh = 128 / bw;
    if (bh > Ho) bh = Ho;
    if (pool) bh &= ~1;
    if (bh < 1) continue;
    int bb = 1;
    if (bw == Wo && bh == Ho) bb = 128 / (bw * bh);
    if (bb < 1) bb = 1;
    // TMA box extents are limited to 256 per dimension; all are <= 128 here
    double covered = (double)Wo * Ho;
    double spent = (double)((Wo + bw - 1) / bw) * ((Ho + bh - 1) / bh) * 128.0 / bb;
    double util = covered / spent;
    if (util > best + 1e-9) {
      best = util;
      *bw_out = bw;
      *bh_out = bh;
      *bb_out = bb;
    }
  }
  return best > 0;
}

size_t tc5_conv_workspace_bytes(int B, int H, int W, int CIN, int COUT, int R) {
  const int pad = (R - 1) / 2;
  return align_up((size_t)B * (H + 2 * pad) * (W + 2 * pad) * CIN, 256) + align_up((size_t)COUT * R * R * CIN, 256) +
         256;
}

// H, W: input extent (without ring).  Strides 1 and 2 (the TMA box extent bw*stride must stay <= 256).
bool tc5_conv_supported(int H, int W, int R, int stride, int pool) {
  if (stride != 1 && stride != 2) return false;
  int bw, bh, bb;
  return tc5_conv_box((H - 1) / stride + 1, (W - 1) / stride + 1, pool, &bw, &bh, &bb);
}

apnn_status tc5_conv_i8(cudaStream_t s, const uint8_t* X8, const uint8_t* W8, void* Out, int B, int Hin, int Win,
                        int CIN, int COUT, int R, int stride, bool w_signed, const apnn_epilogue* epi,
                        int* status_flag) {
  const int pad = (R - 1) / 2;
  const int in_halo = (epi && epi->in_halo) ? epi->in_halo : pad;
  const int Hp = Hin + 2 * in_halo, Wp = Win + 2 * in_halo;
  const int H = (Hin - 1) / stride + 1, W = (Win - 1) / stride + 1;  // output extent
  const int pool = epi ? epi->pool : APNN_POOL_NONE;
  int bw = 0, bh = 0, bb = 0;
  if (!tc5_conv_box(H, W, pool, &bw, &bh, &bb)) return APNN_ERR_UNSUPPORTED;
  cudaError_t e;
  const int sms = device_sm_count();
  Tc5Params p;
  memset(&p, 0, sizeof(p));
  p.is_conv = 1;
  p.bw = bw;
  p.bh = bh;
  p.bb = bb;
  p.tiles_w = (W + bw - 1) / bw;
  p.tiles_h = (H + bh - 1) / bh;
  p.tiles_m = ((B + bb - 1) / bb) * p.tiles_h * p.tiles_w;
  p.Bn = B;
  p.Ho = H;
  p.Wo = W;
  p.cblocks = CIN / BK;
  p.R = R;
  p.in_off = in_halo - pad;
  p.stride = stride;
  p.pool = pool;
  p.out_h = pool ? H / 2 : H;
  p.out_w = pool ? W / 2 : W;
  p.out_halo = epi ? epi->out_halo : 0;
  p.a_box_bytes = (uint32_t)(bw * bh * bb * BK);
  const int bn = pick_bn(p.tiles_m, COUT, sms);
  CUtensorMap map_a, map_b;
  if (!make_activation_map(&map_a, X8, B, Hp, Wp, CIN, bw, bh, bb, stride) ||
      !make_operand_map(&map_b, W8, COUT, (long long)R * R * CIN, bn)) {
    return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  }
  p.out = Out;
  p.thresholds = epi ? epi->thresholds : nullptr;
  p.M = B * H * W;
  p.N = COUT;
  p.kblocks = R * R * p.cblocks;
  p.tiles_n = (COUT + bn - 1) / bn;
  p.out_mode = epi ? epi->out_mode : APNN_OUT_INT32;
  p.out_bits = epi ? epi->out_bits : 0;
  p.out_plane_words =
      (long long)B * (p.out_h + 2 * p.out_halo) * (p.out_w + 2 * p.out_halo) * (COUT / 32);
  p.error_flag = status_flag;
  p.residual_in = epi ? epi->residual_in : nullptr;
  p.residual_out = epi ? epi->residual_out : nullptr;
  p.idesc = make_idesc(false, w_signed, bn);  // A = activations (unsigned), B = filter
  long long tiles = (long long)p.tiles_m * p.tiles_n;
  int grid = (int)(tiles < sms ? tiles : sms);
  e = bn == 256 ? launch_tc5<256>(s, map_a, map_b, p, grid) : launch_tc5<128>(s, map_a, map_b, p, grid);
  if (e != cudaSuccess) return cuda_fail(e, "tc5_conv launch");
  return APNN_OK;
}

apnn_status tc5_conv(cudaStream_t s, int wbits, int xbits, const uint32_t* Wt, const uint32_t* X, void* Out, int B,
                     int H, int W, int CIN, int COUT, int R, int stride, const apnn_epilogue* epi, void* workspace) {
  const int pad = (R - 1) / 2;
  const long long pixels = (long long)B * (H + 2 * pad) * (W + 2 * pad);
  uint8_t* x8 = reinterpret_cast<uint8_t*>(workspace);
  uint8_t* w8 = x8 + align_up((size_t)pixels * CIN, 256);
  int* err = reinterpret_cast<int*>(w8 + align_up((size_t)COUT * R * R * CIN, 256));
  const bool w_signed = epi && epi->signed_operand == APNN_SIGN_W;
  apnn_status st = tc5_expand(s, X, x8, pixels, CIN, xbits, false);
  if (st != APNN_OK) return st;
  st = tc5_expand(s, Wt, w8, COUT, R * R * CIN, wbits, w_signed);
  if (st != APNN_OK) return st;
  return tc5_conv_i8(s, x8, w8, Out, B, H, W, CIN, COUT, R, stride, w_signed, epi, err);
}

int tc5_conv_read_error_flag(cudaStream_t s, const void* workspace, int B, int H, int W, int CIN, int COUT, int R) {
  const int pad = (R - 1) / 2;
  const uint8_t* x8 = reinterpret_cast<const uint8_t*>(workspace);
  const uint8_t* w8 = x8 + align_up((size_t)B * (H + 2 * pad) * (W + 2 * pad) * CIN, 256);
  const int* err = reinterpret_cast<const int*>(w8 + align_up((size_t)COUT * R * R * CIN, 256));
  int v = -1;
  if (cudaMemcpyAsync(&v, err, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
  return v;
}

// Reads back the flag a bounded wait raises; 0 means the last tc5_gemm on this workspace
// ran to completion.  Synchronises the stream.
int tc5_read_error_flag(cudaStream_t s, const void* workspace, int M, int N, int K) {
  const uint8_t* wa = reinterpret_cast<const uint8_t*>(workspace);
  const uint8_t* wb = wa + align_up((size_t)M * K, 256);
  const int* err = reinterpret_cast<const int*>(wb + align_up((size_t)N * K, 256));
  int v = -1;
  if (cudaMemcpyAsync(&v, err, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
  return v;
}

}  // namespace apnn
