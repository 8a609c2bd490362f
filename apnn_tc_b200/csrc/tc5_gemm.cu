// tcgen05 path: GEMMs and convolutions on int8 operands, one CTA per SM.
//
// Step 1 (expand_planes_kernel): an operand is rewritten once from bit planes to one int8 per
// element, value = sum_p bit_p << p (or -1/+1 for a signed 1-bit operand), rows of K bytes in
// the caller's workspace.  Within each group of 32 k the byte order is the "spread" order (bit
// q+8j of the word -> byte 4q+j); both operands use it, so the dot product is unchanged.
// Networks skip this step: a layer's epilogue writes the next layer's int8 rows directly.
//
// Step 2 (tc5_gemm_kernel<BN, BKB, SPLITK, EPI>): persistent, warp-specialised.  Warp 0 streams
// operand tiles with TMA (swizzle span BKB = 128 or 64 bytes of K per row) through mbarrier
// rings; warp 1 issues tcgen05.mma kind::i8 (M=128, N=BN, K=32) from shared-memory descriptors
// into one of two BN-column TMEM accumulators; warps 2-9 drain the other with tcgen05.ld (two
// warps per TMEM lane quarter, alternating 32-column chunks) and run the epilogue: a thread
// owns one row and 32 consecutive columns, i.e. one output word per plane or 32 output bytes.
// No cluster, no multicast.  What bounds it is shared-memory bandwidth (128 B/clk feed both the
// MMA's operand reads and TMA's writes) and the instruction streams of the single producer / MMA
// threads and of the few epilogue warps, so:
//   * the filter stays resident in shared memory when the problem has one tile column;
//   * narrow K blocks are grouped per barrier round trip, and all index arithmetic in the
//     producer / MMA loops is incremental (no divisions);
//   * the epilogue is compiled per family of uses (EPI) instead of branching at run time.
//
// Convolution, stride 1 without pooling ("flat"): output positions are the flattened padded
// pixels q = (b*Hp + h)*Wp + w, a tile is 128 consecutive q, and tap (i, j) reads input rows
// q + i*Wp + j of the flattened int8 image -- so ONE 2-D TMA box of 128 + (R-1)*(Wp+1) rows
// per (tile, channel block) serves every tap through descriptors whose start address is
// shifted by whole rows (the swizzle is a function of the shared-memory address).  Positions in
// the padding ring are computed and dropped.  Other convolutions (stride 2, fused pooling,
// tiny images) fetch one 4-D TMA box of bw x bh x bb output pixels per tap; a 2x2 pooling
// window then lies inside one warp and is reduced with three lane shuffles.
//
// Every mbarrier wait is bounded: on expiry the kernel raises a flag in global memory, stops
// issuing work, and falls through to the common tear-down (TMEM is released).
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "api_internal.h"
#include "apnn_device.cuh"
#include "tc5_common.cuh"
#include "tc5_gemm.h"

namespace apnn {

namespace {

using tc5::BM;
using tc5::BK;

constexpr int THREADS = 320;     // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int EPI_WARPS = 8;     // two per TMEM lane quarter, splitting a tile's 32-column chunks
constexpr int MAX_STAGES = 12;
constexpr int SMEM_LIMIT = 232448;   // 227 KiB of dynamic shared memory per CTA

// Tile shape: 128 rows x BN columns; BKB bytes of K per stage row (= the swizzle span: 128,
// or 64 for operands whose K is a multiple of 64 only, e.g. 64-channel feature maps).
template <int BN, int BKB, bool PAIR = false>
struct TileCfg {
  static constexpr int A_STAGE_BYTES = BM * BKB;
  // rows of the B tile one CTA stages: all BN, or its half when two CTAs share the tile (cta_group::2)
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;
  static constexpr int B_STAGE_BYTES = B_ROWS * BKB;
  static constexpr int TMEM_COLS = 2 * BN;
  // after the operand tiles: barriers, then per epilogue warp 32 threshold entries of 16 bytes
  // and a 32 x 16-word transposition block
  static constexpr int BAR_BYTES = 512;
  static constexpr int THR_BYTES_PER_WARP = 32 * 16;
  static constexpr int XPOSE_BYTES_PER_WARP = 32 * 16 * 4;
  static constexpr int FIXED_BYTES = 1024 /*alignment slack*/ + BAR_BYTES + EPI_WARPS * (THR_BYTES_PER_WARP + XPOSE_BYTES_PER_WARP);
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
  int out_i8;            // quantised outputs as one byte per element (rows of N bytes) instead of packed planes
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
  int res16_in, res16_out;     // residual_in / residual_out hold int16 (values saturate on the way out)
  const float* affine_scale;   // OUT_FLOAT: out = float(value) * scale[c] + bias[c], [N] each
  const float* affine_bias;
  // shared-memory plan (chosen on the host)
  int stages;            // ring depth
  int kgroup;            // K blocks per stage (one barrier round trip and one commit per group)
  int splits;            // split-K instantiation only: the `splits` CTAs of a cluster share one output tile, each
                         // sums its share of the K blocks into its own TMEM; the partial sums meet in shared memory
                         // (distributed shared memory stores) before the epilogue
  int pair;              // host-side note of the PAIR instantiation: tiles_m then counts pairs of tile rows
  int b_resident;        // 1: the whole B operand (one tile column, all K blocks) stays in shared
                         // memory for the life of the CTA and the ring carries A tiles only
  // flat convolution (is_conv == 2): stride 1, no pooling.  Output positions are the flattened
  // padded pixels q = (b*Hp + h)*Wp + w (top-left anchored); a tile is 128 consecutive q, and
  // filter tap (ti, tj) reads input rows q + (ti+in_off)*Wp + tj+in_off of the flattened image
  // -- all taps of a channel block read ONE buffer of consecutive rows through row-shifted
  // descriptors, so the activations enter shared memory once per tile instead of once per tap.
  int flat_wp;           // Wp
  int flat_hpwp;         // Hp * Wp
  // floor(n / flat_hpwp) and floor(n / flat_wp) for 0 <= n < 2^31 as (n * magic) >> shift: the epilogue warps turn
  // a tile row into (image, row, column) once per tile, and a division costs them some twenty instructions
  unsigned long long magic_hpwp, magic_wp;
  int shift_hpwp, shift_wp;
  int flat_nblk;         // row blocks per channel block: 1 (all taps in one box) or R (one per filter row)
  int flat_blk_rows;     // rows per block (multiple of 8, at most 256)
  int flat_na, flat_nb;  // A-buffer ring depth; B-tile ring depth (0 when the filter is resident)
};

// Output row (units of N channels) and validity of tile row r; for pooled outputs only the
// top-left pixel of a window is a writer.
struct RowDst {
  long long row;    // output row, ring included
  long long dense;  // output row without the ring (index of the residual tensors)
  bool valid;
};
// Position of tile row r inside its pixel box: fixed for a thread over the whole kernel.
struct RowInBox {
  int wi, hi, bi;
};
__device__ __forceinline__ RowInBox row_in_box(const Tc5Params& p, int r) {
  RowInBox q = {0, 0, 0};
  if (p.is_conv == 1) {
    q.wi = r % p.bw;
    const int r2 = r / p.bw;
    q.hi = r2 % p.bh;
    q.bi = r2 / p.bh;
  }
  return q;
}
__device__ __forceinline__ RowDst row_destination(const Tc5Params& p, int tm, int r, const RowInBox& q) {
  RowDst d;
  if (!p.is_conv) {
    d.row = (long long)tm * BM + r;
    d.dense = d.row;
    d.valid = d.row < p.M;
    return d;
  }
  int b, ho, wo;
  if (p.is_conv == 2) {
    const int pos = tm * BM + r;   // below 2^31: the host checks the flattened row count
    b = (int)(((unsigned long long)(uint32_t)pos * p.magic_hpwp) >> p.shift_hpwp);
    const int rem = pos - b * p.flat_hpwp;
    ho = (int)(((unsigned long long)(uint32_t)rem * p.magic_wp) >> p.shift_wp);
    wo = rem - ho * p.flat_wp;
    d.valid = b < p.Bn && ho < p.Ho && wo < p.Wo;
  } else {
    const int tw = tm % p.tiles_w;
    const int t2 = tm / p.tiles_w;
    const int th = t2 % p.tiles_h;
    const int bg = t2 / p.tiles_h;
    b = bg * p.bb + q.bi, ho = th * p.bh + q.hi, wo = tw * p.bw + q.wi;
    d.valid = q.bi < p.bb && b < p.Bn && ho < p.Ho && wo < p.Wo;
  }
  int oh = ho, ow = wo;
  if (p.pool != POOL_NONE) {
    d.valid = d.valid && ((q.hi | q.wi) & 1) == 0;
    oh = ho >> 1;
    ow = wo >> 1;
  }
  const int hh = p.out_halo;
  d.row = ((long long)b * (p.out_h + 2 * hh) + oh + hh) * (p.out_w + 2 * hh) + ow + hh;
  d.dense = ((long long)b * p.out_h + oh) * p.out_w + ow;
  return d;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  if (tiles_n == 1) {   // one tile column: the band walk below is the identity
    tm = tile;
    tn = 0;
    return;
  }
  const int band = GROUP_M * tiles_n;
  const int g = tile / band;
  const int first = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first);
  const int r = tile - g * band;
  tm = first + r % rows;
  tn = r / rows;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Cluster-wide barrier with release / acquire semantics (all threads of all CTAs of the cluster).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
// ---- CTA pairs (cta_group::2).  PAIR = true: the even CTA of a pair (the leader) issues every MMA over 256 rows
// (its own 128-row A tile and the peer's) and both halves of the B tile; TMA loads of both CTAs complete on the
// leader's barrier; the leader's commits arrive on the barrier at the same offset in both CTAs.
template <bool PAIR>
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (PAIR) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    tc_mma_i8(d_tmem, adesc, bdesc, idesc, accumulate);
  }
}
// pair_mask: the two CTAs of this pair as bits of the cluster rank (3 << leader rank)
template <bool PAIR>
__device__ __forceinline__ void commit_to(uint32_t bar, uint16_t pair_mask) {
  if constexpr (PAIR) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(pair_mask)
                 : "memory");
  } else {
    tc_commit(bar);
  }
}
// TMA tile loads whose bytes complete on `bar`: this CTA's own barrier, or (PAIR) the leader's barrier given as a
// shared::cluster address.  No multicast.
template <bool PAIR>
__device__ __forceinline__ void load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  if constexpr (PAIR) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
        "[%4];" ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
  } else {
    tma_load_2d(dst, map, x, y, bar);
  }
}
template <bool PAIR>
__device__ __forceinline__ void load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
  if constexpr (PAIR) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, "
        "%5}], [%6];" ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
        : "memory");
  } else {
    tma_load_4d(dst, map, c0, c1, c2, c3, bar);
  }
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// The MMAs of G consecutive K blocks: A tiles G x 128 rows at sa, B tiles G x BN rows at sb.
template <int BN, int BKB, int G, bool PAIR>
__device__ __forceinline__ void issue_group(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t idesc, bool accumulate) {
  constexpr int A_BYTES = BM * BKB, B_BYTES = TileCfg<BN, BKB, PAIR>::B_STAGE_BYTES;
#pragma unroll
  for (int g = 0; g < G; g++) {
    const uint64_t adesc = make_smem_desc_k<BKB>(sa + g * A_BYTES);
    const uint64_t bdesc = make_smem_desc_k<BKB>(sb + g * B_BYTES);
#pragma unroll
    for (int k = 0; k < BKB / 32; k++) {
      // advancing 32 bytes along K inside the swizzle row = +2 in 16-byte units
      mma_i8<PAIR>(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (accumulate || (g | k) != 0) ? 1u : 0u);
    }
  }
}

// Flat convolution, resident filter: the MMAs of all RR x RR taps of one channel block as
// straight-line code.  Descriptors differ only in their 14-bit address field, so they are
// advanced as 32-bit adds on the low word.  a_lo / b_lo: low descriptor words of the buffer and
// of tap 0's filter tile; row_step: 16-byte units between filter rows in the buffer;
// b_step: 16-byte units between consecutive taps' filter tiles.
template <int BKB, int RR, bool PAIR>
__device__ __forceinline__ void flat_issue_taps(uint32_t d_tmem, uint32_t a_lo, uint32_t row_step, uint32_t b_lo,
                                                uint32_t b_step, uint32_t desc_hi, uint32_t idesc, uint32_t& enable) {
#pragma unroll
  for (int ti = 0; ti < RR; ti++) {
#pragma unroll
    for (int tj = 0; tj < RR; tj++) {
      const uint32_t a_tap = a_lo + ti * row_step + tj * (BKB / 16);
      const uint32_t b_tap = b_lo + (ti * RR + tj) * b_step;
#pragma unroll
      for (int k = 0; k < BKB / 32; k++) {
        const uint64_t adesc = ((uint64_t)desc_hi << 32) | (a_tap + 2u * k);
        const uint64_t bdesc = ((uint64_t)desc_hi << 32) | (b_tap + 2u * k);
        mma_i8<PAIR>(d_tmem, adesc, bdesc, idesc, enable);
        enable = 1u;
      }
    }
  }
}

// The same with the filter tiles arriving through their ring: wait, issue, release per tap.
// Returns false when a wait ran out of time.
template <int BKB, int RR, bool PAIR>
__device__ __forceinline__ bool flat_issue_taps_ring(uint32_t d_tmem, uint32_t a_lo, uint32_t row_step, uint32_t lo0,
                                                     uint32_t bring, uint32_t b_bytes, uint32_t bfull0, uint32_t bempty0,
                                                     int nb, int& sb, uint32_t& phb, uint32_t desc_hi, uint32_t idesc,
                                                     uint32_t& enable, uint16_t pair_mask) {
#pragma unroll
  for (int ti = 0; ti < RR; ti++) {
#pragma unroll
    for (int tj = 0; tj < RR; tj++) {
      const uint32_t a_tap = a_lo + ti * row_step + tj * (BKB / 16);
      if (!mbar_wait(bfull0 + 8u * sb, phb)) return false;
      tc_fence_after();
      const uint32_t b_tap = lo0 | (((bring + (uint32_t)sb * b_bytes) & 0x3FFFFu) >> 4);
#pragma unroll
      for (int k = 0; k < BKB / 32; k++) {
        mma_i8<PAIR>(d_tmem, ((uint64_t)desc_hi << 32) | (a_tap + 2u * k), ((uint64_t)desc_hi << 32) | (b_tap + 2u * k), idesc,
                     enable);
        enable = 1u;
      }
      commit_to<PAIR>(bempty0 + 8u * sb, pair_mask);
      if (++sb == nb) { sb = 0; phb ^= 1u; }
    }
  }
  return true;
}

// EPI selects an epilogue compiled for one family of uses (the code of the other paths is
// compiled out; these warps are bound by instruction fetch and issue, so the smaller bodies
// are measurably faster):
//   0  everything decided at run time
//   1  quantise only (thresholds or low bits; packed planes or int8 rows): no pooling, residuals or int32 output
//   2  thresholds of at most 2 bits -> int8 rows, nothing else (hidden layers of the networks)
//   3  as 2 plus residual in / out of either width (second convolution of a ResNet block)
//   4  as 3 with every residual tensor present being int16 (no int32 residual code)
//   5  int32 output only (shortcut convolutions, logits)
//
// SPLITK: the kernel is launched as clusters of p.splits CTAs (2, 4 or 8) with one output tile per
// cluster, for problems with fewer tiles than SMs and a long K.  CTA r of a cluster accumulates K
// blocks [r*kblocks/splits, (r+1)*kblocks/splits) in its own TMEM.  Then, with the operand ring idle, every
// CTA splits its 128 x BN partial tile into p.splits column slices, keeps its own slice in TMEM and stores
// slice o into slot r of CTA o's shared memory (st.shared::cluster); after a cluster barrier CTA o adds the
// slots of its slice to its own partial sums and runs the ordinary epilogue on those columns.  No atomics,
// no global scratch, no second launch.
//
// PAIR: two CTAs of a cluster share every B tile (tcgen05 cta_group::2).  Output tiles are taken in pairs of
// adjacent tile rows: CTA `rank & 1` of a pair owns tile row 2*t + (rank & 1), stages its own 128-row A tile
// and its half of the B tile, and drains its own TMEM; the even CTA issues the MMAs for both (M = 256).  Per
// MMA every SM writes and reads a third fewer operand bytes than alone, which is what bounds the wide
// layers.  With SPLITK the cluster holds `splits` such pairs, and a CTA exchanges partial sums with the
// CTAs of the other pairs that own the same tile row.
// R5: the flat convolution's 5 x 5 taps as straight-line MMAs too (3 x 3 and 1 x 1 always are).  A parameter of its own,
// instantiated for the hidden-layer epilogue only: with the fifty extra MMAs inlined into every instantiation the code
// of the other roles moved and the 3 x 3 layers of ResNet-18 ran 1 % slower.
template <int BN, int BKB, bool SPLITK = false, int EPI = 0, bool PAIR = false, bool R5 = false>
__global__ void __launch_bounds__(THREADS, 1)
tc5_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const Tc5Params p) {
  using Cfg = TileCfg<BN, BKB, PAIR>;
  constexpr int A_STAGE_BYTES = Cfg::A_STAGE_BYTES;
  constexpr int B_STAGE_BYTES = Cfg::B_STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  // layout: [resident B: kblocks x B tile] [stages x (A tile [+ B tile])] [barriers] [thresholds] [transposition]
  const int stages = p.stages;
  const uint32_t bres_bytes = p.b_resident ? (uint32_t)p.kblocks * B_STAGE_BYTES : 0u;
  const int kgroup = p.kgroup;
  const bool flat = p.is_conv == 2;
  const uint32_t flat_a_bytes = (uint32_t)(p.flat_nblk * p.flat_blk_rows) * BKB;
  const uint32_t stage_bytes =
      flat ? flat_a_bytes : (uint32_t)kgroup * (A_STAGE_BYTES + (p.b_resident ? 0 : B_STAGE_BYTES));
  const uint32_t ring = base + bres_bytes;
  const uint32_t bring = ring + (uint32_t)stages * stage_bytes;   // flat: B-tile ring
  const uint32_t bars = bring + (flat ? (uint32_t)p.flat_nb * B_STAGE_BYTES : 0u);
  // barriers (8 bytes each): full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2], b_resident, then the TMEM pointer
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * MAX_STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * MAX_STAGES + 2 + a); };
  const uint32_t bres_bar = bars + 8u * (2 * MAX_STAGES + 4);
  const uint32_t tmem_slot = bars + 8u * (2 * MAX_STAGES + 5);
  // flat convolution: the ring above holds A buffers (full_bar / empty_bar), a second ring of B tiles follows
  auto bfull_bar = [&](int s) { return bars + 8u * (2 * MAX_STAGES + 6 + s); };
  auto bempty_bar = [&](int s) { return bars + 8u * (3 * MAX_STAGES + 6 + s); };
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  uint8_t* epi_smem = smem_raw + (bars + Cfg::BAR_BYTES - raw);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) *p.error_flag = 0;  // only ever raised after a 2 s wait, long after this store
    for (int s = 0; s < stages; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), PAIR ? 2 * EPI_WARPS : EPI_WARPS);   // the leader's collects both CTAs' epilogue warps
    }
    mbar_init(bres_bar, 1);
    if (flat)
      for (int s = 0; s < p.flat_nb; s++) {
        mbar_init(bfull_bar(s), 1);
        mbar_init(bempty_bar(s), 1);
      }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                   "r"(Cfg::TMEM_COLS));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                   "r"(Cfg::TMEM_COLS));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // the peer's barriers exist before anything remote touches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Everything above may overlap the previous kernel's tail (programmatic dependent launch); the roles
  // that touch global memory wait for that kernel below, each before its first access.

  const int num_tiles = p.tiles_m * p.tiles_n;
  // Tiles go round-robin over the grid; with split-K there is one tile per cluster and CTA r of the
  // cluster takes K blocks [r*kblocks/splits, (r+1)*kblocks/splits).  These are evaluated inside each
  // role (TILE_FIRST / TILE_STEP read %ctaid / %nctaid where they are used): hoisting them into
  // variables shared by the roles made the epilogue-bound layer kernels up to 15 % slower.
  // PAIR: p.tiles_m counts pairs of tile rows, a "tile" below is such a pair x one tile column, and this CTA's own
  // tile row is 2 * tm + PRANK.
#define CLUSTER_CTAS ((PAIR ? 2 : 1) * (SPLITK ? p.splits : 1))
#define TILE_FIRST ((SPLITK || PAIR) ? (int)blockIdx.x / CLUSTER_CTAS : (int)blockIdx.x)
#define TILE_STEP ((SPLITK || PAIR) ? (int)gridDim.x / CLUSTER_CTAS : (int)gridDim.x)
#define PRANK (PAIR ? (cluster_ctarank() & 1u) : 0u)                     /* 0: the pair's leader */
#define SPLIT_RANK (PAIR ? (cluster_ctarank() >> 1) : cluster_ctarank()) /* which share of K */
#define KB_FIRST (SPLITK ? (int)(((long long)SPLIT_RANK * p.kblocks) / p.splits) : 0)
#define KB_LAST (SPLITK ? (int)(((long long)(SPLIT_RANK + 1) * p.kblocks) / p.splits) : p.kblocks)

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      grid_dependency_wait();   // the first load of anything an earlier kernel wrote comes after this
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      // PAIR: every load of either CTA completes its bytes on the leader's barrier (same offset, CTA rank & ~1);
      // the leader announces both CTAs' bytes
      const uint32_t prank = PRANK;
      const bool announces = !PAIR || prank == 0;
      const uint32_t tx_mult = PAIR ? 2u : 1u;
      const uint32_t bar_delta = PAIR ? map_to_cta(bars, cluster_ctarank() & ~1u) - bars : 0u;   // own -> leader's window
      const int b_row0 = (int)prank * Cfg::B_ROWS;   // this CTA's rows inside a B tile
      if (p.b_resident && TILE_FIRST < num_tiles) {
        // tiles_n == 1: every tile of this CTA uses the same B rows; fetch all K blocks once
        if (announces) mbar_expect_tx(bres_bar, tx_mult * bres_bytes);
        for (int kb = 0; kb < p.kblocks; kb++)
          load_2d<PAIR>(base + (uint32_t)kb * B_STAGE_BYTES, &map_b, kb * BKB, b_row0, bres_bar + bar_delta);
      }
      const uint32_t stage_tx = (uint32_t)kgroup * ((p.is_conv ? p.a_box_bytes : (uint32_t)A_STAGE_BYTES) +
                                                    (p.b_resident ? 0u : (uint32_t)B_STAGE_BYTES));
      if (flat) {
        // one buffer of consecutive input rows per (tile, channel block); then, unless the filter
        // is resident, the B tile of each tap through its own ring
        int sb = 0;
        uint32_t phb = 0;
        const int taps = p.R * p.R;
        const uint32_t blk_bytes = (uint32_t)p.flat_blk_rows * BKB;
        for (int tile = TILE_FIRST; tile < num_tiles && ok; tile += TILE_STEP) {
          int tm, tn;
          tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
          if constexpr (PAIR) tm = 2 * tm + (int)prank;
          const int q0 = tm * BM + p.in_off * p.flat_wp + p.in_off;
          for (int cb = 0; cb < p.cblocks && ok; cb++) {
            if (!mbar_wait(empty_bar(s), ph ^ 1u)) { ok = false; break; }
            const uint32_t sa = ring + (uint32_t)s * stage_bytes;
            if (announces) mbar_expect_tx(full_bar(s), tx_mult * flat_a_bytes);
            for (int blk = 0; blk < p.flat_nblk; blk++)
              load_2d<PAIR>(sa + blk * blk_bytes, &map_a, cb * BKB, q0 + blk * p.flat_wp, full_bar(s) + bar_delta);
            if (++s == stages) { s = 0; ph ^= 1u; }
            if (!p.b_resident) {
              for (int tap = 0; tap < taps; tap++) {
                if (!mbar_wait(bempty_bar(sb), phb ^ 1u)) { ok = false; break; }
                if (announces) mbar_expect_tx(bfull_bar(sb), tx_mult * B_STAGE_BYTES);
                load_2d<PAIR>(bring + (uint32_t)sb * B_STAGE_BYTES, &map_b, (tap * p.cblocks + cb) * BKB, tn * BN + b_row0,
                              bfull_bar(sb) + bar_delta);
                if (++sb == p.flat_nb) { sb = 0; phb ^= 1u; }
              }
            }
          }
        }
      } else
      for (int tile = TILE_FIRST; tile < num_tiles && ok; tile += TILE_STEP) {
        int tm, tn;
        const int kb0 = KB_FIRST, kb1 = KB_LAST;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        if constexpr (PAIR) tm = 2 * tm + (int)prank;
        int w0 = 0, h0 = 0, b0 = 0;
        if (p.is_conv) {
          w0 = (tm % p.tiles_w) * p.bw;
          const int t2 = tm / p.tiles_w;
          h0 = (t2 % p.tiles_h) * p.bh;
          b0 = (t2 / p.tiles_h) * p.bb;
        }
        int ti = 0, tj = 0, cb = 0;  // conv: K block = (filter tap row, tap column, BKB-channel block)
        if (SPLITK && p.is_conv) {
          cb = kb0 % p.cblocks;
          const int tap = kb0 / p.cblocks;
          tj = tap % p.R;
          ti = tap / p.R;
        }
        const int wbase = w0 * p.stride + p.in_off, hbase = h0 * p.stride + p.in_off;
        for (int kb = kb0; kb < kb1; kb += kgroup) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) { ok = false; break; }
          const uint32_t sa = ring + (uint32_t)s * stage_bytes;
          const uint32_t sb = sa + (uint32_t)kgroup * A_STAGE_BYTES;
          if (announces) mbar_expect_tx(full_bar(s), tx_mult * stage_tx);
          for (int g = 0; g < kgroup; g++) {
            if (!p.is_conv) {
              load_2d<PAIR>(sa + g * A_STAGE_BYTES, &map_a, (kb + g) * BKB, tm * BM, full_bar(s) + bar_delta);
            } else {
              load_4d<PAIR>(sa + g * A_STAGE_BYTES, &map_a, cb * BKB, wbase + tj, hbase + ti, b0, full_bar(s) + bar_delta);
              if (++cb == p.cblocks) {
                cb = 0;
                if (++tj == p.R) { tj = 0; ti++; }
              }
            }
            if (!p.b_resident)
              load_2d<PAIR>(sb + g * B_STAGE_BYTES, &map_b, (kb + g) * BKB, tn * BN + b_row0, full_bar(s) + bar_delta);
          }
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) atomicExch(p.error_flag, 1);
    }
    if constexpr (SPLITK) {   // the two cluster barriers of the partial-sum exchange (every thread takes part)
      __syncwarp();
      cluster_sync_all();
      cluster_sync_all();
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (PAIR: the pair's leader only) ----------------
    if (lane == 0 && PRANK == 0) {
      const uint16_t pair_mask = PAIR ? (uint16_t)(3u << (cluster_ctarank() & ~1u)) : (uint16_t)0;   // both CTAs of this pair
      int s = 0;
      uint32_t ph = 0;
      uint32_t tl = 0;
      bool ok = true;
      if (p.b_resident && TILE_FIRST < num_tiles) {
        ok = mbar_wait(bres_bar, 0u);
        tc_fence_after();
      }
      if (flat) {
        int sb = 0;
        uint32_t phb = 0;
        for (int tile = TILE_FIRST; tile < num_tiles && ok; tile += TILE_STEP, tl++) {
          const uint32_t acc = tl & 1u;
          const uint32_t aph = (tl >> 1) & 1u;
          if (!mbar_wait(tempty_bar(acc), aph ^ 1u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int cb = 0; cb < p.cblocks && ok; cb++) {
            if (!mbar_wait(full_bar(s), ph)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = ring + (uint32_t)s * stage_bytes;
            if (p.R == 3 || p.R == 1 || (R5 && p.R == 5)) {   // straight-line taps; other filters take the loop below
              const uint64_t d0 = make_smem_desc_k<BKB>(0);
              const uint32_t desc_hi = (uint32_t)(d0 >> 32), lo0 = (uint32_t)d0;
              const uint32_t a_lo = lo0 | ((sa & 0x3FFFFu) >> 4);
              const uint32_t row_step = (uint32_t)(p.flat_nblk == 1 ? p.flat_wp : p.flat_blk_rows) * (BKB / 16);
              uint32_t enable = cb != 0 ? 1u : 0u;
              if (p.b_resident) {
                const uint32_t b_lo = lo0 | (((base + (uint32_t)cb * B_STAGE_BYTES) & 0x3FFFFu) >> 4);
                const uint32_t b_step = (uint32_t)p.cblocks * (B_STAGE_BYTES / 16);
                if (R5 && p.R == 5) {
                  if constexpr (R5) flat_issue_taps<BKB, 5, PAIR>(d_tmem, a_lo, row_step, b_lo, b_step, desc_hi, p.idesc, enable);
                } else if (p.R == 3) flat_issue_taps<BKB, 3, PAIR>(d_tmem, a_lo, row_step, b_lo, b_step, desc_hi, p.idesc, enable);
                else flat_issue_taps<BKB, 1, PAIR>(d_tmem, a_lo, row_step, b_lo, b_step, desc_hi, p.idesc, enable);
              } else {
                if (R5 && p.R == 5) {
                  if constexpr (R5)
                    ok = flat_issue_taps_ring<BKB, 5, PAIR>(d_tmem, a_lo, row_step, lo0, bring, B_STAGE_BYTES, bfull_bar(0),
                                                            bempty_bar(0), p.flat_nb, sb, phb, desc_hi, p.idesc, enable, pair_mask);
                } else
                ok = p.R == 3 ? flat_issue_taps_ring<BKB, 3, PAIR>(d_tmem, a_lo, row_step, lo0, bring, B_STAGE_BYTES, bfull_bar(0),
                                                                   bempty_bar(0), p.flat_nb, sb, phb, desc_hi, p.idesc, enable,
                                                                   pair_mask)
                              : flat_issue_taps_ring<BKB, 1, PAIR>(d_tmem, a_lo, row_step, lo0, bring, B_STAGE_BYTES, bfull_bar(0),
                                                                   bempty_bar(0), p.flat_nb, sb, phb, desc_hi, p.idesc, enable,
                                                                   pair_mask);
                if (!ok) break;
              }
              commit_to<PAIR>(empty_bar(s), pair_mask);
              if (++s == stages) { s = 0; ph ^= 1u; }
              continue;
            }
            int tap = 0;
            for (int ti = 0; ti < p.R && ok; ti++) {
              // rows of the buffer this filter row starts at: ti image rows down (one box), or block ti
              const uint32_t row_a = p.flat_nblk == 1 ? (uint32_t)(ti * p.flat_wp) : (uint32_t)(ti * p.flat_blk_rows);
              for (int tj = 0; tj < p.R; tj++, tap++) {
                // a descriptor may start at any row: the swizzle is a function of the shared-memory address
                const uint64_t adesc = make_smem_desc_k<BKB>(sa + (row_a + tj) * BKB);
                uint64_t bdesc;
                if (p.b_resident) {
                  bdesc = make_smem_desc_k<BKB>(base + (uint32_t)(tap * p.cblocks + cb) * B_STAGE_BYTES);
                } else {
                  if (!mbar_wait(bfull_bar(sb), phb)) { ok = false; break; }
                  tc_fence_after();
                  bdesc = make_smem_desc_k<BKB>(bring + (uint32_t)sb * B_STAGE_BYTES);
                }
#pragma unroll
                for (int k = 0; k < BKB / 32; k++)
                  mma_i8<PAIR>(d_tmem, adesc + 2u * k, bdesc + 2u * k, p.idesc, (cb | tap | k) != 0 ? 1u : 0u);
                if (!p.b_resident) {
                  commit_to<PAIR>(bempty_bar(sb), pair_mask);
                  if (++sb == p.flat_nb) { sb = 0; phb ^= 1u; }
                }
              }
            }
            commit_to<PAIR>(empty_bar(s), pair_mask);  // the buffer is free once every tap has read it
            if (++s == stages) { s = 0; ph ^= 1u; }
          }
          if (ok) commit_to<PAIR>(tfull_bar(acc), pair_mask);
        }
      } else
      for (int tile = TILE_FIRST; tile < num_tiles && ok; tile += TILE_STEP, tl++) {
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb0 = KB_FIRST, kb1 = KB_LAST;
        for (int kb = kb0; kb < kb1; kb += kgroup) {
          if (!mbar_wait(full_bar(s), ph)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = ring + (uint32_t)s * stage_bytes;
          const uint32_t sb = sa + (uint32_t)kgroup * A_STAGE_BYTES;
          const uint32_t b0addr = p.b_resident ? base + (uint32_t)kb * B_STAGE_BYTES : sb;
          // unrolled per group size: this thread's instruction stream is on the critical path
          switch (kgroup) {
            case 1: issue_group<BN, BKB, 1, PAIR>(d_tmem, sa, b0addr, p.idesc, kb != kb0); break;
            case 2: issue_group<BN, BKB, 2, PAIR>(d_tmem, sa, b0addr, p.idesc, kb != kb0); break;
            default: issue_group<BN, BKB, 3, PAIR>(d_tmem, sa, b0addr, p.idesc, kb != kb0); break;
          }
          commit_to<PAIR>(empty_bar(s), pair_mask);  // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        if (ok) commit_to<PAIR>(tfull_bar(acc), pair_mask);  // accumulator complete (both CTAs of a pair)
      }
      if (!ok) atomicExch(p.error_flag, 2);
    }
    if constexpr (SPLITK) {
      __syncwarp();
      cluster_sync_all();
      cluster_sync_all();
    }
  } else {
    // ---------------- epilogue warps (2..9) ----------------
    constexpr bool C_NOPOOL = EPI >= 1, C_NORES = EPI == 1 || EPI == 2 || EPI == 5, C_NOINT32 = EPI >= 1 && EPI <= 4;
    constexpr bool C_I8THR = EPI >= 2 && EPI <= 4, C_RES16 = EPI == 4, C_INT32 = EPI == 5;
    grid_dependency_wait();   // residual reads and every store of this kernel come after this
    const int ew = warp - 2;
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
    const int half = ew >> 2;      // this warp drains the tile's 32-column chunks half, half+2, ...
    uint32_t tl = 0;
    bool ok = true;
    const int nl = (1 << p.out_bits) - 1;
    // thresholds of up to 2-bit outputs are staged per chunk in this warp's shared-memory
    // slice, one int4 per column (unused slots = INT_MAX), so a value costs one broadcast
    // 16-byte load instead of nl global loads
    const bool thr_staged = C_I8THR || (!C_INT32 && p.out_mode == OUT_THRESHOLDS && nl <= 3);
    int4* thr_s = reinterpret_cast<int4*>(epi_smem + ew * Cfg::THR_BYTES_PER_WARP);
    // 32 rows x 16 words, 16-byte groups XOR-swizzled by (row >> 1): both the row-per-lane
    // accesses and the 4-lanes-per-row accesses below are free of bank conflicts
    uint32_t* xp = reinterpret_cast<uint32_t*>(epi_smem + EPI_WARPS * Cfg::THR_BYTES_PER_WARP +
                                               ew * Cfg::XPOSE_BYTES_PER_WARP);
    auto swz = [](int r, int g) { return r * 16 + (((g ^ (r >> 1)) & 3) << 2); };
    const bool vec_rows = (p.N & 3) == 0;
    const int sub_r = lane >> 2, grp = lane & 3;
    const RowInBox in_box = row_in_box(p, quarter * 32 + lane);
    constexpr int THR_CHUNKS = BN >= 64 ? BN / 64 : 1;   // chunks per epilogue warp
    int4 thr_of[THR_CHUNKS];
    int thr_tn = -1;
    // 32-column chunks of the tile this CTA finishes: all of them, or (split-K) its slice of the cluster's tile
    const int slice_chunks = SPLITK ? (BN / 32) / p.splits : BN / 32;
    const int crank = SPLITK ? (int)SPLIT_RANK : 0;   // this CTA's share of K = its slot in the exchange
    const int c_first = crank * slice_chunks;
    const int c_end = c_first + slice_chunks;
    const int c_begin = c_first + half;   // this warp's first chunk; it takes every second one
    // Row destinations of a tile: this lane's own row, and (for int32 rows and residuals) the
    // rows it serves in the coalesced 4-lanes-per-row accesses.
    struct TileRows {
      int tn;
      RowDst dst;
      long long row_of[4], dense_of[4];
      bool ok_of[4];
    };
    auto rows_of_tile = [&](int tile, TileRows& t) {
      int tm;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, t.tn);
      if constexpr (PAIR) tm = 2 * tm + (int)PRANK;
      t.dst = row_destination(p, tm, quarter * 32 + lane, in_box);
      if constexpr (!(C_NORES && C_NOINT32)) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          t.row_of[i] = __shfl_sync(0xffffffffu, t.dst.row, 8 * i + sub_r);
          t.dense_of[i] = __shfl_sync(0xffffffffu, t.dst.dense, 8 * i + sub_r);
          t.ok_of[i] = __shfl_sync(0xffffffffu, (int)t.dst.valid, 8 * i + sub_r) != 0;
        }
      }
    };
    // residual rows of a chunk, fetched ahead of their use as 64-byte row segments: the next
    // chunk's while this one finishes, the next TILE's first chunk while this tile finishes
    // (the wait for the accumulator is short when the epilogue is the bound, so a fetch
    // issued at the top of a tile would expose the whole memory latency every tile)
    uint4 rin[8];
    auto fetch_residual = [&](const TileRows& t, int c) {
      const int col0 = t.tn * BN + c * 32;
      if (p.residual_in == nullptr || !vec_rows || col0 + 32 > p.N) return;
      if (C_RES16 || p.res16_in) {
        // int16 rows: 64 bytes per row and chunk, 8 values per lane and load
        const int16_t* R16 = reinterpret_cast<const int16_t*>(p.residual_in);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          rin[i] = make_uint4(0u, 0u, 0u, 0u);
          if (t.ok_of[i]) rin[i] = __ldg(reinterpret_cast<const uint4*>(R16 + t.dense_of[i] * p.N + col0 + 8 * grp));
        }
        return;
      }
      if constexpr (!C_RES16) {
#pragma unroll
        for (int hf = 0; hf < 2; hf++)
#pragma unroll
          for (int i = 0; i < 4; i++) {
            rin[4 * hf + i] = make_uint4(0u, 0u, 0u, 0u);
            if (t.ok_of[i])
              rin[4 * hf + i] =
                  __ldg(reinterpret_cast<const uint4*>(p.residual_in + t.dense_of[i] * p.N + col0 + 16 * hf + 4 * grp));
          }
      }
    };
    TileRows cur, nxt;
    if (TILE_FIRST < num_tiles) {
      rows_of_tile(TILE_FIRST, cur);
      if constexpr (!C_NORES) fetch_residual(cur, c_begin);
    }
    nxt = cur;
    for (int tile = TILE_FIRST; tile < num_tiles && ok; tile += TILE_STEP, tl++) {
      const int tn = cur.tn;
      const uint32_t acc = tl & 1u;
      const uint32_t aph = (tl >> 1) & 1u;
      if (thr_staged && tn != thr_tn) {
        // this lane's column of each chunk the warp drains; reloaded only when the tile column changes
#pragma unroll
        for (int i = 0; i < THR_CHUNKS; i++) {
          const int col = tn * BN + (c_begin + 2 * i) * 32 + lane;
          int4 t4 = make_int4(0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff);
          if (col < p.N) {
            const int32_t* T = p.thresholds + (long long)col * nl;
            t4.x = __ldg(T);
            if (nl > 1) { t4.y = __ldg(T + 1); t4.z = __ldg(T + 2); }
          }
          thr_of[i] = t4;
        }
        thr_tn = tn;
      }
      const RowDst dst = cur.dst;
      const long long row = dst.row;
      const bool row_ok = dst.valid;
      const long long(&row_of)[4] = cur.row_of;
      const long long(&dense_of)[4] = cur.dense_of;
      const bool(&ok_of)[4] = cur.ok_of;
      const bool has_next = tile + TILE_STEP < num_tiles;
      bool nxt_ready = false, nxt_fetched = false;
      if (C_NORES && has_next) {   // no residuals: nothing to overlap, do it before the wait
        rows_of_tile(tile + TILE_STEP, nxt);
        nxt_ready = true;
      }
      const bool acc_ok = mbar_wait(tfull_bar(acc), aph);
      if (!acc_ok) ok = false;
      if (!SPLITK && !acc_ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      // split-K exchange area: the operand ring, idle once every CTA of the cluster has its accumulator.
      // Slot s (the partial sums of CTA s) of this CTA's slice: 16-byte groups of 4 columns, group g of row r
      // at ((s * groups + g) * 128 + r) * 16 -- a warp's accesses are 512 contiguous bytes.
      const uint32_t xch = ring;
      const int row_in_tile = quarter * 32 + lane;
      if constexpr (SPLITK) {
        __syncwarp();
        cluster_sync_all();   // all accumulators of the cluster are complete, all operand rings idle
        const int groups = slice_chunks * 8;   // 16-byte groups per row of a slice
        if (acc_ok) {
#pragma unroll 1
          for (int c = half; c < BN / 32; c += 2) {
            const int owner = c / slice_chunks;
            if (owner == crank) continue;   // this CTA's own slice stays in its TMEM until the sums are formed below
            uint32_t v[32];
            tmem_ld32(taddr + c * 32, v);
            tmem_ld_wait();
            const int g0 = (c - owner * slice_chunks) * 8;
            // the CTA of split `owner` that holds the same tile row: same position inside its pair
            const uint32_t owner_cta = PAIR ? (((uint32_t)owner << 1) | PRANK) : (uint32_t)owner;
            const uint32_t dst = map_to_cta(xch, owner_cta) + (uint32_t)(((crank * groups + g0) * BM + row_in_tile) * 16);
#pragma unroll
            for (int g = 0; g < 8; g++)
              st_cluster_v4(dst + (uint32_t)(g * BM * 16), v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
          }
        }
        __syncwarp();
        cluster_sync_all();   // every slot of every slice has landed
        if (!ok) break;
      }
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 2) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) continue;  // uniform over the warp
        uint32_t v[32];
        if constexpr (SPLITK) {
          // own partial sums from TMEM, the other CTAs' from their slots of the exchange area
          const int groups = slice_chunks * 8;
          const int g0 = (c - c_first) * 8;
          __syncwarp();   // lanes that left the previous chunk early rejoin before the warp-wide TMEM load
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
          for (int sl = 0; sl < p.splits; sl++) {
            if (sl == crank) continue;
            const uint32_t src = xch + (uint32_t)(((sl * groups + g0) * BM + row_in_tile) * 16);
#pragma unroll
            for (int g = 0; g < 8; g++) {
              const uint4 x = ld_shared_v4(src + (uint32_t)(g * BM * 16));
              v[4 * g] += x.x; v[4 * g + 1] += x.y; v[4 * g + 2] += x.z; v[4 * g + 3] += x.w;
            }
          }
        } else {
          // (lanes whose row is outside the output skip the stores of a chunk but meet the others again at the
          // loop increment, so this warp-wide load runs converged; an explicit __syncwarp() here was measured
          // to cost 2 % on the epilogue-bound 64-channel layers)
          tmem_ld32(taddr + c * 32, v);
        }
        if (thr_staged) {
          __syncwarp();   // the previous chunk's readers are done
          thr_s[lane] = thr_of[(c - c_first) >> 1];
          __syncwarp();
        }
        if constexpr (!SPLITK) tmem_ld_wait();
        if (!C_NOPOOL && p.pool != POOL_NONE) {
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
        const bool whole = vec_rows && col0 + 32 <= p.N;   // uniform: 16-byte accesses cover the chunk
        if (!C_NORES && (p.residual_in != nullptr || p.residual_out != nullptr)) {
          if (whole) {
            // int32 rows move through the transposition block so that global accesses are
            // 64 contiguous bytes per row, 8 rows per instruction
            // acc + the signed low / high half of w in one instruction each (a two-way dot product with (1, 0) / (0, 1))
            auto add_lo16 = [](uint32_t acc, uint32_t w) { return (uint32_t)__dp2a_lo((int)w, 0x00000001, (int)acc); };
            auto add_hi16 = [](uint32_t acc, uint32_t w) { return (uint32_t)__dp2a_lo((int)w, 0x00000100, (int)acc); };
            // two int32 -> two saturated int16 in one word (lo in the low half)
            auto sat_pack = [](uint32_t lo, uint32_t hi) {
              uint32_t d;
              asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(d) : "r"((int)hi), "r"((int)lo));
              return d;
            };
            if (p.residual_in != nullptr && (C_RES16 || p.res16_in)) {
#pragma unroll
              for (int i = 0; i < 4; i++) *reinterpret_cast<uint4*>(xp + swz(8 * i + sub_r, grp)) = rin[i];
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 4; j++) {
                const uint4 x = *reinterpret_cast<const uint4*>(xp + swz(lane, j));
                v[8 * j] = add_lo16(v[8 * j], x.x); v[8 * j + 1] = add_hi16(v[8 * j + 1], x.x);
                v[8 * j + 2] = add_lo16(v[8 * j + 2], x.y); v[8 * j + 3] = add_hi16(v[8 * j + 3], x.y);
                v[8 * j + 4] = add_lo16(v[8 * j + 4], x.z); v[8 * j + 5] = add_hi16(v[8 * j + 5], x.z);
                v[8 * j + 6] = add_lo16(v[8 * j + 6], x.w); v[8 * j + 7] = add_hi16(v[8 * j + 7], x.w);
              }
              __syncwarp();
              if (c + 2 < c_end) fetch_residual(cur, c + 2);
              else if (has_next) { rows_of_tile(tile + TILE_STEP, nxt); fetch_residual(nxt, c_begin); nxt_ready = nxt_fetched = true; }
            } else if (!C_RES16 && p.residual_in != nullptr) {
#pragma unroll
              for (int hf = 0; hf < 2; hf++) {
#pragma unroll
                for (int i = 0; i < 4; i++) *reinterpret_cast<uint4*>(xp + swz(8 * i + sub_r, grp)) = rin[4 * hf + i];
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  const uint4 x = *reinterpret_cast<const uint4*>(xp + swz(lane, j));
                  v[16 * hf + 4 * j] += x.x; v[16 * hf + 4 * j + 1] += x.y;
                  v[16 * hf + 4 * j + 2] += x.z; v[16 * hf + 4 * j + 3] += x.w;
                }
                __syncwarp();
              }
              if (c + 2 < c_end) fetch_residual(cur, c + 2);   // the next chunk's rows, in flight during this one's tail
              else if (has_next) { rows_of_tile(tile + TILE_STEP, nxt); fetch_residual(nxt, c_begin); nxt_ready = nxt_fetched = true; }
            }
            if (p.residual_out != nullptr && (C_RES16 || p.res16_out)) {
              int16_t* O16 = reinterpret_cast<int16_t*>(p.residual_out);
#pragma unroll
              for (int j = 0; j < 4; j++)
                *reinterpret_cast<uint4*>(xp + swz(lane, j)) =
                    make_uint4(sat_pack(v[8 * j], v[8 * j + 1]), sat_pack(v[8 * j + 2], v[8 * j + 3]),
                               sat_pack(v[8 * j + 4], v[8 * j + 5]), sat_pack(v[8 * j + 6], v[8 * j + 7]));
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const uint4 x = *reinterpret_cast<const uint4*>(xp + swz(8 * i + sub_r, grp));
                if (ok_of[i]) *reinterpret_cast<uint4*>(O16 + dense_of[i] * p.N + col0 + 8 * grp) = x;
              }
              __syncwarp();
            } else if (!C_RES16 && p.residual_out != nullptr) {
#pragma unroll
              for (int hf = 0; hf < 2; hf++) {
#pragma unroll
                for (int j = 0; j < 4; j++)
                  *reinterpret_cast<uint4*>(xp + swz(lane, j)) =
                      make_uint4(v[16 * hf + 4 * j], v[16 * hf + 4 * j + 1], v[16 * hf + 4 * j + 2], v[16 * hf + 4 * j + 3]);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; i++) {
                  const uint4 x = *reinterpret_cast<const uint4*>(xp + swz(8 * i + sub_r, grp));
                  if (ok_of[i])
                    *reinterpret_cast<uint4*>(p.residual_out + dense_of[i] * p.N + col0 + 16 * hf + 4 * grp) = x;
                }
                __syncwarp();
              }
            }
          } else if (row_ok) {
            const long long at = dst.dense * (long long)p.N + col0;
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < p.N) {
                if (p.residual_in != nullptr)
                  v[j] = (uint32_t)((int)v[j] + (p.res16_in ? (int)__ldg(reinterpret_cast<const int16_t*>(p.residual_in) + at + j)
                                                             : __ldg(p.residual_in + at + j)));
                if (p.residual_out != nullptr) {
                  if (p.res16_out) reinterpret_cast<int16_t*>(p.residual_out)[at + j] = (int16_t)min(max((int)v[j], -32768), 32767);
                  else p.residual_out[at + j] = (int32_t)v[j];
                }
              }
          }
        }
        if (!C_NOINT32 && !C_INT32 && p.out_mode == OUT_FLOAT) {
          // batch-norm affine of an output layer: two separately rounded float operations per element (the
          // CPU check computes the same two); the bits then leave through the 32-bit row stores below
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const int col = min(col0 + j, p.N - 1);
            v[j] = __float_as_uint(__fadd_rn(__fmul_rn((float)(int)v[j], __ldg(p.affine_scale + col)), __ldg(p.affine_bias + col)));
          }
        }
        if (C_INT32 || (!C_NOINT32 && (p.out_mode == OUT_INT32 || p.out_mode == OUT_FLOAT))) {
          if (whole) {
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
#pragma unroll
              for (int j = 0; j < 4; j++)
                *reinterpret_cast<uint4*>(xp + swz(lane, j)) =
                    make_uint4(v[16 * hf + 4 * j], v[16 * hf + 4 * j + 1], v[16 * hf + 4 * j + 2], v[16 * hf + 4 * j + 3]);
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const uint4 x = *reinterpret_cast<const uint4*>(xp + swz(8 * i + sub_r, grp));
                if (ok_of[i])
                  *reinterpret_cast<uint4*>(reinterpret_cast<int32_t*>(p.out) + row_of[i] * p.N + col0 + 16 * hf + 4 * grp) = x;
              }
              __syncwarp();
            }
          } else if (row_ok) {
            int32_t* D = reinterpret_cast<int32_t*>(p.out) + row * p.N + col0;
#pragma unroll
            for (int j = 0; j < 32; j++)
              if (col0 + j < p.N) D[j] = (int32_t)v[j];
          }
        } else if (!C_INT32 && row_ok) {
          if constexpr (C_I8THR) {
            // thresholds -> the next layer's int8 operand in one pass: element j of this 32-column group goes to byte
            // 4*((31-j)&7) + ((31-j)>>3) (the order apnn_expand_planes writes); its level, the number of thresholds it
            // reaches, is added to that byte by up to three predicated adds (a byte never exceeds 3)
            uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const int4 q4 = thr_s[j];
              const int x = (int)v[j];
              const uint32_t inc = 1u << (8 * ((31 - j) >> 3));
              if (x >= q4.x) r[(31 - j) & 7] += inc;
              if (x >= q4.y) r[(31 - j) & 7] += inc;
              if (x >= q4.z) r[(31 - j) & 7] += inc;
            }
            uint8_t* O8 = reinterpret_cast<uint8_t*>(p.out) + row * p.N + col0;
            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(O8), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                         "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                         : "memory");
            continue;
          }
          // packed modes need N % 32 == 0, so this word is whole
          uint32_t lv[32];
          if (!C_I8THR && p.out_mode == OUT_LOWBITS) {
#pragma unroll
            for (int j = 0; j < 32; j++) lv[j] = v[j] & (uint32_t)nl;
          } else if (C_I8THR || thr_staged) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const int4 q4 = thr_s[j];
              const int x = (int)v[j];
              lv[j] = (x >= q4.x ? 1u : 0u) + (x >= q4.y ? 1u : 0u) + (x >= q4.z ? 1u : 0u);
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
          if (C_I8THR || p.out_i8) {
            // the next layer's int8 operand: element j of this 32-column group at byte
            // 4*((31-j)&7) + ((31-j)>>3), the order apnn_expand_planes writes
            uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
            for (int j = 0; j < 32; j++) r[(31 - j) & 7] |= lv[j] << (8 * ((31 - j) >> 3));
            uint8_t* O8 = reinterpret_cast<uint8_t*>(p.out) + row * p.N + col0;
            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(O8), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                         "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                         : "memory");
            continue;
          }
          if constexpr (C_I8THR) continue;   // (not reached: int8 rows left above)
          uint32_t* O = reinterpret_cast<uint32_t*>(p.out);
          for (int b = 0; b < p.out_bits; b++) {
            uint32_t part[4] = {0u, 0u, 0u, 0u};   // four independent chains instead of one of 32 ORs
#pragma unroll
            for (int j = 0; j < 32; j++) part[j & 3] |= ((lv[j] >> b) & 1u) << (31 - j);
            O[b * p.out_plane_words + row * (p.N >> 5) + (col0 >> 5)] = (part[0] | part[1]) | (part[2] | part[3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), cluster_ctarank() & ~1u));   // the leader's barrier
        else mbar_arrive(tempty_bar(acc));
      }
      if (has_next) {
        if (!nxt_ready) rows_of_tile(tile + TILE_STEP, nxt);
        if constexpr (!C_NORES) {
          if (!nxt_fetched) fetch_residual(nxt, c_begin);
        }
        cur = nxt;
      }
    }
    if (!ok && lane == 0) atomicExch(p.error_flag, 3);
  }

  // ---------------- tear-down ----------------
  tc_fence_before();
  __syncthreads();
  // The next kernel of the stream may start its prologue now.  (Triggering at the top of the kernel
  // instead lets its CTAs take SMs in the order they fall idle; measured on the ResNet-18 forward
  // that scattering made every layer kernel 1 - 6 us slower, the late trigger saves 0.4 us per launch.)
  grid_launch_dependents();
  if constexpr (PAIR) cluster_sync_all();   // the peer may not leave while the leader's MMAs or arrivals can still reach it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS));
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS));
  }
}

#undef CLUSTER_CTAS
#undef TILE_FIRST
#undef TILE_STEP
#undef PRANK
#undef SPLIT_RANK
#undef KB_FIRST
#undef KB_LAST

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() { return reinterpret_cast<EncodeTiledFn>(tensor_map_encoder()); }

// rows x K bytes, row-major; box = box_rows x span bytes (span = 128 or 64 = the swizzle span), zero fill outside
bool make_operand_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows, int span = 128) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)span, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// int8 NHWC activations [B][Hp][Wp][CIN]; box = span channels x bw x bh x bb pixels
// With a traversal stride s the box spans bw*s x bh*s stored pixels and picks every s-th one.
bool make_activation_map(CUtensorMap* map, const void* base, int B, int Hp, int Wp, int CIN, int bw, int bh, int bb,
                         int stride, int span) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)CIN, (cuuint64_t)Wp, (cuuint64_t)Hp, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)CIN, (cuuint64_t)Wp * CIN, (cuuint64_t)Hp * Wp * CIN};
  cuuint32_t box[4] = {(cuuint32_t)span, (cuuint32_t)(bw * stride), (cuuint32_t)(bh * stride), (cuuint32_t)bb};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// floor(n / d) == (n * magic) >> shift for every 0 <= n < 2^31 (d >= 1): with L = ceil(log2 d),
// magic = floor(2^(31+L) / d) + 1 and shift = 31 + L; magic <= 2^32, the product stays below 2^63.
void division_magic(int d, unsigned long long* magic, int* shift) {
  int L = 0;
  while ((1ll << L) < d) L++;
  *shift = 31 + L;
  *magic = ((1ull << (31 + L)) / (unsigned long long)d) + 1ull;
}

// Shared-memory plan: keep the whole B operand resident when the problem has one tile column
// and its K blocks leave room for at least three A stages; otherwise a ring of A+B stages.
template <int BN, int BKB, bool PAIR>
void plan_smem(Tc5Params& p, int* smem_bytes) {
  using Cfg = TileCfg<BN, BKB, PAIR>;
  const int room = SMEM_LIMIT - Cfg::FIXED_BYTES;
  const long long bres = (long long)p.kblocks * Cfg::B_STAGE_BYTES;
  p.b_resident = 0;
  int stage = Cfg::A_STAGE_BYTES + Cfg::B_STAGE_BYTES;
  long long fixed = 0;
  if (p.splits <= 1 && p.is_conv && p.tiles_n == 1 && p.tiles_m * (PAIR ? 2 : 1) >= 4 * device_sm_count() &&
      bres + 3LL * Cfg::A_STAGE_BYTES <= room) {
    p.b_resident = 1;
    stage = Cfg::A_STAGE_BYTES;
    fixed = bres;
  }
  // narrow stages are grouped (up to three K blocks per barrier round trip) while at least
  // four groups still fit: the per-stage wait / commit latency of the single issuing thread,
  // not the MMA time, bounds tiles whose K block is only a few KiB
  int kgroup = 1;
  for (int g = 3; g >= 2; g--)
    if (p.splits <= 1 && p.kblocks % g == 0 && stage <= 16384 && (room - fixed) / ((long long)g * stage) >= 4) { kgroup = g; break; }
  p.kgroup = kgroup;
  stage *= kgroup;
  int stages = (int)((room - fixed) / stage);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  p.stages = stages;
  *smem_bytes = (int)(Cfg::FIXED_BYTES + fixed + (long long)stages * stage);
}

// Flat convolution: A-buffer ring plus (unless the filter is resident) a ring of B tiles.
template <int BN, int BKB, bool PAIR>
void plan_flat(Tc5Params& p, int* smem_bytes) {
  using Cfg = TileCfg<BN, BKB, PAIR>;
  const long long room = SMEM_LIMIT - Cfg::FIXED_BYTES;
  const long long a_bytes = (long long)p.flat_nblk * p.flat_blk_rows * BKB;
  const long long bres = (long long)p.kblocks * Cfg::B_STAGE_BYTES;
  p.kgroup = 1;
  p.b_resident = 0;
  long long fixed = 0;
  if (p.tiles_n == 1 && p.tiles_m * (PAIR ? 2 : 1) >= 4 * device_sm_count() && bres + 2 * a_bytes <= room) {
    p.b_resident = 1;
    p.flat_nb = 0;
    fixed = bres;
  } else {
    int nb = 10;   // filter tiles in flight: the taps of a latency-bound small problem wait on these loads
    while (nb > 2 && nb * (long long)Cfg::B_STAGE_BYTES + 2 * a_bytes > room) nb--;
    p.flat_nb = nb;
    fixed = nb * (long long)Cfg::B_STAGE_BYTES;
  }
  long long na = (room - fixed) / a_bytes;
  if (na > 6) na = 6;
  if (na < 1) na = 1;
  p.flat_na = (int)na;
  p.stages = (int)na;
  *smem_bytes = (int)(Cfg::FIXED_BYTES + fixed + na * a_bytes);
}

// One launch through cudaLaunchKernelEx: programmatic dependent launch (the kernels wait with
// griddepcontrol.wait before touching their inputs) and, for split-K, the cluster shape.
template <class Kernel>
cudaError_t launch_kernel(Kernel kernel, cudaStream_t s, int grid, int smem, int cluster, const CUtensorMap& map_a,
                          const CUtensorMap& map_b, const Tc5Params& p) {
  cudaError_t e = ensure_max_smem(reinterpret_cast<const void*>(kernel), SMEM_LIMIT);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int na = pdl_attribute(attr);
  if (cluster > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    na++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)na;
  return cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, p);
}

template <int BN, int BKB, bool PAIR>
cudaError_t launch_tc5_p(cudaStream_t s, const CUtensorMap& map_a, const CUtensorMap& map_b, Tc5Params& p, int grid) {
  int smem = 0;
  if (p.is_conv == 2) plan_flat<BN, BKB, PAIR>(p, &smem);
  else plan_smem<BN, BKB, PAIR>(p, &smem);
  const int pair_ctas = PAIR ? 2 : 1;
  if (p.splits > 1) {
    // split-K over clusters: one instantiation (run-time epilogue) per tile width with 128-byte rows
    if constexpr (BKB == 128 && BN >= 128) {
      using Cfg = TileCfg<BN, BKB, PAIR>;
      if ((long long)p.stages * p.kgroup * (Cfg::A_STAGE_BYTES + Cfg::B_STAGE_BYTES) < (long long)BM * BN * 4)
        return cudaErrorInvalidConfiguration;   // the exchange area is the operand ring
      return launch_kernel(tc5_gemm_kernel<BN, BKB, true, 0, PAIR>, s, grid, smem, pair_ctas * p.splits, map_a, map_b, p);
    } else {
      return cudaErrorInvalidConfiguration;
    }
  }
  const bool quantising = p.out_mode != APNN_OUT_INT32 && p.out_mode != APNN_OUT_FLOAT && p.pool == APNN_POOL_NONE;
  const bool residuals = p.residual_in || p.residual_out;
  const bool thr_i8 = p.out_mode == APNN_OUT_THRESHOLDS && p.out_bits <= 2 && p.out_i8;
  const bool all16 = (!p.residual_in || p.res16_in) && (!p.residual_out || p.res16_out);
  const bool int32_only = p.out_mode == APNN_OUT_INT32 && p.pool == APNN_POOL_NONE && !residuals;
  const int epi = int32_only ? 5 : !quantising ? 0 : (thr_i8 ? (residuals ? (all16 ? 4 : 3) : 2) : (residuals ? 0 : 1));
  if (epi == 1) return launch_kernel(tc5_gemm_kernel<BN, BKB, false, 1, PAIR>, s, grid, smem, pair_ctas, map_a, map_b, p);
  if constexpr (!PAIR) {
    if (epi == 2 && p.is_conv == 2 && p.R == 5)
      return launch_kernel(tc5_gemm_kernel<BN, BKB, false, 2, false, true>, s, grid, smem, pair_ctas, map_a, map_b, p);
  }
  if (epi == 2) return launch_kernel(tc5_gemm_kernel<BN, BKB, false, 2, PAIR>, s, grid, smem, pair_ctas, map_a, map_b, p);
  if (epi == 3) return launch_kernel(tc5_gemm_kernel<BN, BKB, false, 3, PAIR>, s, grid, smem, pair_ctas, map_a, map_b, p);
  if (epi == 4) return launch_kernel(tc5_gemm_kernel<BN, BKB, false, 4, PAIR>, s, grid, smem, pair_ctas, map_a, map_b, p);
  if (epi == 5) return launch_kernel(tc5_gemm_kernel<BN, BKB, false, 5, PAIR>, s, grid, smem, pair_ctas, map_a, map_b, p);
  return launch_kernel(tc5_gemm_kernel<BN, BKB, false, 0, PAIR>, s, grid, smem, pair_ctas, map_a, map_b, p);
}

template <int BN, int BKB>
cudaError_t launch_tc5(cudaStream_t s, const CUtensorMap& map_a, const CUtensorMap& map_b, Tc5Params& p, int grid) {
  if (p.pair) {
    // CTA pairs exist for the widest tile with 128-byte rows only
    if constexpr (BN == 256 && BKB == 128) return launch_tc5_p<BN, BKB, true>(s, map_a, map_b, p, grid);
    else return cudaErrorInvalidConfiguration;
  }
  return launch_tc5_p<BN, BKB, false>(s, map_a, map_b, p, grid);
}

cudaError_t launch_tc5_any(cudaStream_t s, const CUtensorMap& map_a, const CUtensorMap& map_b, Tc5Params& p, int grid,
                           int bn, int span) {
  if (span == 64) {
    if (bn == 64) return launch_tc5<64, 64>(s, map_a, map_b, p, grid);
    if (bn == 128) return launch_tc5<128, 64>(s, map_a, map_b, p, grid);
    return launch_tc5<256, 64>(s, map_a, map_b, p, grid);
  }
  if (bn == 64) return launch_tc5<64, 128>(s, map_a, map_b, p, grid);
  if (bn == 128) return launch_tc5<128, 128>(s, map_a, map_b, p, grid);
  return launch_tc5<256, 128>(s, map_a, map_b, p, grid);
}

// Tile width: 64 for operands of at most 64 columns; else 256 unless that leaves the device
// under-filled and 128 does better.
int pick_bn(long long tiles_m, int N, int sms) {
  if (N <= 64) return 64;
  if (N <= 128) return 128;   // a 256-wide tile would spend half its MMA columns on zero fill
  long long t256 = tiles_m * ((N + 255) / 256), t128 = tiles_m * ((N + 127) / 128);
  if (t256 >= sms) return 256;
  // waves needed with each width, in units of a 256-wide tile's work
  double w256 = (double)((t256 + sms - 1) / sms);
  double w128 = 0.5 * (double)((t128 + sms - 1) / sms);
  return w128 < w256 ? 128 : 256;
}

// How many clusters of `ctas` CTAs of the split-K kernel (single-CTA or CTA-pair form) the device holds at once
// (0 on error); cached.
int cluster_capacity(int bn, bool pair, int ctas) {
  static std::mutex mu;
  static int cache[16][3][4] = {};   // [device][128 / 256 / 256 pair][log2 ctas], value + 1
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16 || ctas < 2 || ctas > 8) return 0;
  const int li = ctas == 2 ? 1 : ctas == 4 ? 2 : 3, bi = pair ? 2 : (bn == 256 ? 1 : 0);
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev][bi][li]) return cache[dev][bi][li] - 1;
  const void* kernel = pair ? reinterpret_cast<const void*>(tc5_gemm_kernel<256, 128, true, 0, true>)
                            : bn == 256 ? reinterpret_cast<const void*>(tc5_gemm_kernel<256, 128, true, 0, false>)
                                        : reinterpret_cast<const void*>(tc5_gemm_kernel<128, 128, true, 0, false>);
  int n = 0;
  if (ensure_max_smem(kernel, SMEM_LIMIT) == cudaSuccess) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(ctas * device_sm_count()), 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_LIMIT;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
  }
  cache[dev][bi][li] = n + 1;
  return n;
}

// Tile plan of one launch: tile width, whether CTA pairs share the B tile, and how many ways K is split over a
// cluster.  Cost of a plan in shared-memory traffic units (what bounds the MMA loop): waves x K blocks per CTA x
// operand rows a CTA stages per K block (128 of A plus its rows of B), plus about four K blocks' worth for the
// partial-sum exchange of a split.  The unsplit single-CTA plan with the width pick_bn chose is kept unless
// another plan is at least a tenth cheaper; splits are only taken when every cluster is resident at once.
struct TilePlan {
  int bn, pair, splits;
  long long cost;   // waves x K blocks per CTA x operand rows per K block
};
TilePlan pick_plan(long long tiles_m, int N, int kblocks, int sms, int bn_plain, bool rows128, bool may_split = true) {
  static const bool no_split = [] { const char* v = getenv("APNN_SPLITK"); return v && v[0] == '0'; }();
  static const bool no_pair = [] { const char* v = getenv("APNN_PAIR_MODE"); return v && v[0] == '0'; }();
  static const bool pair_split = [] { const char* v = getenv("APNN_PAIR_SPLIT"); return v && v[0] == '1'; }();
  auto waves = [](long long units, long long slots) { return (units + slots - 1) / slots; };
  const long long plain_tiles = tiles_m * ((N + bn_plain - 1) / bn_plain);
  const long long plain = waves(plain_tiles, sms) * kblocks * (128 + bn_plain);
  TilePlan best = {bn_plain, 0, 1, plain};
  if (!rows128 || N <= 64) return best;
  long long best_cost = plain * 9 / 10;
  for (int pair = 0; pair <= 1; pair++) {
    if (pair && (no_pair || N <= 128 || tiles_m < 2)) break;
    for (int cand = pair ? 256 : 128; cand <= 256; cand *= 2) {
      if (cand == 256 && N <= 128) break;
      const long long units = (pair ? (tiles_m + 1) / 2 : tiles_m) * ((N + cand - 1) / cand);
      const long long slots = pair ? sms / 2 : sms;
      const int rows = 128 + (pair ? cand / 2 : cand);
      for (int cs = 1; cs <= 8; cs *= 2) {
        if (cs == 1 && !pair) continue;                       // the plain plans are pick_bn's business
        // measured on the ResNet-18 layers: unsplit pairs pay from 18 K blocks on (short K: the cluster set-up and
        // the remote barrier arrivals cost more than the halved filter traffic saves) and with more than one
        // wave of tiles (a single tile per CTA is latency-bound either way)
        if (cs == 1 && pair && (kblocks < 18 || units <= slots)) continue;
        // split plans of CTA pairs run, and are tested with APNN_PAIR_SPLIT=1, but are not chosen: a split problem
        // is one tile per CTA, bound by the MMA chain and the exchange rather than by operand traffic, and measured
        // 1 - 20 % slower as pairs (batch 8, 16x16 convolutions of 640 - 1024 channels)
        if (cs > 1 && pair && !pair_split) break;
        if (cs > 1 && (no_split || !may_split || kblocks < 8 || cs > cand / 32 || kblocks / cs < 4 || (pair ? 2 : 1) * cs > 8)) break;
        if (cs > 1 && (units * cs > slots || units > cluster_capacity(cand, pair != 0, (pair ? 2 : 1) * cs))) break;
        const long long cost = waves(units * cs, slots) * ((kblocks + cs - 1) / cs + (cs > 1 ? 4 : 0)) * rows;
        if (cost < best_cost) {
          best_cost = cost;
          best = {cand, pair, cs, cost};
        }
      }
    }
  }
  return best;
}

uint32_t make_idesc(bool a_signed, bool b_signed, int bn, bool pair = false) {
  // D = s32, A/B = u8 or s8, both K-major, N = bn, M = 128 (256 over a CTA pair)
  return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)((pair ? 2 * BM : BM) >> 4) << 24);
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

// Problems the 256 x 256 CTA-pair kernel takes: enough tiles for every SM pair (or peer destinations, which only
// that kernel writes) and an epilogue it implements.
static bool takes_pair_kernel(int M, int N, int K, const apnn_epilogue* epi) {
  return (tc5_pair_worthwhile(M, N, K) && !(epi && (epi->out_i8 || epi->residual_i16 || epi->out_mode == APNN_OUT_FLOAT))) ||
         (epi && epi->n_peer_out > 0);
}

apnn_status tc5_gemm_i8(cudaStream_t s, const uint8_t* A8, const uint8_t* B8, void* D, int M, int N, int K,
                        bool a_signed, bool b_signed, const apnn_epilogue* epi, int* status_flag) {
  if (takes_pair_kernel(M, N, K, epi))
    return tc5_gemm_i8_pair(s, A8, B8, D, M, N, K, a_signed, b_signed, epi, status_flag);
  cudaError_t e;
  const int sms = device_sm_count();
  Tc5Params p;
  memset(&p, 0, sizeof(p));
  const int tiles_m = (M + BM - 1) / BM;
  int bn = pick_bn(tiles_m, N, sms);
  // few tiles and a long K (the fully connected layers of a network at a small batch): K split over the CTAs of
  // a cluster, whatever the epilogue; wide tiles: CTA pairs sharing the B tile
  const TilePlan plan = pick_plan(tiles_m, N, K / BK, sms, bn, true);
  bn = plan.bn;
  // otherwise a skinny problem that leaves more than half of the SMs idle even with 128-wide tiles is
  // bound by streaming the B operand once: 64-wide tiles put twice as many SMs on that stream
  const long long t128 = (long long)tiles_m * ((N + 127) / 128);
  if (plan.splits == 1 && !plan.pair && bn == 128 && t128 * 2 <= sms) bn = 64;
  p.pair = plan.pair;
  p.tiles_m = plan.pair ? (tiles_m + 1) / 2 : tiles_m;
  CUtensorMap map_a, map_b;
  if (!make_operand_map(&map_a, A8, M, K, BM) || !make_operand_map(&map_b, B8, N, K, plan.pair ? bn / 2 : bn)) {
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
  p.out_i8 = epi ? epi->out_i8 : 0;
  p.out_plane_words = (long long)M * (N / 32);
  p.error_flag = status_flag;
  p.residual_in = epi ? epi->residual_in : nullptr;
  p.residual_out = epi ? epi->residual_out : nullptr;
  p.res16_in = epi ? (epi->residual_i16 & 1) : 0;
  p.res16_out = epi ? ((epi->residual_i16 >> 1) & 1) : 0;
  p.affine_scale = epi ? epi->affine_scale : nullptr;
  p.affine_bias = epi ? epi->affine_bias : nullptr;
  p.idesc = make_idesc(a_signed, b_signed, bn, plan.pair != 0);
  const long long tiles = (long long)p.tiles_m * p.tiles_n;   // tiles, or pairs of tiles
  const int per_tile = plan.pair ? 2 : 1;
  if (plan.splits > 1) {
    p.splits = plan.splits;
    e = launch_tc5_any(s, map_a, map_b, p, (int)tiles * plan.splits * per_tile, bn, 128);
    if (e != cudaSuccess) return cuda_fail(e, "tc5_gemm split-K launch");
    return APNN_OK;
  }
  const long long slots = plan.pair ? sms / 2 : sms;
  int grid = (int)(tiles < slots ? tiles : slots) * per_tile;
  e = launch_tc5_any(s, map_a, map_b, p, grid, bn, 128);
  if (e != cudaSuccess) return cuda_fail(e, "tc5_gemm launch");
  return APNN_OK;
}

apnn_status tc5_gemm(cudaStream_t s, int wbits, int xbits, const uint32_t* W, const uint32_t* X, void* D, int M,
                     int N, int K, const apnn_epilogue* epi, void* workspace, int pair) {
  uint8_t* wa = reinterpret_cast<uint8_t*>(workspace);
  uint8_t* wb = wa + align_up((size_t)M * K, 256);
  int* err = reinterpret_cast<int*>(wb + align_up((size_t)N * K, 256));
  const int sign = epi ? epi->signed_operand : APNN_SIGN_NONE;
  // Operands of at most two bits are exact e2m1 values (levels 0..3, or -1 / +1): the block-scaled 4-bit MMA runs them
  // at twice the int8 rate with every sum exact in fp32 (APNN_FP4=0 keeps the int8 path).
  static const bool fp4_on = [] { const char* v = getenv("APNN_FP4"); return !(v && v[0] == '0'); }();
  if (fp4_on && wbits <= 2 && xbits <= 2 && K % 256 == 0 && (long long)K * 9 < (1ll << 24) &&
      (pair || takes_pair_kernel(M, N, K, epi)) && !(epi && epi->out_mode == APNN_OUT_FLOAT)) {
    uint8_t* xb4 = wa + align_up((size_t)M * (K / 2), 256);
    apnn_status s4 = tc5_expand_fp4(s, W, wa, M, K, wbits, sign == APNN_SIGN_W);
    if (s4 == APNN_OK) s4 = tc5_expand_fp4(s, X, xb4, N, K, xbits, sign == APNN_SIGN_X);
    if (s4 != APNN_OK) return s4;
    return tc5_gemm_fp4_pair(s, wa, xb4, D, M, N, K, epi, err);
  }
  // APNN_XPLANES=1: the CTA-pair kernel spreads the activation planes itself, so only W goes through the expand
  // pass and the activation part of the workspace stays untouched.  Off by default: at 8192^3 that kernel takes
  // 0.45 ms against 0.017 + 0.288 ms for the expand pass and the GEMM over int8 rows.
  static const bool planes_on = [] { const char* v = getenv("APNN_XPLANES"); return v && v[0] == '1'; }();
  if (planes_on && xbits <= 4 && (pair || takes_pair_kernel(M, N, K, epi)) &&
      !(epi && epi->out_mode == APNN_OUT_FLOAT)) {
    apnn_status st1 = tc5_expand(s, W, wa, M, K, wbits, sign == APNN_SIGN_W);
    if (st1 != APNN_OK) return st1;
    return tc5_gemm_i8_pair(s, wa, nullptr, D, M, N, K, sign == APNN_SIGN_W, sign == APNN_SIGN_X, epi, err, X, xbits);
  }
  apnn_status st = tc5_expand2(s, W, wa, M, wbits, sign == APNN_SIGN_W, X, wb, N, xbits, sign == APNN_SIGN_X, K);
  if (st != APNN_OK) return st;
  if (pair) return tc5_gemm_i8_pair(s, wa, wb, D, M, N, K, sign == APNN_SIGN_W, sign == APNN_SIGN_X, epi, err);
  return tc5_gemm_i8(s, wa, wb, D, M, N, K, sign == APNN_SIGN_W, sign == APNN_SIGN_X, epi, err);
}

// ------------------------------------------------------------------ convolution
// Pixel box of an A tile: bw x bh (x bb whole images when an image is smaller than a tile),
// at most 128 pixels, chosen for the fewest wasted MMA rows and, among equals, the widest.  With pooling the box is a
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
    // ties go to the widest box: longer contiguous runs per TMA request
    if (util > best - 1e-9) {
      best = util > best ? util : best;
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
                        int* status_flag, bool x_signed) {
  if (!x_signed && tc5_conv_pair_applies(B, Hin, Win, CIN, COUT, R, stride, epi))
    return tc5_conv_i8_pair(s, X8, W8, Out, B, Hin, Win, CIN, COUT, R, w_signed, epi, status_flag);
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
  const int span = (CIN % 128 == 0) ? 128 : 64;   // bytes of K per stage row; CIN % 64 == 0
  p.cblocks = CIN / span;
  p.R = R;
  p.in_off = in_halo - pad;
  p.stride = stride;
  p.pool = pool;
  p.out_h = pool ? H / 2 : H;
  p.out_w = pool ? W / 2 : W;
  p.out_halo = epi ? epi->out_halo : 0;
  p.a_box_bytes = (uint32_t)(bw * bh * bb * span);
  // stride-1 convolutions without pooling run "flat": tiles of 128 consecutive padded pixels,
  // every tap a row-shifted view of one buffer of consecutive input rows (2-D TMA loads)
  const long long flat_rows = (long long)B * Hp * Wp;
  // ... unless that needs more waves of tiles over the SMs than the pixel boxes would (the ring
  // positions are computed and dropped: tiny images, or a tile count just past a multiple of the
  // SM count).  Cost of a formulation = waves x tile width.
  // The pixel-box formulation can also split K over the CTAs of a cluster when it has few tiles.
  const int kblocks_all = R * R * p.cblocks;
  // (the flat kernel path does not split K)
  auto plan_for = [&](long long tiles_m, bool may_split) {
    return pick_plan(tiles_m, COUT, kblocks_all, sms, pick_bn(tiles_m, COUT, sms), span == 128 && !x_signed, may_split);
  };
  const int tiles_m_box = p.tiles_m;
  const TilePlan pl_box = plan_for(tiles_m_box, true), pl_flat = plan_for((flat_rows + BM - 1) / BM, false);
  // (with many waves a few per cent more tiles still win: a flat tile loads 5-8x fewer rows)
  const long long cost_box = pl_box.cost, cost_flat = pl_flat.cost;
  const long long many = 8LL * kblocks_all * 256;   // about eight waves of 128-wide tiles
  bool flat = stride == 1 && pool == APNN_POOL_NONE && flat_rows < 0x7fffff00LL &&
              (cost_flat <= cost_box || (cost_box >= many && cost_flat * 100 <= cost_box * 105));
  if (flat) {
    // rows of input one (tile, channel block) needs: one box when it has at most 256 rows (the TMA
    // limit), else one box per filter row
    const int all_rows = (BM + (R - 1) * (Wp + 1) + 7) / 8 * 8;
    const int nblk = all_rows <= 256 ? 1 : R;
    const int blk_rows = all_rows <= 256 ? all_rows : (BM + R - 1 + 7) / 8 * 8;
    // the flat plan needs one such buffer plus two filter tiles next to the fixed part; wide
    // filters on wide images (R >= 9, or R = 7 with 256-column tiles) do not fit and take the pixel boxes
    const long long flat_tiles_m = (flat_rows + BM - 1) / BM;
    const int b_rows_flat = pl_flat.pair ? pl_flat.bn / 2 : pl_flat.bn;
    const long long need = (long long)TileCfg<64, 64>::FIXED_BYTES + 2LL * b_rows_flat * span + (long long)nblk * blk_rows * span;
    if (need > SMEM_LIMIT) {
      flat = false;
    } else {
      p.is_conv = 2;
      p.flat_wp = Wp;
      p.flat_hpwp = Hp * Wp;
      division_magic(Wp, &p.magic_wp, &p.shift_wp);
      division_magic(Hp * Wp, &p.magic_hpwp, &p.shift_hpwp);
      p.tiles_m = (int)flat_tiles_m;
      p.flat_nblk = nblk;
      p.flat_blk_rows = blk_rows;
    }
  }
  const TilePlan plan = flat ? pl_flat : pl_box;
  const int bn = plan.bn, splits = plan.splits;
  p.pair = plan.pair;
  if (plan.pair) p.tiles_m = (p.tiles_m + 1) / 2;   // pairs of tile rows
  CUtensorMap map_a, map_b;
  const bool maps_ok =
      (flat ? make_operand_map(&map_a, X8, flat_rows, CIN, p.flat_blk_rows, span)
            : make_activation_map(&map_a, X8, B, Hp, Wp, CIN, bw, bh, bb, stride, span)) &&
      make_operand_map(&map_b, W8, COUT, (long long)R * R * CIN, plan.pair ? bn / 2 : bn, span);
  if (!maps_ok) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  p.out = Out;
  p.thresholds = epi ? epi->thresholds : nullptr;
  p.M = B * H * W;
  p.N = COUT;
  p.kblocks = R * R * p.cblocks;
  p.tiles_n = (COUT + bn - 1) / bn;
  p.out_mode = epi ? epi->out_mode : APNN_OUT_INT32;
  p.out_bits = epi ? epi->out_bits : 0;
  p.out_i8 = epi ? epi->out_i8 : 0;
  p.out_plane_words =
      (long long)B * (p.out_h + 2 * p.out_halo) * (p.out_w + 2 * p.out_halo) * (COUT / 32);
  p.error_flag = status_flag;
  p.residual_in = epi ? epi->residual_in : nullptr;
  p.residual_out = epi ? epi->residual_out : nullptr;
  p.res16_in = epi ? (epi->residual_i16 & 1) : 0;
  p.res16_out = epi ? ((epi->residual_i16 >> 1) & 1) : 0;
  p.affine_scale = epi ? epi->affine_scale : nullptr;
  p.affine_bias = epi ? epi->affine_bias : nullptr;
  p.idesc = make_idesc(x_signed, w_signed, bn, plan.pair != 0);  // A = activations (unsigned levels, or the centred signed bytes), B = filter
  const long long tiles = (long long)p.tiles_m * p.tiles_n;   // tiles, or pairs of tiles
  const int per_tile = plan.pair ? 2 : 1;
  const long long slots = plan.pair ? sms / 2 : sms;
  int grid = (int)(tiles < slots ? tiles : slots) * per_tile;
  if (splits > 1) {
    p.splits = splits;
    grid = (int)tiles * splits * per_tile;
  }
  e = launch_tc5_any(s, map_a, map_b, p, grid, bn, span);
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

int* tc5_flag_slot(void* workspace, int M, int N, int K) {
  uint8_t* wa = reinterpret_cast<uint8_t*>(workspace);
  return reinterpret_cast<int*>(wa + align_up((size_t)M * K, 256) + align_up((size_t)N * K, 256));
}

int* tc5_conv_flag_slot(void* workspace, int B, int H, int W, int CIN, int COUT, int R) {
  const int pad = (R - 1) / 2;
  uint8_t* x8 = reinterpret_cast<uint8_t*>(workspace);
  return reinterpret_cast<int*>(x8 + align_up((size_t)B * (H + 2 * pad) * (W + 2 * pad) * CIN, 256) +
                                align_up((size_t)COUT * R * R * CIN, 256));
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
