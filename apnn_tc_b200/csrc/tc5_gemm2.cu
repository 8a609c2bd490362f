// tcgen05 GEMM on CTA pairs (cta_group::2): one 256 x 256 output tile per pair of SMs.
//
// Each CTA of a 2-CTA cluster stages only its own half of both operands -- 128 rows of A
// (its half of M) and 128 rows of B (its half of N) per 128-byte K block, 32 KiB per stage
// instead of 48 KiB for the same MMA time -- so a 6-stage ring fits and every SM pulls a
// third fewer bytes from L2 per MMA than the single-CTA kernel.  The even CTA (the leader)
// issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32): the tensor cores of both SMs
// read both shared memories, and each SM's TMEM receives its own 128 rows of the tile.
//
// Synchronisation (all waits time-bounded, as in the single-CTA kernel):
//   full[s]      lives in the leader; both CTAs' TMA loads complete their bytes on it
//                (cp.async.bulk.tensor ... cta_group::2 with the leader's barrier address)
//   empty[s]     one per CTA; the leader's tcgen05.commit multicasts the arrival to both
//   tmem_full[a] one per CTA, same multicast commit; each CTA's epilogue warps drain their
//                own TMEM
//   tmem_empty[a] lives in the leader, 8 arrivals (4 epilogue warps x 2 CTAs, the peer's
//                through mapa + a cluster-scope arrive)
// The loads carry no cluster multicast.  A cluster barrier closes the kernel so neither CTA
// exits while the other may still touch its shared memory or barriers.
//
// B from packed planes (template parameter XP = number of planes, 0 = int8 rows through TMA):
// the stage ring splits into a ring of NA_XP A tiles (TMA, as above) and a ring of NB_XP B tiles
// that eight more warps per CTA fill.  They read the B operand's bit planes from global memory
// in groups of four K blocks (64 contiguous bytes per row and plane: a warp-wide load touches
// eight lines instead of thirty-two), one group ahead in registers, spread them to one byte per
// element and store them in the 128-byte-swizzled layout the TMA would have produced; each
// writer then runs a generic -> async proxy fence.  A warp that never loads meets them on a
// named barrier per group and arrives on full_b[t] of the leader (a release at cluster scope
// waits for every memory operation its warp has in flight, prefetched planes included -- hence
// not the expanders themselves).  The activation operand never exists as int8 rows in HBM.
#include <cstring>

#include "api_internal.h"
#include "tc5_common.cuh"
#include "tc5_gemm.h"

namespace apnn {

namespace {

using namespace tc5;

constexpr int TILE_M = 256;   // over the pair
constexpr int TILE_N = 256;
constexpr int HALF = 128;     // rows of A and of B one CTA stages
constexpr int STAGES = 6;
constexpr int STAGE_BYTES = 2 * HALF * BK;  // 32 KiB per CTA
// per epilogue warp, 1024-byte aligned: thresholds (256 x 16 B), or a padded 32 x 32 int32 block, or the swizzled
// 32 x 32 int32 block a bulk tensor store reads
constexpr int THR_BYTES_PER_WARP = 5 * 1024;
constexpr int WORD_BYTES_PER_WARP = 2 * 32 * 8 * 4;  // packed outputs of up to 2 bits: 8 words per row and plane, staged per tile
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 1024 + 4 * THR_BYTES_PER_WARP + 4 * WORD_BYTES_PER_WARP;
static_assert(32 * 36 * 4 <= THR_BYTES_PER_WARP, "padded transposition block");
// MX: a stage is 16 KiB of A and 14 KiB of B.  With the deep ring (seven stages) the epilogue keeps 4 KiB per warp
// (thresholds of a 224-wide tile, or the block of a bulk tensor store) and the layout fills the 227 KiB of an SM
// exactly, so the dynamic shared memory must itself start on a 1024-byte boundary (checked in the kernel).
constexpr int MX_STAGE_BYTES = (HALF + 112) * BK;
constexpr int MX_DEEP_STAGES = 7;
constexpr int MX_DEEP_EPI_BYTES = 4096;
constexpr int SMEM_BYTES_MX = MX_DEEP_STAGES * MX_STAGE_BYTES + 1024 + 4 * MX_DEEP_EPI_BYTES;
static_assert(SMEM_BYTES_MX <= 232448 && SMEM_BYTES_MX >= 6 * MX_STAGE_BYTES + 1024 + 4 * THR_BYTES_PER_WARP, "MX layouts");
constexpr int THREADS = 192;
// B-from-planes instantiations
constexpr int EXPAND_WARPS = 8;                      // warps 6..13, 16 rows of the CTA's B half each
constexpr int THREADS_XP = THREADS + 32 * EXPAND_WARPS + 32;   // + the signalling warp (14)
constexpr int XP_TILES = 12;                         // A tiles + B tiles of 16 KiB: the single ring's shared memory
static_assert(XP_TILES * HALF * BK == STAGES * STAGE_BYTES, "the two rings use the single ring's shared memory");
constexpr int GROUP_M = 8;    // bands of 8 pair-tiles (2048 rows) for L2 reuse

struct PairParams {
  void* out;
  const int32_t* thresholds;
  const int32_t* residual_in;
  int32_t* residual_out;
  int M, N, kblocks;
  int tiles_m, tiles_n;
  int out_mode, out_bits;
  uint32_t idesc;
  long long out_plane_words;
  int* error_flag;
  int n_out;       // destinations of every output tile: out itself, then peer-mapped copies
  void* outs[8];
  // B from packed planes: plane j of row n starts at xplanes + j * xplane_words + n * kwords
  const uint32_t* xplanes;
  long long xplane_words;
  int kwords;
  int x_signed;    // one plane holding -1 / +1
  int tma_out;     // int32 output with one destination and N % 4 == 0: 32 x 32 blocks leave by bulk tensor stores
  int stages;      // MX: ring depth, 7 (4 KiB of epilogue staging per warp) or 6 (5 KiB: the padded transposition block)
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
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
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: data lands in this CTA, the bytes complete on `bar_cluster`
// (a shared::cluster address, here always the leader's barrier)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];" ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  // arrive on the barrier at this offset in both CTAs once the MMAs issued so far are done
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Block-scaled 4-bit floating-point MMA (e2m1 operands packed two per byte, fp32 accumulate), K = 64 per
// instruction: twice the int8 rate.  Scale factors (ue8m0, one per 32 elements) are read from TMEM.
__device__ __forceinline__ void tc_mma_mxf4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// eight 32-bit columns of this warp's 32 TMEM lanes <- one value
__device__ __forceinline__ void tmem_fill8(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %1, %1, %1, %1, %1, %1, %1};" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int band = GROUP_M * tiles_n;
  const int g = tile / band;
  const int first = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first);
  const int r = tile - g * band;
  tm = first + r % rows;
  tn = r / rows;
}

// mbar_wait with acquire semantics at cluster scope: the waiter goes on to have the tensor cores read
// shared memory that threads of the peer CTA wrote before their (release.cluster) arrival
__device__ __forceinline__ bool mbar_wait_cluster_acquire(uint32_t bar, uint32_t parity) {
  unsigned long long t0 = 0;
  for (uint32_t spin = 0;; spin++) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 255u) == 255u) {
      unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) return false;
    }
  }
}

// One 32-k word of XP planes -> 32 bytes (eight 32-bit words of four elements each), in the byte order of
// expand_planes_kernel: output word q, byte i holds the element whose bit sits at position 8*i + q.
template <int XP>
__device__ __forceinline__ void spread_word(const uint32_t (&w)[XP > 0 ? XP : 1], bool is_signed, uint32_t (&r)[8]) {
#pragma unroll
  for (int q = 0; q < 8; q++) {
    uint32_t v = 0;
#pragma unroll
    for (int j = 0; j < XP; j++) {
      const uint32_t sft = (q >= j) ? (w[j] >> (q - j)) : (w[j] << (j - q));
      v |= sft & (0x01010101u << j);
    }
    r[q] = (XP == 1 && is_signed) ? (0xFFFFFFFFu ^ (v * 0xFEu)) : v;
  }
}

// XG: K blocks per expander group (2 or 4); the B ring holds two groups, the A ring the other tiles
// MX: operands are e2m1 nibbles (two per byte, 256 elements per 128-byte K block), kind::mxf4 with unit scale
// factors, fp32 accumulators converted to int32 in the epilogue; one accumulator (the other TMEM columns hold
// the scale factors), so the epilogue of a tile does not overlap the next tile's MMAs.
// MX: operands are e2m1 nibbles (two per byte, 256 elements per 128-byte K block), kind::mxf4 with unit scale
// factors, fp32 accumulators converted to int32 in the epilogue; tiles are 224 wide so that two accumulators and
// the scale factors (32 columns of 0x7F bytes, whatever their layout) fit the 512 TMEM columns.
template <int XP, int XG = 4, bool MX = false>
__global__ void __launch_bounds__(XP ? THREADS_XP : THREADS, 1)
tc5_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_d, const PairParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  // MX fills the SM's shared memory exactly and has no room for alignment slack
  const uint32_t base = MX ? raw : ((raw + 1023u) & ~1023u);
  const int nst = MX ? p.stages : (XP ? 0 : STAGES);                     // depth of the single ring
  const uint32_t stage_bytes = MX ? MX_STAGE_BYTES : STAGE_BYTES;
  const uint32_t bars = base + (MX ? (uint32_t)p.stages * MX_STAGE_BYTES : STAGES * STAGE_BYTES);
  const uint32_t epi_bytes = (MX && p.stages == MX_DEEP_STAGES) ? MX_DEEP_EPI_BYTES : THR_BYTES_PER_WARP;
  if (MX && (raw & 1023u) != 0) {   // never seen; the swizzled tiles and the bulk stores need the alignment
    if (threadIdx.x == 0) atomicExch(p.error_flag, 9);
    return;
  }
  // XP == 0: one ring of STAGES stages (A tile then B tile); XP > 0: NA ring slots of A tiles, then NB of B tiles
  // tile width over the pair: 256, or 224 for MX (two accumulators and the scale factors share the 512 TMEM columns)
  constexpr int TN = MX ? 224 : 256;
  constexpr int BHALF = TN / 2;              // rows of B one CTA stages
  constexpr int XGROUP = XG;
  constexpr int NB_XP = 2 * XGROUP;          // B tiles: two groups
  constexpr int NA_XP = XP_TILES - NB_XP;    // A tiles in flight
  constexpr int KQ_LANES = 32 / XGROUP;      // lanes (rows) per K block of a warp-wide load
  constexpr int XTASKS = 16 / KQ_LANES;      // (row, K block) pieces a thread spreads per group
  static_assert((NB_XP & (NB_XP - 1)) == 0 && XTASKS >= 1, "slot arithmetic below");
  constexpr int NA = XP ? NA_XP : (MX ? MX_DEEP_STAGES : STAGES);   // barriers laid out for the deepest ring
  constexpr int NB = XP ? NB_XP : 0;
  constexpr int A_SLOT_BYTES = HALF * BK;   // XP: size of an A ring slot
  constexpr int RING_BARS = 2 * NA + 2 * NB;
  auto full_bar = [&](int s) { return bars + 8u * s; };                       // A (XP == 0: A and B) landed
  auto empty_bar = [&](int s) { return bars + 8u * (NA + s); };
  auto fullb_bar = [&](int t) { return bars + 8u * (2 * NA + t); };           // XP > 0: B tile t spread
  auto emptyb_bar = [&](int t) { return bars + 8u * (2 * NA + NB + t); };
  auto tfull_bar = [&](int a) { return bars + 8u * (RING_BARS + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (RING_BARS + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (RING_BARS + 4);
  static_assert(8 * (RING_BARS + 4) + 4 <= 256, "barrier block");
  const uint32_t b_ring = base + NA_XP * HALF * BK;   // XP > 0: first B tile
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  uint8_t* thr_stage = smem_raw + (bars + 1024u - raw);   // 1024-byte aligned, as is every warp's part of it

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NA; s++) {
      mbar_init(full_bar(s), 1);    // the leader producer's expect_tx
      mbar_init(empty_bar(s), 1);   // the MMA issuer's commit
    }
    for (int t = 0; t < NB; t++) {
      mbar_init(fullb_bar(t), 2);   // the signalling warp of each CTA
      mbar_init(emptyb_bar(t), 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything remote touches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  constexpr uint32_t SF_COL = 2 * TN;   // MX: scale factors, 32 columns of every lane, every byte ue8m0 1.0 (0x7F)
  if (MX) {
    if (warp >= 2 && warp < 6) {
      const uint32_t t0 = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SF_COL;
#pragma unroll
      for (int i = 0; i < 4; i++) tmem_fill8(t0 + 8 * i, 0x7F7F7F7Fu);
      tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
  }
  // everything above overlapped the previous kernel's tail; from here on its results are visible
  grid_dependency_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) *p.error_flag = 0;

  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      const int ring = XP ? NA : nst;
      int s = 0;          // ring slot and its phase, stepped instead of divided: the ring depth may be a run-time value
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        pair_tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int arow = tm * TILE_M + (int)rank * HALF;
        const int brow = tn * TN + (int)rank * BHALF;
        for (int kb = 0; kb < p.kblocks; kb++, s = (s + 1 == ring) ? 0 : s + 1, ph ^= (s == 0) ? 1u : 0u) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) { ok = false; break; }
          const uint32_t leader_full = map_to_cta(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx(full_bar(s), XP ? 2 * A_SLOT_BYTES : 2 * (HALF + BHALF) * BK);  // both CTAs' bytes
          const uint32_t sa = base + s * (XP ? A_SLOT_BYTES : stage_bytes);
          tma_load_2d_pair(sa, &map_a, kb * BK, arow, leader_full);
          if (XP == 0) tma_load_2d_pair(sa + HALF * BK, &map_b, kb * BK, brow, leader_full);
        }
      }
      if (!ok) atomicExch(p.error_flag, 1);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t it = 0;
      uint32_t tl = 0;
      const int ring = XP ? NA : nst;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, tl++) {
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TN;
        for (int kb = 0; kb < p.kblocks; kb++, it++, s = (s + 1 == ring) ? 0 : s + 1, ph ^= (s == 0) ? 1u : 0u) {
          const int t = XP ? (int)(it % NB_XP) : 0;
          if (!mbar_wait(full_bar(s), ph)) { ok = false; break; }
          // the peer's expanders wrote their half of the B tile with ordinary stores: acquire at cluster scope
          if (XP && !mbar_wait_cluster_acquire(fullb_bar(t), (it / NB_XP) & 1u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * (XP ? A_SLOT_BYTES : stage_bytes);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(XP ? b_ring + t * (HALF * BK) : sa + HALF * BK);
#pragma unroll
          for (int k = 0; k < BK / 32; k++) {
            if (MX) tc_mma_mxf4_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, p.idesc, tmem_base + SF_COL, tmem_base + SF_COL + 16,
                                     (kb | k) != 0 ? 1u : 0u);
            else tc_mma_i8_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, p.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(s));  // frees the stage (the A tile) in both CTAs
          if (XP) tc_commit_pair(emptyb_bar(t));
        }
        if (ok) tc_commit_pair(tfull_bar(acc));  // accumulators complete in both CTAs
      }
      if (!ok) atomicExch(p.error_flag, 2);
    }
  } else if (warp >= 6) {
    // ---------------- B expanders (warps 6..13) and their signalling warp (14), XP > 0 only ----------------
    constexpr int XPN = XP > 0 ? XP : 1;
    constexpr int BAR_THREADS = 32 * EXPAND_WARPS + 32;
    const int my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
    const int groups_per_tile = (p.kblocks + XGROUP - 1) / XGROUP;
    const long long total_groups = (long long)my_tiles * groups_per_tile;
    const uint32_t leader_fullb0 = map_to_cta(fullb_bar(0), 0);
    // K blocks of a group sit in consecutive B tiles, kcount = K blocks before the group (over all tiles of this CTA).
    // Group g meets on named barrier 1 + g % 8: an expander reaches group g + 8 only after a B tile written in
    // group g or later was consumed, hence after the signalling warp left the barrier for group g.
    uint32_t kcount = 0;
    if (warp == 6 + EXPAND_WARPS) {
      int gk = 0;   // group within its tile
      for (long long g = 0; g < total_groups; g++) {
        const int nvalid = min(XGROUP, p.kblocks - gk * XGROUP);
        named_bar_sync(1 + (int)(g & 7), BAR_THREADS);
        if (lane < nvalid) mbar_arrive_cluster(leader_fullb0 + 8u * ((kcount + (uint32_t)lane) & (NB_XP - 1)));
        kcount += (uint32_t)nvalid;
        if (++gk == groups_per_tile) gk = 0;
      }
    } else {
      // A thread spreads, per group, K block kq of two rows: a warp-wide 16-byte load then reads 64 contiguous
      // bytes of each of eight rows, and the eight lanes of a quarter warp store to eight consecutive rows of one
      // tile (conflict-free under the 128-byte swizzle).
      const int kq = lane / KQ_LANES;
      const int r0 = (warp - 6) * 16 + (lane % KQ_LANES);   // rows r0 + i * KQ_LANES of the CTA's half of the B tile
      // fetch cursor: one group ahead of the spreading cursor
      int ptile = pair, pgk = 0;
      const uint32_t* prow[XTASKS];
      auto seek_rows = [&]() {
#pragma unroll
        for (int i = 0; i < XTASKS; i++) prow[i] = nullptr;
        if (ptile < num_tiles) {
          int tm, tn;
          pair_tile_coords(ptile, p.tiles_m, p.tiles_n, tm, tn);
          const long long n = (long long)tn * TN + (int)rank * HALF + r0;
#pragma unroll
          for (int i = 0; i < XTASKS; i++)
            if (n + i * KQ_LANES < p.N) prow[i] = p.xplanes + (n + i * KQ_LANES) * p.kwords;
        }
      };
      seek_rows();
      auto fetch_group = [&](uint4 (&dst)[XTASKS][XPN]) {
        const int kb = pgk * XGROUP + kq;
#pragma unroll
        for (int i = 0; i < XTASKS; i++)
#pragma unroll
          for (int j = 0; j < XPN; j++)
            dst[i][j] = (prow[i] && kb < p.kblocks) ? __ldg(reinterpret_cast<const uint4*>(prow[i] + j * p.xplane_words + 4 * kb))
                                                    : make_uint4(0u, 0u, 0u, 0u);
        if (++pgk == groups_per_tile) {
          pgk = 0;
          ptile += num_pairs;
          seek_rows();
        }
      };
      bool ok = true;
      int gk = 0;
      // After an expired wait the warp keeps meeting the named barriers without touching the tiles, so the
      // signalling warp drains and everyone reaches the tear-down.
      auto spread_group = [&](const uint4 (&src)[XTASKS][XPN], long long g) {
        const int nvalid = min(XGROUP, p.kblocks - gk * XGROUP);
        const bool mine = kq < nvalid;
        const uint32_t idx = kcount + (uint32_t)kq;
        const uint32_t t = idx & (NB_XP - 1);
        if (ok) ok = __all_sync(0xffffffffu, !mine || mbar_wait(emptyb_bar((int)t), ((idx / NB_XP) & 1u) ^ 1u));
        if (ok && mine) {
#pragma unroll
          for (int i = 0; i < XTASKS; i++) {
            const int r = r0 + KQ_LANES * i;
            const uint32_t xr = (uint32_t)(r & 7);
            const uint32_t row_s = b_ring + t * (HALF * BK) + (uint32_t)r * 128u;
#pragma unroll
            for (int gw = 0; gw < 4; gw++) {
              uint32_t w[XPN], o[8];
#pragma unroll
              for (int j = 0; j < XPN; j++)
                w[j] = gw == 0 ? src[i][j].x : gw == 1 ? src[i][j].y : gw == 2 ? src[i][j].z : src[i][j].w;
              spread_word<XP>(w, p.x_signed != 0, o);
              // 16-byte chunk c of a 128-byte row lives at chunk position c ^ (row & 7) (128-byte swizzle)
              st_shared_v4(row_s + (((uint32_t)(2 * gw) ^ xr) << 4), o[0], o[1], o[2], o[3]);
              st_shared_v4(row_s + (((uint32_t)(2 * gw + 1) ^ xr) << 4), o[4], o[5], o[6], o[7]);
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
        }
        named_bar_arrive(1 + (int)(g & 7), BAR_THREADS);
        kcount += (uint32_t)nvalid;
        if (++gk == groups_per_tile) gk = 0;
      };
      uint4 qa[XTASKS][XPN], qb[XTASKS][XPN];
      fetch_group(qa);
      for (long long g = 0; g < total_groups; g += 2) {
        fetch_group(qb);
        spread_group(qa, g);
        if (g + 1 < total_groups) {
          fetch_group(qa);
          spread_group(qb, g + 1);
        }
      }
      if (!ok && lane == 0) atomicExch(p.error_flag, 4);
    }
  } else {
    // ---------------- epilogue warps (2..5) of both CTAs ----------------
    const int quarter = warp & 3;
    uint32_t tl = 0;
    bool ok = true;
    const int nl = (1 << p.out_bits) - 1;
    const bool thr_staged = p.out_mode == OUT_THRESHOLDS && nl <= 3;
    int4* thr_s = reinterpret_cast<int4*>(thr_stage + (warp - 2) * epi_bytes);
    // Packed outputs of one or two bits: a thread's eight words of a tile row (one per 32-column chunk) are
    // collected here and leave as one 32-byte store per plane and destination -- whole sectors for HBM and
    // for NVLink instead of eight scattered 4-byte stores.
    uint32_t* word_s = reinterpret_cast<uint32_t*>(thr_stage + 4 * THR_BYTES_PER_WARP + (warp - 2) * WORD_BYTES_PER_WARP);   // unused by MX
    const bool words_staged = !MX && p.out_mode != OUT_INT32 && p.out_bits <= 2 && ((p.N >> 5) & 3) == 0;   // eight words per tile row
    int staged_tn = -1;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, tl++) {
      int tm, tn;
      pair_tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      if (thr_staged && tn != staged_tn) {
        __syncwarp();
        for (int cidx = lane; cidx < TN; cidx += 32) {
          const int col = tn * TN + cidx;
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
      const long long row = (long long)tm * TILE_M + (int)rank * HALF + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * TN;
#pragma unroll 1
      for (int c = 0; c < TN / 32; c++) {
        uint32_t v[32];
        __syncwarp();   // lanes that left the previous chunk early rejoin before the warp-wide TMEM load
        tmem_ld32(taddr + c * 32, v);
        tmem_ld_wait();
        if (MX) {
          // sums of small integers: exact in fp32 below 2^24
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = (uint32_t)__float2int_rn(__uint_as_float(v[j]));
        }
        const int col0 = tn * TN + c * 32;
        if (col0 >= p.N) continue;                        // uniform over the warp
        if (p.out_mode != OUT_INT32 && !row_ok) continue;  // packed modes: a thread writes only its own row
        if (row_ok && (p.residual_in != nullptr || p.residual_out != nullptr)) {
          const long long at = row * (long long)p.N + col0;
#pragma unroll
          for (int j = 0; j < 32; j++)
            if (col0 + j < p.N) {
              if (p.residual_in != nullptr) v[j] = (uint32_t)((int)v[j] + __ldg(p.residual_in + at + j));
              if (p.residual_out != nullptr) p.residual_out[at + j] = (int32_t)v[j];
            }
        }
        if (p.out_mode == OUT_INT32 && p.tma_out) {
          // The warp's 32 x 32 block goes to shared memory as 32 rows of 128 bytes in the 128-byte swizzle (a thread
          // writes its own row: conflict-free) and leaves as one bulk tensor store, which clips at the matrix edges.
          const long long row0 = (long long)tm * TILE_M + (int)rank * HALF + quarter * 32;
          if (row0 < p.M) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous store has read the block
            __syncwarp();
            const uint32_t blk = smem_u32(thr_s);
            const uint32_t row_s = blk + (uint32_t)lane * 128u;
            const uint32_t xr = (uint32_t)(lane & 7);
#pragma unroll
            for (int j = 0; j < 8; j++)
              st_shared_v4(row_s + (((uint32_t)j ^ xr) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_d), "r"(col0),
                           "r"((int)row0), "r"(blk)
                           : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        } else if (p.out_mode == OUT_INT32) {
          // Transpose the warp's 32 x 32 block through shared memory (rows padded to 36 words,
          // 16-byte accesses, conflict-free) so that every store instruction writes four whole
          // 128-byte row segments: full lines for HBM and, for the fused all-gather, for NVLink.
          // The block goes to the local output and to every peer's buffer.
          uint32_t* tile_s = reinterpret_cast<uint32_t*>(thr_s);  // this warp's slice
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; j++)
            *reinterpret_cast<uint4*>(tile_s + lane * 36 + 4 * j) =
                make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          __syncwarp();
          const long long row0 = (long long)tm * TILE_M + (int)rank * HALF + quarter * 32;
          const int sub_r = lane >> 3, c4 = (lane & 7) * 4;
          const bool vec_ok = (p.N & 3) == 0 && col0 + 32 <= p.N;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int r = 4 * i + sub_r;
            const uint4 x = *reinterpret_cast<const uint4*>(tile_s + r * 36 + c4);
            if (row0 + r < p.M) {
              const long long at = (row0 + r) * (long long)p.N + col0 + c4;
              for (int q = 0; q < p.n_out; q++) {
                uint32_t* dst = reinterpret_cast<uint32_t*>(p.outs[q]) + at;
                if (vec_ok) {
                  *reinterpret_cast<uint4*>(dst) = x;
                } else {
                  if (col0 + c4 < p.N) dst[0] = x.x;
                  if (col0 + c4 + 1 < p.N) dst[1] = x.y;
                  if (col0 + c4 + 2 < p.N) dst[2] = x.z;
                  if (col0 + c4 + 3 < p.N) dst[3] = x.w;
                }
              }
            }
          }
        } else {
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
          const bool tile_whole = words_staged && (tn + 1) * TN <= p.N;
          for (int b = 0; b < p.out_bits; b++) {
            uint32_t part[4] = {0u, 0u, 0u, 0u};   // four independent chains instead of one of 32 ORs
#pragma unroll
            for (int j = 0; j < 32; j++) part[j & 3] |= ((lv[j] >> b) & 1u) << (31 - j);
            const uint32_t word = (part[0] | part[1]) | (part[2] | part[3]);
            if (tile_whole) {
              word_s[(b * 32 + lane) * 8 + c] = word;
            } else {
              for (int q = 0; q < p.n_out; q++)
                reinterpret_cast<uint32_t*>(p.outs[q])[b * p.out_plane_words + row * (p.N >> 5) + (col0 >> 5)] = word;
            }
          }
        }
      }
      if (words_staged && row_ok && (tn + 1) * TN <= p.N) {
        // the row's eight words per plane: 32 contiguous, 32-byte aligned bytes of the packed output
        for (int b = 0; b < p.out_bits; b++) {
          const uint4 lo = *reinterpret_cast<const uint4*>(word_s + (b * 32 + lane) * 8);
          const uint4 hi = *reinterpret_cast<const uint4*>(word_s + (b * 32 + lane) * 8 + 4);
          const long long at = b * p.out_plane_words + row * (p.N >> 5) + tn * (TN >> 5);
          for (int q = 0; q < p.n_out; q++) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(p.outs[q]) + at;   // 16-byte aligned: N/32 is a multiple of 4
            if ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
              asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(lo.x), "r"(lo.y), "r"(lo.z),
                           "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                           : "memory");
            } else {
              *reinterpret_cast<uint4*>(dst) = lo;
              *reinterpret_cast<uint4*>(dst + 4) = hi;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));  // the leader's barrier
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // bulk stores complete before the kernel ends
    if (!ok && lane == 0) atomicExch(p.error_flag, 3);
  }

  // ---------------- tear-down ----------------
  tc_fence_before();
  __syncthreads();
  // The next kernel of the stream may start its prologue now.  (Triggering at the top of the kernel
  // instead lets its CTAs take SMs in the order they fall idle; measured on the ResNet-18 forward
  // that scattering made every layer kernel 1 - 6 us slower, the late trigger saves 0.4 us per launch.)
  grid_launch_dependents();
  cluster_sync_all();  // the peer may not leave while the leader's MMAs or arrivals can still reach it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

// planes[bits][rows][K/32] -> e2m1 nibbles, two elements per byte, 16 bytes per 32-k word.  Levels 0..3 of one or
// two planes (0 -> 0000, 1 -> 0010, 2 -> 0100, 3 -> 0101), or -1 / +1 of a single plane (bit 0 -> 1010, 1 -> 0010).
// Nibble i of output word q holds the element whose bit sits at position 4*i + q: a fixed permutation inside each
// group of 32 k, the same for both operands.
__global__ void __launch_bounds__(256) expand_nibbles_kernel(const uint32_t* __restrict__ planes, uint8_t* __restrict__ out,
                                                             long long total, int bits, int is_signed) {
  // four words per thread and trip, their loads issued together
  constexpr int U = 4;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += U * step) {
    uint32_t w0[U], w1[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const long long i = i0 + u * step;
      w0[u] = i < total ? __ldg(planes + i) : 0u;
      w1[u] = (bits > 1 && i < total) ? __ldg(planes + total + i) : 0u;
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const long long i = i0 + u * step;
      if (i >= total) break;
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const uint32_t t0 = (w0[u] >> q) & 0x11111111u, t1 = (w1[u] >> q) & 0x11111111u;
        o[q] = is_signed ? (0x22222222u | ((t0 ^ 0x11111111u) << 3)) : ((t1 << 2) | ((t0 & ~t1) << 1) | (t0 & t1));
      }
      *reinterpret_cast<uint4*>(out + i * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_half_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows = HALF) {
  EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int XP, int XG = 4, bool MX = false>
cudaError_t launch_pair(cudaStream_t s, const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_d,
                        const PairParams& p, int pairs) {
  constexpr int smem_bytes = MX ? SMEM_BYTES_MX : SMEM_BYTES;
  cudaError_t e = ensure_max_smem(reinterpret_cast<const void*>(tc5_gemm_pair_kernel<XP, XG, MX>), smem_bytes);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(XP ? THREADS_XP : THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + (unsigned)pdl_attribute(attr + 1);
  return cudaLaunchKernelEx(&cfg, tc5_gemm_pair_kernel<XP, XG, MX>, map_a, map_b, map_d, p);
}

// int32 [M][N] output seen as 32 x 32 boxes (128-byte rows, 128-byte swizzle on the shared-memory side)
bool make_out_map(CUtensorMap* map, void* D, long long M, long long N) {
  EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(tensor_map_encoder());
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)N * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, D, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Decides whether the int32 output leaves by bulk tensor stores and builds the map for it (a copy of map_a otherwise:
// the kernel takes three maps whatever it uses).  APNN_TMA_STORE=0 keeps the per-thread stores.
bool plan_out_map(CUtensorMap* map_d, const CUtensorMap& map_a, PairParams* p, void* D, int M, int N) {
  static const bool on = [] { const char* v = getenv("APNN_TMA_STORE"); return !(v && v[0] == '0'); }();
  *map_d = map_a;
  p->tma_out = 0;
  if (!on || p->out_mode != APNN_OUT_INT32 || p->n_out != 1 || (N & 3) != 0) return true;
  if (!make_out_map(map_d, D, M, N)) return false;
  p->tma_out = 1;
  return true;
}

}  // namespace

bool tc5_pair_worthwhile(int M, int N, int K) {
  long long tiles = (long long)((M + TILE_M - 1) / TILE_M) * ((N + TILE_N - 1) / TILE_N);
  return tiles >= device_sm_count() / 2 && K >= 1024;
}

// xplanes == nullptr: B8 holds the int8 rows of B.  Otherwise B8 is ignored and the kernel spreads the xbits
// (1..4) planes at xplanes, [xbits][N][K/32] words, into its stages itself.
apnn_status tc5_gemm_i8_pair(cudaStream_t s, const uint8_t* A8, const uint8_t* B8, void* D, int M, int N, int K,
                             bool a_signed, bool b_signed, const apnn_epilogue* epi, int* status_flag,
                             const uint32_t* xplanes, int xbits) {
  if (epi && epi->out_mode == APNN_OUT_FLOAT) return APNN_ERR_UNSUPPORTED;   // the float affine lives in the single-CTA kernel
  if (xplanes && (xbits < 1 || xbits > 4)) return APNN_ERR_UNSUPPORTED;
  CUtensorMap map_a, map_b;
  if (!make_half_map(&map_a, A8, M, K)) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  if (xplanes) map_b = map_a;   // not read
  else if (!make_half_map(&map_b, B8, N, K)) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  PairParams p;
  memset(&p, 0, sizeof(p));
  p.out = D;
  p.thresholds = epi ? epi->thresholds : nullptr;
  p.residual_in = epi ? epi->residual_in : nullptr;
  p.residual_out = epi ? epi->residual_out : nullptr;
  p.M = M;
  p.N = N;
  p.kblocks = K / BK;
  p.tiles_m = (M + TILE_M - 1) / TILE_M;
  p.tiles_n = (N + TILE_N - 1) / TILE_N;
  p.out_mode = epi ? epi->out_mode : APNN_OUT_INT32;
  p.out_bits = epi ? epi->out_bits : 0;
  p.out_plane_words = (long long)M * (N / 32);
  p.error_flag = status_flag;
  p.n_out = 1;
  p.outs[0] = D;
  if (epi)
    for (int i = 0; i < epi->n_peer_out && p.n_out < 8; i++) p.outs[p.n_out++] = epi->peer_out[i];
  p.xplanes = xplanes;
  p.xplane_words = (long long)N * (K / 32);
  p.kwords = K / 32;
  p.x_signed = b_signed ? 1 : 0;
  // D = s32, A/B = u8 or s8, K-major, N = 256, M = 256 over the pair
  p.idesc = (2u << 4) | ((a_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(TILE_N >> 3) << 17) |
            ((uint32_t)(TILE_M >> 4) << 24);
  CUtensorMap map_d;
  if (!plan_out_map(&map_d, map_a, &p, D, M, N)) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  const int sms = device_sm_count();
  long long tiles = (long long)p.tiles_m * p.tiles_n;
  int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);
  cudaError_t e;
  switch (xplanes ? xbits : 0) {
    case 0: e = launch_pair<0>(s, map_a, map_b, map_d, p, pairs); break;
    case 1: e = launch_pair<1>(s, map_a, map_b, map_d, p, pairs); break;
    case 2: e = launch_pair<2>(s, map_a, map_b, map_d, p, pairs); break;
    case 3: e = launch_pair<3>(s, map_a, map_b, map_d, p, pairs); break;
    default: e = launch_pair<4>(s, map_a, map_b, map_d, p, pairs); break;
  }
  if (e != cudaSuccess) return cuda_fail(e, "tc5_gemm_pair launch");
  return APNN_OK;
}

apnn_status tc5_expand_fp4(cudaStream_t s, const uint32_t* planes, uint8_t* out, long long rows, int K, int bits,
                           bool is_signed) {
  const long long total = rows * (K / 32);
  long long blocks = (total + 4 * 256 - 1) / (4 * 256), cap = (long long)device_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  expand_nibbles_kernel<<<(int)blocks, 256, 0, s>>>(planes, out, total, bits, is_signed ? 1 : 0);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "expand_nibbles launch");
  return APNN_OK;
}

// D = A4 * B4^T over e2m1 nibble rows (K/2 bytes per row, K a multiple of 256), int32 or packed outputs.
apnn_status tc5_gemm_fp4_pair(cudaStream_t s, const uint8_t* A4, const uint8_t* B4, void* D, int M, int N, int K,
                              const apnn_epilogue* epi, int* status_flag) {
  if (epi && epi->out_mode == APNN_OUT_FLOAT) return APNN_ERR_UNSUPPORTED;
  CUtensorMap map_a, map_b;
  constexpr int TN_MX = 224;   // the MX instantiation's tile width
  if (!make_half_map(&map_a, A4, M, K / 2) || !make_half_map(&map_b, B4, N, K / 2, TN_MX / 2))
    return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  PairParams p;
  memset(&p, 0, sizeof(p));
  p.out = D;
  p.thresholds = epi ? epi->thresholds : nullptr;
  p.residual_in = epi ? epi->residual_in : nullptr;
  p.residual_out = epi ? epi->residual_out : nullptr;
  p.M = M;
  p.N = N;
  p.kblocks = (K / 2) / BK;
  p.tiles_m = (M + TILE_M - 1) / TILE_M;
  p.tiles_n = (N + TN_MX - 1) / TN_MX;
  p.out_mode = epi ? epi->out_mode : APNN_OUT_INT32;
  p.out_bits = epi ? epi->out_bits : 0;
  p.out_plane_words = (long long)M * (N / 32);
  p.error_flag = status_flag;
  p.n_out = 1;
  p.outs[0] = D;
  if (epi)
    for (int i = 0; i < epi->n_peer_out && p.n_out < 8; i++) p.outs[p.n_out++] = epi->peer_out[i];
  // block-scaled instruction descriptor: a / b format e2m1 (1) at bits 7 and 10, both K-major, N >> 3 at bit 17,
  // scale format ue8m0 (1) at bit 23, M >> 4 at bit 24, scale-factor ids 0
  p.idesc = (1u << 7) | (1u << 10) | ((uint32_t)(TN_MX >> 3) << 17) | (1u << 23) | ((uint32_t)(TILE_M >> 4) << 24);
  CUtensorMap map_d;
  if (!plan_out_map(&map_d, map_a, &p, D, M, N)) return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  const int sms = device_sm_count();
  long long tiles = (long long)p.tiles_m * p.tiles_n;
  int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);
  // the deep ring leaves 4 KiB of staging per epilogue warp: enough for everything but the padded transposition
  // block of int32 tiles that go to several destinations
  static const bool deep = [] { const char* v = getenv("APNN_MX_STAGES"); return v && v[0] == '7'; }();
  p.stages = (deep && (p.tma_out || p.out_mode != APNN_OUT_INT32)) ? MX_DEEP_STAGES : 6;
  cudaError_t e = launch_pair<0, 4, true>(s, map_a, map_b, map_d, p, pairs);
  if (e != cudaSuccess) return cuda_fail(e, "tc5_gemm_fp4_pair launch");
  return APNN_OK;
}

}  // namespace apnn
