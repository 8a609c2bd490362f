// Flat convolution on CTA pairs (cta_group::2): 256 consecutive flattened padded pixels x 256
// output channels per pair of SMs, for the wide layers (CIN % 128 == 0, COUT % 256 == 0,
// stride 1, no pooling) whose quantised output leaves as int8 rows.
//
// Output positions are the flattened padded pixels q = (b*Hp + h)*Wp + w; filter tap (ti, tj)
// reads input rows q + (ti + in_off)*Wp + tj + in_off of the flattened int8 image.  Per channel
// block of 128 bytes each CTA loads ONE box of 128 + (R-1)*(Wp+1) consecutive rows (its half
// of the pair's 256 positions plus the rows the taps reach) and all R*R taps read it through
// row-shifted descriptors; the filter tile of a (tap, channel block) is split over the pair,
// 128 of its 256 rows per CTA, and the filter ring moves a whole filter row (R taps) per stage.  Against the single-CTA kernel every SM writes half the filter
// bytes into shared memory per MMA, which is what bounds tcgen05.mma kind::i8 there.
//
// Synchronisation follows the CTA-pair GEMM (all waits time-bounded):
//   a_full[i], b_full[s]    in the leader; both CTAs' TMA loads complete their bytes on them
//   a_empty[i], b_empty[s]  one per CTA; the leader's tcgen05.commit multicasts the arrival
//   tmem_full[a]            one per CTA, same multicast commit
//   tmem_empty[a]           in the leader, 16 arrivals (8 epilogue warps x 2 CTAs)
// The loads carry no cluster multicast.
#include <cstdlib>
#include <cstring>

#include "api_internal.h"
#include "tc5_common.cuh"
#include "tc5_gemm.h"

namespace apnn {

namespace {

using namespace tc5;

constexpr int TILE_M = 256;   // flattened positions per pair
constexpr int TILE_N = 256;   // output channels per tile
constexpr int HALF = 128;
constexpr int NA = 2;         // activation buffers (one channel block each)
constexpr int A_BUF_BYTES = 256 * BK;     // at most 256 rows
constexpr int B_TAP_BYTES = HALF * BK;    // one tap's filter tile: 16 KiB per CTA
// The filter ring moves one filter ROW (R taps of a channel block) per stage: one wait, 4*R MMAs of
// straight-line code and one commit per stage keep the issuing thread off the critical path.
constexpr int ring_depth(int RR) { return RR == 1 ? 8 : 3; }
constexpr int B_RING_BYTES = 9 * B_TAP_BYTES;   // 3 stages x 3 taps (R = 3) or 8 stages x 1 tap (R = 1)
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int THR_BYTES_PER_WARP = (TILE_N / 2) * 16;   // one int4 per column the warp drains
constexpr int SMEM_BYTES = NA * A_BUF_BYTES + B_RING_BYTES + 1024 + 256 + EPI_WARPS * THR_BYTES_PER_WARP;
constexpr int MAX_NB = 8;

struct ConvPairParams {
  uint8_t* out;                // int8 rows [B][Ho + 2*out_halo][Wo + 2*out_halo][N]
  const int32_t* thresholds;   // [N][nl]
  int N, CIN, R, cblocks;
  int tiles_m, tiles_n;
  int nl;                      // 2^out_bits - 1 (1 or 3)
  int wp, hpwp, in_off;
  int Bn, Ho, Wo, out_halo;
  uint32_t a_bytes;            // bytes one CTA's activation box deposits
  uint32_t idesc;
  int* error_flag;
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
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: data lands in this CTA, the bytes complete on the leader's barrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], "
      "[%4];" ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
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

template <int RR>
__global__ void __launch_bounds__(THREADS, 1)
tc5_conv_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const ConvPairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bring = base + NA * A_BUF_BYTES;
  constexpr int NB = ring_depth(RR);
  constexpr int B_STAGE_BYTES = RR * B_TAP_BYTES;
  const uint32_t bars = bring + B_RING_BYTES;
  auto afull_bar = [&](int i) { return bars + 8u * i; };
  auto aempty_bar = [&](int i) { return bars + 8u * (NA + i); };
  auto bfull_bar = [&](int s) { return bars + 8u * (2 * NA + s); };
  auto bempty_bar = [&](int s) { return bars + 8u * (2 * NA + MAX_NB + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * NA + 2 * MAX_NB + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * NA + 2 * MAX_NB + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * NA + 2 * MAX_NB + 4);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  uint8_t* thr_stage = smem_raw + (bars + 256u - raw);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NA; i++) {
      mbar_init(afull_bar(i), 1);
      mbar_init(aempty_bar(i), 1);
    }
    for (int s = 0; s < NB; s++) {
      mbar_init(bfull_bar(s), 1);
      mbar_init(bempty_bar(s), 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 2 * EPI_WARPS);
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
  // everything above overlapped the previous kernel's tail; from here on its results are visible
  grid_dependency_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) *p.error_flag = 0;

  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer (one per CTA) ----------------
    if (lane == 0) {
      int ia = 0, sb = 0;
      uint32_t pha = 0, phb = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
        const int q0 = tm * TILE_M + (int)rank * HALF + p.in_off * p.wp + p.in_off;
        const int brow = tn * TILE_N + (int)rank * HALF;
        for (int cb = 0; cb < p.cblocks && ok; cb++) {
          if (!mbar_wait(aempty_bar(ia), pha ^ 1u)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(afull_bar(ia), 2 * p.a_bytes);  // both CTAs' bytes
          tma_load_2d_pair(base + ia * A_BUF_BYTES, &map_a, cb * BK, q0, map_to_cta(afull_bar(ia), 0));
          if (++ia == NA) { ia = 0; pha ^= 1u; }
          int kcol = cb * BK;
          for (int ti = 0; ti < RR; ti++) {
            if (!mbar_wait(bempty_bar(sb), phb ^ 1u)) { ok = false; break; }
            if (rank == 0) mbar_expect_tx(bfull_bar(sb), 2 * B_STAGE_BYTES);
            const uint32_t full = map_to_cta(bfull_bar(sb), 0);
#pragma unroll
            for (int tj = 0; tj < RR; tj++, kcol += p.CIN)
              tma_load_2d_pair(bring + sb * B_STAGE_BYTES + tj * B_TAP_BYTES, &map_b, kcol, brow, full);
            if (++sb == NB) { sb = 0; phb ^= 1u; }
          }
        }
      }
      if (!ok) atomicExch(p.error_flag, 1);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int ia = 0, sb = 0;
      uint32_t pha = 0, phb = 0;
      uint32_t tl = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, tl++) {
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        uint32_t enable = 0;
        for (int cb = 0; cb < p.cblocks && ok; cb++) {
          if (!mbar_wait(afull_bar(ia), pha)) { ok = false; break; }
          tc_fence_after();
          const uint32_t abuf = base + ia * A_BUF_BYTES;
          const uint64_t a0 = make_smem_desc(abuf);
#pragma unroll
          for (int ti = 0; ti < RR; ti++) {
            if (!mbar_wait(bfull_bar(sb), phb)) { ok = false; break; }
            tc_fence_after();
            // tap (ti, tj) reads the box from row ti*Wp + tj on: descriptors shifted by whole rows
            const uint64_t adesc = a0 + (uint32_t)(ti * p.wp) * (BK / 16);
            const uint64_t bdesc = make_smem_desc(bring + sb * B_STAGE_BYTES);
#pragma unroll
            for (int tj = 0; tj < RR; tj++) {
#pragma unroll
              for (int k = 0; k < BK / 32; k++) {
                tc_mma_i8_pair(d_tmem, adesc + tj * (BK / 16) + 2u * k, bdesc + tj * (B_TAP_BYTES / 16) + 2u * k, p.idesc,
                               enable);
                enable = 1u;
              }
            }
            tc_commit_pair(bempty_bar(sb));  // frees the filter stage in both CTAs
            if (++sb == NB) { sb = 0; phb ^= 1u; }
          }
          if (ok) tc_commit_pair(aempty_bar(ia));  // frees the activation buffer in both CTAs
          if (++ia == NA) { ia = 0; pha ^= 1u; }
        }
        if (ok) tc_commit_pair(tfull_bar(acc));  // accumulators complete in both CTAs
      }
      if (!ok) atomicExch(p.error_flag, 2);
    }
  } else {
    // ---------------- epilogue warps (2..9) of both CTAs ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
    const int half = ew >> 2;      // this warp drains the 32-column chunks half, half+2, ...
    uint32_t tl = 0;
    bool ok = true;
    int4* thr_s = reinterpret_cast<int4*>(thr_stage + ew * THR_BYTES_PER_WARP);
    constexpr int CHUNKS = TILE_N / 64;   // per warp
    int thr_tn = -1;
    const int hh = p.out_halo;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, tl++) {
      const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
      if (tn != thr_tn) {
        // thresholds of the columns this warp drains, one int4 per column (unused slots INT_MAX):
        // staged again only when the tile column changes
        __syncwarp();
#pragma unroll
        for (int i = 0; i < CHUNKS; i++) {
          const int32_t* T = p.thresholds + (long long)(tn * TILE_N + (half + 2 * i) * 32 + lane) * p.nl;
          int4 t4 = make_int4(0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff);
          t4.x = __ldg(T);
          if (p.nl > 1) { t4.y = __ldg(T + 1); t4.z = __ldg(T + 2); }
          thr_s[i * 32 + lane] = t4;
        }
        __syncwarp();
        thr_tn = tn;
      }
      // this lane's output position: valid inside the image, everything else is computed and dropped
      const int pos = tm * TILE_M + (int)rank * HALF + quarter * 32 + lane;
      const int b = pos / p.hpwp;
      const int rem = pos - b * p.hpwp;
      const int ho = rem / p.wp, wo = rem - ho * p.wp;
      const bool row_ok = b < p.Bn && ho < p.Ho && wo < p.Wo;
      const long long row = ((long long)b * (p.Ho + 2 * hh) + ho + hh) * (p.Wo + 2 * hh) + wo + hh;
      const uint32_t acc = tl & 1u;
      const uint32_t aph = (tl >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), aph)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * TILE_N;
#pragma unroll 1
      for (int i = 0; i < CHUNKS; i++) {
        const int c = half + 2 * i;
        uint32_t v[32];
        __syncwarp();   // lanes that left the previous chunk early rejoin before the warp-wide TMEM load
        tmem_ld32(taddr + c * 32, v);
        tmem_ld_wait();
        if (!row_ok) continue;
        // the next layer's int8 operand: element j of this 32-column group at byte
        // 4*((31-j)&7) + ((31-j)>>3), the order apnn_expand_planes writes
        uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
        for (int j = 0; j < 32; j++) {
          const int4 q4 = thr_s[i * 32 + j];
          const int x = (int)v[j];
          const uint32_t lv = (x >= q4.x ? 1u : 0u) + (x >= q4.y ? 1u : 0u) + (x >= q4.z ? 1u : 0u);
          r[(31 - j) & 7] |= lv << (8 * ((31 - j) >> 3));
        }
        uint8_t* O8 = p.out + row * p.N + tn * TILE_N + c * 32;
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(O8), "r"(r[0]), "r"(r[1]), "r"(r[2]),
                     "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                     : "memory");
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));  // the leader's barrier
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
  cluster_sync_all();  // the peer may not leave while the leader's MMAs or arrivals can still reach it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// int8 rows [rows][K], boxes of 128 bytes x box_rows rows, 128-byte swizzle
bool make_rows_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
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

int box_rows_of(int R, int Wp) { return (HALF + (R - 1) * (Wp + 1) + 7) / 8 * 8; }

}  // namespace

bool tc5_conv_pair_applies(int B, int Hin, int Win, int CIN, int COUT, int R, int stride, const apnn_epilogue* epi) {
  // APNN_CONV_PAIR=0 in the environment (read once) keeps these layers on the single-CTA kernel, for
  // comparisons; measured on B200 the pair kernel is 7 - 16 % faster on every shape it takes.
  static const bool disabled = [] { const char* v = getenv("APNN_CONV_PAIR"); return v && v[0] == '0'; }();
  if (disabled) return false;
  if (!epi || stride != 1 || CIN % 128 != 0 || COUT % TILE_N != 0 || (R != 1 && R != 3)) return false;
  if (epi->pool != APNN_POOL_NONE || epi->out_mode != APNN_OUT_THRESHOLDS || !epi->out_i8 || !epi->thresholds) return false;
  if (epi->out_bits != 1 && epi->out_bits != 2) return false;
  if (epi->residual_in || epi->residual_out || epi->n_peer_out) return false;
  const int pad = (R - 1) / 2;
  const int in_halo = epi->in_halo ? epi->in_halo : pad;
  const int Hp = Hin + 2 * in_halo, Wp = Win + 2 * in_halo;
  const long long flat_rows = (long long)B * Hp * Wp;
  if (flat_rows >= 0x7fffff00LL || box_rows_of(R, Wp) > 256) return false;
  // at least one tile per SM pair; positions on the ring are computed and dropped, so small images
  // (7x7: 49 of 81 positions useful) stay on the pixel-box kernel
  const long long tiles = ((flat_rows + TILE_M - 1) / TILE_M) * (COUT / TILE_N);
  return tiles >= device_sm_count() / 2 && (long long)Hin * Win * 10 >= (long long)Hp * Wp * 7;
}

apnn_status tc5_conv_i8_pair(cudaStream_t s, const uint8_t* X8, const uint8_t* W8, void* Out, int B, int Hin, int Win,
                             int CIN, int COUT, int R, bool w_signed, const apnn_epilogue* epi, int* status_flag) {
  const int pad = (R - 1) / 2;
  const int in_halo = epi->in_halo ? epi->in_halo : pad;
  const int Hp = Hin + 2 * in_halo, Wp = Win + 2 * in_halo;
  const long long flat_rows = (long long)B * Hp * Wp;
  const int box_rows = box_rows_of(R, Wp);
  CUtensorMap map_a, map_b;
  if (!make_rows_map(&map_a, X8, flat_rows, CIN, box_rows) ||
      !make_rows_map(&map_b, W8, COUT, (long long)R * R * CIN, HALF))
    return cuda_fail(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  cudaError_t e = ensure_max_smem(reinterpret_cast<const void*>(tc5_conv_pair_kernel<1>), SMEM_BYTES);
  if (e == cudaSuccess) e = ensure_max_smem(reinterpret_cast<const void*>(tc5_conv_pair_kernel<3>), SMEM_BYTES);
  if (e != cudaSuccess) return cuda_fail(e, "tc5 conv pair smem attribute");
  ConvPairParams p;
  memset(&p, 0, sizeof(p));
  p.out = reinterpret_cast<uint8_t*>(Out);
  p.thresholds = epi->thresholds;
  p.N = COUT;
  p.CIN = CIN;
  p.R = R;
  p.cblocks = CIN / BK;
  p.tiles_m = (int)((flat_rows + TILE_M - 1) / TILE_M);
  p.tiles_n = COUT / TILE_N;
  p.nl = (1 << epi->out_bits) - 1;
  p.wp = Wp;
  p.hpwp = Hp * Wp;
  p.in_off = in_halo - pad;
  p.Bn = B;
  p.Ho = Hin;
  p.Wo = Win;
  p.out_halo = epi->out_halo;
  p.a_bytes = (uint32_t)box_rows * BK;
  p.error_flag = status_flag;
  // D = s32, A = u8 activations, B = u8 or s8 filter, K-major, N = 256, M = 256 over the pair
  p.idesc = (2u << 4) | ((w_signed ? 1u : 0u) << 10) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
  const int sms = device_sm_count();
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  const int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);

  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1 + (unsigned)pdl_attribute(attr + 1);
  e = R == 3 ? cudaLaunchKernelEx(&cfg, tc5_conv_pair_kernel<3>, map_a, map_b, p)
             : cudaLaunchKernelEx(&cfg, tc5_conv_pair_kernel<1>, map_a, map_b, p);
  if (e != cudaSuccess) return cuda_fail(e, "tc5_conv_pair launch");
  return APNN_OK;
}

}  // namespace apnn
