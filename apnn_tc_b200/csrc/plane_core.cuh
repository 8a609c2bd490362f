// The warp-level plane contraction core (GEMM and implicit-GEMM convolution).
//
// Operands stay bit-packed from HBM to registers: cp.async stages K tiles of every bit
// plane in shared memory (64-byte rows, XOR-swizzled 16-byte chunks), ldmatrix hands each
// thread one 32-bit word per (row, 128-bit chunk), and then either
//   KIND_U8: the words of all planes of an operand are spread into u8 lanes in registers
//            (value = sum_p bit_p << p) and contracted with mma.sync m16n8k32 u8 -- one MMA
//            per 32 k, whatever the bit widths; or
//   KIND_B1: every (A plane, B plane) pair is contracted with mma.sync m16n8k256 b1
//            and.popc into the accumulator of its weight class 2^(pa+pb).
// Because popcount(AND) and the integer dot product do not care about the order of k,
// the u8 path assigns bit q+8j of a word to byte j of expansion register q; A and B use
// the same assignment, so no transposition is ever needed.
//
// The epilogue runs on the accumulator registers: optional +-1 correction from operand
// popcounts gathered in the main loop, optional 2x2 pooling (the four pixels of a window
// are laid out so one thread owns them), then int32 stores or requantise + bit-plane pack.
#pragma once
#include "apnn_device.cuh"

namespace apnn {

enum { KIND_U8 = 0, KIND_B1 = 1 };

// KSPLIT_ warp groups share a tile and split the K chunks of every stage between them (u8 path);
// their partial sums meet in shared memory before the epilogue.  For latency-bound tiny
// problems it shortens the serial chain of one warp by KSPLIT_.
template <int KIND_, int ABITS_, int BBITS_, int MT_, int NT_, int WARPS_M_, int WARPS_N_, int STAGES_, int KSPLIT_ = 1>
struct CoreCfg {
  static constexpr int KIND = KIND_, ABITS = ABITS_, BBITS = BBITS_, MT = MT_, NT = NT_;
  static constexpr int WARPS_M = WARPS_M_, WARPS_N = WARPS_N_, STAGES = STAGES_, KSPLIT = KSPLIT_;
  static constexpr int BM = WARPS_M * MT * 16;
  static constexpr int BN = WARPS_N * NT * 8;
  static constexpr int THREADS = WARPS_M * WARPS_N * KSPLIT * 32;
  static constexpr int A_ROWS = ABITS * BM;
  static constexpr int B_ROWS = BBITS * BN;
  static constexpr int ROW_BYTES = 64;  // one stage holds 512 bits of K per row
  static constexpr int STAGE_BYTES = (A_ROWS + B_ROWS) * ROW_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES;
  static constexpr int NACC = KIND == KIND_U8 ? 1 : ABITS + BBITS - 1;
  static constexpr int RPP = THREADS / 4;  // rows covered by one pass of 16-byte copies
  static constexpr int A_SLOTS = A_ROWS / RPP;
  static constexpr int B_SLOTS = B_ROWS / RPP;
  static_assert(A_ROWS % RPP == 0 && B_ROWS % RPP == 0, "tile rows must divide over the copy passes");
  static_assert(NT % 4 == 0 && MT % 2 == 0, "fragments are fetched four 8-row matrices at a time");
  static_assert(KSPLIT == 1 || (KIND == KIND_U8 && (KSPLIT == 2 || KSPLIT == 4)), "K split: u8 path, 2 or 4 groups");
  static_assert(KSPLIT == 1 || (KSPLIT - 1) * WARPS_M * WARPS_N * 32 * (MT * NT * 4 + MT * 2 + NT) * 4 <= SMEM_BYTES,
                "partial sums must fit the pipeline buffers");
};

// Spread bit (q + 8j) of every plane word into byte j: value = sum_p bit_p << p.
template <int P, int Q>
__device__ __forceinline__ uint32_t spread(const uint32_t (&w)[P]) {
  uint32_t r = 0;
#pragma unroll
  for (int p = 0; p < P; p++) {
    uint32_t s = (Q >= p) ? (w[p] >> (Q - p)) : (w[p] << (p - Q));
    r |= s & (0x01010101u << p);
  }
  return r;
}

struct RowSrc {
  bool valid;
  long long off;  // word offset of the row's first K word inside one plane
};

// Source row of tile-local A row r.  Row, pixel and window counts fit 32 bits (the host
// checks), so the index arithmetic uses 32-bit unsigned division; only the final word
// offset is 64-bit.
template <int BM>
__device__ __forceinline__ RowSrc a_row_source(const CoreParams& p, int tile_m, int r) {
  RowSrc s;
  if (!p.is_conv) {
    const unsigned m = (unsigned)tile_m * BM + r;
    s.valid = m < (unsigned)p.M;
    s.off = (long long)m * p.a_row_words;
    return s;
  }
  unsigned b, ho, wo;
  if (p.pool == POOL_NONE) {
    const unsigned m = (unsigned)tile_m * BM + r;
    s.valid = m < (unsigned)p.M;
    const unsigned t = m / (unsigned)p.Wo;
    wo = m - t * p.Wo;
    b = t / (unsigned)p.Ho;
    ho = t - b * p.Ho;
  } else {
    // rows r, r+8, r+16, r+24 of every 32-row group are the four pixels of one window
    const unsigned u = (unsigned)tile_m * (BM / 4) + (r >> 5) * 8 + (r & 7);
    const unsigned quad = (r >> 3) & 3;
    s.valid = u < (unsigned)p.M / 4;
    const unsigned wh = p.Wo >> 1, hh = p.Ho >> 1;
    const unsigned t = u / wh;
    const unsigned wp = u - t * wh;
    b = t / hh;
    const unsigned hp = t - b * hh;
    ho = 2 * hp + (quad >> 1);
    wo = 2 * wp + (quad & 1);
  }
  s.off = (((long long)b * p.Hp + (long long)ho * p.stride + p.in_off) * p.Wp + (long long)wo * p.stride + p.in_off) *
          p.cin_words;
  return s;
}

// Output row (in units of output rows of N channels) of logical row index idx, where
// idx counts GEMM rows, conv pixels, or pooled windows.  Returns -1 when out of range.
__device__ __forceinline__ long long out_row_of(const CoreParams& p, unsigned idx, unsigned limit) {
  if (idx >= limit) return -1;
  if (!p.is_conv) return idx;
  const unsigned t = idx / (unsigned)p.out_w;
  const unsigned w = idx - t * p.out_w;
  const unsigned b = t / (unsigned)p.out_h;
  const unsigned h = t - b * p.out_h;
  const int hh = p.out_halo;
  return ((long long)b * (p.out_h + 2 * hh) + h + hh) * (p.out_w + 2 * hh) + w + hh;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS) plane_core_kernel(const CoreParams p) {
  constexpr int KIND = Cfg::KIND, ABITS = Cfg::ABITS, BBITS = Cfg::BBITS, MT = Cfg::MT, NT = Cfg::NT;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, STAGES = Cfg::STAGES, NACC = Cfg::NACC;
  constexpr int A_ROWS = Cfg::A_ROWS, RPP = Cfg::RPP, A_SLOTS = Cfg::A_SLOTS, B_SLOTS = Cfg::B_SLOTS;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;

  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  constexpr int KSPLIT = Cfg::KSPLIT;
  const int kgroup = warp / (Cfg::WARPS_M * Cfg::WARPS_N);   // which share of every stage's K chunks
  const int wlocal = warp % (Cfg::WARPS_M * Cfg::WARPS_N);
  const int warp_m = wlocal / Cfg::WARPS_N;
  const int warp_n = wlocal % Cfg::WARPS_N;
  const int g = lane >> 2, t4 = lane & 3;

  const int tiles_n = (p.N + BN - 1) / BN;
  const int tile_m = blockIdx.x / tiles_n;
  const int tile_n = blockIdx.x % tiles_n;
  const int n0 = tile_n * BN;

  // ---- copy plan: thread owns chunk q of rows (tid/4 + i*RPP) -------------------
  const int q = tid & 3;
  const int rbase = tid >> 2;
  const uint32_t dst0 = (uint32_t)((rbase * 4 + (q ^ ((rbase >> 1) & 3))) * 16);
  const uint32_t* a_src[A_SLOTS];
  const uint32_t* b_src[B_SLOTS];
#pragma unroll
  for (int i = 0; i < A_SLOTS; i++) {
    int rr = rbase + i * RPP;
    int plane = rr / BM, r = rr % BM;
    RowSrc s = a_row_source<BM>(p, tile_m, r);
    a_src[i] = s.valid ? p.A + plane * p.a_plane_words + s.off : nullptr;
  }
#pragma unroll
  for (int i = 0; i < B_SLOTS; i++) {
    int rr = rbase + i * RPP;
    int plane = rr / BN, r = rr % BN;
    long long n = (long long)n0 + r;
    b_src[i] = (n < p.N) ? p.B + plane * p.b_plane_words + n * p.b_row_words : nullptr;
  }

  auto load_stage = [&](int stage, int ks) {
    const int kc = ks * 4 + q;
    const bool kvalid = kc < p.kchunks;
    long long a_off = (long long)kc * 4;
    if (p.is_conv) {
      int tap = kc / p.cin_chunks;
      int c = kc - tap * p.cin_chunks;
      int ti = tap / p.R, tj = tap - ti * p.R;
      a_off = ((long long)ti * p.Wp + tj) * p.cin_words + c * 4;
    }
    const long long b_off = (long long)kc * 4;
    const uint32_t sdst = sbase + stage * STAGE_BYTES + dst0;
#pragma unroll
    for (int i = 0; i < A_SLOTS; i++) {
      bool ok = kvalid && a_src[i] != nullptr;
      cp_async16(sdst + i * RPP * 64, ok ? (const void*)(a_src[i] + a_off) : (const void*)p.A, ok ? 16 : 0);
    }
#pragma unroll
    for (int i = 0; i < B_SLOTS; i++) {
      bool ok = kvalid && b_src[i] != nullptr;
      cp_async16(sdst + (A_ROWS + i * RPP) * 64, ok ? (const void*)(b_src[i] + b_off) : (const void*)p.B, ok ? 16 : 0);
    }
  };

  // ---- fragment addressing -------------------------------------------------------
  const int mi = lane >> 3, r8 = lane & 7;
  const int sw = (r8 >> 1) & 3;
  // A: matrices (rows 0-7, chunk c) (rows 8-15, c) (rows 0-7, c+1) (rows 8-15, c+1)
  const uint32_t a_row_off = (uint32_t)((warp_m * MT * 16 + (mi & 1) * 8 + r8) * 64);
  const uint32_t a_chunk0 = (uint32_t)(((mi >> 1) ^ sw) << 4);
  // B: matrices (n-tile j, chunk c) (n-tile j, c+1) (n-tile j+1, c) (n-tile j+1, c+1)
  const uint32_t b_row_off = (uint32_t)((A_ROWS + warp_n * NT * 8 + (mi >> 1) * 8 + r8) * 64);
  const uint32_t b_chunk0 = (uint32_t)(((mi & 1) ^ sw) << 4);

  // u8 path, one chunk at a time:
  //   A matrices (m-tile i rows 0-7) (i rows 8-15) (i+1 rows 0-7) (i+1 rows 8-15)
  //   B matrices (n-tile j) (j+1) (j+2) (j+3)
  const uint32_t a1_row_off = (uint32_t)((warp_m * MT * 16 + mi * 8 + r8) * 64);
  const uint32_t b1_row_off = (uint32_t)((A_ROWS + warp_n * NT * 8 + mi * 8 + r8) * 64);

  int acc[NACC][MT][NT][4];
#pragma unroll
  for (int s = 0; s < NACC; s++)
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
      for (int j = 0; j < NT; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[s][i][j][e] = 0;

  int sum_a[MT][2];  // popcount sums of this thread's A rows (partial over t4)
  int sum_b[NT];     // popcount sums of B row g of every n-tile (partial over t4)
#pragma unroll
  for (int i = 0; i < MT; i++) sum_a[i][0] = sum_a[i][1] = 0;
#pragma unroll
  for (int j = 0; j < NT; j++) sum_b[j] = 0;

  const int ksteps = (p.kchunks + 3) >> 2;

#pragma unroll
  for (int s = 0; s < STAGES - 1; s++) {
    if (s < ksteps) load_stage(s, s);
    cp_async_commit();
  }

  for (int ks = 0; ks < ksteps; ks++) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      int nk = ks + STAGES - 1;
      if (nk < ksteps) load_stage(nk % STAGES, nk);
      cp_async_commit();
    }
    const uint32_t st = sbase + (ks % STAGES) * STAGE_BYTES;

    if constexpr (KIND == KIND_B1) {
      // two 128-bit chunks per m16n8k256 MMA
#pragma unroll
      for (int sub = 0; sub < 2; sub++) {
        uint32_t aw[ABITS][MT][4];
        uint32_t bw[BBITS][NT][2];
#pragma unroll
        for (int pa = 0; pa < ABITS; pa++)
#pragma unroll
          for (int i = 0; i < MT; i++)
            ldmatrix_x4(st + a_row_off + (pa * BM + i * 16) * 64 + (a_chunk0 ^ (sub << 5)), aw[pa][i][0],
                        aw[pa][i][1], aw[pa][i][2], aw[pa][i][3]);
#pragma unroll
        for (int pb = 0; pb < BBITS; pb++)
#pragma unroll
          for (int j = 0; j < NT; j += 2)
            ldmatrix_x4(st + b_row_off + (pb * BN + j * 8) * 64 + (b_chunk0 ^ (sub << 5)), bw[pb][j][0],
                        bw[pb][j][1], bw[pb][j + 1][0], bw[pb][j + 1][1]);
        if (p.sign == SIGN_B) {
#pragma unroll
          for (int pa = 0; pa < ABITS; pa++)
#pragma unroll
            for (int i = 0; i < MT; i++) {
              sum_a[i][0] += (__popc(aw[pa][i][0]) + __popc(aw[pa][i][2])) << pa;
              sum_a[i][1] += (__popc(aw[pa][i][1]) + __popc(aw[pa][i][3])) << pa;
            }
        } else if (p.sign == SIGN_A) {
#pragma unroll
          for (int pb = 0; pb < BBITS; pb++)
#pragma unroll
            for (int j = 0; j < NT; j++) sum_b[j] += (__popc(bw[pb][j][0]) + __popc(bw[pb][j][1])) << pb;
        }
#pragma unroll
        for (int pa = 0; pa < ABITS; pa++)
#pragma unroll
          for (int pb = 0; pb < BBITS; pb++)
#pragma unroll
            for (int i = 0; i < MT; i++)
#pragma unroll
              for (int j = 0; j < NT; j++)
                mma_b1(acc[pa + pb][i][j], aw[pa][i][0], aw[pa][i][1], aw[pa][i][2], aw[pa][i][3], bw[pb][j][0],
                       bw[pb][j][1]);
      }
    } else {
      // one 128-bit chunk per iteration: a compact body (four k32 steps) that stays in the
      // instruction cache, executed four times per stage
#pragma unroll 1
      for (int c = kgroup; c < 4; c += KSPLIT) {
        uint32_t aw[ABITS][MT][2];  // [plane][m-tile][rows g / g+8]: word t4 of the chunk
        uint32_t bw[BBITS][NT];     // [plane][n-tile]: word t4 of row g
        const uint32_t a_ch = (uint32_t)((c ^ sw) << 4);
#pragma unroll
        for (int pa = 0; pa < ABITS; pa++)
#pragma unroll
          for (int i = 0; i < MT; i += 2)
            ldmatrix_x4(st + a1_row_off + (pa * BM + i * 16) * 64 + a_ch, aw[pa][i][0], aw[pa][i][1],
                        aw[pa][i + 1][0], aw[pa][i + 1][1]);
#pragma unroll
        for (int pb = 0; pb < BBITS; pb++)
#pragma unroll
          for (int j = 0; j < NT; j += 4)
            ldmatrix_x4(st + b1_row_off + (pb * BN + j * 8) * 64 + a_ch, bw[pb][j], bw[pb][j + 1], bw[pb][j + 2],
                        bw[pb][j + 3]);
        if (p.sign == SIGN_B) {
#pragma unroll
          for (int pa = 0; pa < ABITS; pa++)
#pragma unroll
            for (int i = 0; i < MT; i++) {
              sum_a[i][0] += __popc(aw[pa][i][0]) << pa;
              sum_a[i][1] += __popc(aw[pa][i][1]) << pa;
            }
        } else if (p.sign == SIGN_A) {
#pragma unroll
          for (int pb = 0; pb < BBITS; pb++)
#pragma unroll
            for (int j = 0; j < NT; j++) sum_b[j] += __popc(bw[pb][j]) << pb;
        }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
          uint32_t ea[MT][4];
          uint32_t eb[NT][2];
#pragma unroll
          for (int i = 0; i < MT; i++) {
            uint32_t lo[ABITS], hi[ABITS];
#pragma unroll
            for (int pa = 0; pa < ABITS; pa++) {
              lo[pa] = aw[pa][i][0];
              hi[pa] = aw[pa][i][1];
            }
            // kk is a compile-time constant after unrolling; dispatch the shift amounts
            switch (kk) {
              case 0: ea[i][0] = spread<ABITS, 0>(lo); ea[i][1] = spread<ABITS, 0>(hi);
                      ea[i][2] = spread<ABITS, 1>(lo); ea[i][3] = spread<ABITS, 1>(hi); break;
              case 1: ea[i][0] = spread<ABITS, 2>(lo); ea[i][1] = spread<ABITS, 2>(hi);
                      ea[i][2] = spread<ABITS, 3>(lo); ea[i][3] = spread<ABITS, 3>(hi); break;
              case 2: ea[i][0] = spread<ABITS, 4>(lo); ea[i][1] = spread<ABITS, 4>(hi);
                      ea[i][2] = spread<ABITS, 5>(lo); ea[i][3] = spread<ABITS, 5>(hi); break;
              default: ea[i][0] = spread<ABITS, 6>(lo); ea[i][1] = spread<ABITS, 6>(hi);
                       ea[i][2] = spread<ABITS, 7>(lo); ea[i][3] = spread<ABITS, 7>(hi); break;
            }
          }
#pragma unroll
          for (int j = 0; j < NT; j++) {
            uint32_t wv[BBITS];
#pragma unroll
            for (int pb = 0; pb < BBITS; pb++) wv[pb] = bw[pb][j];
            switch (kk) {
              case 0: eb[j][0] = spread<BBITS, 0>(wv); eb[j][1] = spread<BBITS, 1>(wv); break;
              case 1: eb[j][0] = spread<BBITS, 2>(wv); eb[j][1] = spread<BBITS, 3>(wv); break;
              case 2: eb[j][0] = spread<BBITS, 4>(wv); eb[j][1] = spread<BBITS, 5>(wv); break;
              default: eb[j][0] = spread<BBITS, 6>(wv); eb[j][1] = spread<BBITS, 7>(wv); break;
            }
          }
#pragma unroll
          for (int i = 0; i < MT; i++)
#pragma unroll
            for (int j = 0; j < NT; j++)
              mma_u8(acc[0][i][j], ea[i][0], ea[i][1], ea[i][2], ea[i][3], eb[j][0], eb[j][1]);
        }
      }
    }
  }
  cp_async_wait<0>();

  if constexpr (KSPLIT > 1) {
    // the groups' partial accumulators and popcount sums meet in the (now idle) pipeline buffers
    constexpr int PER_THREAD = MT * NT * 4 + MT * 2 + NT;
    int* red = reinterpret_cast<int*>(smem);
    __syncthreads();   // every warp is done with the last stage
    if (kgroup > 0) {
      int* mine = red + ((kgroup - 1) * Cfg::WARPS_M * Cfg::WARPS_N * 32 + wlocal * 32 + lane);
      constexpr int STRIDE = (KSPLIT - 1) * Cfg::WARPS_M * Cfg::WARPS_N * 32;   // element-major: conflict-free
      int n = 0;
#pragma unroll
      for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int e = 0; e < 4; e++) mine[(n++) * STRIDE] = acc[0][i][j][e];
#pragma unroll
      for (int i = 0; i < MT; i++) { mine[(n++) * STRIDE] = sum_a[i][0]; mine[(n++) * STRIDE] = sum_a[i][1]; }
#pragma unroll
      for (int j = 0; j < NT; j++) mine[(n++) * STRIDE] = sum_b[j];
      static_assert(PER_THREAD == MT * NT * 4 + MT * 2 + NT, "layout");
    }
    __syncthreads();
    if (kgroup == 0) {
      constexpr int STRIDE = (KSPLIT - 1) * Cfg::WARPS_M * Cfg::WARPS_N * 32;
#pragma unroll
      for (int gk = 1; gk < KSPLIT; gk++) {
        const int* theirs = red + ((gk - 1) * Cfg::WARPS_M * Cfg::WARPS_N * 32 + wlocal * 32 + lane);
        int n = 0;
#pragma unroll
        for (int i = 0; i < MT; i++)
#pragma unroll
          for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[0][i][j][e] += theirs[(n++) * STRIDE];
#pragma unroll
        for (int i = 0; i < MT; i++) { sum_a[i][0] += theirs[(n++) * STRIDE]; sum_a[i][1] += theirs[(n++) * STRIDE]; }
#pragma unroll
        for (int j = 0; j < NT; j++) sum_b[j] += theirs[(n++) * STRIDE];
      }
    }
    __syncthreads();   // the buffers may be reused (threshold staging) once everyone has read
  }
  const bool writer = KSPLIT == 1 || kgroup == 0;   // the other groups only keep the barriers company

  // ---- epilogue -------------------------------------------------------------------
  // fold the weight classes (b1 path) into acc[0]
  if constexpr (NACC > 1) {
#pragma unroll
    for (int s = 1; s < NACC; s++)
#pragma unroll
      for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int e = 0; e < 4; e++) acc[0][i][j][e] += acc[s][i][j][e] << s;
  }

  if (p.sign == SIGN_B) {
    // B holds -1/+1: value = 2*acc - (sum of A's row)
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
      for (int h = 0; h < 2; h++) {
        int s = sum_a[i][h];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
#pragma unroll
        for (int j = 0; j < NT; j++) {
          acc[0][i][j][h * 2 + 0] = 2 * acc[0][i][j][h * 2 + 0] - s;
          acc[0][i][j][h * 2 + 1] = 2 * acc[0][i][j][h * 2 + 1] - s;
        }
      }
  } else if (p.sign == SIGN_A) {
    // A holds -1/+1: value = 2*acc - (sum of B's row n); sums live with lanes g == column
#pragma unroll
    for (int j = 0; j < NT; j++) {
      int s = sum_b[j];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      int s0 = __shfl_sync(0xffffffffu, s, (2 * t4) * 4);
      int s1 = __shfl_sync(0xffffffffu, s, (2 * t4 + 1) * 4);
#pragma unroll
      for (int i = 0; i < MT; i++) {
        acc[0][i][j][0] = 2 * acc[0][i][j][0] - s0;
        acc[0][i][j][1] = 2 * acc[0][i][j][1] - s1;
        acc[0][i][j][2] = 2 * acc[0][i][j][2] - s0;
        acc[0][i][j][3] = 2 * acc[0][i][j][3] - s1;
      }
    }
  }

  const int ncol0 = n0 + warp_n * NT * 8;  // first column of this warp
  const int nl = (1 << p.out_bits) - 1;

  // Thresholds of up to 2-bit outputs are staged once per CTA in the (now idle) pipeline
  // buffers, one int4 per column with unused slots at INT_MAX: one shared-memory load per
  // value instead of nl global loads.
  const bool thr_staged = p.out_mode == OUT_THRESHOLDS && nl <= 3;
  const int4* thr_s = reinterpret_cast<const int4*>(smem);
  if (thr_staged) {
    __syncthreads();  // every warp is done with the last stage
    for (int cidx = tid; cidx < BN; cidx += Cfg::THREADS) {
      const int col = n0 + cidx;
      int4 t4 = make_int4(0x7fffffff, 0x7fffffff, 0x7fffffff, 0x7fffffff);
      if (col < p.N) {
        const int32_t* T = p.thresholds + (long long)col * nl;
        t4.x = __ldg(T);
        if (nl > 1) { t4.y = __ldg(T + 1); t4.z = __ldg(T + 2); }
      }
      reinterpret_cast<int4*>(smem)[cidx] = t4;
    }
    __syncthreads();
  }
  if (!writer) return;   // no block-wide barrier follows

  auto level_of = [&](int v, int col) -> uint32_t {
    if (p.out_mode == OUT_LOWBITS) return (uint32_t)v & (uint32_t)nl;
    if (thr_staged) {
      const int4 t4 = thr_s[col - n0];
      return (v >= t4.x ? 1u : 0u) + (v >= t4.y ? 1u : 0u) + (v >= t4.z ? 1u : 0u);
    }
    uint32_t l = 0;
    const int32_t* T = p.thresholds + (long long)col * nl;
    for (int j2 = 0; j2 < nl; j2++) l += (v >= __ldg(T + j2)) ? 1u : 0u;
    return l;
  };

  // Emits one output row: vals[j][e] is the value at column ncol0 + j*8 + 2*t4 + e.
  // orow: output row including the optional ring; dense: row index without it (the index of
  // the residual tensors); both negative when the row is out of range.
  auto emit_row = [&](long long orow, long long dense, int (&vals)[NT][2]) {
    if (p.residual_in != nullptr || p.residual_out != nullptr) {
      if (dense >= 0) {
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int col = ncol0 + j * 8 + 2 * t4 + e;
            if (col < p.N) {
              const long long at = dense * (long long)p.N + col;
              if (p.residual_in != nullptr) vals[j][e] += __ldg(p.residual_in + at);
              if (p.residual_out != nullptr) p.residual_out[at] = vals[j][e];
            }
          }
      }
    }
    if (p.out_mode == OUT_INT32) {
      if (orow < 0) return;
      int32_t* D = reinterpret_cast<int32_t*>(p.out) + orow * (long long)p.N;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        int col = ncol0 + j * 8 + 2 * t4;
        if (((p.N & 1) == 0) && col + 1 < p.N) {
          *reinterpret_cast<int2*>(D + col) = make_int2(vals[j][0], vals[j][1]);
        } else {
          if (col < p.N) D[col] = vals[j][0];
          if (col + 1 < p.N) D[col + 1] = vals[j][1];
        }
      }
    } else if constexpr (NT % 4 == 0) {
      // 32 columns per word, first column in bit 31; the 4 lanes of a row group hold 8 each
      uint32_t* O = reinterpret_cast<uint32_t*>(p.out);
      const int nwords = p.N >> 5;
#pragma unroll
      for (int wgrp = 0; wgrp < NT / 4; wgrp++) {
        int colw = ncol0 + wgrp * 32;
        uint32_t lv[4][2];
#pragma unroll
        for (int jj = 0; jj < 4; jj++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            int col = colw + jj * 8 + 2 * t4 + e;
            lv[jj][e] = (col < p.N && orow >= 0) ? level_of(vals[wgrp * 4 + jj][e], col) : 0u;
          }
        for (int b = 0; b < p.out_bits; b++) {
          uint32_t word = 0;
#pragma unroll
          for (int jj = 0; jj < 4; jj++)
#pragma unroll
            for (int e = 0; e < 2; e++) word |= ((lv[jj][e] >> b) & 1u) << (31 - (jj * 8 + 2 * t4 + e));
          word |= __shfl_xor_sync(0xffffffffu, word, 1);
          word |= __shfl_xor_sync(0xffffffffu, word, 2);
          if (t4 == (b & 3) && orow >= 0 && colw < p.N)
            O[b * p.out_plane_words + orow * nwords + (colw >> 5)] = word;
        }
      }
    }
  };

  if (p.pool == POOL_NONE) {
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
      for (int h = 0; h < 2; h++) {
        unsigned idx = (unsigned)tile_m * BM + warp_m * MT * 16 + i * 16 + h * 8 + g;
        long long orow = out_row_of(p, idx, (unsigned)p.M);
        long long dense = orow < 0 ? -1 : (long long)idx;
        int vals[NT][2];
#pragma unroll
        for (int j = 0; j < NT; j++) {
          vals[j][0] = acc[0][i][j][h * 2 + 0];
          vals[j][1] = acc[0][i][j][h * 2 + 1];
        }
        emit_row(orow, dense, vals);
      }
  } else {
    if constexpr (MT % 2 == 0) {
#pragma unroll
      for (int i = 0; i < MT; i += 2) {
        unsigned u = (unsigned)tile_m * (BM / 4) + ((warp_m * MT * 16 + i * 16) >> 5) * 8 + g;
        long long orow = out_row_of(p, u, (unsigned)p.M / 4);
        long long dense = orow < 0 ? -1 : (long long)u;
        int vals[NT][2];
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            int v0 = acc[0][i][j][e], v1 = acc[0][i][j][2 + e];
            int v2 = acc[0][i + 1][j][e], v3 = acc[0][i + 1][j][2 + e];
            vals[j][e] = (p.pool == POOL_AVG2) ? (v0 + v1 + v2 + v3) / 4 : max(max(v0, v1), max(v2, v3));
          }
        emit_row(orow, dense, vals);
      }
    }
  }
}

}  // namespace apnn
