// Checker-side timing harness, never part of the product: launches ONE of the reference's own GPU
// kernels, unmodified, with the launch configuration its own main() uses
// (<<<multiProcessorCount, 256, 65536>>> after raising the dynamic shared memory limit,
// APNN-TC-lib/bmmaTensorCoreGemm/src/71_bmmaTensorCoreGemm.cu:519-536 and 67_...cu:577-593), on a
// shape given on the command line, and reports the mean device time per launch.  The reference
// source file is pulled in by the compiler (`-include <file> -Dmain=apnn_ref_main`, see the
// Makefile's `ref_gpu` target); nothing of it is copied here.  Built once per reference program:
//
//   -DBAR_GEMM -DBAR_KERNEL=apmm_w1a2 -DBAR_WB=1 -DBAR_XB=2     (71, 72, 78)
//   -DBAR_CONV -DBAR_KERNEL=APConv_w1a2_pack -DBAR_WB=1 -DBAR_XB=2   (67, 70)
//
// usage:  bar gemm <rows_w> <rows_x> <depth> <iters> [in.bin out.bin]
//         bar conv <height> <width> <cin> <cout> <iters> [in.bin out.bin]
// in.bin holds the W planes then the X planes exactly as the kernel reads them; out.bin receives
// the kernel's output words.  Without files the operands are filled by a 64-bit LCG.
//
// The reference's macros M, N and K are live in this translation unit, hence the long names.
#undef main   // the command line renames the reference program's own main(); ours keeps the name
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <cuda_runtime.h>

#define BAR_STR2(x) #x
#define BAR_STR(x) BAR_STR2(x)

#define BAR_CHECK(x)                                                                   \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));                  \
      return 2;                                                                        \
    }                                                                                  \
  } while (0)

static void bar_fill(std::vector<unsigned>& v, unsigned long long seed) {
  unsigned long long s = seed * 0x9E3779B97F4A7C15ull + 1;
  for (size_t i = 0; i < v.size(); i++) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    v[i] = (unsigned)(s >> 32);
  }
}

static bool bar_read(const char* path, std::vector<unsigned>& a, std::vector<unsigned>& b) {
  FILE* f = fopen(path, "rb");
  if (!f) return false;
  bool ok = fread(a.data(), 4, a.size(), f) == a.size() && fread(b.data(), 4, b.size(), f) == b.size();
  fclose(f);
  return ok;
}

int main(int argc, char** argv) {
  if (argc < 2) { fprintf(stderr, "usage: see the header of ref_gpu_bar.cu\n"); return 1; }
  cudaDeviceProp prop;
  BAR_CHECK(cudaGetDeviceProperties(&prop, 0));
  const int shmem_bytes = 65536;
  BAR_CHECK(cudaFuncSetAttribute(BAR_KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, shmem_bytes));
  const char* in_path = nullptr;
  const char* out_path = nullptr;
  size_t w_words, x_words, out_words;
  int iters;
  double ops;
#ifdef BAR_GEMM
  if (argc < 6 || strcmp(argv[1], "gemm")) { fprintf(stderr, "this binary times a GEMM kernel\n"); return 1; }
  const int rows_w = atoi(argv[2]), rows_x = atoi(argv[3]), depth = atoi(argv[4]);
  iters = atoi(argv[5]);
  if (argc >= 8) { in_path = argv[6]; out_path = argv[7]; }
  // the shape rules the kernels assume and never check (71:112-119, 72:80-84, 78:75-77)
  const int row_tile = BAR_WB == 1 ? 64 : 32, col_tile = BAR_XB == 4 ? 16 : 32;
  if (rows_w % row_tile || rows_x % col_tile || depth % 128 || rows_w <= 0 || rows_x <= 0 || depth <= 0) {
    fprintf(stderr, "shape not accepted by this kernel\n");
    return 1;
  }
  w_words = (size_t)BAR_WB * rows_w * (depth / 32);
  x_words = (size_t)BAR_XB * rows_x * (depth / 32);
  out_words = (size_t)rows_w * rows_x;
  ops = 2.0 * rows_w * rows_x * depth;
#else
  if (argc < 7 || strcmp(argv[1], "conv")) { fprintf(stderr, "this binary times a conv kernel\n"); return 1; }
  const int height = atoi(argv[2]), width = atoi(argv[3]), cin = atoi(argv[4]), cout = atoi(argv[5]);
  iters = atoi(argv[6]);
  if (argc >= 9) { in_path = argv[7]; out_path = argv[8]; }
  // 67:64-70, 70:64-70: 4 x 8 pixel tiles, 64 (w1) or 32 (w2) output channels per CTA
  if (height % 4 || width % 8 || cin % 128 || cout % (BAR_WB == 1 ? 64 : 32) || height <= 0 || width <= 0) {
    fprintf(stderr, "shape not accepted by this kernel\n");
    return 1;
  }
  w_words = (size_t)BAR_WB * cout * 9 * (cin / 32);
  x_words = (size_t)BAR_XB * (height + 2) * (width + 2) * (cin / 32);
  out_words = (size_t)2 * height * width * (cout / 32);   // 2-bit packed output
  ops = 2.0 * height * width * (double)cout * 9.0 * cin;
#endif
  if (iters < 1 || iters > 100000) return 1;

  std::vector<unsigned> w_h(w_words), x_h(x_words), out_h(out_words);
  if (in_path) {
    if (!bar_read(in_path, w_h, x_h)) { fprintf(stderr, "cannot read %s\n", in_path); return 1; }
  } else {
    bar_fill(w_h, 1);
    bar_fill(x_h, 2);
  }
  unsigned *w_d, *x_d, *out_d;
  BAR_CHECK(cudaMalloc(&w_d, w_words * 4));
  BAR_CHECK(cudaMalloc(&x_d, x_words * 4));
  BAR_CHECK(cudaMalloc(&out_d, out_words * 4));
  BAR_CHECK(cudaMemcpy(w_d, w_h.data(), w_words * 4, cudaMemcpyHostToDevice));
  BAR_CHECK(cudaMemcpy(x_d, x_h.data(), x_words * 4, cudaMemcpyHostToDevice));
  BAR_CHECK(cudaMemset(out_d, 0xff, out_words * 4));

  cudaEvent_t t0, t1;
  BAR_CHECK(cudaEventCreate(&t0));
  BAR_CHECK(cudaEventCreate(&t1));
  const int grid = prop.multiProcessorCount;
  float ms = 0.f;
  for (int pass = 0; pass < 2; pass++) {   // pass 0 warms up (3 launches), pass 1 is timed
    const int n = pass == 0 ? 3 : iters;
    BAR_CHECK(cudaEventRecord(t0));
    for (int i = 0; i < n; i++) {
#ifdef BAR_GEMM
      BAR_KERNEL<<<grid, 256, shmem_bytes>>>((const int4*)w_d, (const int4*)x_d, (int*)out_d, rows_w, rows_x,
                                             depth, BAR_WB, BAR_XB);
#else
      BAR_KERNEL<<<grid, 256, shmem_bytes>>>((const int4*)w_d, (const int4*)x_d, (int*)out_d, height, width,
                                             cin, cout);
#endif
    }
    BAR_CHECK(cudaGetLastError());
    BAR_CHECK(cudaEventRecord(t1));
    BAR_CHECK(cudaEventSynchronize(t1));
    BAR_CHECK(cudaEventElapsedTime(&ms, t0, t1));
  }
  const double us = 1e3 * ms / iters;
  printf("{\"kernel\": \"%s\", \"us_per_launch\": %.3f, \"tops\": %.3f, \"iters\": %d, \"sms\": %d}\n",
         BAR_STR(BAR_KERNEL), us, ops / (us * 1e-6) / 1e12, iters, grid);
  if (out_path) {
    BAR_CHECK(cudaMemcpy(out_h.data(), out_d, out_words * 4, cudaMemcpyDeviceToHost));
    FILE* f = fopen(out_path, "wb");
    if (!f || fwrite(out_h.data(), 4, out_words, f) != out_words) { fprintf(stderr, "cannot write output\n"); return 1; }
    fclose(f);
  }
  cudaFree(w_d); cudaFree(x_d); cudaFree(out_d);
  return 0;
}
