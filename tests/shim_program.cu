// Test program (built and run by tests/test_shims_gpu.py): a caller written against the reference's own
// names.  Operands come from the reference's init_matrices, the kernels are called through
// include/apnn_b200_shims.h exactly as the reference's main() programs and layer wrappers call theirs, and the
// results go to the reference's own compute_ref / compute_ref_pack + validate_results[_pack] -- all of them
// the reference's unmodified host functions, linked from oracle/_ref/libref_66.so.
//   GEMM int32       : APNN-TC-lib/bmmaTensorCoreGemm/src/71_bmmaTensorCoreGemm.cu:305-376, 428-447, 498-571
//   GEMM low-bit pack: 66_bmmaTensorCoreGemm.cuh:356-408 through FC_new_global (APNN-TC-nn/src/kernel.cuh:313-318)
//   conv low-bit pack: 67_bmmaTensorCoreGemm.cu:324-350, 412-478 through Conv_new_global (kernel.cuh:285-289)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "apnn_b200_shims.h"

// the reference's host functions (C++ linkage, as compiled from its sources)
void init_matrices(int4* W, int4* X, int M_GLOBAL, int N_GLOBAL, int K_GLOBAL, int W_BIT, int X_BIT);
void compute_ref(int4* W, int4* X, int* ref_C, int M_GLOBAL, int N_GLOBAL, int K_GLOBAL, int W_BIT, int X_BIT);
void compute_ref_pack(int4* W, int4* X, int* ref_C, int M_GLOBAL, int N_GLOBAL, int K_GLOBAL, int W_BIT, int X_BIT, int OUT_BIT);
void validate_results(int* C, int* ref_C, int M_, int N_);
void validate_results_pack(int* C, int* ref_C, int M_, int N_, int OUT_BIT);
void init_matrices(int4* X, int4* W, int Height, int Width, int CIN, int COUT, int X_BIT, int W_BIT);
void compute_ref_pack(int4* W, int4* X, int* ref_C, int Height, int Width, int CIN, int COUT, int W_BIT, int X_BIT, int OUT_BIT);
void validate_results_pack(int* C, int* ref_C, int Height, int Width, int COUT, int OUT_BIT);

// layer structures with the reference's field names (APNN-TC-nn/src/param.h:1044-1082, 219-385)
struct ConvParam {
  uin32 *filter_gpu, *input_gpu, *output_gpu;
  int batch, input_height, input_width, input_channels, output_channels;
};
struct FcParam {
  uin32 *input_gpu, *weight_gpu, *output_gpu;
  int input_height, input_width, weight_width;
};

#define CK(x)                                                                      \
  do {                                                                             \
    cudaError_t e_ = (x);                                                          \
    if (e_ != cudaSuccess) {                                                       \
      printf("%s failed: %s\n", #x, cudaGetErrorString(e_));                       \
      return 2;                                                                    \
    }                                                                              \
  } while (0)

template <class T>
static T* to_device(const void* host, size_t bytes) {
  void* d = nullptr;
  if (cudaMalloc(&d, bytes) != cudaSuccess) return nullptr;
  cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice);
  return reinterpret_cast<T*>(d);
}

int main() {
  int failures = 0;
  {  // ---- apmm_w1a2, the reference's CPU-runnable case: M = 64, N = K = 1024
    const int M = 64, N = 1024, K = 1024, WB = 1, XB = 2;
    std::vector<int> W(WB * M * K / 32), X(XB * N * K / 32), D(M * N), ref(M * N);
    init_matrices((int4*)W.data(), (int4*)X.data(), M, N, K, WB, XB);
    int4* dW = to_device<int4>(W.data(), W.size() * 4);
    int4* dX = to_device<int4>(X.data(), X.size() * 4);
    int* dD = nullptr;
    CK(cudaMalloc(&dD, D.size() * 4));
    apmm_w1a2(dW, dX, dD, M, N, K);
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(D.data(), dD, D.size() * 4, cudaMemcpyDeviceToHost));
    compute_ref((int4*)W.data(), (int4*)X.data(), ref.data(), M, N, K, WB, XB);
    validate_results(D.data(), ref.data(), M, N);
    if (memcmp(D.data(), ref.data(), D.size() * 4) != 0) failures++;
    long long sum = 0;
    for (int v : D) sum += v;
    printf("apmm_w1a2 checksum %lld\n", sum);
    cudaFree(dW); cudaFree(dX); cudaFree(dD);
  }
  {  // ---- FC_new_global over a layer structure: activations are the 1-bit first operand, weights the 2-bit second
    FcParam p;
    p.input_height = 8;      // batch rows (PAD8)
    p.input_width = 256;     // features in (PAD128)
    p.weight_width = 128;    // features out
    const int M = 8, N = 128, K = 256;
    std::vector<int> A(1 * M * K / 32), Wt(2 * N * K / 32), out(2 * M * N / 32), ref(2 * M * N / 32);
    init_matrices((int4*)A.data(), (int4*)Wt.data(), M, N, K, 1, 2);
    p.input_gpu = to_device<uin32>(A.data(), A.size() * 4);
    p.weight_gpu = to_device<uin32>(Wt.data(), Wt.size() * 4);
    CK(cudaMalloc(&p.output_gpu, out.size() * 4));
    FC_new_global(&p);
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(out.data(), p.output_gpu, out.size() * 4, cudaMemcpyDeviceToHost));
    compute_ref_pack((int4*)A.data(), (int4*)Wt.data(), ref.data(), M, N, K, 1, 2, 2);
    validate_results_pack(out.data(), ref.data(), M, N, 2);
    if (memcmp(out.data(), ref.data(), out.size() * 4) != 0) failures++;
    cudaFree(p.input_gpu); cudaFree(p.weight_gpu); cudaFree(p.output_gpu);
  }
  {  // ---- Conv_new_global over a layer structure: the batch (PAD8) is folded into the height, as the reference does
    ConvParam p;
    p.batch = 1;
    p.input_height = 4;
    p.input_width = 8;
    p.input_channels = 128;
    p.output_channels = 64;
    const int H = 8 * p.input_height, Wd = p.input_width, CIN = 128, COUT = 64;
    std::vector<int> X(2 * (H + 2) * (Wd + 2) * CIN / 32), Wt(1 * COUT * 9 * CIN / 32), out(2 * H * Wd * COUT / 32),
        ref(2 * H * Wd * COUT / 32);
    init_matrices((int4*)X.data(), (int4*)Wt.data(), H, Wd, CIN, COUT, 2, 1);
    p.input_gpu = to_device<uin32>(X.data(), X.size() * 4);
    p.filter_gpu = to_device<uin32>(Wt.data(), Wt.size() * 4);
    CK(cudaMalloc(&p.output_gpu, out.size() * 4));
    Conv_new_global(&p);
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(out.data(), p.output_gpu, out.size() * 4, cudaMemcpyDeviceToHost));
    compute_ref_pack((int4*)Wt.data(), (int4*)X.data(), ref.data(), H, Wd, CIN, COUT, 1, 2, 2);
    validate_results_pack(out.data(), ref.data(), H, Wd, COUT, 2);
    if (memcmp(out.data(), ref.data(), out.size() * 4) != 0) failures++;
    cudaFree(p.input_gpu); cudaFree(p.filter_gpu); cudaFree(p.output_gpu);
  }
  printf("failures %d\n", failures);
  return failures ? 1 : 0;
}
