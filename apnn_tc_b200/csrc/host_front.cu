// Host-buffer front end: a handle that owns a stream and a grow-only device arena, for
// callers that keep operands in host memory and want one call per layer.
#include <cstdlib>
#include <cstring>

#include "../../include/apnn_b200.h"
#include "api_internal.h"

struct apnn_handle_s {
  int device;
  cudaStream_t stream;
  void* arena;
  size_t arena_bytes;
};

namespace {

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

apnn_status ensure_arena(apnn_handle h, size_t bytes) {
  if (bytes <= h->arena_bytes) return APNN_OK;
  cudaError_t e;
  if (h->arena) {
    e = cudaStreamSynchronize(h->stream);
    if (e != cudaSuccess) return apnn::cuda_fail(e, "arena sync");
    cudaFree(h->arena);
    h->arena = nullptr;
    h->arena_bytes = 0;
  }
  e = cudaMalloc(&h->arena, bytes);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "arena cudaMalloc");
  h->arena_bytes = bytes;
  return APNN_OK;
}

struct Carver {
  char* base;
  size_t off;
  void* take(size_t bytes) {
    void* p = base ? base + off : nullptr;
    off += round_up(bytes, 256);
    return p;
  }
};

size_t out_bytes_of(const apnn_epilogue* epi, long long rows, int channels) {
  if (!epi || epi->out_mode == APNN_OUT_INT32 || epi->out_mode == APNN_OUT_FLOAT) return (size_t)rows * channels * 4;
  return (size_t)epi->out_bits * rows * (channels / 32) * 4;
}

}  // namespace

extern "C" {

apnn_status apnn_create(apnn_handle* h, int device) {
  if (!h) return APNN_ERR_INVALID_ARG;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return APNN_ERR_NO_DEVICE;
  int major = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (major != 10) return APNN_ERR_NO_DEVICE;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "cudaSetDevice");
  apnn_handle_s* hs = (apnn_handle_s*)calloc(1, sizeof(apnn_handle_s));
  if (!hs) return APNN_ERR_INVALID_ARG;
  hs->device = device;
  e = cudaStreamCreateWithFlags(&hs->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    free(hs);
    return apnn::cuda_fail(e, "cudaStreamCreate");
  }
  *h = hs;
  return APNN_OK;
}

apnn_status apnn_destroy(apnn_handle h) {
  if (!h) return APNN_ERR_INVALID_ARG;
  cudaSetDevice(h->device);
  cudaStreamSynchronize(h->stream);
  if (h->arena) cudaFree(h->arena);
  cudaStreamDestroy(h->stream);
  free(h);
  return APNN_OK;
}

apnn_status apnn_gemm_host(apnn_handle h, int algo, int wbits, int xbits, const void* W_host, const void* X_host,
                           void* D_host, int M, int N, int K, const apnn_epilogue* epi) {
  if (!h || !W_host || !X_host || !D_host) return APNN_ERR_INVALID_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || wbits < 1 || xbits < 1) return APNN_ERR_INVALID_ARG;
  if (K % 128 != 0) return APNN_ERR_ALIGNMENT;
  cudaError_t e = cudaSetDevice(h->device);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "cudaSetDevice");
  // the descriptor is validated before any size is derived from it
  apnn_status st = apnn::check_epilogue(epi, N, false, wbits, xbits);
  if (st != APNN_OK) return st;
  const size_t wb = (size_t)wbits * M * (K / 8), xb = (size_t)xbits * N * (K / 8);
  const size_t db = out_bytes_of(epi, M, N);
  const bool thr = epi && epi->out_mode == APNN_OUT_THRESHOLDS;
  const size_t tb = thr ? (size_t)N * ((1u << epi->out_bits) - 1) * 4 : 0;
  int use_algo = algo;
  size_t ws = apnn_gemm_workspace_bytes(APNN_ALGO_TCGEN05, wbits, xbits, M, N, K);
  if (algo != APNN_ALGO_TCGEN05 && algo != APNN_ALGO_AUTO) ws = 0;

  Carver sizing{nullptr, 0};
  sizing.take(wb); sizing.take(xb); sizing.take(db); sizing.take(tb); sizing.take(ws);
  st = ensure_arena(h, sizing.off);
  if (st != APNN_OK) return st;
  Carver c{(char*)h->arena, 0};
  void* dW = c.take(wb);
  void* dX = c.take(xb);
  void* dD = c.take(db);
  void* dT = c.take(tb);
  void* dWs = c.take(ws);

  e = cudaMemcpyAsync(dW, W_host, wb, cudaMemcpyHostToDevice, h->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(dX, X_host, xb, cudaMemcpyHostToDevice, h->stream);
  if (e == cudaSuccess && thr) e = cudaMemcpyAsync(dT, epi->thresholds, tb, cudaMemcpyHostToDevice, h->stream);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "host->device copy");
  apnn_epilogue dev_epi;
  const apnn_epilogue* pe = nullptr;
  if (epi) {
    dev_epi = *epi;
    dev_epi.thresholds = (const int32_t*)dT;
    dev_epi.residual_in = nullptr;  // residual tensors are device-side only
    dev_epi.residual_out = nullptr;
    pe = &dev_epi;
  }
  st = apnn_gemm_ex(h->stream, use_algo, wbits, xbits, dW, dX, dD, M, N, K, pe, ws ? dWs : nullptr, ws);
  if (st != APNN_OK) return st;
  e = cudaMemcpyAsync(D_host, dD, db, cudaMemcpyDeviceToHost, h->stream);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "device->host copy");
  // synchronises; with a workspace it also reads the flag a bounded wait raises (apnn_gemm_ex clears the
  // flag when it ends up on a kernel that has no waits), so an incomplete result is never returned as OK
  if (ws) return apnn_gemm_check(h->stream, dWs, M, N, K);
  e = cudaStreamSynchronize(h->stream);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "device->host copy");
  return APNN_OK;
}

apnn_status apnn_conv2d_host(apnn_handle h, int wbits, int xbits, const void* Wt_host, const void* X_host,
                             void* Out_host, int B, int H, int W, int CIN, int COUT, int R, int stride,
                             const apnn_epilogue* epi) {
  if (!h || !Wt_host || !X_host || !Out_host) return APNN_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || W <= 0 || CIN <= 0 || COUT <= 0 || wbits < 1 || xbits < 1) return APNN_ERR_INVALID_ARG;
  if (R < 1 || R > 11 || (R & 1) == 0) return APNN_ERR_UNSUPPORTED;
  if (stride < 1 || stride > 4) return APNN_ERR_UNSUPPORTED;
  if (CIN % 128 != 0) return APNN_ERR_ALIGNMENT;
  cudaError_t e = cudaSetDevice(h->device);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "cudaSetDevice");
  apnn_status st = apnn::check_epilogue(epi, COUT, true, wbits, xbits);
  if (st != APNN_OK) return st;
  // the host image is copied with exactly the ring the filter needs; a wider stored ring is a device-side notion
  if (epi && epi->in_halo != 0 && epi->in_halo != (R - 1) / 2) return APNN_ERR_UNSUPPORTED;
  const int pad = (R - 1) / 2;
  const int Ho = (H - 1) / stride + 1, Wo = (W - 1) / stride + 1;
  const int pool = epi ? epi->pool : APNN_POOL_NONE;
  const int halo = epi ? epi->out_halo : 0;
  const int oh = (pool ? Ho / 2 : Ho) + 2 * halo, ow = (pool ? Wo / 2 : Wo) + 2 * halo;
  const size_t xb = (size_t)xbits * B * (H + 2 * pad) * (W + 2 * pad) * (CIN / 8);
  const size_t wb = (size_t)wbits * COUT * R * R * (CIN / 8);
  const size_t ob = out_bytes_of(epi, (long long)B * oh * ow, COUT);
  const bool thr = epi && epi->out_mode == APNN_OUT_THRESHOLDS;
  const size_t tb = thr ? (size_t)COUT * ((1u << epi->out_bits) - 1) * 4 : 0;
  // with a workspace apnn_conv2d_ex(APNN_ALGO_AUTO) takes the tcgen05 path for sizeable problems
  const size_t ws = apnn_conv2d_workspace_bytes(APNN_ALGO_TCGEN05, B, H, W, CIN, COUT, R);

  Carver sizing{nullptr, 0};
  sizing.take(wb); sizing.take(xb); sizing.take(ob); sizing.take(tb); sizing.take(ws);
  st = ensure_arena(h, sizing.off);
  if (st != APNN_OK) return st;
  Carver c{(char*)h->arena, 0};
  void* dW = c.take(wb);
  void* dX = c.take(xb);
  void* dO = c.take(ob);
  void* dT = c.take(tb);
  void* dWs = c.take(ws);
  e = cudaMemcpyAsync(dW, Wt_host, wb, cudaMemcpyHostToDevice, h->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(dX, X_host, xb, cudaMemcpyHostToDevice, h->stream);
  if (e == cudaSuccess && thr) e = cudaMemcpyAsync(dT, epi->thresholds, tb, cudaMemcpyHostToDevice, h->stream);
  if (e == cudaSuccess && halo > 0) e = cudaMemsetAsync(dO, 0, ob, h->stream);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "host->device copy");
  apnn_epilogue dev_epi;
  const apnn_epilogue* pe = nullptr;
  if (epi) {
    dev_epi = *epi;
    dev_epi.thresholds = (const int32_t*)dT;
    dev_epi.residual_in = nullptr;  // residual tensors are device-side only
    dev_epi.residual_out = nullptr;
    pe = &dev_epi;
  }
  st = apnn_conv2d_ex(h->stream, APNN_ALGO_AUTO, wbits, xbits, dW, dX, dO, B, H, W, CIN, COUT, R, stride, pe,
                      ws ? dWs : nullptr, ws);
  if (st != APNN_OK) return st;
  e = cudaMemcpyAsync(Out_host, dO, ob, cudaMemcpyDeviceToHost, h->stream);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "device->host copy");
  if (ws) return apnn_conv2d_check(h->stream, dWs, B, H, W, CIN, COUT, R);   // synchronises, reads the wait flag
  e = cudaStreamSynchronize(h->stream);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "device->host copy");
  return APNN_OK;
}

}  // extern "C"
