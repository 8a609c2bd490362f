// apnn_gemm_static_scratch: the tcgen05 GEMM for callers that cannot allocate.
//
// The regular tcgen05 entry point (apnn_gemm_ex with APNN_ALGO_TCGEN05) needs a workspace
// the caller has to cudaMalloc.  Some callers have no way to do that: a plug-in living
// inside a host application whose own pool already holds all of the device's memory (a raw
// cudaMalloc there fails or fights the pool), or a latency-critical loop that must not pay
// the device-wide synchronisation cudaMalloc and cudaFree imply and has no spare buffer to
// hand over.  For them the int8 images of the two operands go into a fixed array that is
// part of the library image itself.
//
// Cost and limits, stated plainly:
//   * every GPU that loads the library carries APNN_STATIC_SCRATCH_BYTES (32 MiB) of device
//     memory from load until process exit, used or not;
//   * a problem fits only if align256(M*K) + align256(N*K) <= APNN_STATIC_SCRATCH_BYTES,
//     e.g. 2048 x 2048 x 8192 or 4096 x 4096 x 4096; larger ones are refused with
//     APNN_ERR_WORKSPACE before anything is launched;
//   * there is one array per device and every call uses it, so two calls whose kernels can
//     overlap on the GPU (different streams, no dependency between them) race on it and
//     corrupt each other's operands -- serialise such calls;
//   * the array keeps whatever the previous call left.  Nothing in it needs to start at
//     zero: the expand kernels overwrite every byte the GEMM reads (rows beyond M or N are
//     zero-filled by the TMA unit, not read from the array), and the only state that must
//     start cleared, the 4-byte status flag, lives in caller memory and is reset on the
//     stream by every call.
//
// The array's name is only a host-side handle in host code, not a device address, so the
// device address is looked up with cudaGetSymbolAddress.  That look-up happens in the first
// call made on each device (with that device current) and is cached; make that first call
// outside any stream capture.  No call here allocates or frees memory.
#include <mutex>

#include "../../include/apnn_b200.h"
#include "api_internal.h"
#include "tc5_gemm.h"

namespace {

constexpr size_t kScratchBytes = APNN_STATIC_SCRATCH_BYTES;

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Device address of the array on the current device; looked up once per device.
apnn_status scratch_address(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return apnn::cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return APNN_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return apnn::cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    if (!p) return apnn::cuda_fail(cudaErrorInvalidSymbol, "cudaGetSymbolAddress returned null");
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return APNN_OK;
}

}  // namespace

extern "C" apnn_status apnn_gemm_static_scratch(void* stream, int wbits, int xbits, const void* W, const void* X,
                                                void* D, int M, int N, int K, const apnn_epilogue* epi,
                                                int* status_flag) {
  if (!W || !X || !D || !status_flag) return APNN_ERR_INVALID_ARG;
  if (M <= 0 || N <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  if (wbits < 1 || wbits > 4 || xbits < 1 || xbits > 4) return APNN_ERR_UNSUPPORTED;
  if (K % 128 != 0) return APNN_ERR_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(D)) & 15u)
    return APNN_ERR_ALIGNMENT;
  apnn_status st = apnn::check_epilogue(epi, N, false, wbits, xbits);
  if (st != APNN_OK) return st;
  // refuse what does not fit, before touching the device
  const size_t need = align256((size_t)M * K) + align256((size_t)N * K);
  if (need > kScratchBytes) return APNN_ERR_WORKSPACE;

  unsigned char* base = nullptr;
  st = scratch_address(&base);
  if (st != APNN_OK) return st;
  unsigned char* w8 = base;
  unsigned char* x8 = base + align256((size_t)M * K);

  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int sign = epi ? epi->signed_operand : APNN_SIGN_NONE;
  st = apnn::tc5_expand(s, static_cast<const uint32_t*>(W), w8, M, K, wbits, sign == APNN_SIGN_W);
  if (st != APNN_OK) return st;
  st = apnn::tc5_expand(s, static_cast<const uint32_t*>(X), x8, N, K, xbits, sign == APNN_SIGN_X);
  if (st != APNN_OK) return st;
  // the sign is now in the bytes; the GEMM's epilogue must not correct a second time
  apnn_epilogue e2;
  const apnn_epilogue* pe = nullptr;
  if (epi) {
    e2 = *epi;
    e2.signed_operand = APNN_SIGN_NONE;
    pe = &e2;
  }
  // resets *status_flag on the stream, then launches the GEMM
  return apnn::tc5_gemm_i8(s, w8, x8, D, M, N, K, sign == APNN_SIGN_W, sign == APNN_SIGN_X, pe, status_flag);
}
