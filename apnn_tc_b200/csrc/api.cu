// C ABI of the library (include/apnn_b200.h): argument checking, problem set-up and
// dispatch.  No entry point allocates device memory except the host-buffer front end's
// handle (host_front.cu), and none falls back to a CPU path.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/apnn_b200.h"
#include "api_internal.h"
#include "core_launch.h"
#include "tc5_gemm.h"

namespace apnn {

static thread_local char g_cuda_err[256] = "";

apnn_status cuda_fail(cudaError_t e, const char* where) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", where, cudaGetErrorString(e));
  return APNN_ERR_CUDA;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
// the expand kernel writes the int8 images with 32-byte stores
static bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

int device_sm_count() {
  static int sms[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 16 && sms[dev]) return sms[dev];
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 16) sms[dev] = n;
  return n;
}

apnn_status check_epilogue(const apnn_epilogue* e, int channels, bool is_conv, int abits_signed_w, int abits_signed_x,
                           bool i8_rows_ok) {
  if (!e) return APNN_OK;
  if (e->struct_size != sizeof(apnn_epilogue)) return APNN_ERR_INVALID_ARG;   // built against another layout
  if (e->residual_i16 != 0 && (e->residual_i16 < 0 || e->residual_i16 > 3 || !i8_rows_ok || e->n_peer_out != 0))
    return (e->residual_i16 > 0 && e->residual_i16 <= 3 && !i8_rows_ok) ? APNN_ERR_UNSUPPORTED : APNN_ERR_INVALID_ARG;
  if (e->out_i8 != 0 && (e->out_i8 != 1 || !i8_rows_ok || e->out_mode == APNN_OUT_INT32 || e->n_peer_out != 0))
    return e->out_i8 == 1 && !i8_rows_ok ? APNN_ERR_UNSUPPORTED : APNN_ERR_INVALID_ARG;
  if (e->out_mode < APNN_OUT_INT32 || e->out_mode > APNN_OUT_FLOAT) return APNN_ERR_INVALID_ARG;
  if (e->out_mode == APNN_OUT_FLOAT) {
    // the float affine exists in the tcgen05 kernels' run-time epilogue and in apnn_requantize_i32
    if (!i8_rows_ok) return APNN_ERR_UNSUPPORTED;
    if (!e->affine_scale || !e->affine_bias || e->out_i8 || e->n_peer_out) return APNN_ERR_INVALID_ARG;
  } else if (e->out_mode != APNN_OUT_INT32) {
    if (e->out_bits < 1 || e->out_bits > 8) return APNN_ERR_INVALID_ARG;
    if (channels % 32 != 0) return APNN_ERR_UNSUPPORTED;
    if (e->out_mode == APNN_OUT_THRESHOLDS && !e->thresholds) return APNN_ERR_INVALID_ARG;
  }
  if (e->signed_operand < APNN_SIGN_NONE || e->signed_operand > APNN_SIGN_X) return APNN_ERR_INVALID_ARG;
  if (e->signed_operand == APNN_SIGN_W && abits_signed_w != 1) return APNN_ERR_UNSUPPORTED;
  if (e->signed_operand == APNN_SIGN_X && abits_signed_x != 1) return APNN_ERR_UNSUPPORTED;
  if (e->pool < APNN_POOL_NONE || e->pool > APNN_POOL_MAX2) return APNN_ERR_INVALID_ARG;
  if (!is_conv && (e->pool != APNN_POOL_NONE || e->out_halo != 0)) return APNN_ERR_INVALID_ARG;
  if (e->out_halo < 0 || e->out_halo > 8) return APNN_ERR_INVALID_ARG;
  if (e->in_halo < 0 || e->in_halo > 8 || (!is_conv && e->in_halo != 0)) return APNN_ERR_INVALID_ARG;
  if (e->n_peer_out < 0 || e->n_peer_out > 7 || (is_conv && e->n_peer_out != 0)) return APNN_ERR_INVALID_ARG;
  for (int i = 0; i < e->n_peer_out; i++)
    if (!e->peer_out[i] || (reinterpret_cast<uintptr_t>(e->peer_out[i]) & 15u)) return APNN_ERR_INVALID_ARG;
  return APNN_OK;
}

cudaError_t ensure_max_smem(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::vector<std::pair<const void*, int>> done;   // (kernel, device)
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  for (const auto& d : done)
    if (d.first == kernel && d.second == dev) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.emplace_back(kernel, dev);
  return e;
}

void* tensor_map_encoder() {
  static std::once_flag once;
  static void* fn = nullptr;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = ptr;
  });
  return fn;
}

int pdl_attribute(cudaLaunchAttribute* attrs) {
  static const bool enabled = [] { const char* v = getenv("APNN_PDL"); return !(v && v[0] == '0'); }();
  if (!enabled) return 0;
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  return 1;
}

// Plane counts the int8 (tcgen05) path takes: every level of up to 8 bits fits one byte.
bool tc5_bits_ok(int bits) { return (bits >= 1 && bits <= 4) || bits == 8; }

}  // namespace apnn

using namespace apnn;

extern "C" {

const char* apnn_status_string(apnn_status s) {
  switch (s) {
    case APNN_OK: return "ok";
    case APNN_ERR_INVALID_ARG: return "invalid argument";
    case APNN_ERR_UNSUPPORTED: return "unsupported bit widths or shape";
    case APNN_ERR_ALIGNMENT: return "pointer not 16-byte aligned or K not a multiple of 128";
    case APNN_ERR_WORKSPACE: return "workspace missing or too small";
    case APNN_ERR_CUDA: return "CUDA error";
    case APNN_ERR_NO_DEVICE: return "no sm_100 device";
    case APNN_ERR_TIMEOUT: return "a bounded device-side wait expired";
  }
  return "unknown status";
}

const char* apnn_last_cuda_error(void) { return g_cuda_err; }

int apnn_version(void) { return 100; }

size_t apnn_gemm_workspace_bytes(int algo, int wbits, int xbits, int M, int N, int K) {
  (void)wbits;
  (void)xbits;
  if (algo != APNN_ALGO_TCGEN05 && algo != APNN_ALGO_TCGEN05_PAIR) return 0;
  return tc5_workspace_bytes(M, N, K);
}

apnn_status apnn_gemm_check(void* stream, const void* workspace, int M, int N, int K) {
  if (!workspace || M <= 0 || N <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  int flag = tc5_read_error_flag(reinterpret_cast<cudaStream_t>(stream), workspace, M, N, K);
  if (flag < 0) return cuda_fail(cudaGetLastError(), "apnn_gemm_check");
  return flag == 0 ? APNN_OK : APNN_ERR_TIMEOUT;
}

apnn_status apnn_expand_planes(void* stream, const void* planes, void* out_i8, long rows, int K, int bits,
                               int is_signed) {
  if (!planes || !out_i8 || rows <= 0 || K <= 0 || bits < 1 || bits > 8) return APNN_ERR_INVALID_ARG;
  if (bits > 4 && bits < 8) return APNN_ERR_UNSUPPORTED;
  if (is_signed && bits != 1) return APNN_ERR_UNSUPPORTED;
  if (K % 64 != 0 || !aligned16(planes) || !aligned32(out_i8)) return APNN_ERR_ALIGNMENT;
  return tc5_expand(reinterpret_cast<cudaStream_t>(stream), (const uint32_t*)planes, (uint8_t*)out_i8, rows, K, bits,
                    is_signed != 0);
}

apnn_status apnn_expand_planes_pair(void* stream, const void* planes_w, void* w_i8, long rows_w, int wbits,
                                    int w_signed, const void* planes_x, void* x_i8, long rows_x, int xbits,
                                    int x_signed, int K) {
  if (!planes_w || !w_i8 || !planes_x || !x_i8 || rows_w <= 0 || rows_x <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  if (wbits < 1 || wbits > 8 || xbits < 1 || xbits > 8) return APNN_ERR_INVALID_ARG;
  if ((wbits > 4 && wbits < 8) || (xbits > 4 && xbits < 8)) return APNN_ERR_UNSUPPORTED;
  if ((w_signed && wbits != 1) || (x_signed && xbits != 1)) return APNN_ERR_UNSUPPORTED;
  if (K % 128 != 0 || !aligned16(planes_w) || !aligned32(w_i8) || !aligned16(planes_x) || !aligned32(x_i8))
    return APNN_ERR_ALIGNMENT;
  return tc5_expand2(reinterpret_cast<cudaStream_t>(stream), (const uint32_t*)planes_w, (uint8_t*)w_i8, rows_w, wbits,
                     w_signed != 0, (const uint32_t*)planes_x, (uint8_t*)x_i8, rows_x, xbits, x_signed != 0, K);
}

apnn_status apnn_gemm_i8(void* stream, const void* W8, const void* X8, void* D, int M, int N, int K, int w_signed,
                         int x_signed, const apnn_epilogue* epi, int* status_flag) {
  if (!W8 || !X8 || !D || !status_flag || M <= 0 || N <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  if (K % 128 != 0 || !aligned16(W8) || !aligned16(X8) || !aligned16(D)) return APNN_ERR_ALIGNMENT;
  if (epi) {
    // the sign lives in the expanded bytes; the epilogue must not correct again
    if (epi->signed_operand != APNN_SIGN_NONE) return APNN_ERR_INVALID_ARG;
    apnn_status st = check_epilogue(epi, N, false, 1, 1, true);
    if (st == APNN_OK && epi->out_i8 && !aligned32(D)) st = APNN_ERR_ALIGNMENT;
    if (st != APNN_OK) return st;
  }
  return tc5_gemm_i8(reinterpret_cast<cudaStream_t>(stream), (const uint8_t*)W8, (const uint8_t*)X8, D, M, N, K,
                     w_signed != 0, x_signed != 0, epi, status_flag);
}

apnn_status apnn_expand_planes_fp4(void* stream, const void* planes, void* out_fp4, long rows, int K, int bits, int is_signed) {
  if (!planes || !out_fp4 || rows <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  if (bits < 1 || bits > 2 || (is_signed && bits != 1)) return APNN_ERR_UNSUPPORTED;
  if (K % 256 != 0 || !aligned16(planes) || !aligned16(out_fp4)) return APNN_ERR_ALIGNMENT;
  return tc5_expand_fp4(reinterpret_cast<cudaStream_t>(stream), (const uint32_t*)planes, (uint8_t*)out_fp4, rows, K, bits,
                        is_signed != 0);
}

apnn_status apnn_gemm_fp4(void* stream, const void* W4, const void* X4, void* D, int M, int N, int K,
                          const apnn_epilogue* epi, int* status_flag) {
  if (!W4 || !X4 || !D || !status_flag || M <= 0 || N <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  if (K % 256 != 0 || !aligned16(W4) || !aligned16(X4) || !aligned16(D)) return APNN_ERR_ALIGNMENT;
  if ((long long)K * 9 >= (1ll << 24)) return APNN_ERR_UNSUPPORTED;   // sums must stay exact in fp32
  if (epi) {
    if (epi->signed_operand != APNN_SIGN_NONE) return APNN_ERR_INVALID_ARG;
    apnn_status st = check_epilogue(epi, N, false, 1, 1, true);
    if (st != APNN_OK) return st;
    if (epi->out_i8 || epi->residual_i16 || epi->out_mode == APNN_OUT_FLOAT) return APNN_ERR_UNSUPPORTED;
  }
  return tc5_gemm_fp4_pair(reinterpret_cast<cudaStream_t>(stream), (const uint8_t*)W4, (const uint8_t*)X4, D, M, N, K, epi,
                           status_flag);
}

apnn_status apnn_gemm_w8(void* stream, const void* W8, int xbits, const void* X, void* D, int M, int N, int K,
                         int w_signed, int x_signed, const apnn_epilogue* epi, int* status_flag) {
  if (!W8 || !X || !D || !status_flag || M <= 0 || N <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  if (xbits < 1 || xbits > 4 || (x_signed && xbits != 1)) return APNN_ERR_UNSUPPORTED;
  if (K % 128 != 0 || !aligned16(W8) || !aligned16(X) || !aligned16(D)) return APNN_ERR_ALIGNMENT;
  if (epi) {
    if (epi->signed_operand != APNN_SIGN_NONE) return APNN_ERR_INVALID_ARG;
    apnn_status st = check_epilogue(epi, N, false, 1, 1, true);
    if (st != APNN_OK) return st;
    // epilogues of the single-CTA kernel only
    if (epi->out_i8 || epi->residual_i16 || epi->out_mode == APNN_OUT_FLOAT) return APNN_ERR_UNSUPPORTED;
  }
  return tc5_gemm_i8_pair(reinterpret_cast<cudaStream_t>(stream), (const uint8_t*)W8, nullptr, D, M, N, K, w_signed != 0,
                          x_signed != 0, epi, status_flag, (const uint32_t*)X, xbits);
}

apnn_status apnn_gemm_ex(void* stream, int algo, int wbits, int xbits, const void* W, const void* X, void* D, int M,
                         int N, int K, const apnn_epilogue* epi, void* workspace, size_t workspace_bytes) {
  if (!W || !X || !D) return APNN_ERR_INVALID_ARG;
  if (M <= 0 || N <= 0 || K <= 0) return APNN_ERR_INVALID_ARG;
  if (algo < APNN_ALGO_AUTO || algo > APNN_ALGO_TCGEN05_PAIR) return APNN_ERR_INVALID_ARG;
  if (K % 128 != 0) return APNN_ERR_ALIGNMENT;
  if (!aligned16(W) || !aligned16(X) || !aligned16(D)) return APNN_ERR_ALIGNMENT;
  // the warp-level kernels are instantiated for the reference's pairs (w1a1..w1a4, w2a2 and
  // their mirrors); wider pairs (w4a4, w1a8, w2a8 ...) exist on the int8 tcgen05 path only
  const bool warp_ok = core_supports(wbits, xbits);
  if (!warp_ok && !(tc5_bits_ok(wbits) && tc5_bits_ok(xbits))) return APNN_ERR_UNSUPPORTED;
  apnn_status st = check_epilogue(epi, N, false, wbits, xbits);
  if (st != APNN_OK) return st;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);

  if (algo == APNN_ALGO_AUTO) {
    bool ws_ok = workspace && workspace_bytes >= tc5_workspace_bytes(M, N, K);
    algo = (ws_ok && (tc5_worthwhile(M, N, K) || !warp_ok)) ? APNN_ALGO_TCGEN05 : APNN_ALGO_IMMA;
  }
  if (!warp_ok && algo != APNN_ALGO_TCGEN05 && algo != APNN_ALGO_TCGEN05_PAIR)
    return workspace ? APNN_ERR_UNSUPPORTED : APNN_ERR_WORKSPACE;
  if (algo == APNN_ALGO_TCGEN05 || algo == APNN_ALGO_TCGEN05_PAIR) {
    if (!workspace || workspace_bytes < tc5_workspace_bytes(M, N, K)) return APNN_ERR_WORKSPACE;
    if (!aligned32(workspace)) return APNN_ERR_ALIGNMENT;
    return tc5_gemm(s, wbits, xbits, (const uint32_t*)W, (const uint32_t*)X, D, M, N, K, epi, workspace,
                    algo == APNN_ALGO_TCGEN05_PAIR ? 1 : 0);
  }

  if (epi && epi->n_peer_out != 0) return APNN_ERR_UNSUPPORTED;  // peer stores exist in the pair kernel only
  if (workspace && workspace_bytes >= tc5_workspace_bytes(M, N, K)) {
    // the warp-level kernels have no waits and never touch the flag apnn_gemm_check reads: clear it
    cudaError_t ce = cudaMemsetAsync(tc5_flag_slot(workspace, M, N, K), 0, sizeof(int), s);
    if (ce != cudaSuccess) return cuda_fail(ce, "status flag reset");
  }
  CoreParams p;
  memset(&p, 0, sizeof(p));
  p.A = (const uint32_t*)W;
  p.B = (const uint32_t*)X;
  p.a_plane_words = (long long)M * (K / 32);
  p.b_plane_words = (long long)N * (K / 32);
  p.M = M;
  p.N = N;
  p.kchunks = K / 128;
  p.a_row_words = K / 32;
  p.b_row_words = K / 32;
  p.out = D;
  p.out_mode = APNN_OUT_INT32;
  if (epi) {
    p.out_mode = epi->out_mode;
    p.out_bits = epi->out_bits;
    p.thresholds = epi->thresholds;
    p.sign = epi->signed_operand == APNN_SIGN_W ? SIGN_A : epi->signed_operand == APNN_SIGN_X ? SIGN_B : SIGN_NONE;
    p.out_plane_words = (long long)M * (N / 32);
    p.residual_in = epi->residual_in;
    p.residual_out = epi->residual_out;
  }
  int kind = algo == APNN_ALGO_BMMA ? CORE_B1 : CORE_U8;
  cudaError_t e = launch_core(kind, wbits, xbits, p, s, core_pick_tile(p, device_sm_count()));
  if (e != cudaSuccess) return cuda_fail(e, "apnn_gemm launch");
  return APNN_OK;
}

apnn_status apnn_gemm(void* stream, int wbits, int xbits, const void* W, const void* X, int32_t* D, int M, int N,
                      int K) {
  return apnn_gemm_ex(stream, APNN_ALGO_AUTO, wbits, xbits, W, X, D, M, N, K, nullptr, nullptr, 0);
}

size_t apnn_conv2d_workspace_bytes(int algo, int B, int H, int W, int CIN, int COUT, int R) {
  if (algo != APNN_ALGO_TCGEN05 || B <= 0 || H <= 0 || W <= 0 || CIN <= 0 || COUT <= 0 || (R < 1 || R > 11 || (R & 1) == 0)) return 0;
  return tc5_conv_workspace_bytes(B, H, W, CIN, COUT, R);
}

apnn_status apnn_conv2d_check(void* stream, const void* workspace, int B, int H, int W, int CIN, int COUT, int R) {
  if (!workspace || B <= 0 || H <= 0 || W <= 0 || CIN <= 0 || COUT <= 0) return APNN_ERR_INVALID_ARG;
  int flag = tc5_conv_read_error_flag(reinterpret_cast<cudaStream_t>(stream), workspace, B, H, W, CIN, COUT, R);
  if (flag < 0) return cuda_fail(cudaGetLastError(), "apnn_conv2d_check");
  return flag == 0 ? APNN_OK : APNN_ERR_TIMEOUT;
}

apnn_status apnn_conv2d_i8(void* stream, const void* W8, const void* X8, void* Out, int B, int H, int W, int CIN,
                           int COUT, int R, int stride, int w_signed, const apnn_epilogue* epi, int* status_flag) {
  if (!W8 || !X8 || !Out || !status_flag) return APNN_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || W <= 0 || CIN <= 0 || COUT <= 0) return APNN_ERR_INVALID_ARG;
  if (R < 1 || R > 11 || (R & 1) == 0) return APNN_ERR_UNSUPPORTED;
  if (CIN % 64 != 0 || !aligned16(W8) || !aligned16(X8) || !aligned16(Out)) return APNN_ERR_ALIGNMENT;
  if (epi) {
    if (epi->signed_operand != APNN_SIGN_NONE) return APNN_ERR_INVALID_ARG;  // the sign is in the bytes
    apnn_status st = check_epilogue(epi, COUT, true, 1, 1, true);
    if (st == APNN_OK && epi->out_i8 && !aligned32(Out)) st = APNN_ERR_ALIGNMENT;
    if (st != APNN_OK) return st;
    if (epi->pool != APNN_POOL_NONE && ((((H - 1) / (stride > 0 ? stride : 1) + 1) & 1) ||
                                        (((W - 1) / (stride > 0 ? stride : 1) + 1) & 1)))
      return APNN_ERR_UNSUPPORTED;
    if (epi->in_halo != 0 && epi->in_halo < (R - 1) / 2) return APNN_ERR_INVALID_ARG;
  }
  if (!tc5_conv_supported(H, W, R, stride, epi ? epi->pool : APNN_POOL_NONE)) return APNN_ERR_UNSUPPORTED;
  if (w_signed < 0 || w_signed > 3) return APNN_ERR_INVALID_ARG;
  return tc5_conv_i8(reinterpret_cast<cudaStream_t>(stream), (const uint8_t*)X8, (const uint8_t*)W8, Out, B, H, W,
                     CIN, COUT, R, stride, (w_signed & 1) != 0, epi, status_flag, (w_signed & 2) != 0);
}

apnn_status apnn_conv2d(void* stream, int wbits, int xbits, const void* Wt, const void* X, void* Out, int B, int H,
                        int Wd, int CIN, int COUT, int R, int stride, const apnn_epilogue* epi) {
  return apnn_conv2d_ex(stream, APNN_ALGO_IMMA, wbits, xbits, Wt, X, Out, B, H, Wd, CIN, COUT, R, stride, epi, nullptr,
                        0);
}

apnn_status apnn_conv2d_ex(void* stream, int algo, int wbits, int xbits, const void* Wt, const void* X, void* Out,
                           int B, int H, int Wd, int CIN, int COUT, int R, int stride, const apnn_epilogue* epi,
                           void* workspace, size_t workspace_bytes) {
  if (!Wt || !X || !Out) return APNN_ERR_INVALID_ARG;
  if (algo != APNN_ALGO_AUTO && algo != APNN_ALGO_IMMA && algo != APNN_ALGO_TCGEN05) return APNN_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || Wd <= 0 || CIN <= 0 || COUT <= 0) return APNN_ERR_INVALID_ARG;
  if (R < 1 || R > 11 || (R & 1) == 0) return APNN_ERR_UNSUPPORTED;
  if (stride < 1 || stride > 4) return APNN_ERR_UNSUPPORTED;
  // 64-channel feature maps run on the tcgen05 path only (64-byte swizzle rows)
  if (CIN % 128 != 0 && !(CIN % 64 == 0 && algo == APNN_ALGO_TCGEN05)) return APNN_ERR_ALIGNMENT;
  if (!aligned16(Wt) || !aligned16(X) || !aligned16(Out)) return APNN_ERR_ALIGNMENT;
  // core operand A = activations (xbits), B = filter (wbits)
  const bool warp_ok = core_supports(xbits, wbits);
  if (!warp_ok && !(tc5_bits_ok(wbits) && tc5_bits_ok(xbits))) return APNN_ERR_UNSUPPORTED;
  apnn_status st = check_epilogue(epi, COUT, true, wbits, xbits);
  if (st != APNN_OK) return st;
  const int pad = (R - 1) / 2;
  const int Ho = (H - 1) / stride + 1, Wo = (Wd - 1) / stride + 1;
  const int pool = epi ? epi->pool : APNN_POOL_NONE;
  if (pool != APNN_POOL_NONE && ((Ho & 1) || (Wo & 1))) return APNN_ERR_UNSUPPORTED;
  const long long pixels = (long long)B * Ho * Wo;
  if (pixels > 0x7fffffffLL) return APNN_ERR_UNSUPPORTED;

  if (algo == APNN_ALGO_AUTO) {
    // the tcgen05 path pays two expand launches; worth it once the contraction is sizeable
    const bool ws_ok = workspace && workspace_bytes >= tc5_conv_workspace_bytes(B, H, Wd, CIN, COUT, R);
    const double flops = 2.0 * (double)pixels * COUT * R * R * CIN;
    const bool exact_ring = !epi || epi->in_halo == 0 || epi->in_halo == pad;
    algo = (ws_ok && exact_ring && tc5_conv_supported(H, Wd, R, stride, pool) && (flops >= 2e9 || !warp_ok))
               ? APNN_ALGO_TCGEN05
               : APNN_ALGO_IMMA;
  }
  if (!warp_ok && algo != APNN_ALGO_TCGEN05) return workspace ? APNN_ERR_UNSUPPORTED : APNN_ERR_WORKSPACE;
  if (algo == APNN_ALGO_TCGEN05) {
    if (!tc5_conv_supported(H, Wd, R, stride, pool)) return APNN_ERR_UNSUPPORTED;
    if (epi && epi->in_halo != 0 && epi->in_halo != pad) return APNN_ERR_UNSUPPORTED;  // use apnn_conv2d_i8
    if (epi && epi->signed_operand == APNN_SIGN_X) return APNN_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < tc5_conv_workspace_bytes(B, H, Wd, CIN, COUT, R)) return APNN_ERR_WORKSPACE;
    if (!aligned32(workspace)) return APNN_ERR_ALIGNMENT;
    return tc5_conv(reinterpret_cast<cudaStream_t>(stream), wbits, xbits, (const uint32_t*)Wt, (const uint32_t*)X, Out,
                    B, H, Wd, CIN, COUT, R, stride, epi, workspace);
  }

  if (workspace && workspace_bytes >= tc5_conv_workspace_bytes(B, H, Wd, CIN, COUT, R)) {
    cudaError_t ce = cudaMemsetAsync(tc5_conv_flag_slot(workspace, B, H, Wd, CIN, COUT, R), 0, sizeof(int),
                                     reinterpret_cast<cudaStream_t>(stream));
    if (ce != cudaSuccess) return cuda_fail(ce, "status flag reset");
  }
  CoreParams p;
  memset(&p, 0, sizeof(p));
  p.A = (const uint32_t*)X;
  p.B = (const uint32_t*)Wt;
  const int in_halo = (epi && epi->in_halo) ? epi->in_halo : pad;
  if (in_halo < pad) return APNN_ERR_INVALID_ARG;
  p.Hp = H + 2 * in_halo;
  p.Wp = Wd + 2 * in_halo;
  p.in_off = in_halo - pad;
  p.cin_words = CIN / 32;
  p.cin_chunks = CIN / 128;
  p.a_plane_words = (long long)B * p.Hp * p.Wp * p.cin_words;
  p.b_row_words = R * R * p.cin_words;
  p.b_plane_words = (long long)COUT * p.b_row_words;
  p.M = (int)pixels;
  p.N = COUT;
  p.kchunks = R * R * p.cin_chunks;
  p.is_conv = 1;
  p.Ho = Ho;
  p.Wo = Wo;
  p.R = R;
  p.stride = stride;
  p.out = Out;
  p.out_mode = APNN_OUT_INT32;
  p.pool = pool;
  p.out_h = pool ? Ho / 2 : Ho;
  p.out_w = pool ? Wo / 2 : Wo;
  if (epi) {
    p.out_mode = epi->out_mode;
    p.out_bits = epi->out_bits;
    p.thresholds = epi->thresholds;
    // the filter is core operand B, the activations core operand A
    p.sign = epi->signed_operand == APNN_SIGN_W ? SIGN_B : epi->signed_operand == APNN_SIGN_X ? SIGN_A : SIGN_NONE;
    p.out_halo = epi->out_halo;
    p.residual_in = epi->residual_in;
    p.residual_out = epi->residual_out;
  }
  p.out_plane_words =
      (long long)B * (p.out_h + 2 * p.out_halo) * (p.out_w + 2 * p.out_halo) * (COUT / 32);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = launch_core(CORE_U8, xbits, wbits, p, s, core_pick_tile(p, device_sm_count()));
  if (e != cudaSuccess) return cuda_fail(e, "apnn_conv2d launch");
  return APNN_OK;
}

}  // extern "C"
