"""GPU test of apnn_gemm_static_scratch, the GEMM entry point for callers that cannot
allocate a workspace (its operands' int8 images live in a fixed array inside the library).

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test.  It calls the entry point through the C ABI twice in a row -- the
second, smaller problem lands on top of the first one's left-overs in the shared array --
and compares each result bit for bit with the CPU oracle and with the regular entry point
apnn_gemm_ex, and checks with cudaMemGetInfo that the calls left the amount of free device
memory unchanged.  It needs no state from other tests and leaves none behind.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from apnn_tc_b200 import _cabi

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 32 * 1024 * 1024


def _words(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randint(-2**31, 2**31 - 1, shape, dtype=torch.int32, device="cuda", generator=g)


def _host(t):
    return t.cpu().numpy().view(np.uint32)


def _static(L, W, X, M, N, K, wb, xb, epi=None):
    out_shape = (M, N) if epi is None or epi.out_mode == 0 else (epi.out_bits, M, N // 32)
    D = torch.full(out_shape, -1, dtype=torch.int32, device="cuda")
    flag = torch.full((1,), 7, dtype=torch.int32, device="cuda")  # must be reset by the call

    def call():
        st = L.apnn_gemm_static_scratch(torch.cuda.current_stream().cuda_stream, wb, xb, W.data_ptr(), X.data_ptr(),
                                        D.data_ptr(), M, N, K, ctypes.byref(epi) if epi is not None else None,
                                        flag.data_ptr())
        _cabi.check(st, "apnn_gemm_static_scratch")
        torch.cuda.synchronize()
        assert int(flag.item()) == 0

    call()   # the first use of a kernel may load its code onto the device (lazy module loading)
    first = D.clone()
    D.fill_(-1)
    flag.fill_(7)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()   # cudaMemGetInfo; every buffer of the call exists already
    call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the entry point must not allocate or free device memory"
    assert torch.equal(first, D)
    return D


def _regular(L, W, X, M, N, K, wb, xb, epi=None):
    out_shape = (M, N) if epi is None or epi.out_mode == 0 else (epi.out_bits, M, N // 32)
    D = torch.full(out_shape, -2, dtype=torch.int32, device="cuda")
    st = L.apnn_gemm_ex(torch.cuda.current_stream().cuda_stream, _cabi.ALGO_IMMA, wb, xb, W.data_ptr(), X.data_ptr(),
                        D.data_ptr(), M, N, K, ctypes.byref(epi) if epi is not None else None, None, 0)
    _cabi.check(st, "apnn_gemm_ex")
    torch.cuda.synchronize()
    return D


def test_static_scratch_matches_regular_entry_point_twice(cuda_device):
    L = _cabi.lib()
    # call 1: fills most of the array (w1a2, 1536 x 2304 x 4096: 15.0 MiB of int8 images)
    M, N, K = 1536, 2304, 4096
    W, X = _words((1, M, K // 32), 1), _words((2, N, K // 32), 2)
    D = _static(L, W, X, M, N, K, 1, 2)
    assert np.array_equal(D.cpu().numpy(), oracle.gemm_popc(_host(W), _host(X), threads=8))
    assert torch.equal(D, _regular(L, W, X, M, N, K, 1, 2))
    # call 2, straight after: a smaller, ragged w2a2 problem written over call 1's left-overs,
    # with the low-bit packed epilogue
    M, N, K = 200, 352, 768
    W, X = _words((2, M, K // 32), 3), _words((2, N, K // 32), 4)
    epi = _cabi.Epilogue(out_mode=_cabi.OUT_LOWBITS, out_bits=2)
    P = _static(L, W, X, M, N, K, 2, 2, epi)
    assert np.array_equal(_host(P), oracle.requant_pack(oracle.gemm_popc(_host(W), _host(X), threads=4), 2, 1))
    assert torch.equal(P, _regular(L, W, X, M, N, K, 2, 2, epi))
    # call 3: +-1 weights, int32 output, same array again
    M, N, K = 130, 257, 640
    W, X = _words((1, M, K // 32), 5), _words((3, N, K // 32), 6)
    epi = _cabi.Epilogue(out_mode=_cabi.OUT_INT32, signed_operand=_cabi.SIGN_W)
    D = _static(L, W, X, M, N, K, 1, 3, epi)
    want = oracle.signed_correct(oracle.gemm_popc(_host(W), _host(X), threads=4), oracle.row_sums(_host(X)), 1)
    assert np.array_equal(D.cpu().numpy(), want)
    assert torch.equal(D, _regular(L, W, X, M, N, K, 1, 3, epi))


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    L = _cabi.lib()
    M = N = 4096
    K = 4096 + 128  # (M + N) * K just over 32 MiB
    assert (M + N) * K > SCRATCH_BYTES
    W, X = _words((1, M, K // 32), 7), _words((2, N, K // 32), 8)
    D = torch.zeros((8,), dtype=torch.int32, device="cuda")  # never written: the call must refuse first
    flag = torch.zeros((1,), dtype=torch.int32, device="cuda")
    st = L.apnn_gemm_static_scratch(torch.cuda.current_stream().cuda_stream, 1, 2, W.data_ptr(), X.data_ptr(),
                                    D.data_ptr(), M, N, K, None, flag.data_ptr())
    assert st == 4  # APNN_ERR_WORKSPACE
    assert L.apnn_status_string(st) == b"workspace missing or too small"
    # the largest problem that fits is accepted: 4096 x 4096 x 4096 uses the array exactly
    K = 4096
    W, X = _words((1, M, K // 32), 9), _words((2, N, K // 32), 10)
    D = _static(L, W, X, M, N, K, 1, 2)
    rows = np.array([0, 127, 128, 2049, 4095])
    want = oracle.gemm_popc(np.ascontiguousarray(_host(W)[:, rows]), _host(X), threads=8)
    assert np.array_equal(D[torch.from_numpy(rows).cuda()].cpu().numpy(), want)
    assert torch.equal(D, _regular(L, W, X, M, N, K, 1, 2))
    # bad arguments come back as status codes too
    assert L.apnn_gemm_static_scratch(None, 1, 2, W.data_ptr(), X.data_ptr(), D.data_ptr(), M, N, K, None, None) == 1
    assert L.apnn_gemm_static_scratch(None, 5, 2, W.data_ptr(), X.data_ptr(), D.data_ptr(), M, N, K, None,
                                      flag.data_ptr()) == 2
