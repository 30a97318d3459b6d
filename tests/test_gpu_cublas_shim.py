"""The relink-level cuBLAS shim: cublasSgemm_v2 / cublasSgemmBatched / cublasSgemmStridedBatched with
cuBLAS's own signatures and a real cuBLAS handle compute what tcec_sgemm computes (bit for bit),
on the handle's stream; the reference's own benchmark, linked against the shim unchanged, runs."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import cpu
from wmma_extension_b200 import tcec

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "wmma_extension_b200", "libtcec_cublas_shim.so")
OP_N, OP_T = 0, 1
DEV = "cuda:0"


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def test_cublas_signatures_compute_the_tcec_product():
    if not os.path.exists(SHIM):
        pytest.skip("the shim library is not built")
    cublas = ctypes.CDLL("libcublas.so.12", mode=ctypes.RTLD_GLOBAL)
    shim = ctypes.CDLL(SHIM)
    handle = ctypes.c_void_p()
    assert cublas.cublasCreate_v2(ctypes.byref(handle)) == 0
    side = torch.cuda.Stream()
    assert cublas.cublasSetStream_v2(handle, ctypes.c_void_p(side.cuda_stream)) == 0
    i, p, ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong
    fp = ctypes.POINTER(ctypes.c_float)
    shim.cublasSgemm_v2.argtypes = [p, i, i, i, i, i, fp, p, i, p, i, fp, p, i]
    cublas.cublasSgemm_v2.argtypes = shim.cublasSgemm_v2.argtypes
    shim.cublasSgemmBatched.argtypes = [p, i, i, i, i, i, fp, p, i, p, i, fp, p, i, i]
    shim.cublasSgemmStridedBatched.argtypes = [p, i, i, i, i, i, fp, p, i, ll, p, i, ll, fp, p, i, ll, i]
    rng = np.random.default_rng(80)
    m, n, k, batch = 300, 200, 160, 3
    a = rng.standard_normal((batch, m, k)).astype(np.float32)   # logical A: row-major m x k = column-major k x m
    b = rng.standard_normal((batch, k, n)).astype(np.float32)
    c0 = rng.standard_normal((batch, m, n)).astype(np.float32)
    alpha, beta = ctypes.c_float(1.25), ctypes.c_float(-0.5)
    # the reference's argument list: OP_T on a row-major A (lda = k), OP_N on a column-major B (ldb = k), C column-major
    a_mem, b_mem = _t(a), _t(b.transpose(0, 2, 1))
    c_shim = _t(c0.transpose(0, 2, 1)).clone()
    c_real = c_shim.clone()
    c_tcec = c_shim.clone()
    torch.cuda.synchronize()
    st = shim.cublasSgemm_v2(handle, OP_T, OP_N, m, n, k, ctypes.byref(alpha), a_mem[0].data_ptr(), k,
                             b_mem[0].data_ptr(), k, ctypes.byref(beta), c_shim[0].data_ptr(), m)
    assert st == 0
    ptrs = [torch.tensor([x[j].data_ptr() for j in range(1, batch)], dtype=torch.int64, device=DEV)
            for x in (a_mem, b_mem, c_shim)]
    st = shim.cublasSgemmBatched(handle, OP_T, OP_N, m, n, k, ctypes.byref(alpha), ptrs[0].data_ptr(), k,
                                 ptrs[1].data_ptr(), k, ctypes.byref(beta), ptrs[2].data_ptr(), m, batch - 1)
    assert st == 0
    side.synchronize()
    tcec.device_status()
    lib = tcec.load()
    for j in range(batch):
        assert lib.tcec_sgemm_cublas(OP_T, OP_N, m, n, k, ctypes.byref(alpha), a_mem[j].data_ptr(), k, b_mem[j].data_ptr(),
                                     k, ctypes.byref(beta), c_tcec[j].data_ptr(), m, 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(c_shim, c_tcec)  # the shim is this library, not cuBLAS
    got = c_shim.cpu().numpy().transpose(0, 2, 1)
    for j in range(batch):
        want = 1.25 * cpu.gemm_f64(a[j], b[j]) - 0.5 * c0[j]
        assert cpu.errors(got[j], want)["max_rel"] < 1e-6
    # the strided form, against the real cuBLAS's result as the FP32 class
    c_str = _t(c0.transpose(0, 2, 1)).clone()
    st = shim.cublasSgemmStridedBatched(handle, OP_T, OP_N, m, n, k, ctypes.byref(alpha), a_mem.data_ptr(), k, m * k,
                                        b_mem.data_ptr(), k, k * n, ctypes.byref(beta), c_str.data_ptr(), m, m * n, batch)
    assert st == 0
    side.synchronize()
    assert torch.equal(c_str, c_tcec)
    assert cublas.cublasSgemm_v2(handle, OP_T, OP_N, m, n, k, ctypes.byref(alpha), a_mem[0].data_ptr(), k,
                                 b_mem[0].data_ptr(), k, ctypes.byref(beta), c_real[0].data_ptr(), m) == 0
    side.synchronize()
    assert torch.allclose(c_real[0], c_shim[0], rtol=0, atol=1e-3) and not torch.equal(c_real[0], c_shim[0])
    cublas.cublasDestroy_v2(handle)


def test_reference_benchmark_links_against_the_shim_unchanged():
    """test/tcec/batch_gemm.cu, compiled from where it lies with the reference's headers and linked with
    the shim before libcublas: it starts, and its cuBLAS leg resolves to this library."""
    exe = os.path.join(ROOT, "oracle", "_ref", "reftest_batch_gemm.shim")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/reftest_batch_gemm.shim was not built")
    out = subprocess.run(["ldd", exe], capture_output=True, text=True)
    libs = out.stdout
    assert "libtcec_cublas_shim.so" in libs and libs.index("libtcec_cublas_shim.so") < libs.index("libcublas.so")
