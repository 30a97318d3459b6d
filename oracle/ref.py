"""ctypes view of ``_ref/libtcec_ref.so``: the reference's own device code built for sm_100a.

TEST INFRASTRUCTURE ONLY.  Used on a GPU box to produce golden fixtures and as the
GPU comparator in parity tests.  ``available()`` is False when the library was
not built (the reference tree exists only where the build ran).
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libtcec_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(LIB_PATH)
        p, i, u, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_float, ctypes.c_size_t
        lib.ref_split.argtypes = [p, p, p, sz, i]
        lib.ref_split.restype = i
        lib.ref_warp_mma.argtypes = [i, i, i, p, p, p, p, i]
        lib.ref_warp_mma.restype = i
        lib.ref_bgemm.argtypes = [i, i, u, u, u, f, p, u, p, u, f, p, u, u]
        lib.ref_bgemm.restype = i
        _lib = lib
    return _lib


def split(x: torch.Tensor, tf32: bool):
    x = x.contiguous()
    hi, lo = torch.empty_like(x), torch.empty_like(x)
    rc = load().ref_split(x.data_ptr(), hi.data_ptr(), lo.data_ptr(), x.numel(), int(tf32))
    torch.cuda.synchronize()
    assert rc == 0, rc
    return hi, lo


def warp_mma(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor | None, tf32: bool, op_wmma: bool, ec: bool,
             rz: bool = False) -> torch.Tensor:
    """32x32x32 on one warp. a: (32,32) row-major A; b: (32,32) holding B (k x n); returns D row-major."""
    a = a.contiguous()
    b_col = b.t().contiguous()  # column-major storage of B
    d = torch.empty(32, 32, device=a.device, dtype=torch.float32)
    cp = c.contiguous().data_ptr() if c is not None else None
    rc = load().ref_warp_mma(int(tf32), int(op_wmma), int(ec), d.data_ptr(), a.data_ptr(), b_col.data_ptr(), cp,
                             int(rz))
    torch.cuda.synchronize()
    assert rc == 0, rc
    return d


def bgemm(a: torch.Tensor, b: torch.Tensor, tf32: bool = False, per: int = 4, alpha: float = 1.0) -> torch.Tensor:
    """Reference batched TCEC GEMM. a: (batch, m, k), b: (batch, k, n) -> (batch, m, n).

    The reference kernel wants A row-major, B column-major and writes C column-major,
    so B is handed over transposed and C is read back transposed; the products and
    their k order are unchanged.  Launches on the default stream.
    """
    batch, m, k = a.shape
    n = b.shape[2]
    a = a.contiguous()
    bt = b.transpose(1, 2).contiguous()  # (batch, n, k): column-major k x n
    ct = torch.empty(batch, n, m, device=a.device, dtype=torch.float32)  # column-major m x n
    pa = torch.tensor([a[i].data_ptr() for i in range(batch)], dtype=torch.int64, device=a.device)
    pb = torch.tensor([bt[i].data_ptr() for i in range(batch)], dtype=torch.int64, device=a.device)
    pc = torch.tensor([ct[i].data_ptr() for i in range(batch)], dtype=torch.int64, device=a.device)
    torch.cuda.synchronize()
    rc = load().ref_bgemm(int(tf32), per, m, n, k, alpha, pa.data_ptr(), k, pb.data_ptr(), k, 0.0, pc.data_ptr(),
                          m, batch)
    torch.cuda.synchronize()
    assert rc == 0, rc
    return ct.transpose(1, 2)
