"""ctypes/numpy view of ``liboracle.so`` (the CPU restatement in ``tcec_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and
the CPU-baseline legs of ``bench.py``; the product library never touches it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build() -> None:
    subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        build()
    lib = ctypes.CDLL(LIB_PATH)
    f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
    i, ll, f, sz = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_size_t
    lib.oracle_round_fp16.argtypes = [f]
    lib.oracle_round_fp16.restype = f
    lib.oracle_round_tf32.argtypes = [f]
    lib.oracle_round_tf32.restype = f
    lib.oracle_split.argtypes = [f32p, f32p, f32p, sz, i]
    lib.oracle_split.restype = None
    lib.oracle_tcec_gemm.argtypes = [i, i, i, i, i, i, f, f32p, ll, f32p, ll, f, f32p, ll, i, i, i, i]
    lib.oracle_tcec_gemm.restype = None
    lib.oracle_gemm_f64.argtypes = [i, i, i, i, i, f32p, ll, f32p, ll, f64p, ll, i, i]
    lib.oracle_gemm_f64.restype = None
    lib.oracle_gemm_f32.argtypes = [i, i, i, i, i, f32p, ll, f32p, ll, f32p, ll, i, i]
    lib.oracle_gemm_f32.restype = None
    lib.oracle_errors.argtypes = [f32p, f64p, sz, f64p]
    lib.oracle_errors.restype = None
    lib.oracle_set_num_threads.argtypes = [i]
    lib.oracle_set_num_threads.restype = None
    lib.oracle_num_threads.argtypes = []
    lib.oracle_num_threads.restype = i
    _lib = lib
    return lib


def _is_tf32(policy: str) -> int:
    return 1 if policy.startswith("tf32") else 0


def _is_ec(policy: str) -> int:
    return 0 if policy.endswith("no_ec") else 1


def split(x: np.ndarray, policy: str = "fp16_ec"):
    """hi, lo (lo scaled by 2^11 for fp16) of every element, widened to float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    hi = np.empty_like(x)
    lo = np.empty_like(x)
    load().oracle_split(x.reshape(-1), hi.reshape(-1), lo.reshape(-1), x.size, _is_tf32(policy))
    return hi, lo


def _mat(x: np.ndarray):
    """(array to pass, col_major flag, ld) for a 2-D float32 array, C- or F-ordered."""
    if x.flags["C_CONTIGUOUS"]:
        return x, 0, x.shape[1]
    if x.flags["F_CONTIGUOUS"]:
        return x.T, 1, x.shape[0]
    x = np.ascontiguousarray(x)
    return x, 0, x.shape[1]


def tcec_gemm(a: np.ndarray, b: np.ndarray, c: np.ndarray | None = None, alpha: float = 1.0,
              beta: float = 0.0, policy: str = "fp16_ec", rn_block: int = 1, tc_rz: bool = False) -> np.ndarray:
    """The reference's arithmetic on the CPU; returns a C-ordered (m, n) float32 array."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    m, k = a.shape
    _, n = b.shape
    out = np.zeros((m, n), dtype=np.float32) if c is None else np.ascontiguousarray(c, dtype=np.float32).copy()
    aa, acol, lda = _mat(a)
    bb, bcol, ldb = _mat(b)
    load().oracle_tcec_gemm(acol, bcol, 0, m, n, k, alpha, np.ascontiguousarray(aa).reshape(-1), lda,
                            np.ascontiguousarray(bb).reshape(-1), ldb, beta, out.reshape(-1), n,
                            _is_tf32(policy), _is_ec(policy), rn_block, int(tc_rz))
    return out


def tcec_cgemm(a: np.ndarray, b: np.ndarray, policy: str = "fp16_ec", rn_block: int = 1) -> np.ndarray:
    """Complex product from four real TCEC products in the reference's order
    (include/wmma_extension/tcec/complex.hpp:712-727): imag = Ai Br, then += Ar Bi;
    real = Ar Br, then += Ai (-Bi).  Returns a complex64 (m, n) array."""
    a = np.asarray(a, dtype=np.complex64)
    b = np.asarray(b, dtype=np.complex64)
    ar, ai = np.ascontiguousarray(a.real), np.ascontiguousarray(a.imag)
    br, bi = np.ascontiguousarray(b.real), np.ascontiguousarray(b.imag)
    im = tcec_gemm(ai, br, policy=policy, rn_block=rn_block)
    im = tcec_gemm(ar, bi, c=im, beta=1.0, policy=policy, rn_block=rn_block)
    re = tcec_gemm(ar, br, policy=policy, rn_block=rn_block)
    re = tcec_gemm(ai, -bi, c=re, beta=1.0, policy=policy, rn_block=rn_block)
    return (re + 1j * im).astype(np.complex64)


def gemm_f64(a: np.ndarray, b: np.ndarray, row0: int = 0, row1: int | None = None) -> np.ndarray:
    """FP64 ground truth for rows [row0, row1) of A @ B."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    m, k = a.shape
    _, n = b.shape
    row1 = m if row1 is None else row1
    out = np.empty((row1 - row0, n), dtype=np.float64)
    aa, acol, lda = _mat(a)
    bb, bcol, ldb = _mat(b)
    load().oracle_gemm_f64(acol, bcol, m, n, k, np.ascontiguousarray(aa).reshape(-1), lda,
                           np.ascontiguousarray(bb).reshape(-1), ldb, out.reshape(-1), n, row0, row1)
    return out


def gemm_f32(a: np.ndarray, b: np.ndarray, row0: int = 0, row1: int | None = None) -> np.ndarray:
    """Sequential FP32-FMA GEMM (the accuracy class of an FP32 SIMT SGEMM)."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    m, k = a.shape
    _, n = b.shape
    row1 = m if row1 is None else row1
    out = np.empty((row1 - row0, n), dtype=np.float32)
    aa, acol, lda = _mat(a)
    bb, bcol, ldb = _mat(b)
    load().oracle_gemm_f32(acol, bcol, m, n, k, np.ascontiguousarray(aa).reshape(-1), lda,
                           np.ascontiguousarray(bb).reshape(-1), ldb, out.reshape(-1), n, row0, row1)
    return out


def errors(c: np.ndarray, ref: np.ndarray) -> dict:
    """max-rel (max|d|/max|ref|), relative Frobenius residual and max-abs error."""
    c = np.ascontiguousarray(c, dtype=np.float32).reshape(-1)
    ref = np.ascontiguousarray(ref, dtype=np.float64).reshape(-1)
    out = np.zeros(3, dtype=np.float64)
    load().oracle_errors(c, ref, c.size, out)
    return {"max_rel": float(out[0]), "fro_rel": float(out[1]), "max_abs": float(out[2])}


def use_all_cores() -> int:
    """Lets the host loops use every core of the machine, whatever the launcher put into
    OMP_NUM_THREADS or the affinity mask (torchrun sets OMP_NUM_THREADS=1); returns the count."""
    n = os.cpu_count() or 1
    try:
        os.sched_setaffinity(0, range(n))
    except (AttributeError, OSError):
        pass
    load().oracle_set_num_threads(n)
    return num_threads()


def num_threads() -> int:
    return int(load().oracle_num_threads())
