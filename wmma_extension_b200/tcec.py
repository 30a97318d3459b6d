"""ctypes binding of the C ABI in ``include/tcec.h`` for torch CUDA tensors.

PyTorch is used for device memory and streams only; all arithmetic happens in
the sm_100a kernels of ``libtcec_b200.so``.  There is no CPU or eager fallback:
if the shared library is missing, or no sm_100 device is present, calls raise.

Policy names follow the reference's fragment type and error-correction tags
(``half`` / ``tf32`` x ``with_ec`` / ``without_ec``,
include/wmma_extension/tcec/detail/policy.hpp:12-20).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtcec_b200.so")

ROW_MAJOR, COL_MAJOR = 0, 1
POLICIES = {"fp16_ec": 0, "tf32_ec": 1, "fp16_no_ec": 2, "tf32_no_ec": 3}
OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_ALLOC, ERR_TOO_LARGE, ERR_COMM = range(8)
COMM_ID_BYTES = 128

EXPORTED_SYMBOLS = (
    "tcec_sgemm",
    "tcec_sgemm_batched",
    "tcec_sgemm_strided_batched",
    "tcec_packed_bytes",
    "tcec_packed_row_offset",
    "tcec_pack_a",
    "tcec_pack_b",
    "tcec_sgemm_packed",
    "tcec_split",
    "tcec_cgemm",
    "tcec_sgemm_cublas",
    "tcec_sgemm_batched_cublas",
    "tcec_sgemm_host",
    "tcec_sgemm_multi",
    "tcec_sgemm_batched_multi",
    "tcec_comm_set_library",
    "tcec_comm_unique_id",
    "tcec_comm_init_rank",
    "tcec_comm_destroy",
    "tcec_sgemm_column_shard",
    "tcec_sgemm_column_shard_host",
    "tcec_sgemm_static",
    "tcec_static_scratch_bytes",
    "tcec_static_status",
    "tcec_set_option",
    "tcec_get_option",
    "tcec_device_status",
    "tcec_workspace_bytes",
    "tcec_destroy",
    "tcec_status_string",
    "tcec_version",
)

_lib = None


class TcecError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: status {status} ({status_string(status)})")


def load() -> ctypes.CDLL:
    """Load the in-tree shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no fallback path)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    i, ll, f, p, sz = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
    lib.tcec_sgemm.argtypes = [i, i, i, i, i, i, f, p, ll, p, ll, f, p, ll, i, p]
    lib.tcec_sgemm.restype = i
    lib.tcec_sgemm_batched.argtypes = [i, i, i, i, i, i, f, p, ll, p, ll, f, p, ll, i, i, p]
    lib.tcec_sgemm_batched.restype = i
    lib.tcec_sgemm_strided_batched.argtypes = [i, i, i, i, i, i, f, p, ll, ll, p, ll, ll, f, p, ll, ll, i, i, p]
    lib.tcec_sgemm_strided_batched.restype = i
    lib.tcec_packed_bytes.argtypes = [i, i, i]
    lib.tcec_packed_bytes.restype = sz
    lib.tcec_packed_row_offset.argtypes = [i, i, i]
    lib.tcec_packed_row_offset.restype = sz
    lib.tcec_pack_a.argtypes = [i, i, i, p, ll, p, i, p]
    lib.tcec_pack_a.restype = i
    lib.tcec_pack_b.argtypes = [i, i, i, p, ll, p, i, p]
    lib.tcec_pack_b.restype = i
    lib.tcec_sgemm_packed.argtypes = [i, i, i, i, f, p, p, f, p, ll, i, p]
    lib.tcec_sgemm_packed.restype = i
    fp = ctypes.POINTER(ctypes.c_float)
    lib.tcec_sgemm_cublas.argtypes = [i, i, i, i, i, fp, p, i, p, i, fp, p, i, i, p]
    lib.tcec_sgemm_cublas.restype = i
    lib.tcec_sgemm_batched_cublas.argtypes = [i, i, i, i, i, fp, p, i, p, i, fp, p, i, i, i, p]
    lib.tcec_sgemm_batched_cublas.restype = i
    lib.tcec_sgemm_static.argtypes = [i, i, i, i, i, i, f, p, ll, p, ll, f, p, ll, i, p]
    lib.tcec_sgemm_static.restype = i
    lib.tcec_static_scratch_bytes.argtypes = []
    lib.tcec_static_scratch_bytes.restype = sz
    lib.tcec_static_status.argtypes = [ctypes.POINTER(i)]
    lib.tcec_static_status.restype = i
    lib.tcec_sgemm_host.argtypes = [i, i, i, i, i, i, f, p, ll, p, ll, f, p, ll, i, i, p]
    lib.tcec_sgemm_host.restype = i
    ip, pp, llp = ctypes.POINTER(i), ctypes.POINTER(p), ctypes.POINTER(ll)
    lib.tcec_sgemm_multi.argtypes = [i, ip, i, i, i, i, ip, i, f, p, ll, pp, llp, f, pp, llp, i, pp]
    lib.tcec_sgemm_multi.restype = i
    lib.tcec_sgemm_batched_multi.argtypes = [i, ip, i, i, i, i, i, i, f, pp, ll, ll, pp, ll, ll, f, pp, ll, ll, ip, i, pp]
    lib.tcec_sgemm_batched_multi.restype = i
    lib.tcec_comm_set_library.argtypes = [ctypes.c_char_p]
    lib.tcec_comm_set_library.restype = i
    lib.tcec_comm_unique_id.argtypes = [p]
    lib.tcec_comm_unique_id.restype = i
    lib.tcec_comm_init_rank.argtypes = [i, i, p]
    lib.tcec_comm_init_rank.restype = i
    lib.tcec_comm_destroy.argtypes = []
    lib.tcec_comm_destroy.restype = i
    lib.tcec_sgemm_column_shard.argtypes = [i, i, i, i, i, i, i, f, p, ll, p, ll, f, p, ll, i, p]
    lib.tcec_sgemm_column_shard.restype = i
    lib.tcec_sgemm_column_shard_host.argtypes = [i, i, i, i, i, i, i, f, p, ll, p, ll, f, p, ll, i, i, p]
    lib.tcec_sgemm_column_shard_host.restype = i
    lib.tcec_cgemm.argtypes = [i, i, i, i, i, i, fp, p, ll, p, ll, fp, p, ll, i, p]
    lib.tcec_cgemm.restype = i
    lib.tcec_split.argtypes = [p, p, p, sz, i, p]
    lib.tcec_split.restype = i
    lib.tcec_set_option.argtypes = [ctypes.c_char_p, i]
    lib.tcec_set_option.restype = i
    lib.tcec_get_option.argtypes = [ctypes.c_char_p, ctypes.POINTER(i)]
    lib.tcec_get_option.restype = i
    lib.tcec_device_status.argtypes = [ctypes.POINTER(i)]
    lib.tcec_device_status.restype = i
    lib.tcec_workspace_bytes.argtypes = [i, i, i, i, i]
    lib.tcec_workspace_bytes.restype = sz
    lib.tcec_destroy.argtypes = []
    lib.tcec_destroy.restype = i
    lib.tcec_status_string.argtypes = [i]
    lib.tcec_status_string.restype = ctypes.c_char_p
    lib.tcec_version.argtypes = []
    lib.tcec_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().tcec_status_string(status).decode()


def _check(status: int, what: str) -> None:
    if status != OK:
        raise TcecError(status, what)


def _policy(policy) -> int:
    if isinstance(policy, str):
        return POLICIES[policy]
    return int(policy)


def _layout_ld(t: torch.Tensor):
    """(layout, leading dimension) of a 2-D view, from its strides."""
    r, c = t.shape[-2], t.shape[-1]
    s0, s1 = t.stride(-2), t.stride(-1)
    if s1 == 1 and (s0 >= c or r == 1):
        return ROW_MAJOR, max(s0, c)
    if s0 == 1 and (s1 >= r or c == 1):
        return COL_MAJOR, max(s1, r)
    raise ValueError("matrix must have unit stride along rows or columns")


def _require_cuda_f32(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_cuda or t.dtype != torch.float32:
            raise ValueError("operands must be float32 CUDA tensors")


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def set_option(name: str, value: int) -> None:
    _check(load().tcec_set_option(name.encode(), int(value)), f"tcec_set_option({name})")


def get_option(name: str) -> int:
    v = ctypes.c_int(0)
    _check(load().tcec_get_option(name.encode(), ctypes.byref(v)), f"tcec_get_option({name})")
    return v.value


def device_status() -> int:
    """Synchronise and raise if a kernel gave up a bounded wait."""
    detail = ctypes.c_int(0)
    st = load().tcec_device_status(ctypes.byref(detail))
    if st != OK:
        raise TcecError(st, f"device status word {detail.value}")
    return detail.value


def sgemm(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, *, alpha: float = 1.0,
          beta: float = 0.0, policy="fp16_ec") -> torch.Tensor:
    """C = alpha * A @ B + beta * C for 2-D float32 CUDA tensors (row- or column-major views)."""
    _require_cuda_f32(a, b)
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise ValueError("inner dimensions differ")
    if c is None:
        c = torch.empty((m, n), dtype=torch.float32, device=a.device)
    _require_cuda_f32(c)
    la, lda = _layout_ld(a)
    lb, ldb = _layout_ld(b)
    lc, ldc = _layout_ld(c)
    with torch.cuda.device(a.device):
        st = load().tcec_sgemm(la, lb, lc, m, n, k, alpha, a.data_ptr(), lda, b.data_ptr(), ldb, beta,
                               c.data_ptr(), ldc, _policy(policy), _stream_ptr())
    _check(st, "tcec_sgemm")
    return c


def cgemm(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, *, alpha: complex = 1.0,
          beta: complex = 0.0, policy="fp16_ec") -> torch.Tensor:
    """C = alpha * A @ B + beta * C for 2-D complex64 CUDA tensors (row- or column-major views)."""
    for t in (a, b) + ((c,) if c is not None else ()):
        if not t.is_cuda or t.dtype != torch.complex64:
            raise ValueError("operands must be complex64 CUDA tensors")
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise ValueError("inner dimensions differ")
    if c is None:
        c = torch.empty((m, n), dtype=torch.complex64, device=a.device)
    la, lda = _layout_ld(a)
    lb, ldb = _layout_ld(b)
    lc, ldc = _layout_ld(c)
    al = (ctypes.c_float * 2)(complex(alpha).real, complex(alpha).imag)
    be = (ctypes.c_float * 2)(complex(beta).real, complex(beta).imag)
    with torch.cuda.device(a.device):
        st = load().tcec_cgemm(la, lb, lc, m, n, k, al, a.data_ptr(), lda, b.data_ptr(), ldb, be,
                               c.data_ptr(), ldc, _policy(policy), _stream_ptr())
    _check(st, "tcec_cgemm")
    return c


def sgemm_static(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, *, alpha: float = 1.0, beta: float = 0.0,
                 policy="fp16_ec") -> torch.Tensor:
    """``sgemm`` through the entry point that allocates nothing (``tcec_sgemm_static``).

    For callers that cannot allocate device memory when they need the product; the split
    operands go to a fixed array inside the library, so the problem must fit it
    (``TcecError`` with ``ERR_TOO_LARGE`` otherwise) and ``c`` must be supplied.  Calls that
    overlap on the GPU share that array and race: keep them on one stream.
    """
    _require_cuda_f32(a, b, c)
    m, k = a.shape
    k2, n = b.shape
    if k != k2 or tuple(c.shape) != (m, n):
        raise ValueError("shape mismatch")
    la, lda = _layout_ld(a)
    lb, ldb = _layout_ld(b)
    lc, ldc = _layout_ld(c)
    with torch.cuda.device(a.device):
        st = load().tcec_sgemm_static(la, lb, lc, m, n, k, alpha, a.data_ptr(), lda, b.data_ptr(), ldb, beta,
                                      c.data_ptr(), ldc, _policy(policy), _stream_ptr())
    _check(st, "tcec_sgemm_static")
    return c


def static_status() -> int:
    """Synchronise and raise if a kernel launched by ``sgemm_static`` gave up a bounded wait."""
    detail = ctypes.c_int(0)
    st = load().tcec_static_status(ctypes.byref(detail))
    if st != OK:
        raise TcecError(st, f"static status word {detail.value}")
    return detail.value


def sgemm_strided_batched(a: torch.Tensor, b: torch.Tensor, c: Optional[torch.Tensor] = None, *,
                          alpha: float = 1.0, beta: float = 0.0, policy="fp16_ec") -> torch.Tensor:
    """Batched product of 3-D tensors [batch, m, k] x [batch, k, n] with a uniform batch stride."""
    _require_cuda_f32(a, b)
    batch, m, k = a.shape
    _, k2, n = b.shape
    if k != k2 or b.shape[0] != batch:
        raise ValueError("shape mismatch")
    if c is None:
        c = torch.empty((batch, m, n), dtype=torch.float32, device=a.device)
    _require_cuda_f32(c)
    la, lda = _layout_ld(a)
    lb, ldb = _layout_ld(b)
    lc, ldc = _layout_ld(c)
    with torch.cuda.device(a.device):
        st = load().tcec_sgemm_strided_batched(
            la, lb, lc, m, n, k, alpha, a.data_ptr(), lda, a.stride(0), b.data_ptr(), ldb, b.stride(0), beta,
            c.data_ptr(), ldc, c.stride(0), batch, _policy(policy), _stream_ptr())
    _check(st, "tcec_sgemm_strided_batched")
    return c


def sgemm_batched(a_list: Sequence[torch.Tensor], b_list: Sequence[torch.Tensor],
                  c_list: Sequence[torch.Tensor], *, alpha: float = 1.0, beta: float = 0.0,
                  policy="fp16_ec") -> Sequence[torch.Tensor]:
    """Pointer-array batch: one independent matrix per list entry, equal shapes and strides."""
    batch = len(a_list)
    if batch == 0:
        return c_list
    _require_cuda_f32(*a_list, *b_list, *c_list)
    m, k = a_list[0].shape
    _, n = b_list[0].shape
    la, lda = _layout_ld(a_list[0])
    lb, ldb = _layout_ld(b_list[0])
    lc, ldc = _layout_ld(c_list[0])
    dev = a_list[0].device

    def ptrs(ts):
        return torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64).to(dev)

    pa, pb, pc = ptrs(a_list), ptrs(b_list), ptrs(c_list)
    with torch.cuda.device(dev):
        st = load().tcec_sgemm_batched(la, lb, lc, m, n, k, alpha, pa.data_ptr(), lda, pb.data_ptr(), ldb, beta,
                                       pc.data_ptr(), ldc, batch, _policy(policy), _stream_ptr())
        _check(st, "tcec_sgemm_batched")
        # the pointer tables must outlive the kernels that read them
        torch.cuda.current_stream().synchronize()
    return c_list


def packed_bytes(rows: int, k: int, policy="fp16_ec") -> int:
    return int(load().tcec_packed_bytes(rows, k, _policy(policy)))


def packed_row_offset(row: int, k: int, policy="fp16_ec") -> int:
    return int(load().tcec_packed_row_offset(row, k, _policy(policy)))


def pack_a(a: torch.Tensor, policy="fp16_ec", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Split A (m x k) once into operand panels; returns the uint8 panel buffer."""
    _require_cuda_f32(a)
    m, k = a.shape
    la, lda = _layout_ld(a)
    if out is None:
        out = torch.empty(packed_bytes(m, k, policy), dtype=torch.uint8, device=a.device)
    with torch.cuda.device(a.device):
        st = load().tcec_pack_a(la, m, k, a.data_ptr(), lda, out.data_ptr(), _policy(policy), _stream_ptr())
    _check(st, "tcec_pack_a")
    return out


def pack_b(b: torch.Tensor, policy="fp16_ec", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Split B (k x n) once into operand panels; returns the uint8 panel buffer."""
    _require_cuda_f32(b)
    k, n = b.shape
    lb, ldb = _layout_ld(b)
    if out is None:
        out = torch.empty(packed_bytes(n, k, policy), dtype=torch.uint8, device=b.device)
    with torch.cuda.device(b.device):
        st = load().tcec_pack_b(lb, k, n, b.data_ptr(), ldb, out.data_ptr(), _policy(policy), _stream_ptr())
    _check(st, "tcec_pack_b")
    return out


def sgemm_packed(a_packed: torch.Tensor, b_packed: torch.Tensor, m: int, n: int, k: int,
                 c: Optional[torch.Tensor] = None, *, alpha: float = 1.0, beta: float = 0.0,
                 policy="fp16_ec") -> torch.Tensor:
    """C = alpha * A @ B + beta * C on operands packed by pack_a / pack_b."""
    if c is None:
        c = torch.empty((m, n), dtype=torch.float32, device=a_packed.device)
    _require_cuda_f32(c)
    lc, ldc = _layout_ld(c)
    with torch.cuda.device(c.device):
        st = load().tcec_sgemm_packed(lc, m, n, k, alpha, a_packed.data_ptr(), b_packed.data_ptr(), beta,
                                      c.data_ptr(), ldc, _policy(policy), _stream_ptr())
    _check(st, "tcec_sgemm_packed")
    return c


def _require_host_f32(*ts: torch.Tensor) -> None:
    for t in ts:
        if t.is_cuda or t.dtype != torch.float32:
            raise ValueError("host operands must be float32 CPU tensors")


def sgemm_host(a_host: torch.Tensor, b_host: torch.Tensor, c_host: torch.Tensor, *, alpha: float = 1.0,
               beta: float = 0.0, policy="fp16_ec", panel_rows: int = 0,
               device: Optional[torch.device] = None) -> torch.Tensor:
    """C = alpha * A @ B + beta * C for operands in (pinned) HOST memory, through ``tcec_sgemm_host``.

    B is copied and split once; A travels in row panels, so that the copy-in of panel p+1, the
    GEMM on panel p and the copy-out of panel p-1 overlap on three streams.  The call returns
    when everything is queued: ``c_host`` is complete once the current CUDA stream has reached
    the end of the call's work (synchronise it before reading).
    """
    _require_host_f32(a_host, b_host, c_host)
    m, k = a_host.shape
    k2, n = b_host.shape
    if k != k2 or tuple(c_host.shape) != (m, n):
        raise ValueError("shape mismatch")
    la, lda = _layout_ld(a_host)
    lb, ldb = _layout_ld(b_host)
    lc, ldc = _layout_ld(c_host)
    dev = device or torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        st = load().tcec_sgemm_host(la, lb, lc, m, n, k, alpha, a_host.data_ptr(), lda, b_host.data_ptr(), ldb, beta,
                                    c_host.data_ptr(), ldc, _policy(policy), int(panel_rows), _stream_ptr())
    _check(st, "tcec_sgemm_host")
    return c_host


# ---------------------------------------------------------------- several GPUs
def comm_unique_id() -> bytes:
    """Rank 0's communicator id (``tcec_comm_unique_id``), to be handed to every rank."""
    buf = ctypes.create_string_buffer(COMM_ID_BYTES)
    _check(load().tcec_comm_unique_id(buf), "tcec_comm_unique_id")
    return buf.raw


def comm_init_rank(nranks: int, rank: int, uid: bytes) -> None:
    """Creates this process's communicator on the current device (``tcec_comm_init_rank``)."""
    if len(uid) != COMM_ID_BYTES:
        raise ValueError("communicator id has the wrong size")
    buf = ctypes.create_string_buffer(uid, COMM_ID_BYTES)
    _check(load().tcec_comm_init_rank(int(nranks), int(rank), buf), "tcec_comm_init_rank")


def comm_destroy() -> None:
    _check(load().tcec_comm_destroy(), "tcec_comm_destroy")


def _opt_mat(t: Optional[torch.Tensor]):
    if t is None:
        return ROW_MAJOR, 0, None
    la, lda = _layout_ld(t)
    return la, lda, t.data_ptr()


def sgemm_column_shard(a: Optional[torch.Tensor], b_local: torch.Tensor, c_local: torch.Tensor, m: int, k: int, *,
                       root: int = 0, alpha: float = 1.0, beta: float = 0.0, policy="fp16_ec") -> torch.Tensor:
    """This rank's part of the column-sharded GEMM (``tcec_sgemm_column_shard``): ``a`` (m x k) is
    needed on ``root`` only; ``b_local`` is k x n_local, ``c_local`` m x n_local, on the current device."""
    _require_cuda_f32(b_local, c_local)
    la, lda, ap = _opt_mat(a)
    lb, ldb = _layout_ld(b_local)
    lc, ldc = _layout_ld(c_local)
    with torch.cuda.device(c_local.device):
        st = load().tcec_sgemm_column_shard(root, la, lb, lc, m, b_local.shape[1], k, alpha, ap, lda, b_local.data_ptr(),
                                            ldb, beta, c_local.data_ptr(), ldc, _policy(policy), _stream_ptr())
    _check(st, "tcec_sgemm_column_shard")
    return c_local


def sgemm_column_shard_host(a_host: Optional[torch.Tensor], b_host: torch.Tensor, c_host: torch.Tensor, m: int, k: int,
                            *, root: int = 0, alpha: float = 1.0, beta: float = 0.0, policy="fp16_ec",
                            panel_rows: int = 2048) -> torch.Tensor:
    """The same with host operands (``tcec_sgemm_column_shard_host``): copy-in, broadcast, GEMM and
    copy-out pipelined in row panels; complete when the current stream has reached the end of it."""
    _require_host_f32(b_host, c_host)
    la, lda, ap = _opt_mat(a_host)
    lb, ldb = _layout_ld(b_host)
    lc, ldc = _layout_ld(c_host)
    st = load().tcec_sgemm_column_shard_host(root, la, lb, lc, m, b_host.shape[1], k, alpha, ap, lda, b_host.data_ptr(),
                                             ldb, beta, c_host.data_ptr(), ldc, _policy(policy), int(panel_rows),
                                             _stream_ptr())
    _check(st, "tcec_sgemm_column_shard_host")
    return c_host


def _parr(ctype, values):
    return (ctype * len(values))(*values)


def sgemm_multi(a: torch.Tensor, b_blocks: Sequence[torch.Tensor], c_blocks: Sequence[torch.Tensor], *,
                alpha: float = 1.0, beta: float = 0.0, policy="fp16_ec") -> Sequence[torch.Tensor]:
    """One process driving several GPUs (``tcec_sgemm_multi``): block i of B and C lives on its own
    device, A on the device of block 0.  Returns when everything is queued on every device's current stream."""
    devices = [t.device.index for t in c_blocks]
    m, k = a.shape
    la, lda = _layout_ld(a)
    lays = [(_layout_ld(bb), _layout_ld(cc)) for bb, cc in zip(b_blocks, c_blocks)]
    if len({(x[0][0], x[1][0]) for x in lays}) != 1:
        raise ValueError("blocks must share their layouts")
    lb, lc = lays[0][0][0], lays[0][1][0]
    streams = [torch.cuda.current_stream(t.device).cuda_stream for t in c_blocks]
    st = load().tcec_sgemm_multi(
        len(devices), _parr(ctypes.c_int, devices), la, lb, lc, m, _parr(ctypes.c_int, [t.shape[1] for t in b_blocks]), k,
        alpha, a.data_ptr(), lda, _parr(ctypes.c_void_p, [t.data_ptr() for t in b_blocks]),
        _parr(ctypes.c_longlong, [x[0][1] for x in lays]), beta, _parr(ctypes.c_void_p, [t.data_ptr() for t in c_blocks]),
        _parr(ctypes.c_longlong, [x[1][1] for x in lays]), _policy(policy), _parr(ctypes.c_void_p, streams))
    _check(st, "tcec_sgemm_multi")
    return c_blocks


def sgemm_batched_multi(a_parts: Sequence[torch.Tensor], b_parts: Sequence[torch.Tensor],
                        c_parts: Sequence[torch.Tensor], *, alpha: float = 1.0, beta: float = 0.0,
                        policy="fp16_ec") -> Sequence[torch.Tensor]:
    """A batch divided among several GPUs driven by one process (``tcec_sgemm_batched_multi``):
    part i ([count_i, m, k] x [count_i, k, n]) lives on its own device; no collective."""
    devices = [t.device.index for t in c_parts]
    _, m, k = a_parts[0].shape
    n = b_parts[0].shape[2]
    la, lda = _layout_ld(a_parts[0])
    lb, ldb = _layout_ld(b_parts[0])
    lc, ldc = _layout_ld(c_parts[0])
    streams = [torch.cuda.current_stream(t.device).cuda_stream for t in c_parts]
    st = load().tcec_sgemm_batched_multi(
        len(devices), _parr(ctypes.c_int, devices), la, lb, lc, m, n, k, alpha,
        _parr(ctypes.c_void_p, [t.data_ptr() for t in a_parts]), lda, a_parts[0].stride(0),
        _parr(ctypes.c_void_p, [t.data_ptr() for t in b_parts]), ldb, b_parts[0].stride(0), beta,
        _parr(ctypes.c_void_p, [t.data_ptr() for t in c_parts]), ldc, c_parts[0].stride(0),
        _parr(ctypes.c_int, [t.shape[0] for t in a_parts]), _policy(policy), _parr(ctypes.c_void_p, streams))
    _check(st, "tcec_sgemm_batched_multi")
    return c_parts


def split(x: torch.Tensor, policy="fp16_ec"):
    """Element-wise hi / scaled-lo split, widened to float32 (for bit-exact checks)."""
    _require_cuda_f32(x)
    x = x.contiguous()
    hi = torch.empty_like(x)
    lo = torch.empty_like(x)
    with torch.cuda.device(x.device):
        st = load().tcec_split(x.data_ptr(), hi.data_ptr(), lo.data_ptr(), x.numel(), _policy(policy), _stream_ptr())
    _check(st, "tcec_split")
    return hi, lo


def workspace_bytes(m: int, n: int, k: int, batch: int = 1, policy="fp16_ec") -> int:
    return int(load().tcec_workspace_bytes(m, n, k, batch, _policy(policy)))


def destroy() -> None:
    _check(load().tcec_destroy(), "tcec_destroy")
