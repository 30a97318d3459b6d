"""The bounded waits of the kernels, made to run out on purpose - by a stall made on the host side
of the launch, never by a fault: a build of the library with a short wait limit is told (through a
development switch that only that build has) to leave one ring stage unfilled, so the MMA thread's
wait gives up, every role of every CTA returns, and the host reads TCEC_ERR_TIMEOUT.  The context
stays usable: the next call gives correct results."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import cpu

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TEST_LIB = os.path.join(ROOT, "tests", "_build", "libtcec_b200_shortwait.so")
ERR_TIMEOUT = 4


def test_a_wait_that_runs_out_is_reported_and_leaves_the_context_usable():
    if not os.path.exists(TEST_LIB):
        pytest.skip("the short-wait test build of the library is missing (run build())")
    lib = ctypes.CDLL(TEST_LIB)
    i, ll, f, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
    lib.tcec_sgemm.argtypes = [i, i, i, i, i, i, f, p, ll, p, ll, f, p, ll, i, p]
    lib.tcec_device_status.argtypes = [ctypes.POINTER(i)]
    lib.tcec_set_option.argtypes = [ctypes.c_char_p, i]
    rng = np.random.default_rng(3)
    m, n, k = 128, 256, 512  # one tile, 16 K blocks: more than the ring holds
    a = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float32)).cuda()
    b = torch.from_numpy(rng.uniform(-1, 1, (k, n)).astype(np.float32)).cuda()
    c = torch.zeros((m, n), device="cuda")

    def run():
        return lib.tcec_sgemm(0, 0, 0, m, n, k, 1.0, a.data_ptr(), k, b.data_ptr(), n, 0.0, c.data_ptr(), n, 0, None)

    detail = i(0)
    assert lib.tcec_set_option(b"path", 1) == 0
    assert run() == 0 and lib.tcec_device_status(ctypes.byref(detail)) == 0  # the build works
    assert lib.tcec_set_option(b"debug_flags", 32) == 0  # one stage is never filled
    try:
        assert run() == 0  # the launch itself succeeds
        st = lib.tcec_device_status(ctypes.byref(detail))
    finally:
        lib.tcec_set_option(b"debug_flags", 0)
    assert st == ERR_TIMEOUT, st
    assert detail.value in (1, 2, 3)  # which role gave up first (producer, MMA thread or epilogue)
    assert lib.tcec_device_status(ctypes.byref(detail)) == 0  # reading the status clears it
    # the context is intact: a normal call gives the right answer
    c.fill_(float("nan"))
    assert run() == 0 and lib.tcec_device_status(ctypes.byref(detail)) == 0
    exact = cpu.gemm_f64(a.cpu().numpy(), b.cpu().numpy())
    assert cpu.errors(c.cpu().numpy(), exact)["max_rel"] < 1e-6
    lib.tcec_destroy()
