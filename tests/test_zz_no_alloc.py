"""The entry point that allocates nothing, ``tcec_sgemm_static``.

Some users of this library cannot allocate device memory at the point where they need a GEMM
(their memory pool owns the whole GPU, or they run inside a loop or a host application that
forbids cudaMalloc after start-up).  ``tcec_sgemm_static`` keeps the split operands in a fixed
array inside the library instead of a cudaMalloc'ed workspace.  This file checks, through the
C ABI, that it gives what ``tcec_sgemm`` gives, on two calls in a row (the array is shared and
keeps the previous call's contents), and that it refuses problems larger than the array.
It is collected last so that a failure here cannot hide one elsewhere.
"""
import ctypes

import numpy as np
import pytest
import torch

from wmma_extension_b200 import tcec

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(fn_name, a, b, c, alpha, beta, policy):
    lib = tcec.load()
    m, k = a.shape
    n = b.shape[1]
    st = getattr(lib, fn_name)(tcec.ROW_MAJOR, tcec.ROW_MAJOR, tcec.ROW_MAJOR, m, n, k, alpha, a.data_ptr(), k,
                               b.data_ptr(), n, beta, c.data_ptr(), n, tcec.POLICIES[policy],
                               torch.cuda.current_stream().cuda_stream)
    assert st == tcec.OK, tcec.status_string(st)


def test_static_entry_matches_the_allocating_one_twice_in_a_row():
    gen = torch.Generator(device=DEV)
    gen.manual_seed(90)
    # two different shapes back to back: the second call finds the first call's panels in the array
    for (m, n, k, policy, alpha, beta) in [(384, 512, 1000, "fp16_ec", 1.0, 0.0), (200, 130, 70, "tf32_ec", 1.5, 0.5),
                                             (300, 400, 200, "fp16_no_ec", 1.0, 0.0)]:
        a = torch.rand((m, k), generator=gen, device=DEV) * 2 - 1
        b = torch.rand((k, n), generator=gen, device=DEV) * 2 - 1
        c0 = torch.rand((m, n), generator=gen, device=DEV)
        want, got = c0.clone(), c0.clone()
        _call("tcec_sgemm", a, b, want, alpha, beta, policy)
        _call("tcec_sgemm_static", a, b, got, alpha, beta, policy)
        tcec.device_status()
        tcec.static_status()
        exact = alpha * (a.double() @ b.double()) + beta * c0.double()
        # the tolerances of the GEMM parity tests (one product only without error correction)
        tol = (2e-3 if policy.endswith("no_ec") else 1e-6) * exact.abs().max().item()
        assert (got.double() - want.double()).abs().max().item() <= tol
        assert (got.double() - exact).abs().max().item() <= tol
        assert torch.equal(got, want)  # same kernels on the same panels: not a bit differs


def test_static_entry_allocates_nothing():
    """The property the entry point exists for: after its one-time set-up, a call leaves the
    device's free memory exactly as it found it - also for a shape that makes the allocating
    entry point take a new workspace from the device."""
    tcec.destroy()  # drop every cached workspace, so that tcec_sgemm has to allocate again below
    a1, b1, c1 = torch.rand((1024, 512), device=DEV), torch.rand((512, 768), device=DEV), torch.empty((1024, 768), device=DEV)
    a2, b2, c2 = torch.rand((2048, 256), device=DEV), torch.rand((256, 1536), device=DEV), torch.empty((2048, 1536), device=DEV)
    want = torch.empty((2048, 1536), device=DEV)
    tcec.sgemm_static(a1, b1, c1)  # first call on the device: looks up the array's address, sets kernel attributes
    tcec.static_status()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    tcec.sgemm_static(a2, b2, c2)  # a larger problem than any before it
    tcec.sgemm_static(a1, b1, c1)
    tcec.static_status()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "tcec_sgemm_static changed the device's free memory"
    # the allocating entry point, by contrast, takes its workspace from the device here
    tcec.sgemm(a2, b2, want)
    torch.cuda.synchronize()
    free_alloc, _ = torch.cuda.mem_get_info()
    assert free_alloc <= free_after - tcec.workspace_bytes(2048, 1536, 256) // 2
    assert torch.equal(c2, want)


def test_static_entry_rejects_what_does_not_fit_and_bad_arguments():
    lib = tcec.load()
    limit = lib.tcec_static_scratch_bytes()
    assert limit == 32 << 20
    big = 4096
    assert tcec.packed_bytes(big, big) * 2 > limit
    x = torch.zeros(1, device=DEV)  # never dereferenced: the size check comes first
    st = lib.tcec_sgemm_static(0, 0, 0, big, big, big, 1.0, x.data_ptr(), big, x.data_ptr(), big, 0.0, x.data_ptr(),
                               big, 0, None)
    assert st == tcec.ERR_TOO_LARGE
    assert "scratch" in tcec.status_string(st)
    assert lib.tcec_sgemm_static(0, 0, 0, 4, 4, 4, 1.0, None, 4, x.data_ptr(), 4, 0.0, x.data_ptr(), 4, 0,
                                 None) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_static(0, 0, 0, 0, 4, 4, 1.0, None, 4, None, 4, 0.0, None, 4, 0, None) == tcec.OK
    # the largest cube that fits
    n = 2048
    assert tcec.packed_bytes(n, n) * 2 <= limit
    a = torch.rand(n, n, device=DEV) - 0.5
    b = torch.rand(n, n, device=DEV) - 0.5
    got, want = torch.empty(n, n, device=DEV), torch.empty(n, n, device=DEV)
    tcec.sgemm_static(a, b, got)
    tcec.sgemm(a, b, want)
    tcec.static_status()
    assert torch.equal(got, want)
