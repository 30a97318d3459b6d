"""The warp-level mtk::wmma::tcec header surface of this repository, run as one-warp kernels
(tests/header_api_harness.cu) and checked against the reference's own results: golden
fixtures, the live reference build when present, and the CPU restatement."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest
import torch

from oracle import cpu, ref

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "tests", "_build", "libtcec_header_test.so")
DEV = "cuda:0"


@pytest.fixture(scope="module")
def hdr():
    if not os.path.exists(LIB):
        pytest.fail(f"{LIB} missing: run __graft_entry__.build()")
    lib = ctypes.CDLL(LIB)
    p, i = ctypes.c_void_p, ctypes.c_int
    lib.hdr_warp_mma.argtypes = [i, i, i, p, p, p, p, i]
    lib.hdr_warp_mma.restype = i
    lib.hdr_matvec.argtypes = [i, i, i, p, p, p]
    lib.hdr_matvec.restype = i
    lib.hdr_dump.argtypes = [i, p, p, p]
    lib.hdr_dump.restype = i
    lib.hdr_dump_tf32.argtypes = [i, p, p, p]
    lib.hdr_dump_tf32.restype = i
    lib.hdr_wmma_map_mismatches.argtypes = [p]
    lib.hdr_wmma_map_mismatches.restype = i
    return lib


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(DEV)


def run_mma(lib, a, b, c, tf32, op_wmma, ec, mode=0):
    """a (32x32), b (32x32, k x n), c or None as logical matrices; mode picks memory orders."""
    a_mem = a.T if mode & 1 else a            # column-major A = transposed buffer
    b_mem = b if mode & 2 else b.T            # default: column-major B
    c_mem = None if c is None else (c.T if mode & 4 else c)
    d = torch.empty(32, 32, device=DEV)
    at, bt = _t(a_mem), _t(b_mem)  # keep the buffers alive across the launch
    ct = None if c_mem is None else _t(c_mem)
    rc = lib.hdr_warp_mma(int(tf32), int(op_wmma), int(ec), d.data_ptr(), at.data_ptr(), bt.data_ptr(),
                          None if ct is None else ct.data_ptr(), mode)
    torch.cuda.synchronize()
    assert rc == 0
    out = d.cpu().numpy()
    return out.T if mode & 4 else out


@pytest.fixture(scope="module")
def fixture(golden_dir):
    return np.load(os.path.join(golden_dir, "ref_warp_mma.npz"))


@pytest.mark.parametrize("tf32", [False, True])
@pytest.mark.parametrize("op_wmma", [False, True])
@pytest.mark.parametrize("ec", [False, True])
@pytest.mark.parametrize("with_c", [False, True])
@pytest.mark.parametrize("rz", [False, True])
def test_matches_reference_fixtures(hdr, fixture, tf32, op_wmma, ec, with_c, rz):
    a, b, c = fixture["a"], fixture["b"], fixture["c"]
    key = f"d_{'tf32' if tf32 else 'fp16'}_{'wmma' if op_wmma else 'mma'}_{'ec' if ec else 'noec'}" \
          f"_{'abcd' if with_c else 'abd'}_{'rz' if rz else 'default'}"
    got = run_mma(hdr, a, b, c if with_c else None, tf32, op_wmma, ec, mode=16 if rz else 0)
    want = fixture[key]
    exact = a.astype(np.float64) @ b.astype(np.float64) + (c if with_c else 0)
    # the reference's own thresholds (test/tcec/mma.cu:5-19)
    assert np.max(np.abs(got - exact)) < (1e-5 if ec else 1e-2)
    # same split, same products, same order: only tensor-core accumulation order inside one
    # instruction may differ between the 16-wide wmma tile and two n8 mma tiles
    assert np.max(np.abs(got - want)) < 3e-6, key
    if not op_wmma:
        # identical instruction sequence as the reference's op_mma path
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), key


@pytest.mark.parametrize("mode", [1, 2, 3, 4, 7, 8, 8 | 4 | 1, 32])
@pytest.mark.parametrize("tf32", [False, True])
def test_memory_layouts_with_mul_and_rn(hdr, fixture, mode, tf32):
    a, b, c = fixture["a"], fixture["b"], fixture["c"]
    base = run_mma(hdr, a, b, c, tf32, False, True, mode=0)
    got = run_mma(hdr, a, b, c, tf32, False, True, mode=mode)
    if mode & 8:
        # A scaled by 2 before the split and D by 0.5 at the store: D = 0.5 * (2A B + C)
        want = (2 * a.astype(np.float64)) @ b.astype(np.float64) + c
        assert np.max(np.abs(got - 0.5 * want)) < 1e-5
    else:
        # memory order is independent of the fragment's register order: same bits
        assert np.array_equal(got.view(np.uint32), base.view(np.uint32))


def test_against_cpu_restatement_random(hdr):
    rng = np.random.default_rng(77)
    for trial in range(4):
        a = rng.uniform(-1, 1, (32, 32)).astype(np.float32)
        b = rng.uniform(-1, 1, (32, 32)).astype(np.float32)
        for tf32 in (False, True):
            pol = "tf32_ec" if tf32 else "fp16_ec"
            got = run_mma(hdr, a, b, None, tf32, False, True)
            want = cpu.tcec_gemm(a, b, policy=pol, rn_block=1)
            assert np.max(np.abs(got - want)) < 3e-6
            assert cpu.errors(got, cpu.gemm_f64(a, b))["max_abs"] < 1e-5


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref was not built")
def test_bitwise_equal_to_live_reference_op_mma(hdr):
    rng = np.random.default_rng(78)
    a = rng.standard_normal((32, 32)).astype(np.float32)
    b = rng.standard_normal((32, 32)).astype(np.float32)
    c = rng.standard_normal((32, 32)).astype(np.float32)
    for tf32 in (False, True):
        for ec in (False, True):
            for with_c in (False, True):
                want = ref.warp_mma(_t(a), _t(b), _t(c) if with_c else None, tf32, False, ec).cpu().numpy()
                got = run_mma(hdr, a, b, c if with_c else None, tf32, False, ec)
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (tf32, ec, with_c)


def test_matvec_through_vectors(hdr):
    rng = np.random.default_rng(79)
    a = rng.uniform(-1, 1, (32, 32)).astype(np.float32)
    x = rng.uniform(-1, 1, 32).astype(np.float32)
    exact = a.astype(np.float64) @ x.astype(np.float64)
    for tf32 in (False, True):
        for op_wmma in (False, True):
            for ec in (False, True):
                y = torch.empty(32, device=DEV)
                at, xt = _t(a.T), _t(x)
                rc = hdr.hdr_matvec(int(tf32), int(op_wmma), int(ec), y.data_ptr(), at.data_ptr(), xt.data_ptr())
                torch.cuda.synchronize()
                assert rc == 0
                # thresholds of the reference's matvec test (test/tcec/matvec.cu:5-19)
                assert np.max(np.abs(y.cpu().numpy() - exact)) < (1e-5 if ec else 1e-2)


def test_element_map_of_op_mma_half_fragments(hdr):
    """x(i) of the op_mma half fragments follows the PTX m16n8k16 register order
    (reference include/wmma_extension/detail/m16n8k16.hpp:100-176)."""
    src = (np.arange(32 * 32, dtype=np.float32)).reshape(32, 32) / 8.0  # exactly representable in fp16
    for use, shape in ((0, (16, 16)), (1, (16, 8)), (2, (16, 8))):
        rows, cols = shape
        ne = rows * cols // 32
        blocks_m, blocks_n = 32 // rows, 32 // cols
        hi = torch.zeros(32, ne * blocks_m * blocks_n, device=DEV)
        lo = torch.zeros_like(hi)
        st = _t(src)
        assert hdr.hdr_dump(use, hi.data_ptr(), lo.data_ptr(), st.data_ptr()) == 0
        torch.cuda.synchronize()
        h = hi.cpu().numpy()
        for lane in range(32):
            g, t = lane // 4, lane % 4
            for f in range(blocks_m * blocks_n):
                bm, bn = f % blocks_m, f // blocks_m
                for r in range(ne):
                    if use == 0:
                        c_, rr, e = r // 4, (r // 2) % 2, r % 2
                        i, j = g + 8 * rr, 8 * c_ + 2 * t + e
                    elif use == 1:
                        kh, e = (r // 2) % 2, r % 2
                        i, j = 2 * t + 8 * kh + e, g
                    else:
                        rr, e = (r // 2) % 2, r % 2
                        i, j = g + 8 * rr, 2 * t + e
                    assert h[lane, f * ne + r] == src[i + bm * rows, j + bn * cols], (use, lane, f, r)


def test_op_wmma_sub_fragments_are_nvcuda_fragments_with_nvcuda_element_order(hdr):
    """With the op_wmma policy the sub-fragments are nvcuda::wmma::fragment objects (reference
    include/wmma_extension/tcec/detail/policy.hpp:107-112) and x(i) follows nvcuda's (undocumented)
    register order (detail/sm_80.hpp:95-173, detail/sm_80_tf32.hpp:102-184): on the GPU the test runs
    on, every register equals what nvcuda::wmma::load_matrix_sync puts there, for half and tf32,
    A and B in both layouts, and the accumulator."""
    bad = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert hdr.hdr_wmma_map_mismatches(bad.data_ptr()) == 0
    torch.cuda.synchronize()
    assert int(bad.item()) == 0


def test_element_map_of_op_mma_tf32_fragments(hdr):
    """x(i) of the op_mma tf32 fragments follows the PTX m16n8k8 register order (reference
    include/wmma_extension/detail/m16n8k8_tf32.hpp:68-112; accumulator as m16n8k8 float,
    detail/m16n8k8.hpp:136-165): A x0..x3 = (r, c), (r+8, c), (r, c+4), (r+8, c+4) with r = lane/4,
    c = lane%4; B x0, x1 = (k = lane%4, n = lane/4), (k+4, n); C x0..x3 = (r, 2c), (r, 2c+1), (r+8, 2c), (r+8, 2c+1)."""
    src = (np.arange(32 * 32, dtype=np.float32)).reshape(32, 32) / 8.0  # exactly representable in tf32
    for use, shape in ((0, (16, 8)), (1, (8, 8)), (2, (16, 8))):
        rows, cols = shape
        ne = rows * cols // 32
        blocks_m, blocks_n = 32 // rows, 32 // cols
        hi = torch.zeros(32, ne * blocks_m * blocks_n, device=DEV)
        lo = torch.zeros_like(hi)
        st = _t(src)
        assert hdr.hdr_dump_tf32(use, hi.data_ptr(), lo.data_ptr(), st.data_ptr()) == 0
        torch.cuda.synchronize()
        h = hi.cpu().numpy()
        for lane in range(32):
            g, t = lane // 4, lane % 4
            for f in range(blocks_m * blocks_n):
                bm, bn = f % blocks_m, f // blocks_m
                for r in range(ne):
                    if use == 0:
                        i, j = g + 8 * (r % 2), t + 4 * (r // 2)
                    elif use == 1:
                        i, j = t + 4 * r, g
                    else:
                        i, j = g + 8 * (r // 2), 2 * t + (r % 2)
                    assert h[lane, f * ne + r] == src[i + bm * rows, j + bn * cols], (use, lane, f, r)
        assert not lo.any()  # exactly representable values leave no residual


def test_reference_vector_test_program_reports_no_error_on_these_headers():
    """test/tcec/vector.cu of the reference, compiled unchanged against these headers: load_vector must
    equal load_matrix_sync of the zero-padded matrix lane by lane (test/tcec/vector.cu:15-60) and
    store_vector must give back the vector (:62-75); the program prints the errors, all must be zero."""
    text = _run_reference_test_binary("reftest_vector.newhdr")
    lane_errors = [float(x) for x in re.findall(r"^\[\d+\]\s+(\S+)\s*$", text, flags=re.M)]
    store_errors = [float(x) for x in re.findall(r"^Error\s*:\s*(\S+)\s*$", text, flags=re.M)]
    assert len(lane_errors) >= 32 * 8 and len(store_errors) >= 4, (len(lane_errors), len(store_errors))
    assert max(lane_errors) == 0.0 and max(store_errors) == 0.0


def _run_reference_test_binary(name):
    path = os.path.join(ROOT, "oracle", "_ref", name)
    if not os.path.exists(path):
        pytest.skip(f"{name} was not built (needs the reference tree at build time)")
    out = subprocess.run([path], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    return out.stdout


def test_reference_mma_test_program_passes_on_these_headers():
    """The reference's own test/tcec/mma.cu, compiled unchanged against include/ of this
    repository: every enumerated case must report PASSED."""
    text = _run_reference_test_binary("reftest_mma.newhdr")
    m = re.search(r"passed\s*:\s*(\d+)\s*/\s*(\d+)", text)
    assert m, text[-500:]
    assert m.group(1) == m.group(2) and int(m.group(2)) >= 300, m.group(0)


def test_reference_complex_mma_test_program_passes_on_these_headers():
    """test/tcec/mma_complex.cu of the reference (fragment_complex, four real products per
    complex product), compiled unchanged against this repository's complex.hpp."""
    text = _run_reference_test_binary("reftest_mma_complex.newhdr")
    m = re.search(r"passed\s*:\s*(\d+)\s*/\s*(\d+)", text)
    assert m, text[-500:]
    assert m.group(1) == m.group(2) and int(m.group(2)) >= 100, m.group(0)


def test_reference_matvec_test_program_passes_on_these_headers():
    text = _run_reference_test_binary("reftest_matvec.newhdr")
    assert "FAILED" not in text and text.count("PASSED") >= 4, text[-800:]
