"""Parity of the CUDA path, called through the C ABI, against the CPU restatement,
the FP64 ground truth, the reference's golden fixtures and (when oracle/_ref was
built) the reference's own kernels run live on the same inputs."""
import os

import numpy as np
import pytest
import torch

from oracle import cpu, ref
from wmma_extension_b200 import tcec

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def _t(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def _gemm(a, b, **kw):
    c = tcec.sgemm(_t(a), _t(b), **kw)
    tcec.device_status()
    return c.cpu().numpy()


@pytest.fixture(autouse=True)
def _defaults():
    tcec.set_option("promote_k", -1)
    tcec.set_option("tile_n", 0)
    tcec.set_option("path", 0)
    tcec.set_option("cta_pair", -1)
    tcec.set_option("half_tiles", 1)
    yield
    tcec.set_option("promote_k", -1)
    tcec.set_option("tile_n", 0)
    tcec.set_option("path", 0)
    tcec.set_option("cta_pair", -1)
    tcec.set_option("half_tiles", 1)


# ---------------------------------------------------------------- split (bit-exact)
def test_split_bit_exact_vs_golden_and_oracle(golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_split.npz"))
    rng = np.random.default_rng(12)
    extra = (rng.uniform(-1, 1, 1 << 20) * np.exp2(rng.integers(-40, 20, 1 << 20))).astype(np.float32)
    for name in ("fp16", "tf32"):
        hi, lo = tcec.split(_t(g["x"]), name + "_ec")
        assert np.array_equal(_bits(hi.cpu().numpy()), _bits(g["hi_" + name]))
        assert np.array_equal(_bits(lo.cpu().numpy()), _bits(g["lo_" + name]))
        hi, lo = tcec.split(_t(extra), name + "_ec")
        ohi, olo = cpu.split(extra, name + "_ec")
        assert np.array_equal(_bits(hi.cpu().numpy()), _bits(ohi))
        assert np.array_equal(_bits(lo.cpu().numpy()), _bits(olo))


def test_packed_panels_hold_the_oracle_split():
    """The operand panels the GEMM kernel streams contain exactly the oracle's hi / lo bits."""
    rng = np.random.default_rng(13)
    m, k = 200, 70
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    for layout in ("row", "col"):
        at = _t(a) if layout == "row" else _t(a.T).t()
        packed = tcec.pack_a(at, "fp16_ec").cpu().numpy()
        ohi, olo = cpu.split(a, "fp16_ec")
        nkb = (k + 31) // 32
        blocks = packed.reshape(-1, nkb, 2, 16, 4, 8, 16).view(np.float16)  # [rb][kb][hi/lo][r8][c][r%8][8 halves]
        # element (r, kk): rb=r//128, r8=(r%128)//8, rr=r%8, kb=kk//32, c=(kk%32)//8, e=kk%8
        r, kk = np.meshgrid(np.arange(m), np.arange(k), indexing="ij")
        got_hi = blocks[r // 128, kk // 32, 0, (r % 128) // 8, (kk % 32) // 8, r % 8, kk % 8].astype(np.float32)
        got_lo = blocks[r // 128, kk // 32, 1, (r % 128) // 8, (kk % 32) // 8, r % 8, kk % 8].astype(np.float32)
        assert np.array_equal(_bits(got_hi), _bits(ohi)), layout
        assert np.array_equal(_bits(got_lo), _bits(olo)), layout


# ---------------------------------------------------------------- GEMM vs oracle / FP64
POLICY_BOUND = {"fp16_ec": 1e-6, "tf32_ec": 1e-6, "fp16_no_ec": 2e-3, "tf32_no_ec": 2e-3}


@pytest.mark.parametrize("policy", list(POLICY_BOUND))
@pytest.mark.parametrize("shape", [(16, 16, 16), (32, 32, 32), (128, 256, 64), (256, 512, 256), (37, 41, 19),
                                   (1, 1, 1), (130, 257, 33), (129, 127, 515), (512, 384, 1000)])
def test_gemm_matches_oracle(policy, shape):
    m, n, k = shape
    rng = np.random.default_rng(100 + m + n + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    exact = cpu.gemm_f64(a, b)
    got = _gemm(a, b, policy=policy)
    pk = 64  # the library's automatic promotion interval for these K
    want = cpu.tcec_gemm(a, b, policy=policy, rn_block=pk // (16 if policy.startswith("fp16") else 8))
    e_got, e_orc = cpu.errors(got, exact), cpu.errors(want, exact)
    assert e_got["max_rel"] < POLICY_BOUND[policy]
    if policy.endswith("no_ec"):
        assert e_got["max_rel"] < 2 * e_orc["max_rel"] + 1e-6
    else:
        # same split bits, same products; only the accumulator roundings may differ
        assert np.max(np.abs(got - want)) <= 1e-6 * max(1.0, np.max(np.abs(exact)))
        e_f32 = cpu.errors(cpu.gemm_f32(a, b), exact)
        assert e_got["max_rel"] <= 2 * max(e_orc["max_rel"], e_f32["max_rel"])
        if m == n == k == 32:
            assert e_got["max_abs"] < 1e-5  # the reference's unit-test threshold (test/tcec/mma.cu:8)


@pytest.mark.parametrize("policy", ["fp16_ec", "tf32_ec", "fp16_no_ec"])
def test_non_finite_and_out_of_range_values_follow_the_reference_semantics(policy):
    """Values beyond the fp16 range (heads become inf), inf, NaN and subnormals in the operands: every
    element of C is NaN, +inf, -inf or finite exactly where the CPU restatement says, and the finite
    ones agree with it (tcec.hpp:219-223: the split itself produces the inf / NaN parts)."""
    rng = np.random.default_rng(77)
    m, n, k = 96, 160, 64
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    a[3, 5], a[10, 7], b[9, 2] = 1e5, -7e4, 6.6e4           # beyond fp16: the heads overflow
    a[20, 1], b[30, 40] = np.inf, np.nan
    a[40, 3], b[3, 50], a[50, 60] = 1e-30, 3e-41, -2e-39    # tiny and subnormal FP32 values
    got = _gemm(a, b, policy=policy)
    want = cpu.tcec_gemm(a, b, policy=policy, rn_block=64 // (16 if policy.startswith("fp16") else 8))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(np.isposinf(got), np.isposinf(want))
    assert np.array_equal(np.isneginf(got), np.isneginf(want))
    fin = np.isfinite(want)
    assert fin.sum() > 0.9 * fin.size and (~fin).sum() > 100
    tol = 2e-3 if "no_ec" in policy else 1e-6
    assert np.max(np.abs(got[fin] - want[fin])) <= tol * max(1.0, np.max(np.abs(want[fin])))
    if policy.startswith("fp16"):
        # the FP32-tile kernel splits in registers: the same classes, and the same bits where finite
        tcec.set_option("path", 2)
        fused = _gemm(a, b, policy=policy)
        assert np.array_equal(np.isnan(fused), np.isnan(got))
        assert np.array_equal(np.isposinf(fused), np.isposinf(got)) and np.array_equal(np.isneginf(fused), np.isneginf(got))
        assert np.array_equal(_bits(fused[fin]), _bits(got[fin]))


@pytest.mark.parametrize("la", ["row", "col"])
@pytest.mark.parametrize("lb", ["row", "col"])
@pytest.mark.parametrize("lc", ["row", "col"])
def test_layouts_alpha_beta_and_padded_leading_dimensions(la, lb, lc):
    rng = np.random.default_rng(31)
    m, n, k = 200, 300, 100
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)

    def view(x, layout, pad):
        r, c = x.shape
        if layout == "row":
            buf = torch.full((r, c + pad), float("nan"), device=DEV)
            buf[:, :c] = _t(x)
            return buf[:, :c]
        buf = torch.full((c, r + pad), float("nan"), device=DEV)
        buf[:, :r] = _t(x.T)
        return buf[:, :r].t()

    for pad in (0, 4, 3):  # 3: leading dimension not a multiple of 4 -> scalar paths
        A, B, C = view(a, la, pad), view(b, lb, pad), view(c0, lc, pad)
        tcec.sgemm(A, B, C, alpha=1.5, beta=0.5)
        tcec.device_status()
        want = 1.5 * cpu.gemm_f64(a, b) + 0.5 * c0
        assert cpu.errors(C.cpu().numpy(), want)["max_rel"] < 1e-6, (la, lb, lc, pad)
        assert torch.isnan(C.as_strided((C._base.shape), C._base.stride())).sum() == (
            C._base.numel() - m * n), "wrote outside the matrix"


def test_beta_zero_never_reads_c_and_alpha_zero_scales():
    rng = np.random.default_rng(32)
    a = rng.uniform(-1, 1, (64, 64)).astype(np.float32)
    b = rng.uniform(-1, 1, (64, 64)).astype(np.float32)
    c = torch.full((64, 64), float("nan"), device=DEV)
    tcec.sgemm(_t(a), _t(b), c, beta=0.0)
    assert torch.isfinite(c).all()
    c2 = torch.ones(64, 64, device=DEV)
    tcec.sgemm(_t(a), _t(b), c2, alpha=0.0, beta=3.0)
    assert torch.equal(c2, torch.full_like(c2, 3.0))
    c3 = torch.full((64, 64), float("nan"), device=DEV)
    tcec.sgemm(_t(a[:, :0]), _t(b[:0, :]), c3, beta=0.0)  # k == 0
    assert torch.equal(c3, torch.zeros_like(c3))
    tcec.device_status()


def test_promotion_interval_option():
    """promote_k = 0 reproduces the in-accumulator (round-toward-zero) variant; the default beats it."""
    rng = np.random.default_rng(33)
    a = rng.uniform(0, 1, (256, 4096)).astype(np.float32)
    b = rng.uniform(0, 1, (4096, 256)).astype(np.float32)
    exact = cpu.gemm_f64(a, b)
    errs = {}
    for pk in (0, 32, 128, 512):
        tcec.set_option("promote_k", pk)
        errs[pk] = cpu.errors(_gemm(a, b), exact)["max_rel"]
    e_f32 = cpu.errors(cpu.gemm_f32(a, b), exact)["max_rel"]
    assert errs[128] < e_f32 and errs[32] < e_f32
    assert errs[0] > 4 * errs[128]


def test_direct_store_option_is_bit_identical():
    """store_turn = 0 (direct stores, smaller shared-memory footprint) changes no result."""
    rng = np.random.default_rng(5)
    a = _t(rng.uniform(-1, 1, (300, 200)).astype(np.float32))
    b = _t(rng.uniform(-1, 1, (200, 700)).astype(np.float32))
    c0 = _t(rng.uniform(-1, 1, (300, 700)).astype(np.float32))
    tcec.set_option("path", 1)
    out = {}
    try:
        for turn in (1, 0):
            tcec.set_option("store_turn", turn)
            out[turn] = tcec.sgemm(a, b, c0.clone(), alpha=1.5, beta=-0.5)
            tcec.device_status()
    finally:
        tcec.set_option("store_turn", 1)
    assert torch.equal(out[0], out[1])


def test_tile_order_options_are_bit_identical():
    """Tiles drawn from the device-wide counter, by static striding, and with SMs held back all
    give the same bits; the counters are left at zero, so calls can follow one another."""
    rng = np.random.default_rng(6)
    a = _t(rng.uniform(-1, 1, (2000, 300)).astype(np.float32))
    b = _t(rng.uniform(-1, 1, (300, 5000)).astype(np.float32))  # 16 x 20 = 320 tiles: more than two per SM
    tcec.set_option("path", 1)
    try:
        tcec.set_option("static_tiles", 1)
        ref = tcec.sgemm(a, b)
        tcec.set_option("static_tiles", 0)
        for _ in range(3):
            assert torch.equal(tcec.sgemm(a, b), ref)
        tcec.set_option("reserve_sms", 20)
        assert torch.equal(tcec.sgemm(a, b), ref)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):  # a second stream has counters of its own
            c2 = tcec.sgemm(a, b)
        side.synchronize()
        assert torch.equal(c2, ref)
        tcec.device_status()
    finally:
        tcec.set_option("static_tiles", 0)
        tcec.set_option("reserve_sms", 0)
    exact = cpu.gemm_f64(a.cpu().numpy()[:64], b.cpu().numpy())
    assert cpu.errors(ref[:64].cpu().numpy(), exact)["max_rel"] < 1e-6


def test_tile_width_option_gives_same_quality():
    rng = np.random.default_rng(34)
    a = rng.standard_normal((256, 512)).astype(np.float32)
    b = rng.standard_normal((512, 512)).astype(np.float32)
    exact = cpu.gemm_f64(a, b)
    for tn in (128, 256):
        tcec.set_option("tile_n", tn)
        assert cpu.errors(_gemm(a, b), exact)["max_rel"] < 1e-6


# ---------------------------------------------------------------- FP32-tile (in-kernel split) path
@pytest.mark.parametrize("la", ["row", "col"])
@pytest.mark.parametrize("lb", ["row", "col"])
@pytest.mark.parametrize("shape", [(128, 256, 32), (200, 300, 100), (37, 260, 19), (384, 512, 1000)])
def test_fp32_tile_kernel_matches_panel_kernel(la, lb, shape):
    """The kernel that TMA-loads FP32 tiles and splits them in registers computes the same
    products from the same split as the two-kernel path: equal up to the last alpha/beta FMA."""
    m, n, k = shape
    rng = np.random.default_rng(200 + m + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    A = _t(a) if la == "row" else _t(a.T).t()
    B = _t(b) if lb == "row" else _t(b.T).t()
    out = {}
    for path in (1, 2):
        tcec.set_option("path", path)
        out[path] = tcec.sgemm(A, B).cpu().numpy()
        tcec.device_status()
    exact = cpu.gemm_f64(a, b)
    assert np.array_equal(out[1].view(np.uint32), out[2].view(np.uint32))  # alpha = 1, beta = 0: same bits
    assert cpu.errors(out[2], exact)["max_rel"] < 1e-6
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    tcec.set_option("path", 2)
    got = tcec.sgemm(A, B, _t(c0).clone(), alpha=1.5, beta=-0.5, policy="fp16_no_ec").cpu().numpy()
    assert cpu.errors(got, 1.5 * exact - 0.5 * c0)["max_rel"] < 2e-3


def test_fp32_tile_kernel_batched_and_fallback():
    rng = np.random.default_rng(210)
    a = rng.standard_normal((6, 256, 256)).astype(np.float32)
    b = rng.standard_normal((6, 256, 256)).astype(np.float32)
    tcec.set_option("path", 1)
    want = tcec.sgemm_strided_batched(_t(a), _t(b))
    tcec.set_option("path", 0)  # automatic: short-K batches take the FP32-tile kernel
    got = tcec.sgemm_strided_batched(_t(a), _t(b))
    tcec.device_status()
    assert torch.equal(got, want)
    # operands the TMA cannot address (leading dimension not a multiple of 4) fall back to panels
    tcec.set_option("path", 2)
    buf = torch.zeros(256, 259, device=DEV)
    buf[:, :256] = _t(a[0])
    odd = tcec.sgemm(buf[:, :256], _t(b[0]))
    assert torch.equal(odd, want[0])
    # tf32 policies always use panels
    t32 = tcec.sgemm(_t(a[0]), _t(b[0]), policy="tf32_ec").cpu().numpy()
    assert cpu.errors(t32, cpu.gemm_f64(a[0], b[0]))["max_rel"] < 1e-6
    tcec.device_status()


# ---------------------------------------------------------------- CTA-pair kernel (cta_group::2)
@pytest.mark.parametrize("shape,policy", [((256, 256, 32), "fp16_ec"), ((300, 300, 100), "fp16_ec"),
                                          ((129, 257, 33), "tf32_ec"), ((1000, 700, 300), "fp16_no_ec"),
                                          ((1024, 1024, 2048), "fp16_ec")])
def test_cta_pair_kernel_is_bit_identical(shape, policy):
    """Two SMs sharing a 256 x 256 tile compute every output row exactly as one SM does."""
    m, n, k = shape
    rng = np.random.default_rng(300 + m + k)
    a = _t(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = _t(rng.uniform(-1, 1, (k, n)).astype(np.float32))
    tcec.set_option("path", 1)
    out = {}
    for pair in (0, 1):
        tcec.set_option("cta_pair", pair)
        out[pair] = tcec.sgemm(a, b, policy=policy)
        tcec.device_status()
    assert torch.equal(out[0], out[1])
    # batched, with a tile row that only the leader CTA has rows in (m = 150 < 256)
    ab = _t(rng.standard_normal((5, 150, 96)).astype(np.float32))
    bb = _t(rng.standard_normal((5, 96, 260)).astype(np.float32))
    tcec.set_option("cta_pair", 0)
    want = tcec.sgemm_strided_batched(ab, bb, policy=policy)
    tcec.set_option("cta_pair", 1)
    got = tcec.sgemm_strided_batched(ab, bb, policy=policy)
    tcec.device_status()
    assert torch.equal(got, want)


@pytest.mark.parametrize("shape,policy", [((1024, 1024, 512), "fp16_ec"), ((1500, 1400, 96), "tf32_ec"),
                                          ((1024, 1000, 160), "fp16_no_ec"), ((700, 2300, 64), "tf32_no_ec"),
                                          ((300, 130, 64), "fp16_ec")])
def test_half_width_tiles_are_bit_identical(shape, policy):
    """A call with at most 37 pair tiles (half of the 74 SM pairs) runs on 256 x 128 half tiles (N = 128
    MMAs, 64 columns per epilogue warp); every element of C is the same as with whole tiles, and
    as from the one-SM kernel."""
    m, n, k = shape
    rng = np.random.default_rng(900 + m + n + k)
    a = _t(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = _t(rng.uniform(-1, 1, (k, n)).astype(np.float32))
    tcec.set_option("path", 1)
    tcec.set_option("cta_pair", 1)
    out = {}
    for halves in (0, 1):
        tcec.set_option("half_tiles", halves)
        c = torch.full((m + 1, n + 3), float("nan"), dtype=torch.float32, device="cuda")
        tcec.sgemm(a, b, c[:m, :n], policy=policy)
        tcec.device_status()
        assert torch.isnan(c[m:, :]).all() and torch.isnan(c[:, n:]).all()
        out[halves] = c[:m, :n].clone()
    assert torch.equal(out[0], out[1])
    tcec.set_option("cta_pair", 0)
    assert torch.equal(tcec.sgemm(a, b, policy=policy), out[1])
    # a batch in half tiles: 30 matrices of one pair tile each
    ab = _t(rng.standard_normal((30, 256, 64)).astype(np.float32))
    bb = _t(rng.standard_normal((30, 64, 256)).astype(np.float32))
    want = tcec.sgemm_strided_batched(ab, bb, policy=policy)
    tcec.set_option("cta_pair", 1)
    got = tcec.sgemm_strided_batched(ab, bb, policy=policy)
    tcec.device_status()
    assert torch.equal(got, want)


# ---------------------------------------------------------------- complex GEMM
def _crand(rng, shape):
    return (rng.uniform(-1, 1, shape) + 1j * rng.uniform(-1, 1, shape)).astype(np.complex64)


@pytest.mark.parametrize("policy", ["fp16_ec", "tf32_ec", "fp16_no_ec"])
@pytest.mark.parametrize("shape", [(32, 32, 32), (130, 257, 33), (256, 512, 300), (1, 1, 1), (500, 300, 1000)])
def test_cgemm_matches_oracle_and_complex128(policy, shape):
    m, n, k = shape
    rng = np.random.default_rng(500 + m + n + k)
    a, b = _crand(rng, (m, k)), _crand(rng, (k, n))
    exact = a.astype(np.complex128) @ b.astype(np.complex128)
    got = tcec.cgemm(_t(a), _t(b), policy=policy)
    tcec.device_status()
    got = got.cpu().numpy()
    scale = np.max(np.abs(exact))
    e_got = np.max(np.abs(got - exact)) / scale
    want = cpu.tcec_cgemm(a, b, policy=policy)
    e_orc = np.max(np.abs(want - exact)) / scale
    if policy.endswith("no_ec"):
        assert e_got < 2e-3 and e_got < 2 * e_orc + 1e-6
    else:
        assert e_got < 1e-6
        assert np.max(np.abs(got - want)) <= 2e-6 * max(1.0, scale)
        # the FP32 class: torch's complex64 product of the same operands
        e_f32 = np.max(np.abs((_t(a) @ _t(b)).cpu().numpy() - exact)) / scale
        assert e_got <= 2 * max(e_orc, e_f32)
        if m == n == k == 32:
            assert np.max(np.abs(got - exact)) < 1e-5 * np.sqrt(2)  # threshold of test/tcec/mma_complex.cu per part


@pytest.mark.parametrize("la", ["row", "col"])
@pytest.mark.parametrize("lb", ["row", "col"])
@pytest.mark.parametrize("lc", ["row", "col"])
def test_cgemm_layouts_alpha_beta(la, lb, lc):
    m, n, k = 150, 200, 70
    rng = np.random.default_rng(77)
    a, b, c0 = _crand(rng, (m, k)), _crand(rng, (k, n)), _crand(rng, (m, n))
    alpha, beta = 0.5 - 1.25j, -0.75 + 2j

    def place(x, layout, pad):
        r, c = x.shape
        if layout == "row":
            buf = torch.full((r, c + pad), 7 + 7j, dtype=torch.complex64, device=DEV)
            view = buf[:, :c]
        else:
            buf = torch.full((c, r + pad), 7 + 7j, dtype=torch.complex64, device=DEV)
            view = buf.t()[:r, :]
        view.copy_(_t(x))
        return buf, view

    _, av = place(a, la, 3)
    _, bv = place(b, lb, 5)
    cbuf, cv = place(c0, lc, 2)
    tcec.cgemm(av, bv, cv, alpha=alpha, beta=beta)
    tcec.device_status()
    exact = alpha * (a.astype(np.complex128) @ b.astype(np.complex128)) + beta * c0.astype(np.complex128)
    got = cv.cpu().numpy()
    assert np.max(np.abs(got - exact)) / np.max(np.abs(exact)) < 1e-6
    # the padding of C is untouched
    pad = cbuf[:, -2:].cpu().numpy()
    assert np.all(pad == 7 + 7j)
    # alpha = 0 scales only; k = 0 likewise
    tcec.cgemm(av, bv, cv, alpha=0.0, beta=2.0)
    tcec.device_status()
    assert np.allclose(cv.cpu().numpy(), 2 * got, rtol=1e-6, atol=1e-6)


def test_cgemm_full_size_linearity():
    """4096^3 complex: sampled rows against complex128 and C(A, B1 + B2) = C(A, B1) + C(A, B2) to rounding."""
    n = 4096
    g = torch.Generator(device=DEV).manual_seed(11)
    def crand():
        return torch.complex(torch.rand(n, n, device=DEV, generator=g) * 2 - 1,
                             torch.rand(n, n, device=DEV, generator=g) * 2 - 1)
    a, b1, b2 = crand(), crand(), crand()
    c1, c2, c12 = tcec.cgemm(a, b1), tcec.cgemm(a, b2), tcec.cgemm(a, b1 + b2)
    tcec.device_status()
    rows = torch.tensor([0, 1, 127, 128, 2049, 4095], device=DEV)
    exact = a[rows].to(torch.complex128) @ b1.to(torch.complex128)
    err = ((c1[rows].to(torch.complex128) - exact).abs().max() / exact.abs().max()).item()
    assert err < 1e-6
    lin = ((c12 - (c1 + c2)).abs().max() / c12.abs().max()).item()
    assert lin < 2e-6


# ---------------------------------------------------------------- golden fixtures of the reference
def test_against_reference_warp_fixtures(golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_warp_mma.npz"))
    a, b, c = g["a"], g["b"], g["c"]
    for name in ("fp16", "tf32"):
        got = _gemm(a, b, policy=name + "_ec")
        assert np.max(np.abs(got - g[f"d_{name}_mma_ec_abd_default"])) < 4e-6
        got_c = tcec.sgemm(_t(a), _t(b), _t(c).clone(), beta=1.0, policy=name + "_ec").cpu().numpy()
        assert np.max(np.abs(got_c - g[f"d_{name}_mma_ec_abcd_default"])) < 4e-6
        got_n = _gemm(a, b, policy=name + "_no_ec")
        assert np.max(np.abs(got_n - g[f"d_{name}_mma_noec_abd_default"])) < 4e-6


def test_against_reference_bgemm_fixtures(golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_bgemm.npz"))
    a, b = g["a"], g["b"]
    for name in ("fp16", "tf32"):
        got = tcec.sgemm_strided_batched(_t(a), _t(b), policy=name + "_ec").cpu().numpy()
        for i in range(a.shape[0]):
            exact = cpu.gemm_f64(a[i], b[i])
            e_ref = cpu.errors(g["c_" + name][i], exact)["max_rel"]
            e_got = cpu.errors(got[i], exact)["max_rel"]
            assert e_got <= 2 * e_ref
    got = _gemm(g["a_iota"][0], g["b_iota"][0])
    exact = cpu.gemm_f64(g["a_iota"][0], g["b_iota"][0])
    assert cpu.errors(got, exact)["fro_rel"] <= 2 * cpu.errors(g["c_iota_fp16"][0], exact)["fro_rel"] + 1e-9
    tcec.device_status()


# ---------------------------------------------------------------- batched forms
def test_batched_forms_agree_and_match_fp64():
    rng = np.random.default_rng(4)
    batch, m, n, k = 12, 256, 256, 256
    a = rng.standard_normal((batch, m, k)).astype(np.float32)
    b = rng.standard_normal((batch, k, n)).astype(np.float32)
    at, bt = _t(a), _t(b)
    c_str = tcec.sgemm_strided_batched(at, bt)
    c_list = [torch.empty(m, n, device=DEV) for _ in range(batch)]
    tcec.sgemm_batched(list(at.unbind(0)), list(bt.unbind(0)), c_list)
    tcec.device_status()
    assert torch.equal(torch.stack(c_list), c_str)
    for i in (0, batch // 2, batch - 1):
        single = tcec.sgemm(at[i], bt[i])
        assert torch.equal(single, c_str[i])  # batching does not change a single bit
        assert cpu.errors(c_str[i].cpu().numpy(), cpu.gemm_f64(a[i], b[i]))["max_rel"] < 1e-6


def test_ragged_batch_shapes():
    rng = np.random.default_rng(41)
    for (batch, m, n, k) in [(3, 100, 60, 50), (1, 129, 257, 31), (5, 16, 16, 16)]:
        a = rng.standard_normal((batch, m, k)).astype(np.float32)
        b = rng.standard_normal((batch, k, n)).astype(np.float32)
        got = tcec.sgemm_strided_batched(_t(a), _t(b)).cpu().numpy()
        for i in range(batch):
            assert cpu.errors(got[i], cpu.gemm_f64(a[i], b[i]))["max_rel"] < 1e-6
    tcec.device_status()


def test_more_matrices_than_a_grid_dimension_holds():
    """70 000 tiny matrices: the batch index of the split kernel is a grid dimension (65 535 at
    most), so such a batch takes several launches; every matrix must still be right."""
    if _free_gib() < 12:
        pytest.skip("needs 12 GiB of free device memory")
    g = torch.Generator(device=DEV).manual_seed(44)
    nb = 70000
    a = torch.randn((nb, 16, 16), generator=g, device=DEV)
    b = torch.randn((nb, 16, 16), generator=g, device=DEV)
    c = tcec.sgemm_strided_batched(a, b)
    tcec.device_status()
    exact = torch.matmul(a.double(), b.double())
    err = ((c.double() - exact).abs().amax(dim=(1, 2)) / exact.abs().amax(dim=(1, 2))).max().item()
    assert err < 1e-6
    tcec.destroy()  # gives the 4.6 GB workspace back


def test_packed_entry_points_match_plain_call():
    rng = np.random.default_rng(42)
    m, n, k = 384, 300, 200
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    at, bt = _t(a), _t(b)
    want = tcec.sgemm(at, bt)
    ap, bp = tcec.pack_a(at), tcec.pack_b(bt)
    assert torch.equal(tcec.sgemm_packed(ap, bp, m, n, k), want)
    # a row sub-range of packed A that starts at a multiple of 256 rows is itself a packed A
    off = tcec.packed_row_offset(256, k)
    part = tcec.sgemm_packed(ap[off:], bp, m - 256, n, k)
    assert torch.equal(part, want[256:])
    tcec.device_status()


@pytest.mark.parametrize("policy", ["fp16_ec", "fp16_no_ec", "tf32_ec"])
def test_packed_sub_ranges_stay_inside_exactly_sized_buffers(policy):
    """Sub-ranges of packed A and B (the 256-wide tiles and the CTA-pair kernel read row blocks in
    pairs) placed at the very end of a buffer: nothing beyond the operand may be read, and the
    result equals the matching rows and columns of the full product."""
    rng = np.random.default_rng(43)
    m, n, k = 768, 1024, 160
    a = _t(rng.standard_normal((m, k)).astype(np.float32))
    b = _t(rng.standard_normal((k, n)).astype(np.float32))
    want = tcec.sgemm(a, b, policy=policy)
    na, nb = tcec.packed_bytes(m, k, policy), tcec.packed_bytes(n, k, policy)
    # one arena: [A packed][B packed]; the last sub-range of each ends exactly at its operand's end
    arena = torch.full((na + nb,), 0xFF, dtype=torch.uint8, device=DEV)  # 0xFFFF = a NaN in fp16, 0xFFFFFFFF in tf32
    tcec.pack_a(a, policy, out=arena[:na])
    tcec.pack_b(b, policy, out=arena[na:])
    oa, ob = tcec.packed_row_offset(512, k, policy), tcec.packed_row_offset(768, k, policy)
    assert oa and ob and na - oa == tcec.packed_bytes(256, k, policy) and nb - ob == tcec.packed_bytes(256, k, policy)
    # A's last 256 rows: the sub-range ends where B's NaN-free data begins, so an over-read would change nothing
    # visible; therefore use a second arena whose tail is NaN for the check of A
    tail = torch.full((na + 4096,), 0xFF, dtype=torch.uint8, device=DEV)
    tail[:na] = arena[:na]
    got_a = tcec.sgemm_packed(tail[oa:], arena[na:], 256, n, k, policy=policy)
    got_b = tcec.sgemm_packed(arena[:na], torch.cat([arena[na:], torch.full((4096,), 0xFF, dtype=torch.uint8, device=DEV)])[ob:],
                              m, 256, k, policy=policy)
    tcec.device_status()
    assert torch.equal(got_a, want[512:])
    assert torch.equal(got_b, want[:, 768:])


# ---------------------------------------------------------------- cuBLAS-convention entry points
def test_cublas_convention_calls():
    """Column-major storage with transposition flags, exactly the argument list of the
    cublasSgemmBatched call the reference benchmarks against (OP_T, OP_N, lda = ldb = k, ldc = m)."""
    import ctypes

    lib = tcec.load()
    rng = np.random.default_rng(60)
    m, n, k, batch = 200, 130, 96, 3
    a = rng.standard_normal((batch, m, k)).astype(np.float32)  # logical A (m x k)
    b = rng.standard_normal((batch, k, n)).astype(np.float32)  # logical B (k x n)
    c0 = rng.standard_normal((batch, m, n)).astype(np.float32)
    alpha, beta = ctypes.c_float(1.25), ctypes.c_float(-0.5)
    for ta in (0, 1):
        for tb in (0, 1):
            # N: column-major storage of the logical matrix; T: column-major storage of its transpose
            a_mem = _t(a.transpose(0, 2, 1)) if ta == 0 else _t(a)   # (k, m) rows = col-major m x k ; T: rows of A
            b_mem = _t(b.transpose(0, 2, 1)) if tb == 0 else _t(b)
            lda = m if ta == 0 else k
            ldb = k if tb == 0 else n
            c_mem = _t(c0.transpose(0, 2, 1)).clone()                # column-major m x n, ldc = m
            st = lib.tcec_sgemm_cublas(ta, tb, m, n, k, ctypes.byref(alpha), a_mem[0].data_ptr(), lda,
                                       b_mem[0].data_ptr(), ldb, ctypes.byref(beta), c_mem[0].data_ptr(), m, 0, None)
            assert st == tcec.OK
            ptrs = [torch.tensor([x[i].data_ptr() for i in range(1, batch)], dtype=torch.int64, device=DEV)
                    for x in (a_mem, b_mem, c_mem)]
            st = lib.tcec_sgemm_batched_cublas(ta, tb, m, n, k, ctypes.byref(alpha), ptrs[0].data_ptr(), lda,
                                               ptrs[1].data_ptr(), ldb, ctypes.byref(beta), ptrs[2].data_ptr(), m,
                                               batch - 1, 0, None)
            assert st == tcec.OK
            tcec.device_status()
            got = c_mem.cpu().numpy().transpose(0, 2, 1)
            for i in range(batch):
                want = 1.25 * cpu.gemm_f64(a[i], b[i]) - 0.5 * c0[i]
                assert cpu.errors(got[i], want)["max_rel"] < 1e-6, (ta, tb, i)
    assert lib.tcec_sgemm_cublas(5, 0, 4, 4, 4, ctypes.byref(alpha), None, 4, None, 4, ctypes.byref(beta), None, 4,
                                 0, None) == tcec.ERR_INVALID_ARGUMENT


# ---------------------------------------------------------------- randomised differential test
def test_random_shapes_layouts_and_scalars_agree_across_kernels():
    """Sixty seeded random calls (shape, layouts, padded leading dimensions, alpha, beta, policy): whatever
    kernel the library picks gives the bits of the one-SM panel kernel, writes nothing outside C, and stays
    within the policy's error bound against FP64."""
    rng = np.random.default_rng(20260)
    for case in range(60):
        m, n, k = (int(rng.integers(1, 700)), int(rng.integers(1, 900)), int(rng.integers(1, 600)))
        if case % 10 == 0:
            m, n, k = int(rng.integers(1000, 2600)), int(rng.integers(1000, 2600)), int(rng.integers(32, 300))
        policy = ["fp16_ec", "tf32_ec", "fp16_no_ec", "tf32_no_ec"][int(rng.integers(0, 4))]
        la, lb, lc = (["row", "col"][int(rng.integers(0, 2))] for _ in range(3))
        pad = int(rng.choice([0, 0, 4, 3, 8]))
        alpha = float(rng.choice([1.0, 1.0, -0.5, 2.25]))
        beta = float(rng.choice([0.0, 0.0, 1.0, -0.75]))
        a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)

        def view(x, layout):
            r, c = x.shape
            if layout == "row":
                buf = torch.full((r, c + pad), float("nan"), device=DEV)
                buf[:, :c] = _t(x)
                return buf[:, :c]
            buf = torch.full((c, r + pad), float("nan"), device=DEV)
            buf[:, :r] = _t(x.T)
            return buf[:, :r].t()

        A, B = view(a, la), view(b, lb)
        out = {}
        for forced in (False, True):
            tcec.set_option("path", 1 if forced else 0)
            tcec.set_option("cta_pair", 0 if forced else -1)
            C = view(c0, lc)
            tcec.sgemm(A, B, C, alpha=alpha, beta=beta, policy=policy)
            tcec.device_status()
            base = C._base
            assert int(torch.isnan(base).sum()) == base.numel() - m * n, (case, "wrote outside the matrix")
            out[forced] = C.clone()
        what = (case, m, n, k, policy, la, lb, lc, pad, alpha, beta)
        assert torch.equal(out[False], out[True]), what
        want = alpha * cpu.gemm_f64(a, b) + beta * c0
        bound = (2e-3 if "no_ec" in policy else 1e-6) * (abs(alpha) + abs(beta) + 1)
        assert cpu.errors(out[False].cpu().numpy(), want)["max_rel"] < bound, what


def test_random_batches_agree_with_single_calls():
    """Thirty seeded random batches (strided and pointer-array forms, fp16 and tf32, alpha and beta): every
    matrix of the batch has the bits of a single tcec_sgemm call on it, whichever kernel the batch ran on
    (FP32 tiles for short K, panels on one SM or on pairs otherwise)."""
    rng = np.random.default_rng(20261)
    for case in range(30):
        batch = int(rng.integers(1, 40))
        m, n, k = int(rng.integers(1, 420)), int(rng.integers(1, 520)), int(rng.integers(1, 700))
        if case % 6 == 0:
            m, n, k = 256, 256, int(rng.choice([64, 256, 512]))
        policy = ["fp16_ec", "tf32_ec", "fp16_no_ec"][int(rng.integers(0, 3))]
        alpha = float(rng.choice([1.0, 1.0, 0.5]))
        beta = float(rng.choice([0.0, 0.0, -1.25]))
        a = _t(rng.standard_normal((batch, m, k)).astype(np.float32))
        b = _t(rng.standard_normal((batch, k, n)).astype(np.float32))
        c0 = _t(rng.standard_normal((batch, m, n)).astype(np.float32))
        tcec.set_option("path", 1)
        tcec.set_option("cta_pair", 0)
        single = torch.stack([tcec.sgemm(a[i], b[i], c0[i].clone(), alpha=alpha, beta=beta, policy=policy)
                              for i in range(batch)])
        tcec.set_option("path", 0)
        tcec.set_option("cta_pair", -1)
        strided = tcec.sgemm_strided_batched(a, b, c0.clone(), alpha=alpha, beta=beta, policy=policy)
        cl = [c0[i].clone() for i in range(batch)]
        tcec.sgemm_batched([a[i] for i in range(batch)], [b[i] for i in range(batch)], cl, alpha=alpha, beta=beta,
                           policy=policy)
        tcec.device_status()
        what = (case, batch, m, n, k, policy, alpha, beta)
        assert torch.equal(strided, single), what
        assert torch.equal(torch.stack(cl), single), what


# ---------------------------------------------------------------- CUDA graphs
@pytest.mark.parametrize("shape,policy", [((512, 768, 256), "fp16_ec"), ((2048, 2304, 512), "tf32_ec"),
                                          ((300, 200, 100), "fp16_no_ec")])
def test_calls_can_be_captured_in_a_cuda_graph_and_replayed(shape, policy):
    """After one call on a stream (which sizes the stream's workspace), tcec_sgemm on that stream is
    launches only: captured into a CUDA graph and replayed on new operand values it gives the bits of
    a direct call (the kernels leave their tile counters at zero for the next launch)."""
    m, n, k = shape
    rng = np.random.default_rng(2000 + m)
    a = _t(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = _t(rng.uniform(-1, 1, (k, n)).astype(np.float32))
    c = torch.zeros((m, n), dtype=torch.float32, device=DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        tcec.sgemm(a, b, c, policy=policy)  # sizes the workspace of this stream
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        tcec.sgemm(a, b, c, policy=policy)
    for rep in range(3):
        a.copy_(_t(rng.uniform(-1, 1, (m, k)).astype(np.float32)))
        b.copy_(_t(rng.uniform(-1, 1, (k, n)).astype(np.float32)))
        c.zero_()
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(c, tcec.sgemm(a, b, policy=policy)), rep
    tcec.device_status()


# ---------------------------------------------------------------- host threads
def test_host_threads_on_their_own_streams_do_not_disturb_each_other():
    """Four host threads, each with its own stream and shapes, call the library at the same time (ctypes
    releases the interpreter lock during a call): every result equals the one the same call gives alone.
    Workspaces and tile counters are per (device, stream); the state mutex only covers their lookup."""
    import threading

    shapes = [(512, 384, 256, "fp16_ec"), (1300, 700, 96, "tf32_ec"), (256, 2304, 512, "fp16_ec"), (700, 300, 1000, "fp16_no_ec")]
    rng = np.random.default_rng(4242)
    work = []
    for m, n, k, pol in shapes:
        a = _t(rng.uniform(-1, 1, (m, k)).astype(np.float32))
        b = _t(rng.uniform(-1, 1, (k, n)).astype(np.float32))
        work.append((a, b, pol, tcec.sgemm(a, b, policy=pol)))
    torch.cuda.synchronize()
    errors = []

    def run(idx):
        try:
            a, b, pol, want = work[idx]
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for _ in range(25):
                    got = tcec.sgemm(a, b, policy=pol)
                stream.synchronize()
                if not torch.equal(got, want):
                    errors.append(f"thread {idx}: result differs")
        except Exception as e:  # surfaced below: an exception in a thread would otherwise pass silently
            errors.append(f"thread {idx}: {e!r}")

    threads = [threading.Thread(target=run, args=(i,)) for i in range(len(work))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads)
    assert not errors, errors
    tcec.device_status()


# ---------------------------------------------------------------- live reference comparator
@pytest.mark.skipif(not ref.available(), reason="oracle/_ref was not built")
@pytest.mark.parametrize("policy", ["fp16_ec", "tf32_ec"])
@pytest.mark.parametrize("dist_name", ["uniform", "normal", "positive"])
@pytest.mark.parametrize("k", [4096, 16384, 32768])
def test_error_no_worse_than_twice_the_reference(policy, dist_name, k):
    """Acceptance bound: max relative error vs FP64 <= 2x the reference TCEC kernel's and
    <= 2x an FP32 SGEMM's, on identical inputs.  K = 16384 and 32768 are where the automatic
    promotion interval is longest (512), i.e. where the margin is thinnest."""
    torch.manual_seed(50)
    m, n = (1024, 768) if k == 4096 else (1024, 1024)
    if dist_name == "uniform":
        a, b = torch.rand(m, k, device=DEV) * 2 - 1, torch.rand(k, n, device=DEV) * 2 - 1
    elif dist_name == "normal":
        a, b = torch.randn(m, k, device=DEV), torch.randn(k, n, device=DEV)
    else:
        a, b = torch.rand(m, k, device=DEV), torch.rand(k, n, device=DEV)
    exact = a.double() @ b.double()
    scale = exact.abs().max()

    def err(c):
        return ((c.double() - exact).abs().max() / scale).item()

    e_ref = err(ref.bgemm(a[None], b[None], tf32=policy.startswith("tf32"), per=4)[0])
    e_got = err(tcec.sgemm(a, b, policy=policy))
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    e_f32 = err(a @ b)
    torch.backends.cuda.matmul.allow_tf32 = prev
    tcec.device_status()
    assert e_got <= 2 * e_ref, (e_got, e_ref)
    assert e_got <= 2 * e_f32, (e_got, e_f32)


# ---------------------------------------------------------------- full-size properties
def test_full_size_sampled_rows_and_linearity():
    """M=N=K=16384-class problem checked through size-independent properties: sampled rows
    against the FP64 host GEMM, and linearity in alpha."""
    torch.manual_seed(3)
    n = 8192
    sign = torch.where(torch.rand(n, n, device=DEV) < 0.5, -1.0, 1.0)
    a = sign * (1 + torch.rand(n, n, device=DEV)) * torch.exp2(torch.randint(-15, 16, (n, n), device=DEV).float())
    b = torch.randn(n, n, device=DEV)
    a.clamp_(-65000, 65000)  # keep fp16 heads finite so both policies can be compared
    rows = [0, 1, 127, 128, 4095, 4096, 8191]
    a_rows = a[rows].cpu().numpy()
    bh = b.cpu().numpy()
    exact = cpu.gemm_f64(a_rows, bh)
    for policy in ("tf32_ec", "fp16_ec"):
        c = tcec.sgemm(a, b, policy=policy)
        tcec.device_status()
        e = cpu.errors(c[rows].cpu().numpy(), exact)
        e32 = cpu.errors(cpu.gemm_f32(a_rows, bh), exact)
        assert e["max_rel"] <= 2 * e32["max_rel"], (policy, e, e32)
        c2 = tcec.sgemm(a, b, alpha=2.0, policy=policy)
        assert torch.equal(c2, 2 * c)  # scaling by a power of two is exact
        del c, c2


def _free_gib():
    free, _ = torch.cuda.mem_get_info()
    return free / 2 ** 30


def test_batched_configuration_full_size_properties():
    """8192 independent 256^3 products, N(0,1): first/last/sampled matrices against FP64, and the
    row checksums of every matrix, C 1 = A (B 1), which no wrong tile anywhere can satisfy."""
    if _free_gib() < 12:
        pytest.skip("needs 12 GiB of free device memory")
    nb, n = 8192, 256
    g = torch.Generator(device=DEV).manual_seed(4)
    a = torch.randn((nb, n, n), generator=g, device=DEV)
    b = torch.randn((nb, n, n), generator=g, device=DEV)
    c = tcec.sgemm_strided_batched(a, b)
    tcec.device_status()
    idx = [0, 1, 1023, 1024, 4095, 4096, 8190, 8191]
    exact = torch.matmul(a[idx].double(), b[idx].double())
    err = ((c[idx].double() - exact).abs().amax(dim=(1, 2)) / exact.abs().amax(dim=(1, 2))).max().item()
    f32 = torch.matmul(a[idx], b[idx])
    err32 = ((f32.double() - exact).abs().amax(dim=(1, 2)) / exact.abs().amax(dim=(1, 2))).max().item()
    assert err < 1e-6 and err <= 2 * err32, (err, err32)
    ones = torch.ones((nb, n, 1), dtype=torch.float64, device=DEV)
    want = torch.matmul(a.double(), torch.matmul(b.double(), ones)).squeeze(-1)
    got = c.double().sum(dim=2)
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() < 1e-4 * scale  # 256 terms of ~1e-7 relative error each
    # the pointer-array form gives the same bits
    c2 = [torch.empty((n, n), device=DEV) for _ in range(64)]
    tcec.sgemm_batched(list(a[:64]), list(b[:64]), c2)
    tcec.device_status()
    # the pointer-array form goes through the panel kernel, the strided form through the FP32-tile
    # kernel: same split, same products, same rounding points, so not a bit differs
    assert all(torch.equal(x, y) for x, y in zip(c2, c[:64]))


def test_column_block_configuration_full_size_properties():
    """M = N = 65536, K = 8192, N(0,1) on one GPU in column blocks (what each rank of the sharded
    configuration computes): sampled rows against FP64 and the row checksums of the whole result."""
    if _free_gib() < 40:
        pytest.skip("needs 40 GiB of free device memory")
    m = n = 65536
    k = 8192
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn((m, k), generator=g, device=DEV)
    b = torch.randn((k, n), generator=g, device=DEV)
    c = torch.empty((m, n), dtype=torch.float32, device=DEV)
    block = n // 8
    for j in range(8):  # the eight column blocks of the 8-GPU sharding, through strided views of B and C
        tcec.sgemm(a, b[:, j * block:(j + 1) * block], c[:, j * block:(j + 1) * block])
    tcec.device_status()
    rows = torch.tensor([0, 127, 128, 32767, 32768, 65535], device=DEV)
    bd = b.double()
    exact = a[rows].double() @ bd
    err = ((c[rows].double() - exact).abs().max() / exact.abs().max()).item()
    err32 = (((a[rows] @ b).double() - exact).abs().max() / exact.abs().max()).item()
    assert err < 2e-6 and err <= 2 * err32, (err, err32)
    want = a.double() @ (bd @ torch.ones((n, 1), dtype=torch.float64, device=DEV))
    del bd
    got = torch.zeros((m, 1), dtype=torch.float64, device=DEV)
    for j in range(8):
        got += c[:, j * block:(j + 1) * block].double().sum(dim=1, keepdim=True)
    assert ((got - want).abs().max() / want.abs().max()).item() < 1e-5


def test_column_sharded_driver_on_one_gpu(tmp_path):
    """The multi-GPU driver with a world of one rank: row panels of A against a B packed once."""
    import torch.distributed as dist
    from wmma_extension_b200 import sharded

    dist.init_process_group("gloo", init_method=f"file://{tmp_path}/store", rank=0, world_size=1)
    try:
        m, n, k = 700, 520, 300
        g = torch.Generator(device=DEV).manual_seed(9)
        a = torch.randn((m, k), generator=g, device=DEV)
        b = torch.randn((k, n), generator=g, device=DEV)
        c = torch.full((m, n), float("nan"), device=DEV)
        tcec.set_option("comm_panel_rows", 256)  # several panels at this size
        try:
            sharded.sgemm_column_sharded(a, b, c, m, k, root=0)
        finally:
            tcec.set_option("comm_panel_rows", 2048)
        tcec.device_status()
        assert torch.equal(c, tcec.sgemm(a, b))
        first, count = sharded.batch_shard(10, 0, 1)
        ab, bb = torch.randn((10, 64, 96), device=DEV), torch.randn((10, 96, 130), device=DEV)
        assert torch.equal(sharded.sgemm_batch_sharded(ab[first:first + count], bb[first:first + count]),
                           tcec.sgemm_strided_batched(ab, bb))
    finally:
        dist.destroy_process_group()


# ---------------------------------------------------------------- host operands
@pytest.mark.parametrize("la,lb,lc", [("row", "row", "row"), ("col", "row", "col"), ("row", "col", "row")])
def test_host_operand_gemm_matches_device_call(la, lb, lc):
    """tcec_sgemm_host (copy-in, GEMM and copy-out pipelined in row panels) gives the bits of
    tcec_sgemm on the same operands, for every layout, with alpha and beta, padded leading
    dimensions, and a result that is complete once the stream is."""
    rng = np.random.default_rng(70)
    m, n, k = 900, 520, 300

    def host(x, layout, pad):
        r, c = x.shape
        if layout == "row":
            buf = torch.full((r, c + pad), float("nan")).pin_memory()
            v = buf[:, :c]
        else:
            buf = torch.full((c, r + pad), float("nan")).pin_memory()
            v = buf[:, :r].t()
        v.copy_(torch.from_numpy(x))
        return buf, v

    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    _, ah = host(a, la, 4)
    _, bh = host(b, lb, 0)
    for alpha, beta in ((1.0, 0.0), (1.5, -0.5)):
        cbuf, ch = host(c0, lc, 3)
        tcec.sgemm_host(ah, bh, ch, alpha=alpha, beta=beta, panel_rows=256)
        torch.cuda.current_stream().synchronize()
        tcec.device_status()
        cd = _t(c0).clone() if lc == "row" else _t(c0.T).clone().t()
        want = tcec.sgemm(_t(a), _t(b), cd, alpha=alpha, beta=beta)
        assert torch.equal(ch, want.cpu()), (la, lb, lc, alpha)
        assert torch.isnan(cbuf).sum() == cbuf.numel() - m * n  # the padding of C is untouched
    # k == 0 scales C only
    cbuf, ch = host(c0, lc, 0)
    tcec.sgemm_host(ah[:, :0], bh[:0, :], ch, beta=2.0)
    torch.cuda.current_stream().synchronize()
    assert torch.equal(ch, torch.from_numpy(2 * c0))
