"""The CPU restatement against the reference's own outputs (golden fixtures made by
tests/golden/make_golden.py from the reference built for sm_100a) and against
independent numpy arithmetic.  No GPU needed."""
import os

import numpy as np
import pytest

from oracle import cpu


def _bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def test_fp16_rounding_matches_numpy_everywhere():
    rng = np.random.default_rng(5)
    x = (rng.uniform(-1, 1, 400000) * np.exp2(rng.integers(-45, 20, 400000))).astype(np.float32)
    x = np.concatenate([x, np.array([0.0, -0.0, 65504, 65519.996, 65520, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25,
                                      np.nextafter(np.float32(2.0 ** -25), np.float32(1)), 6.1e-5], np.float32)])
    hi, _ = cpu.split(x, "fp16_ec")
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(_bits(hi), _bits(want))


def test_tf32_rounding_is_nearest_ties_away():
    base = np.float32(1.0)
    ulp = np.float32(2.0 ** -10)  # tf32 keeps 10 mantissa bits
    assert cpu.load().oracle_round_tf32(float(base + ulp / 2)) == float(base + ulp)  # tie goes away from zero
    assert cpu.load().oracle_round_tf32(float(-(base + ulp / 2))) == float(-(base + ulp))
    assert cpu.load().oracle_round_tf32(float(base + ulp / 4)) == float(base)
    x = np.random.default_rng(6).uniform(-4, 4, 10000).astype(np.float32)
    hi, lo = cpu.split(x, "tf32_ec")
    assert np.all((_bits(hi) & 0x1FFF) == 0) and np.all((_bits(lo) & 0x1FFF) == 0)
    assert np.all(np.abs(x - hi) <= np.abs(x) * 2.0 ** -11 * 1.0001)


def test_split_bit_exact_against_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_split.npz"))
    for name in ("fp16", "tf32"):
        hi, lo = cpu.split(g["x"], name + "_ec")
        assert np.array_equal(_bits(hi), _bits(g["hi_" + name])), name
        assert np.array_equal(_bits(lo), _bits(g["lo_" + name])), name


def test_fp16_split_reconstructs_to_22_bits():
    x = np.random.default_rng(7).uniform(-1, 1, 50000).astype(np.float32)
    hi, lo = cpu.split(x, "fp16_ec")
    rec = hi.astype(np.float64) + lo.astype(np.float64) / 2048.0
    assert np.max(np.abs(rec - x)) <= 2.0 ** -22


def test_gemm_f64_matches_numpy():
    rng = np.random.default_rng(8)
    a = rng.standard_normal((37, 53)).astype(np.float32)
    b = rng.standard_normal((53, 29)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.allclose(cpu.gemm_f64(a, b), want, rtol=1e-13, atol=1e-13)
    assert np.allclose(cpu.gemm_f64(np.asfortranarray(a), np.asfortranarray(b)), want, rtol=1e-13, atol=1e-13)
    assert np.allclose(cpu.gemm_f64(a, b, 5, 9), want[5:9], rtol=1e-13, atol=1e-13)


def _policy_of(key):
    return ("tf32" if "tf32" in key else "fp16") + ("_ec" if "_ec_" in key else "_no_ec")


def test_warp_mma_fixtures(golden_dir):
    """Reference one-warp 32x32x32 results: inside the reference's own thresholds
    (test/tcec/mma.cu:5-19) and reproduced by the restatement to a few ulps."""
    g = np.load(os.path.join(golden_dir, "ref_warp_mma.npz"))
    a, b, c = g["a"], g["b"], g["c"]
    exact = a.astype(np.float64) @ b.astype(np.float64)
    keys = [k for k in g.files if k.startswith("d_")]
    assert len(keys) == 32
    for key in keys:
        pol = _policy_of(key)
        ec = pol.endswith("_ec") and not pol.endswith("no_ec")
        with_c = "abcd" in key
        want = exact + (c if with_c else 0)
        thr = 1e-5 if ec else 1e-2
        assert np.max(np.abs(g[key] - want)) < thr, key
        # without_ec rounds C to T when it is loaded (no_cor.hpp:165-166): mirror that quirk
        c_in = None
        if with_c:
            c_in = c if ec else cpu.split(c, pol)[0]
        rn_block = 0 if (not ec or key.endswith("_rz")) else 1
        got = cpu.tcec_gemm(a, b, c_in, beta=1.0 if with_c else 0.0, policy=pol, rn_block=rn_block)
        assert np.max(np.abs(got - g[key])) < 4e-6, (key, np.max(np.abs(got - g[key])))


def test_bgemm_fixtures(golden_dir):
    g = np.load(os.path.join(golden_dir, "ref_bgemm.npz"))
    a, b = g["a"], g["b"]
    for name in ("fp16", "tf32"):
        for i in range(a.shape[0]):
            exact = cpu.gemm_f64(a[i], b[i])
            e_ref = cpu.errors(g["c_" + name][i], exact)
            got = cpu.tcec_gemm(a[i], b[i], policy=name + "_ec")
            e_got = cpu.errors(got, exact)
            assert e_ref["max_rel"] < 1e-6 and e_got["max_rel"] < 1e-6
            assert np.max(np.abs(got - g["c_" + name][i])) <= 2e-6 * np.max(np.abs(exact))
    # the reference's own deterministic inputs (test/tcec/batch_gemm.cu:507-513)
    exact = cpu.gemm_f64(g["a_iota"][0], g["b_iota"][0])
    got = cpu.tcec_gemm(g["a_iota"][0], g["b_iota"][0], policy="fp16_ec")
    assert cpu.errors(g["c_iota_fp16"][0], exact)["fro_rel"] < 1e-6
    assert cpu.errors(got, exact)["fro_rel"] < 1e-6


@pytest.mark.parametrize("policy,bound", [("fp16_ec", 1e-6), ("tf32_ec", 1e-6), ("fp16_no_ec", 2e-3),
                                          ("tf32_no_ec", 2e-3)])
def test_restatement_error_levels(policy, bound):
    rng = np.random.default_rng(9)
    a = rng.uniform(-1, 1, (96, 160)).astype(np.float32)
    b = rng.uniform(-1, 1, (160, 80)).astype(np.float32)
    exact = cpu.gemm_f64(a, b)
    assert cpu.errors(cpu.tcec_gemm(a, b, policy=policy), exact)["max_rel"] < bound
    c0 = rng.uniform(-1, 1, (96, 80)).astype(np.float32)
    got = cpu.tcec_gemm(a, b, c0, alpha=0.5, beta=-2.0, policy=policy)
    assert cpu.errors(got, 0.5 * exact - 2.0 * c0)["max_rel"] < bound * 2


@pytest.mark.parametrize("policy,bound", [("fp16_ec", 1e-6), ("tf32_ec", 1e-6), ("fp16_no_ec", 2e-3)])
def test_complex_product_from_four_real_products(policy, bound):
    """The reference's complex fragments (complex.hpp:646-727; threshold of test/tcec/mma_complex.cu)."""
    rng = np.random.default_rng(21)
    a = (rng.uniform(-1, 1, (32, 32)) + 1j * rng.uniform(-1, 1, (32, 32))).astype(np.complex64)
    b = (rng.uniform(-1, 1, (32, 32)) + 1j * rng.uniform(-1, 1, (32, 32))).astype(np.complex64)
    exact = a.astype(np.complex128) @ b.astype(np.complex128)
    got = cpu.tcec_cgemm(a, b, policy=policy)
    assert np.max(np.abs(got - exact)) / np.max(np.abs(exact)) < bound
    if not policy.endswith("no_ec"):
        assert np.max(np.abs(got - exact)) < 1e-5 * np.sqrt(2)


def test_wide_exponent_inputs():
    """The 16384^3 configuration's value distribution, sign * U[1,2) * 2^U{-15..15}: tf32 keeps
    the FP32 exponent range; fp16 heads overflow to inf from 65520 up (reference semantics,
    scale.hpp:11-20 only rescues the residual), which poisons the rows that meet such a value."""
    rng = np.random.default_rng(3)
    shape_a, shape_b = (64, 256), (256, 64)

    def gen(shape):
        return (rng.choice([-1.0, 1.0], shape) * rng.uniform(1, 2, shape) * np.exp2(rng.integers(-15, 16, shape))
                ).astype(np.float32)

    a, b = gen(shape_a), gen(shape_b)
    exact = cpu.gemm_f64(a, b)
    e_tf32 = cpu.errors(cpu.tcec_gemm(a, b, policy="tf32_ec"), exact)["max_rel"]
    e_fp16 = cpu.errors(cpu.tcec_gemm(a, b, policy="fp16_ec"), exact)["max_rel"]
    e_f32 = cpu.errors(cpu.gemm_f32(a, b), exact)["max_rel"]
    assert e_tf32 < 2 * max(e_f32, 1e-7)
    assert e_fp16 < 2 * max(e_f32, 1e-7)  # no value of this draw reaches 65520
    a[3, 5] = 65530.0  # in range of the distribution, beyond the largest finite fp16
    exact = cpu.gemm_f64(a, b)
    bad = cpu.tcec_gemm(a, b, policy="fp16_ec")
    assert not np.all(np.isfinite(bad[3])) and np.all(np.isfinite(np.delete(bad, 3, axis=0)))
    assert cpu.errors(cpu.tcec_gemm(a, b, policy="tf32_ec"), exact)["max_rel"] < 2 * max(e_f32, 1e-7)
