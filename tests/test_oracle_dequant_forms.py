"""The level-2 kernels de-quantise the packed 4-bit keys in bf16 arithmetic (one rounding per operation),
the oracle in fp32 with a rounding to bf16 after each operation (two roundings).  The two forms must give
the same bits for every input the path can meet; this checks the claim on the CPU, exhaustively for the
product (16 codes x every finite bf16 scale) and on millions of (value, zero) pairs for the difference,
against an exact evaluation in float64."""
import numpy as np


def _round_f64_to_bf16(x):
    """Round-to-nearest-even of exact float64 values to bf16 (subnormals kept), as float64."""
    x = np.asarray(x, np.float64)
    _, e = np.frexp(x)
    lead = np.maximum(e - 1, -126)
    q = np.ldexp(1.0, lead - 7)
    with np.errstate(invalid="ignore"):
        r = np.rint(x / q) * q
        r = np.where(np.abs(r) > 3.3895313892515355e38, np.sign(r) * np.inf, r)
    return np.where(np.isfinite(x), r, x)


def _bf16r(x32):
    """The oracle's rounding of fp32 to bf16 (loda_oracle.bf16_rn), as float64 for comparison."""
    from oracle import loda_oracle as oc
    return oc.bf16_rn(np.asarray(x32, np.float32)).astype(np.float64)


def _finite_bf16():
    allb = (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)
    return allb[np.isfinite(allb)]


def test_code_times_scale_rounds_once_in_both_forms():
    fin = _finite_bf16()
    for code in range(16):
        with np.errstate(over="ignore"):
            two_roundings = _bf16r(np.float32(code) * fin)
        one_rounding = _round_f64_to_bf16(np.float64(code) * fin.astype(np.float64))
        assert np.array_equal(two_roundings, one_rounding), code


def test_difference_of_two_bf16_numbers_rounds_the_same_in_both_forms():
    fin = _finite_bf16()
    rng = np.random.default_rng(0)
    for _ in range(4):
        t = fin[rng.integers(0, len(fin), 1_000_000)]
        z = fin[rng.integers(0, len(fin), 1_000_000)]
        _, et = np.frexp(t.astype(np.float64))
        _, ez = np.frexp(z.astype(np.float64))
        exact = (np.abs(et - ez) <= 40) | (t == 0) | (z == 0)        # the float64 difference is exact there
        with np.errstate(all="ignore"):
            a = _bf16r(t - z)
            b = _round_f64_to_bf16(t.astype(np.float64) - z.astype(np.float64))
        assert np.array_equal(a[exact], b[exact])
    # every pair of mantissas at every exponent distance where the fp32 difference is, and is not, exact
    mant = np.arange(128, dtype=np.uint32)
    for dist in range(0, 30):
        for sign in (0, 0x8000):
            tb = (np.uint32(0x3F80 + (20 << 7)) + mant)[:, None] << 16
            zb = ((np.uint32(0x3F80 + ((20 - dist) << 7)) + mant)[None, :] | sign) << 16
            t = np.broadcast_to(tb, (128, 128)).astype(np.uint32).view(np.float32).ravel()
            z = np.broadcast_to(zb, (128, 128)).astype(np.uint32).view(np.float32).ravel()
            a = _bf16r(t - z)
            b = _round_f64_to_bf16(t.astype(np.float64) - z.astype(np.float64))
            assert np.array_equal(a, b), (dist, sign)
