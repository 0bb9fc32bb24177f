"""CPU proofs (numpy, exhaustive where the domain is small) of the arithmetic identities the fused
quantizer relies on to be bit-exact without IEEE divides or compares.  Each test restates in numpy
what the kernel computes (svdquant_kernels_b200/csrc/quantize_fused.cu) and compares it with the
definition the oracle uses."""
import numpy as np

from oracle import nvfp4_oracle as O

f32 = np.float32


def _fma(a, b, c):
    # a*b is exact in float64 for float32 inputs; the sums below stay far inside 53 bits
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def _smooth_table_entry(s):
    """(r_hi, r_lo) as the table builder makes them: r_hi = RU(1/s), r_lo = RN((1 - s r_hi) r_hi) <= 0,
    -0 when the reciprocal is exact (qmath::smooth_table_entry)."""
    r = f32(f32(1.0) / s)
    if np.float64(r) * np.float64(s) < 1.0:                 # the product is exact in float64: 24 x 11 bits
        r = np.nextafter(r, f32(np.inf))
    assert np.float64(r) * np.float64(s) >= 1.0
    e = 1.0 - np.float64(r) * np.float64(s)                 # exact, <= 0, at most 11 significant bits
    e32 = f32(e)
    assert np.float64(e32) == e
    return r, (f32(np.float64(e32) * np.float64(r)) if e32 != 0 else f32(-0.0))


def test_two_step_quotient_equals_ieee_division_for_11_bit_mantissas():
    """q = fma(x, r_hi, RN(x * r_lo)) equals RN(x/s) for every pair of 11-bit mantissas (fp16 and, a
    fortiori, bf16 inputs widened to fp32), and either zero comes out as +0.  The fma is evaluated in
    80-bit extended precision, whose 64-bit significand holds x*r_hi + t exactly."""
    ld = np.longdouble
    assert np.finfo(ld).nmant >= 63, "needs x87 extended precision to model the fma exactly"
    x = np.arange(1024, 2048, dtype=np.float32)
    bad = bad_zero = 0
    for ms in range(1024, 2048):
        s = f32(ms)
        r_hi, r_lo = _smooth_table_entry(s)
        assert r_lo <= 0 and np.signbit(r_lo)
        t = (x.astype(np.float64) * np.float64(r_lo)).astype(np.float32)
        q = (x.astype(ld) * ld(r_hi) + t.astype(ld)).astype(np.float32)
        bad += int((q != (x / s).astype(np.float32)).sum())
        for z in (f32(0.0), f32(-0.0)):
            tz = f32(np.float64(z) * np.float64(r_lo))
            qz = f32(ld(z) * ld(r_hi) + ld(tz))
            bad_zero += int(qz != 0 or np.signbit(qz))
    assert bad == 0 and bad_zero == 0


def test_three_step_division_by_six_is_exact_on_sampled_binades():
    """amax / 6 through the same three steps with RN(1/6), over every mantissa of five binades."""
    r6 = f32(1.0) / f32(6.0)
    bad = 0
    for start in range(0, 1 << 23, 1 << 21):
        m = np.arange(start, start + (1 << 21), dtype=np.uint32)
        for ebits in (100, 127, 128, 129, 140):
            a = ((np.uint32(ebits) << 23) | m).view(np.float32)
            q0 = (a * r6).astype(np.float32)
            e = a.astype(np.float64) - 6.0 * q0.astype(np.float64)
            e32 = e.astype(np.float32)
            assert (e32.astype(np.float64) == e).all()          # the remainder is exact
            q = (q0.astype(np.float64) + e32.astype(np.float64) * np.float64(r6)).astype(np.float32)
            bad += int((q != (a / f32(6.0)).astype(np.float32)).sum())
    assert bad == 0


def test_quotient_compare_equals_product_compare():
    """RN(a / s) >= b  <=>  a >= s*b for every positive e4m3 scale, every E2M1 bound and the fp32
    neighbours of the product (s*b is exact: 4 x 3 significant bits)."""
    bounds = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    for s in O._E4M3_POS[1:]:
        for b in bounds:
            p = f32(s) * f32(b)
            assert np.float64(p) == np.float64(s) * np.float64(b)
            cands, lo, hi = [p], p, p
            for _ in range(4):
                lo, hi = np.nextafter(lo, f32(0)), np.nextafter(hi, f32(1e30))
                cands += [lo, hi]
            a = np.array(cands, dtype=np.float32)
            assert (((a / f32(s)).astype(np.float32) >= b) == (a >= p)).all(), (s, b)


_LEVELS = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float64)


def _rne_e2m1(w):
    """float -> E2M1 code, round to nearest, ties to the even code, saturating: the documented
    behaviour of cvt.rn.satfinite.e2m1x2.f32."""
    out = np.zeros(w.shape, dtype=np.int64)
    for i, x in np.ndenumerate(w.astype(np.float64)):
        if x >= 6:
            out[i] = 7
            continue
        hi = int(np.searchsorted(_LEVELS, x, side="right"))
        lo = hi - 1
        dl, dh = x - _LEVELS[lo], _LEVELS[hi] - x
        out[i] = lo if dl < dh else hi if dh < dl else (lo if lo % 2 == 0 else hi)
    return out


def test_hardware_conversion_of_scaled_floor_counts_the_bounds():
    """With scale = J * 2^E and m = floor(4|v| / 2^E): the E2M1 conversion of
    RN(m * RN(RN(1/(4J)) * (1 + 2^-20))) equals #{n in {1,3,5,7,10,14,20} : n*J <= m} for every
    J in 1..15 and every m up to well past saturation, and never lands on a rounding tie (so the
    tie rule of the conversion does not matter)."""
    fudge = f32(1.0) + f32(2.0 ** -20)
    for J in range(1, 16):
        rj = f32(f32(f32(1.0) / f32(4 * J)) * fudge)
        m = np.arange(0, 40 * J + 5, dtype=np.float32)
        w = (m * rj).astype(np.float32)
        ref = sum((n * J <= m.astype(np.int64)).astype(np.int64) for n in (1, 3, 5, 7, 10, 14, 20))
        assert (_rne_e2m1(w) == ref).all(), J
        ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
        assert not np.isin(w.astype(np.float64), ties).any(), J


def test_signed_truncation_carries_the_sign_through_the_rescale():
    """The kernel forms trunc(4 v / 2^E) * rj with the sign of v riding along: for negative v this is
    minus the value for |v| (rounding to nearest is symmetric), and a small negative v gives -0, the
    'negative zero' code the reference produces for it."""
    rng = np.random.default_rng(1)
    t = (rng.random(200000) * 400).astype(np.float32)
    for J in (1, 3, 7, 15):
        rj = f32(f32(f32(1.0) / f32(4 * J)) * (f32(1.0) + f32(2.0 ** -20)))
        pos = (np.trunc(t) * rj).astype(np.float32)
        neg = (np.trunc(-t) * rj).astype(np.float32)
        assert (neg == -pos).all()
        assert np.signbit(neg[t < 1]).all() and (neg[t < 1] == 0).all()


def _round_to_f32(fr):
    """Correctly rounded (nearest, ties to even) float32 of an exact rational, normal range only."""
    from fractions import Fraction
    if fr == 0:
        return np.float32(0.0)
    sign = -1 if fr < 0 else 1
    fr = abs(fr)
    e = 0
    while fr >= Fraction(1 << 24):
        fr /= 2
        e += 1
    while fr < Fraction(1 << 23):
        fr *= 2
        e -= 1
    n = fr.numerator // fr.denominator
    rem = fr - n
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and (n & 1)):
        n += 1
    return np.float32(sign * float(n) * 2.0 ** e)        # n < 2^24 + 1 and a power of two: exact


def test_division_through_the_rounded_reciprocal_equals_ieee_division_on_samples():
    """The next-layer epilogue's divide: q0 = RN(a r), e = a - s q0 (one fma, exact), q = RN(q0 + e r) with
    r = RN(1 / s), for fp32 dividends and divisors of at most 11 significant bits, against the correctly
    rounded quotient worked out with rationals.  (The library's device self-test does all 2^23 x 2^10
    significand pairs; this is the same statement on a sample, for boxes without a GPU.)"""
    from fractions import Fraction
    rng = np.random.default_rng(5)
    # divisors: every 64th 11-bit significand plus the extremes, over a few binades; dividends: random fp32
    sig = sorted(set(list(range(1024, 2048, 64)) + [1024, 1025, 2046, 2047]))
    divisors = [np.float32(m * 2.0 ** (k - 10)) for m in sig for k in (-12, -1, 0, 3, 14)]
    bad = 0
    checked = 0
    for s in divisors:
        r = np.float32(1.0) / s                                  # numpy divides correctly rounded
        a = (rng.standard_normal(40).astype(np.float32) * np.float32(2.0) ** rng.integers(-20, 20, 40)).astype(np.float32)
        a[:4] = [np.float32(1.0), np.float32(-3.0), np.nextafter(np.float32(1.0), np.float32(2.0)), s]
        for av in a:
            fa, fs, fr = Fraction(float(av)), Fraction(float(s)), Fraction(float(r))
            q0 = np.float32(av * r)
            fe = fa - fs * Fraction(float(q0))                    # the fma's exact value ...
            e = _round_to_f32(fe)
            assert Fraction(float(e)) == fe, "... which fp32 holds exactly"
            q = _round_to_f32(Fraction(float(q0)) + fe * fr)
            want = _round_to_f32(fa / fs)
            bad += int(q != want)
            checked += 1
    assert checked > 3000 and bad == 0
