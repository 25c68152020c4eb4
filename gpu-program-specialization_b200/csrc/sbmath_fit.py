"""Derives the polynomial coefficients used by sbmath.cuh.

Each polynomial is fitted in float64 with Lawson's iteratively re-weighted least squares
(an approximation of the minimax fit) on a dense grid, rounded to float32, and its worst
error is reported by re-evaluating it in emulated float32 fused-multiply-add arithmetic
against the float64 function.  Run:  python sbmath_fit.py  (prints the constants).
"""
import numpy as np


def lawson(basis, target, weight, iters=60):
    w = np.ones(len(target))
    for _ in range(iters):
        sw = np.sqrt(w) * weight
        coef, *_ = np.linalg.lstsq(basis * sw[:, None], target * sw, rcond=None)
        err = np.abs(basis @ coef - target) * weight
        w = w * (err / err.max() + 1e-3)
        w /= w.sum()
    return coef


def f32(x):
    return np.asarray(x, dtype=np.float32)


def fma(a, b, c):
    return f32(np.float64(a) * np.float64(b) + np.float64(c))


def ulp_err(got, exact):
    got = np.float64(got)
    ulp = np.spacing(np.abs(f32(exact))).astype(np.float64)
    return np.abs(got - exact) / ulp


def fit_sin():
    r = np.linspace(-np.pi / 4, np.pi / 4, 40001)
    r = r[r != 0]
    z = r * r
    # sin r = r + r^3 (s0 + s1 z + s2 z^2)
    target = (np.sin(r) - r) / r ** 3
    basis = np.stack([z ** k for k in range(3)], axis=1)
    coef = lawson(basis, target, np.abs(r ** 3 / np.sin(r)))
    c = f32(coef)
    rf = f32(r)
    zf = f32(rf * rf)
    p = fma(fma(c[2], zf, c[1]), zf, c[0])
    got = fma(f32(rf * zf), p, rf)
    return c, ulp_err(got, np.sin(np.float64(rf))).max()


def fit_cos():
    r = np.linspace(-np.pi / 4, np.pi / 4, 40001)
    z = r * r
    # cos r = 1 - z/2 + z^2 (c0 + c1 z + c2 z^2)
    zz = np.where(z == 0, 1, z)
    target = np.where(z == 0, 1 / 24.0, (np.cos(r) - 1 + z / 2) / zz ** 2)
    basis = np.stack([z ** k for k in range(4)], axis=1)
    coef = lawson(basis, target, z ** 2 / np.cos(r))
    c = f32(coef)
    rf = f32(r)
    zf = f32(rf * rf)
    p = fma(fma(fma(c[3], zf, c[2]), zf, c[1]), zf, c[0])
    got = f32(f32(1.0) + fma(f32(zf * zf), p, f32(-0.5) * zf))
    return c, ulp_err(got, np.cos(np.float64(rf))).max()


def fit_exp():
    h = np.log(2) / 2 * 1.0001
    r = np.linspace(-h, h, 40001)
    r = r[r != 0]
    # exp r = 1 + r + r^2 (e0 + e1 r + ... + e4 r^4)
    target = (np.exp(r) - 1 - r) / r ** 2
    basis = np.stack([r ** k for k in range(6)], axis=1)
    coef = lawson(basis, target, r ** 2 / np.exp(r))
    c = f32(coef)
    rf = f32(r)
    p = c[5]
    for k in (4, 3, 2, 1, 0):
        p = fma(p, rf, c[k])
    got = f32(f32(1.0) + fma(f32(rf * rf), p, rf))
    return c, ulp_err(got, np.exp(np.float64(rf))).max()


def fit_log():
    lo, hi = np.sqrt(0.5), np.sqrt(2.0)
    m = np.linspace(lo, hi, 60001)
    f = m - 1
    f = f[f != 0]
    # log(1+f) = f - f^2/2 + f^3 (l0 + l1 f + ... + l6 f^6)
    target = (np.log1p(f) - f + f * f / 2) / f ** 3
    basis = np.stack([f ** k for k in range(8)], axis=1)
    coef = lawson(basis, target, np.abs(f ** 3 / np.log1p(f)))
    c = f32(coef)
    ff = f32(f)
    p = c[7]
    for k in (6, 5, 4, 3, 2, 1, 0):
        p = fma(p, ff, c[k])
    f2 = f32(ff * ff)
    got = f32(ff + fma(f32(ff * f2), p, f32(-0.5) * f2))
    return c, ulp_err(got, np.log1p(np.float64(ff))).max()


def split(value, bits):
    """value = hi + mid + lo with hi, mid holding `bits` significant bits each."""
    parts = []
    rest = value
    for _ in range(2):
        m, e = np.frexp(rest)
        hi = np.ldexp(np.round(m * 2 ** bits) / 2 ** bits, e)
        parts.append(hi)
        rest -= hi
    parts.append(rest)
    return parts


if __name__ == "__main__":
    np.set_printoptions(precision=10)
    for name, fn in (("sin", fit_sin), ("cos", fit_cos), ("exp", fit_exp), ("log", fit_log)):
        c, err = fn()
        print(name, [f"{float(x):.9e}f" for x in c], f"max error {err:.3f} ulp (polynomial only)")
    print("pi/2 split", [f"{float(f32(x)):.9e}f" for x in split(np.pi / 2, 24)])
    print("ln2 split", [f"{float(f32(x)):.9e}f" for x in split(np.log(2), 16)[:2]], "rest folded:",
          f"{float(f32(np.log(2) - float(f32(split(np.log(2), 16)[0])))):.9e}f")
    # 2/pi as 32-bit words after the binary point, enough for |x| < 2^128
    from fractions import Fraction
    from math import factorial

    def pi_fraction(terms=260):  # Chudnovsky is overkill; use Machin with exact rationals
        def atan_inv(n, terms):
            s = Fraction(0)
            for k in range(terms):
                s += Fraction((-1) ** k, (2 * k + 1) * n ** (2 * k + 1))
            return s
        return 4 * (4 * atan_inv(5, terms) - atan_inv(239, terms // 3))

    two_over_pi = 2 / pi_fraction()
    words = []
    x = two_over_pi
    for _ in range(8):
        x *= 2 ** 32
        w = int(x)
        words.append(w)
        x -= w
    print("2/pi words", ", ".join(f"0x{w:08x}u" for w in words))
