"""Derives the polynomial coefficients hard-coded in gv_transcendentals.h.

erf and exp are approximated by Chebyshev interpolants (converted to monomials in
a centred, scaled variable) so that the CPU oracle and the CUDA kernels evaluate
the very same fp32 fmaf chain and therefore agree bit for bit.  Run:

    python fit_transcendentals.py        # prints C initialisers + max errors
"""
import numpy as np
from numpy.polynomial import chebyshev as C
from scipy.special import erf


def cheb_mono(f, lo, hi, deg):
    c, h = (lo + hi) / 2.0, (hi - lo) / 2.0
    n = deg + 1
    k = np.arange(n)
    x = np.cos(np.pi * (k + 0.5) / n)
    return c, h, C.cheb2poly(C.chebfit(x, f(c + h * x), deg))


def horner32(mono, x):
    acc = np.full_like(x, np.float32(mono[-1]))
    for co in mono[-2::-1]:
        acc = (acc.astype(np.float64) * x.astype(np.float64)
               + np.float64(np.float32(co))).astype(np.float32)
    return acc


def fmt(mono, width):
    m = list(mono) + [0.0] * (width - len(mono))
    return "{" + ", ".join(f"{np.float32(v):.9e}f" for v in m) + "}"


def main():
    # erf on [0,4): eight intervals of width 0.5, degree 6 in u = a - centre
    worst = 0.0
    print("#define GV_ERF_TABLE_INIT {\\")
    for i in range(8):
        lo, hi = 0.5 * i, 0.5 * (i + 1)
        c, h, m = cheb_mono(erf, lo, hi, 6)
        m = m / (h ** np.arange(len(m)))  # monomial in (a - c)
        a = np.linspace(lo, hi, 100001)[:-1].astype(np.float32)
        u = (a - np.float32(c)).astype(np.float32)
        worst = max(worst, np.abs(horner32(m, u).astype(np.float64) - erf(a.astype(np.float64))).max())
        print("  " + fmt(m, 7)[:-1] + ", 0.0f},\\")
    print("}")
    print(f"// erf table max abs err {worst:.3e}")
    # exp on [-ln2/2, ln2/2]
    half = np.log(2.0) / 2
    c, h, m = cheb_mono(np.exp, -half, half, 6)
    r = np.linspace(-half, half, 400001).astype(np.float32)
    x = (r * np.float32(1 / h)).astype(np.float32)
    # fold 1/h into the coefficients so the kernel evaluates p(r) directly
    m2 = m / (h ** np.arange(len(m)))
    e = np.abs(horner32(m2, r).astype(np.float64) / np.exp(r.astype(np.float64)) - 1).max()
    print(f"// exp core max rel err {e:.3e}")
    print("GV_EXP_POLY =", fmt(m2, 7))


if __name__ == "__main__":
    main()
