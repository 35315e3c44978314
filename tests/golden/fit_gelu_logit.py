"""Derives the coefficients of `gelu_pair_fast` in hawk-pytorch_b200/csrc/glue.cu (needs numpy and scipy; not used at run time).

The bf16 GELU kernels evaluate the exact (erf) GELU as a * Phi(a) with Phi(a) = 1 / (1 + exp(-a q(a^2))),
where a q(a^2) = log(Phi(a) / Phi(-a)) exactly.  q is smooth and grows slowly, so a low-degree polynomial
in s = a^2 reproduces it; this script fits degree 6 by Lawson-weighted least squares (towards the minimax
fit), weighting by the sensitivity of a * Phi(a) to an error in q, and prints the coefficients of
-log2(e) * q(s), highest degree first, as the kernel's Horner chain uses them, together with the error
of the fp32 evaluation over |a| <= 60 and at the largest magnitudes.

    python tests/golden/fit_gelu_logit.py
"""
import numpy as np
from scipy.special import log_ndtr, ndtr

DEG, S_MAX = 6, 30.25  # fitted for |a| <= 5.5; beyond it the polynomial keeps growing, so Phi saturates by itself


def q_of_s(s):
    a = np.sqrt(s)
    logit = log_ndtr(a) - log_ndtr(-a)
    return np.where(a > 1e-6, logit / np.maximum(a, 1e-300), 4.0 / np.sqrt(2 * np.pi))


def fit(deg=DEG, s_max=S_MAX, iters=60):
    a = np.linspace(0, np.sqrt(s_max), 20001)
    s = a * a
    q = q_of_s(s)
    phi = ndtr(a)
    sens = phi * (1 - phi) * a * a + 1e-12  # d(a Phi) / dq
    w = np.ones_like(s)
    vander = np.vander(s / s_max, deg + 1, increasing=True)
    for _ in range(iters):
        ww = w * sens
        c, *_ = np.linalg.lstsq(vander * ww[:, None], q * ww, rcond=None)
        err = np.abs((vander @ c - q) * sens)
        w = w * (err / err.max() + 1e-3) ** 0.5
        w /= w.max()
    return c / s_max ** np.arange(deg + 1)  # increasing powers of s


def check(c):
    a = np.concatenate([np.linspace(-60, 60, 1200001), [-1e3, 1e3, -1e10, 1e10, -3e38, 3e38]])
    a32 = a.astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        s = (a32 * a32).astype(np.float32)
        q = np.zeros_like(s) + np.float32(c[-1])
        for k in range(len(c) - 2, -1, -1):
            q = (q * s + np.float32(c[k])).astype(np.float32)
        e = (a32 * q).astype(np.float32)
        phi = (1.0 / (1.0 + np.exp(-e.astype(np.float64)))).astype(np.float32)
        g = (a32 * phi).astype(np.float64)
    true = a * ndtr(a)
    body = slice(0, -6)
    rel = np.abs(g - true) / np.maximum(np.abs(true), 1e-4)
    return dict(min_q=float(q.min()), any_nan=bool(np.isnan(q).any()), max_abs=float(np.abs(g - true)[body].max()),
                max_rel_floor_1e_4=float(rel[body].max()), extremes=g[-6:].tolist())


if __name__ == "__main__":
    coeffs = fit()
    print("q(s), increasing powers:", [f"{v:.10e}" for v in coeffs])
    print("-log2(e) q(s), highest degree first:", [f"{v:.7e}" for v in (-np.log2(np.e) * coeffs)[::-1]])
    print(check(coeffs))
