"""Error metrics shared by the GPU parity tests.

`strict_rel` is the elementwise metric stated for f32 results: |a - b| / max(|b|, 1e-6 * max|b|).

For contractions it is applied against the ENVELOPE of the oracle's two variants: an OpenCL compiler may
contract `c += a * b` into a fused multiply-add or not (the oracle's USE_FMA switch), so the reference itself
has two legal answers per element.  An element passes when it is within `tol` of either answer by the strict
metric, or lies between them.  Outputs that cancel to ~0 can still miss (any two fp32 summation orders differ
there by more than 1e-4 of the value), so the result is the FRACTION of elements that miss and the worst one;
the tests assert a bound on the fraction and keep the rms-floored metric beside it.

The bound is calibrated by the data itself: the correctly rounded float64 product — the best any f32 kernel
could return — also misses the envelope on some elements, because the oracle's sequential sums carry their own
rounding (measured with U(-1, 1) operands: 1.4e-3 of the elements at K = 1024, 3.5e-3 at K = 4608, 1e-4 at
K = 63).  A result passes when it misses on at most 1.5 x as many elements as that exact product (+ 3 elements),
and never on more than `max_fraction` of them.
"""
import numpy as np

from oracle import sage_ref as R


def strict_rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    scale = np.maximum(np.abs(b), 1e-6 * max(float(np.abs(b).max(initial=0.0)), 1e-30))
    return np.abs(a - b) / scale


def oracle_envelope(fn):
    """Evaluates `fn()` (which builds and evaluates an oracle graph) with and without FMA contraction."""
    saved = R.USE_FMA
    try:
        outs = []
        for fma in (0, 1):
            R.USE_FMA = fma
            outs.append(np.asarray(fn()))
    finally:
        R.USE_FMA = saved
    return outs


def envelope_report(got, refs, tol=1e-4):
    """-> dict(fraction, failing, size, worst, worst_value): elements of `got` outside the envelope of `refs`."""
    got = np.asarray(got, np.float64)
    lo = np.minimum(refs[0], refs[1]).astype(np.float64)
    hi = np.maximum(refs[0], refs[1]).astype(np.float64)
    assert got.shape == lo.shape, (got.shape, lo.shape)
    e = np.minimum(strict_rel(got, refs[0]), strict_rel(got, refs[1]))
    ok = (e <= tol) | ((got >= lo) & (got <= hi))
    bad = ~ok
    n_bad = int(bad.sum())
    worst = float(e[bad].max()) if n_bad else float(e.max(initial=0.0))
    where = int(np.argmax(np.where(bad, e, -1.0))) if n_bad else int(np.argmax(e)) if e.size else 0
    return dict(fraction=n_bad / max(got.size, 1), failing=n_bad, size=int(got.size), worst=worst,
                worst_value=float(np.asarray(refs[1], np.float64).flat[where]) if got.size else 0.0)


def check_envelope(name, got, fn, exact, max_fraction=1e-2, tol=1e-4):
    """`fn` evaluates the oracle; `exact` is the float64 result of the same contraction."""
    refs = oracle_envelope(fn)
    rep = envelope_report(got, refs, tol)
    best = envelope_report(np.asarray(exact, np.float64).astype(np.float32), refs, tol)
    print("\n[envelope] %s: %d of %d elements (%.2e) outside the FMA/non-FMA envelope at %.0e; worst %.3e on a value of %.3e; "
          "the exact product rounded to f32 misses on %d"
          % (name, rep["failing"], rep["size"], rep["fraction"], tol, rep["worst"], rep["worst_value"], best["failing"]))
    assert rep["failing"] <= 1.5 * best["failing"] + 3, (rep, best)
    assert rep["fraction"] <= max_fraction, rep
    return rep
