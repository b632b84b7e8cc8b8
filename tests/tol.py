"""The one tolerance rule of the floating-point parity tests.

FP32-accumulated results must match the reference within rel 1e-3 / abs 1e-4. The absolute
term is stated for outputs of unit scale: a contraction over K terms of magnitude a.b has
outputs (and an f32 reference whose own rounding error is) proportional to the magnitudes it
sums, so for a tensor whose largest reference magnitude is m the absolute bar is
1e-4 * max(1, m / 8). Elementwise results never need the scaling (m is O(1) there)."""
import numpy as np

RTOL, ATOL = 1e-3, 1e-4


def abs_bar(want) -> float:
    m = float(np.max(np.abs(want))) if np.size(want) else 0.0
    return ATOL * max(1.0, m / 8.0)


def assert_close(got, want, name="", rtol=RTOL):
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    assert got.shape == want.shape, name
    err = np.abs(got - want)
    bar = abs_bar(want) + rtol * np.abs(want)
    bad = err > bar
    assert not bad.any(), (f"{name}: {int(bad.sum())} of {want.size} outside rel {rtol:g} / abs {abs_bar(want):.3g}; "
                           f"max err {err.max():.3e} at |ref| {np.abs(want)[err.argmax()]:.3e}, max |ref| {np.abs(want).max():.3e}")
