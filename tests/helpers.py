"""Comparison helpers shared by the parity tests."""
import numpy as np


def assert_exact(D, I, D_ref, I_ref):
    """Bit-exact distances and identical ids."""
    np.testing.assert_array_equal(I, I_ref)
    np.testing.assert_array_equal(D.view(np.uint32), D_ref.view(np.uint32))


def assert_close_gap_aware(D, I, D_ref, I_ref, rtol, what=""):
    """Distances within rtol (relative); ids identical wherever the reference gap to both
    neighbours in rank exceeds the tolerance (a tie within tolerance may swap ranks)."""
    assert D.shape == D_ref.shape and I.shape == I_ref.shape
    scale = np.maximum(np.abs(D_ref), 1e-30)
    pad = I_ref < 0
    err = np.abs(D - D_ref) / scale
    err[pad] = 0
    assert np.all((I < 0) == pad), f"{what}: padding differs"
    assert err.max() <= rtol, f"{what}: max relative distance error {err.max():.3e} > {rtol}"
    mism = (I != I_ref) & ~pad
    if mism.any():
        k = D_ref.shape[1]
        tol = rtol * np.abs(D_ref) * 2
        gap_prev = np.full_like(D_ref, np.inf)
        gap_next = np.full_like(D_ref, np.inf)
        gap_prev[:, 1:] = np.abs(D_ref[:, 1:] - D_ref[:, :-1])
        gap_next[:, :-1] = gap_prev[:, 1:]
        # the last rank competes with the (k+1)-th element, which the caller cannot see: allow it
        gap_next[:, k - 1] = 0
        clear = (gap_prev > tol) & (gap_next > tol)
        bad = mism & clear
        assert not bad.any(), f"{what}: {bad.sum()} ids differ where the distance gap exceeds tolerance"
