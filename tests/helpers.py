"""Shared checks for the GPU parity tests."""
import numpy as np

# Tolerance of the attention outputs against the reference's fp32 CPU path.
MAX_ABS = 2e-3
REL_L2 = 1e-3


def assert_close(got, want, what="", max_abs=MAX_ABS, rel_l2=REL_L2):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - want).max()
    rel = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    assert err <= max_abs and rel <= rel_l2, f"{what}: max-abs {err:.3e} (limit {max_abs}), rel-L2 {rel:.3e} (limit {rel_l2})"
    return err, rel
