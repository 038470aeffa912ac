"""Shared comparison helpers for the parity tests."""
import numpy as np


def rel_err(a, b):
    """||a-b|| / ||b|| in float64 (b is the reference)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / (den if den > 0 else 1.0))


def max_rel_err(a, b):
    """max|a-b| / max|b|."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.abs(b).max()
    return float(np.abs(a - b).max() / (den if den > 0 else 1.0))


def assert_close(a, b, tol, what=""):
    r, m = rel_err(a, b), max_rel_err(a, b)
    assert r <= tol and m <= tol, f"{what}: rel {r:.3e} max-rel {m:.3e} > tol {tol:.1e}"


def checksum(*ts):
    import torch
    return np.array([float(t.double().sum()) for t in ts] + [float(t.double().abs().sum()) for t in ts])
