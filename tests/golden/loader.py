"""Loader for tests/golden/reference_vectors.npz (written by make_golden.py)."""

from __future__ import annotations

import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")


def load_golden() -> dict:
    """Return {name: ndarray}; arrays stored as bf16 bit patterns come back as fp32."""
    out = {}
    with np.load(_PATH) as z:
        for key in z.files:
            arr = z[key]
            if key.endswith("__bf16"):
                out[key[:-6]] = (arr.astype(np.uint32) << 16).view(np.float32)
            else:
                out[key] = arr
    return out
