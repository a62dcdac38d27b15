"""Loader for tests/golden/reference_vectors.npz (written by make_golden.py)."""

from __future__ import annotations

import os

import numpy as np

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")


_GRAD_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_grad_vectors.npz")


def load_golden(grads: bool = False) -> dict:
    """Return {name: ndarray}; arrays stored as bf16 bit patterns come back as fp32.
    ``grads`` selects the gradient vectors (reference_grad_vectors.npz)."""
    out = {}
    with np.load(_GRAD_PATH if grads else _PATH) as z:
        for key in z.files:
            arr = z[key]
            if key.endswith("__bf16"):
                out[key[:-6]] = (arr.astype(np.uint32) << 16).view(np.float32)
            elif key.endswith("__f16"):
                out[key[:-5]] = arr.astype(np.float32)
            else:
                out[key] = arr
    return out
