"""The gradient oracle (oracle.sps_oracle.prefill_attention_grads) against dQ, dK, dV obtained by
autograd through the reference's own SDPA oracles (tests/golden/make_golden.py: grad_cases)."""

import numpy as np
import pytest
import torch

from oracle import sps_oracle as orc
from tests.golden.loader import load_golden


@pytest.fixture(scope="module")
def grads():
    return load_golden(grads=True)


def _t(a):
    return torch.from_numpy(np.asarray(a))


SPS_TAGS = ["t16_nodoc", "t16_doc", "n200", "n384", "n256_d128"]


def _check(got, g, name):
    for x, key in zip(got, ("dq", "dk", "dv")):
        ref = _t(g[f"{name}_{key}"])
        # the stored gradients are rounded to fp16
        assert float((x - ref).abs().max()) <= 2e-3 + 2e-3 * float(ref.abs().max()), (name, key)


@pytest.mark.parametrize("tag", SPS_TAGS)
def test_sps_grads_match_reference_autograd(grads, tag):
    name = f"grad_sps_{tag}"
    q, k, v, g = (_t(grads[f"{name}_{x}"]) for x in ("q", "k", "v", "do"))
    docs = _t(grads[f"{name}_docs"]) if f"{name}_docs" in grads else None
    got = orc.prefill_attention_grads(q, k, v, g, 1.0 / np.sqrt(q.shape[-1]), persistent_parity=orc.PARITY_EVEN,
                                      temporary_window=int(grads[f"{name}_w"]), docs=docs)
    _check(got, grads, name)


def test_full_grads_match_reference_autograd(grads):
    q, k, v, g = (_t(grads[f"grad_full_{x}"]) for x in ("q", "k", "v", "do"))
    got = orc.prefill_attention_grads(q, k, v, g, 0.125, persistent_parity=orc.PARITY_NONE,
                                      docs=_t(grads["grad_full_docs"]))
    _check(got, grads, "grad_full")


@pytest.mark.parametrize("rem", [0, 1])
def test_persistent_window_grads_match_reference_autograd(grads, rem):
    name = f"grad_pkw{rem}"
    q, k, v, g = (_t(grads[f"{name}_{x}"]) for x in ("q", "k", "v", "do"))
    got = orc.prefill_attention_grads(q, k, v, g, 0.125, persistent_parity=rem, temporary_window=2,
                                      persistent_window=5)
    _check(got, grads, name)
