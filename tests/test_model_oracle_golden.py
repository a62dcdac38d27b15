"""The model-level oracle against logits and greedy tokens of the reference's own SPS and
Reverse-SPS models (tests/golden/make_golden.py::model_cases).  CPU only."""

import numpy as np
import pytest
import torch

from oracle import sps_model_oracle as mo
from tests.golden.loader import load_golden

G = load_golden()
TAGS = {"sps": "sps", "sps_w5": "sps", "rsps": "reverse_sps", "ds": "delayed_state"}


def golden_model(tag):
    """(weights, dims) of one committed reference model."""
    d = [int(x) for x in G[f"model_{tag}_dims"]]
    dims = mo.Dims(block_size=d[0], vocab_size=d[1], n_layer=d[2], n_head=d[3], hidden_size=d[4],
                   intermediate_size=d[5], eos_token_id=d[6], pad_token_id=d[7], predict_token_id=d[8],
                   window_size=d[9])
    prefix = f"model_{tag}_w__"
    weights = {k[len(prefix):]: torch.from_numpy(np.asarray(v)) for k, v in G.items() if k.startswith(prefix)}
    return weights, dims


@pytest.mark.parametrize("tag", list(TAGS))
def test_dense_logits_match_reference_forward(tag):
    weights, dims = golden_model(tag)
    idx = torch.from_numpy(G[f"model_{tag}_dense_idx"])
    # the reference's dense forward rounds q, k, v to bf16 (sps/core.py:53-55); the fixture's
    # attention stand-in returned fp32, so the output is not rounded
    got = mo.logits(weights, dims, idx, variant=TAGS[tag], round_output=False)
    ref = torch.from_numpy(G[f"model_{tag}_dense_logits"])
    assert (got - ref).abs().max().item() < 2e-4


@pytest.mark.parametrize("tag", list(TAGS))
def test_fp32_logits_match_reference_stepwise_decode(tag):
    weights, dims = golden_model(tag)
    idx = torch.from_numpy(G[f"model_{tag}_dense_idx"])
    got = mo.logits(weights, dims, idx, variant=TAGS[tag], operand_dtype=torch.float32)
    ref = torch.from_numpy(G[f"model_{tag}_stepwise_logits"])
    assert (got - ref).abs().max().item() < 2e-4


@pytest.mark.parametrize("tag", list(TAGS))
def test_left_padded_logits_match_reference(tag):
    weights, dims = golden_model(tag)
    idx = torch.from_numpy(G[f"model_{tag}_padded_idx"])
    pos = mo.left_padded_positions(idx, dims.pad_token_id)
    got = mo.logits(weights, dims, idx, variant=TAGS[tag], positions=pos, operand_dtype=torch.float32)
    ref = torch.from_numpy(G[f"model_{tag}_padded_logits"])
    real = idx != dims.pad_token_id
    assert (got - ref)[real].abs().max().item() < 2e-4
    assert ref[~real].abs().max().item() == 0.0     # the reference returns zeros at pad positions


@pytest.mark.parametrize("tag", list(TAGS))
def test_greedy_tokens_match_reference(tag):
    weights, dims = golden_model(tag)
    idx = torch.from_numpy(G[f"model_{tag}_padded_idx"])
    ref = torch.from_numpy(G[f"model_{tag}_greedy"])
    n_new = ref.shape[1] - idx.shape[1]
    got, margins = mo.generate(weights, dims, idx, n_new, variant=TAGS[tag], stop_on_eos=False,
                               operand_dtype=torch.float32, return_margins=True)
    assert torch.equal(got, ref)
    assert np.allclose(margins.numpy(), G[f"model_{tag}_greedy_margin"], atol=1e-3)


def test_document_ids_known_answer():
    # model.py:67-99 on a left-padded row with an EOS inside
    idx = torch.tensor([[62, 62, 11, 63, 12, 13], [21, 22, 23, 24, 25, 26]])
    doc = mo.document_idx(idx, eos=63, pad=62)
    assert doc.tolist() == [[0, 1, 2, 2, 3, 3], [0, 0, 0, 0, 0, 0]]
    assert mo.left_padded_positions(idx, 62).tolist() == [[0, 0, 0, 1, 2, 3], [0, 1, 2, 3, 4, 5]]


E, P = 63, 62   # EOS and pad ids used below

# (token ids, document ids): the known answers of the reference's tests/core/test_document_idx.py
DOC_ID_CASES = [
    ([[1, 2, 3, 4, 5, 6, 7, 8, 9, 10]], [[0] * 10]),                                    # :22-31
    ([[1, 2, 3, E, 4, 5, 6, 7, 8, 9]], [[0, 0, 0, 0, 1, 1, 1, 1, 1, 1]]),               # :34-43 EOS closes its document
    ([[1, 2, E, 3, 4, E, 5, 6, 7, 8]], [[0, 0, 0, 1, 1, 1, 2, 2, 2, 2]]),               # :46-55
    ([[E, 1, 2, 3, 4]], [[0, 1, 1, 1, 1]]),                                             # :58-67 EOS first
    ([[1, 2, 3, 4, E]], [[0, 0, 0, 0, 0]]),                                             # :69-72 EOS last
    ([[1, E, E, E, 2, 3]], [[0, 0, 1, 2, 3, 3]]),                                       # :75-84 consecutive EOS
    ([[1, 2, E, 3, 4, 5, 6, 7, 8, 9], [1, E, 2, 3, E, 4, 5, 6, 7, 8], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]],
     [[0, 0, 0, 1, 1, 1, 1, 1, 1, 1], [0, 0, 1, 1, 1, 2, 2, 2, 2, 2], [0] * 10]),       # :87-103 batch
    ([[P, P, 1, 2, E, 3, 4]], [[0, 1, 2, 2, 2, 3, 3]]),                                 # :105-115 left padding
]


@pytest.mark.parametrize("case", range(len(DOC_ID_CASES)))
def test_document_ids_match_the_reference_known_answers(case):
    """Oracle and the package's host function against the literal tensors of the reference's tests."""
    from sps_b200.generation import left_padded_document_idx
    idx, want = (torch.tensor(x) for x in DOC_ID_CASES[case])
    assert torch.equal(mo.document_idx(idx, eos=E, pad=P), want)
    assert torch.equal(left_padded_document_idx(idx, E, P), want)


def test_standard_model_logits_and_greedy_tokens_match_reference():
    """The Standard model (no <predict> rows): prefill logits over left-padded prompts with an EOS
    inside, its cached greedy decode, and a prompt that ends on EOS."""
    weights, dims = golden_model("std")
    idx = torch.from_numpy(G["model_std_padded_idx"])
    pos = mo.left_padded_positions(idx, dims.pad_token_id)
    got = mo.logits(weights, dims, idx, variant="standard", positions=pos, operand_dtype=torch.float32)
    ref = torch.from_numpy(G["model_std_padded_logits"])
    real = idx != dims.pad_token_id
    assert (got - ref)[real].abs().max().item() < 2e-4
    want = torch.from_numpy(G["model_std_greedy"])
    out, margins = mo.generate(weights, dims, idx, 8, variant="standard", stop_on_eos=False,
                               operand_dtype=torch.float32, return_margins=True)
    assert torch.equal(out, want)
    assert np.allclose(margins.numpy(), G["model_std_greedy_margin"], atol=1e-3)
    ends = torch.from_numpy(G["model_std_eos_end_idx"])
    out2 = mo.generate(weights, dims, ends, 5, variant="standard", stop_on_eos=False, operand_dtype=torch.float32)
    assert torch.equal(out2, torch.from_numpy(G["model_std_eos_end_greedy"]))
