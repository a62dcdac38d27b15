"""The reference's own model classes running on these kernels: sps_b200.install() rebinds the
module-level names, then SPSModel / ReverseSPSModel / DelayedStateModel / the Standard model are
driven exactly as the reference's model tests drive them (src/modeling/tests/models/sps/
test_dense_only.py:226-285, :338-387): dense forward against stepwise forward_efficient, batched
generation prefill against stepwise, greedy generate against stepwise greedy, left-padding
invariance.  A second group runs the same model once on the reference's Triton kernels and once
on these and compares logits and gradients.

The reference package is read from baseline/_ref (a pip --target install of it that travels with
the repository snapshot); without it, or without Triton, the tests are skipped with that reason.
Needs a B200."""

import importlib
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ref():
    """The reference's model modules, importable, or a skip that says why not."""
    if not os.path.isdir(os.path.join(REF, "modeling", "models")):
        pytest.skip("unavailable on this box: baseline/_ref holds no install of the reference")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    try:
        mods = {name: importlib.import_module(f"modeling.models.{name}")
                for name in ("sps", "reverse_sps", "delayed_state", "full_attention_model")}
    except Exception as e:
        pytest.skip(f"unavailable on this box: the reference does not import ({e!r})")
    return mods


@pytest.fixture()
def installed(ref):
    """install(strict=True) for one test, the reference's own names restored afterwards."""
    inst = importlib.import_module("sps_b200.install")
    originals = {(m, a): getattr(importlib.import_module(m), a) for m, a, _ in inst._BINDINGS}
    done = inst.install(strict=True)
    assert len(done) == len(inst._BINDINGS)
    yield ref
    for (m, a), fn in originals.items():
        setattr(importlib.import_module(m), a, fn)


_FAMILY = {"sps": ("sps", "SPSConfig", "SPSModel"),
           "reverse_sps": ("reverse_sps", "ReverseSPSConfig", "ReverseSPSModel"),
           "delayed_state": ("delayed_state", "DelayedStateConfig", "DelayedStateModel")}


def _make(ref, family, seed, hidden=128, inter=256, n_head=2, window=2, block=32):
    mod, cfg_name, model_name = _FAMILY[family]
    cfg = getattr(ref[mod], cfg_name)(
        block_size=block, vocab_size=64, n_layer=2, n_head=n_head, hidden_size=hidden,
        intermediate_size=inter, dropout=0.0, bias=False, eos_token_id=63, pad_token_id=62,
        predict_token_id=61, window_size=window, enable_triton_attention=True, warp_specialize=False)
    torch.manual_seed(seed)
    model = getattr(ref[mod], model_name)(cfg)
    return model.eval().to(_dev())


def _greedy_next(model, idx):
    z = model.forward_efficient(idx)[:, -1, :].clone()
    z[:, model.config.predict_token_id] = float("-inf")
    z[:, model.config.pad_token_id] = float("-inf")
    return z.argmax(dim=-1, keepdim=True).to(idx.dtype)


@pytest.mark.parametrize("family", list(_FAMILY))
def test_dense_forward_matches_forward_efficient(installed, family):
    model = _make(installed, family, seed=2)
    eos = model.config.eos_token_id
    idx = torch.tensor([[4, 5, 6, 7], [8, eos, 9, 10]], dtype=torch.long, device=_dev())
    with torch.no_grad():
        dense = model(idx)
        stepwise = model.forward_efficient(idx)
    torch.testing.assert_close(dense, stepwise, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("family", list(_FAMILY))
def test_batched_generation_prefill_matches_forward_efficient(installed, family):
    model = _make(installed, family, seed=4)
    eos = model.config.eos_token_id
    dev = _dev()
    idx = torch.tensor([[4, 5, 6, 7], [8, eos, 9, 10]], dtype=torch.long, device=dev)
    on = torch.ones(2, device=dev, dtype=torch.bool)
    with torch.no_grad():
        state, next_logits, mode = model._prefill_generation_state(idx, max_new_tokens=2, require_batched=True)
        expected_next = model.forward_efficient(idx)[:, -1, :]
        z = next_logits.clone()
        z[:, model.config.predict_token_id] = float("-inf")
        z[:, model.config.pad_token_id] = float("-inf")
        tok = z.argmax(dim=-1).to(torch.long)
        decoded = model._decode_generation_state(state, tok, on)
        model._advance_decode_state(state, tok, on)
        expected_decoded = model.forward_efficient(torch.cat([idx, tok[:, None]], dim=1))[:, -1, :]
    assert mode == "batched_prefill"
    torch.testing.assert_close(next_logits, expected_next, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(decoded, expected_decoded, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("family", list(_FAMILY))
def test_generate_greedy_matches_stepwise(installed, family):
    model = _make(installed, family, seed=0)
    eos = model.config.eos_token_id
    prompt = torch.tensor([[5, eos, 7, 8]], dtype=torch.long, device=_dev())
    with torch.no_grad():
        generated = model.generate(prompt, max_new_tokens=3, do_sample=False)
        expected = prompt.clone()
        for _ in range(3):
            expected = torch.cat([expected, _greedy_next(model, expected)], dim=1)
    assert torch.equal(generated, expected)


def test_generate_left_padded_batch_matches_unpadded_rows(installed):
    model = _make(installed, "sps", seed=1)
    pad, eos = model.config.pad_token_id, model.config.eos_token_id
    prompts = torch.tensor([[pad, pad, 11, eos, 12, 13], [21, 22, 23, 24, 25, 26]], dtype=torch.long, device=_dev())
    with torch.no_grad():
        batched = model.generate(prompts, max_new_tokens=4, do_sample=False)
        for r, prompt in enumerate(prompts):
            first = int((prompt != pad).nonzero(as_tuple=False)[0].item())
            single = model.generate(prompt[first:].unsqueeze(0), max_new_tokens=4, do_sample=False)
            assert bool((batched[r, :first] == pad).all())
            assert torch.equal(batched[r, first:], single[0])


def test_standard_model_runs_on_the_bound_kernels(installed):
    """Standard model (full_attention_model.py): dense forward through full_attention, cached
    decode through masked_kv_attention; greedy generate against a dense re-forward per token, as
    src/modeling/tests/models/shared/test_full_attention_generation.py:20-44 compares them."""
    fam = installed["full_attention_model"]
    cfg = fam.ModelConfig(block_size=32, vocab_size=64, n_layer=2, n_head=2, hidden_size=128,
                          intermediate_size=256, dropout=0.0, bias=False, eos_token_id=63, pad_token_id=62,
                          use_triton_full_attention=True, warp_specialize=False)
    torch.manual_seed(5)
    model = fam.Model(cfg).eval().to(_dev())
    prompt = torch.tensor([[5, 63, 7, 8, 9]], dtype=torch.long, device=_dev())
    with torch.no_grad():
        generated = model.generate(prompt, max_new_tokens=3, do_sample=False)
        expected = prompt.clone()
        for _ in range(3):
            hidden, _ = model._forward_generation_hidden_states(expected)
            z = model.lm_head(hidden)[:, -1, :].float().clone()
            z[:, cfg.pad_token_id] = float("-inf")
            expected = torch.cat([expected, z.argmax(dim=-1, keepdim=True)], dim=1)
    assert torch.equal(generated, expected)


@pytest.mark.parametrize("family", ["sps", "reverse_sps"])
def test_same_model_on_reference_triton_kernels_and_on_these(ref, family):
    """One model, one batch: logits and parameter gradients with the reference's own Triton
    kernels bound, then with these kernels bound.  (If the reference's kernels cannot run on
    this box the test is skipped with the error, not failed: they are the other side of the
    comparison, not the product.)"""
    model = _make(ref, family, seed=7, hidden=256, inter=512, n_head=4, window=3, block=64)
    eos = model.config.eos_token_id
    g = torch.Generator().manual_seed(9)
    idx = torch.randint(0, 60, (2, 48), generator=g)
    idx[0, 13] = eos
    idx[1, 30] = eos
    idx = idx.to(_dev())

    def run():
        model.zero_grad(set_to_none=True)
        logits = model(idx)
        loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(),
                                                 idx[:, 1:].reshape(-1))
        loss.backward()
        grads = {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if p.grad is not None}
        return logits.detach().float(), grads

    try:
        ref_logits, ref_grads = run()
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"unavailable on this box: the reference's Triton kernels did not run ({e!r})")
    inst = importlib.import_module("sps_b200.install")
    originals = {(m, a): getattr(importlib.import_module(m), a) for m, a, _ in inst._BINDINGS}
    try:
        inst.install(strict=True)
        our_logits, our_grads = run()
        torch.cuda.synchronize()
    finally:
        for (m, a), fn in originals.items():
            setattr(importlib.import_module(m), a, fn)
    torch.testing.assert_close(our_logits, ref_logits, atol=3e-2, rtol=3e-2)
    assert set(our_grads) == set(ref_grads)
    for name, gr in ref_grads.items():
        scale = float(gr.abs().max()) + 1e-6
        err = float((our_grads[name] - gr).abs().max())
        assert err <= 4e-2 * scale + 1e-4, (name, err, scale)
