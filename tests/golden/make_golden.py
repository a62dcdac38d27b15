"""Generate tests/golden/reference_vectors.npz and reference_grad_vectors.npz (``--grads-only``
writes just the second) from the reference's own CPU oracles.

Run once, in a container that has the reference checkout (it cannot travel to
another machine, so the vectors are committed):

    REFERENCE_ROOT=/path/to/reference python tests/golden/make_golden.py

It imports, unmodified, from the reference:
  * ``_sdpa_reference_attention_sps``      src/modeling/tests/attention/triton/test_sps_attention.py:25-74
  * ``_reference_persistent_key_window_attention``
                                            src/modeling/tests/models/attention/test_persistent_key_window.py:14-51
  * ``_pytorch_reference_attention``       src/modeling/tests/attention/triton/test_full_flash_attention.py:29-59
  * ``_reference_q2_attention``            src/modeling/tests/models/attention/test_segmented_q2_attention.py:25-62
  * ``masked_kv_attention`` (SDPA path)    src/modeling/models/utils/decode_attention.py:597-704
  * ``window_score_mod_factory``           src/modeling/tests/_sliding_window_reference.py:15-34
  * the eager cache update methods         src/modeling/models/reverse_sps/inference.py:137-167, :240-268
    and the prefill -> decode hand-over     src/modeling/models/reverse_sps/inference.py:568-613
    through the reference's own tiny Delayed-State / SPS test models.
  * ``apply_rotary_emb``, ``precompute_freqs_cis``  src/modeling/models/model.py:134-230
  * the Standard ``Model`` (src/modeling/models/full_attention_model.py): prefill logits and its
    own cached greedy ``generate`` on CPU.
  * ``SPSModel`` / ``ReverseSPSModel`` / ``DelayedStateModel`` themselves (src/modeling/models/sps/, reverse_sps/): dense
    ``forward`` (its attention name rebound to the SDPA oracle above, since the Triton kernel needs
    a GPU), stepwise ``forward_efficient`` (with the eager cache updates) and greedy tokens
    obtained the way tests/models/sps/test_dense_only.py:212-249 obtains them.

Every case stores its inputs (bf16/fp16 values widened to fp32, integer tensors
as int64) next to the reference output so the tests need nothing but numpy.
"""

from __future__ import annotations

import math
import os
import sys

sys.dont_write_bytecode = True
REF = os.environ.get("REFERENCE_ROOT")
if not REF:
    raise SystemExit("set REFERENCE_ROOT to the checkout of the reference project")
sys.path[:0] = [os.path.join(REF, "src"), REF]

import numpy as np
import torch

from modeling.models.utils.decode_attention import KVSegment, masked_kv_attention
from modeling.tests._sliding_window_reference import window_score_mod_factory
from modeling.tests.attention.triton.test_full_flash_attention import _pytorch_reference_attention
from modeling.tests.attention.triton.test_sps_attention import _sdpa_reference_attention_sps
from modeling.tests.models.attention.test_persistent_key_window import (
    _reference_persistent_key_window_attention,
)
from modeling.tests.models.attention.test_segmented_q2_attention import _reference_q2_attention

OUT = {}


def put(name, t, half=False):
    """Store one array; floats that are exactly bf16-representable are stored as
    their 16-bit patterns under ``<name>__bf16`` (tests/golden/loader.py widens them);
    ``half`` stores a float tensor rounded to fp16 under ``<name>__f16`` (gradients, which are
    compared at 4e-2)."""
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu()
        if t.is_floating_point():
            t = t.float()
            if half:
                OUT[name + "__f16"] = t.half().numpy()
                return
            if t.numel() > 64 and torch.equal(t.bfloat16().float(), t):
                OUT[name + "__bf16"] = t.bfloat16().view(torch.int16).numpy().view(np.uint16)
                return
            t = t.numpy()
        else:
            t = t.long().numpy()
    OUT[name] = np.asarray(t)


def geometric_docs(batch, t, mean, seed):
    rng = np.random.default_rng(seed)
    rows = []
    for _ in range(batch):
        ids, d = [], 0
        while len(ids) < t:
            ids += [d] * int(rng.geometric(1.0 / mean))
            d += 1
        rows.append(ids[:t])
    return torch.tensor(rows, dtype=torch.long).repeat_interleave(2, dim=1)


def sps_cases():
    # the reference's own kernel-parity case (test_sps_attention.py:77-131)
    for tag, with_docs in (("nodoc", False), ("doc", True)):
        torch.manual_seed(17)
        b, h, t, d, w = 1, 2, 16, 64, 3
        q, k, v = (torch.randn(b, h, 2 * t, d).bfloat16().float() for _ in range(3))
        docs = None
        if with_docs:
            docs = torch.tensor([[0] * 6 + [1] * 8 + [2] * 2]).repeat_interleave(2, dim=1)
            put(f"sps_{tag}_docs", docs)
        put(f"sps_{tag}_q", q), put(f"sps_{tag}_k", k), put(f"sps_{tag}_v", v)
        put(f"sps_{tag}_w", np.int64(w))
        put(f"sps_{tag}_out", _sdpa_reference_attention_sps(q, k, v, w, documents_idx_BxT=docs))
    # ragged / odd sizes: 2T in {8, 24, 200}, several windows, packed documents
    for n, w, mean, seed in ((8, 1, 3, 1), (24, 2, 5, 2), (200, 7, 30, 3), (384, 64, 60, 4)):
        g = torch.Generator().manual_seed(100 + n)
        q, k, v = (torch.randn(2, 2, n, 64, generator=g).bfloat16().float() for _ in range(3))
        docs = geometric_docs(2, n // 2, mean, seed)
        tag = f"sps_n{n}"
        put(f"{tag}_q", q), put(f"{tag}_k", k), put(f"{tag}_v", v), put(f"{tag}_docs", docs)
        put(f"{tag}_w", np.int64(w))
        put(f"{tag}_out", _sdpa_reference_attention_sps(q, k, v, w, documents_idx_BxT=docs))
    # the CPU-runnable benchmark shape: [2,8,512,64] fp32, w=64, documents ~ Geometric(mean 100);
    # inputs are regenerated from the seed by the test, only 2 heads of output are kept
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 8, 512, 64, generator=g) for _ in range(3))
    docs = geometric_docs(2, 256, 100, 0)
    out = _sdpa_reference_attention_sps(q, k, v, 64, documents_idx_BxT=docs)
    put("sps_cfg0_docs", docs)
    put("sps_cfg0_q_checksum", q.double().sum() + 2 * k.double().sum() + 3 * v.double().sum())
    put("sps_cfg0_out_h0h5", out[:, [0, 5]])


def persistent_window_cases():
    # test_persistent_key_window.py:54-98, both parities (fp16 inputs)
    for rem in (0, 1):
        torch.manual_seed(0)
        q = torch.randn(1, 1, 8, 64).half().float()
        k, v = torch.randn_like(q).half().float(), torch.randn_like(q).half().float()
        out = _reference_persistent_key_window_attention(
            q, k, v, persistent_key_window=1, persistent_key_remainder=rem, temporary_key_window=8)
        put(f"pkw{rem}_q", q), put(f"pkw{rem}_k", k), put(f"pkw{rem}_v", v), put(f"pkw{rem}_out", out)
    # a larger one with a real temporary window as well
    for rem in (0, 1):
        g = torch.Generator().manual_seed(7 + rem)
        q, k, v = (torch.randn(1, 2, 96, 64, generator=g).bfloat16().float() for _ in range(3))
        out = _reference_persistent_key_window_attention(
            q, k, v, persistent_key_window=5, persistent_key_remainder=rem, temporary_key_window=2)
        put(f"pkwL{rem}_q", q), put(f"pkwL{rem}_k", k), put(f"pkwL{rem}_v", v), put(f"pkwL{rem}_out", out)


def full_cases():
    for n, d, seed in ((128, 64, 5), (200, 128, 6)):
        g = torch.Generator().manual_seed(seed)
        q, k, v = (torch.randn(2, 2, n, d, generator=g).bfloat16().float() for _ in range(3))
        docs = geometric_docs(2, n, 40, seed)[:, ::2].contiguous()
        tag = f"full_n{n}"
        put(f"{tag}_q", q), put(f"{tag}_k", k), put(f"{tag}_v", v), put(f"{tag}_docs", docs)
        put(f"{tag}_out", _pytorch_reference_attention(q, k, v, 1.0 / math.sqrt(d), docs))
        put(f"{tag}_out_nodoc", _pytorch_reference_attention(q, k, v, 1.0 / math.sqrt(d), None))


def decode_cases():
    # test_segmented_q2_attention.py:65-117 on CPU tensors
    for tag in ("shared", "empty"):
        torch.manual_seed(123)
        bsz, nh, hd = 2, 3, 16
        q = torch.randn(bsz, 2, nh, hd).bfloat16()
        k0 = torch.randn(bsz, nh, 7, hd).bfloat16()
        v0 = torch.randn_like(k0)
        k1 = torch.randn(bsz, nh, 11, hd).bfloat16()
        v1 = torch.randn_like(k1)
        if tag == "empty":
            len0, cap0 = torch.zeros((bsz,), dtype=torch.long), 0
        else:
            len0, cap0 = torch.tensor([2, 5]), 5
        len1 = torch.tensor([[1, 3, 6], [2, 4, 7]])
        segs = [KVSegment(k0, v0, len0, max_len_cap=cap0), KVSegment(k1, v1, len1, max_len_cap=8)]
        cnk = torch.randn(bsz, nh, hd).bfloat16()
        cnv, cpk, cpv = torch.randn_like(cnk), torch.randn_like(cnk), torch.randn_like(cnk)
        out = _reference_q2_attention(q, segs, current_normal_k_BxHxD=cnk, current_normal_v_BxHxD=cnv,
                                      current_predict_k_BxHxD=cpk, current_predict_v_BxHxD=cpv)
        for nm, t in (("q", q), ("k0", k0), ("v0", v0), ("k1", k1), ("v1", v1), ("len0", len0),
                      ("len1", len1), ("cnk", cnk), ("cnv", cnv), ("cpk", cpk), ("cpv", cpv),
                      ("out", out)):
            put(f"q2_{tag}_{nm}", t)
        put(f"q2_{tag}_cap0", np.int64(cap0))
        # the reference's own SDPA fallback, one query at a time, must agree with it
        o0 = masked_kv_attention(q[:, 0].float(), segs, extra_kv=[(cnk, cnv)], attn_dtype=torch.float32)
        o1 = masked_kv_attention(q[:, 1].float(), segs, extra_kv=[(cnk, cnv), (cpk, cpv)],
                                 attn_dtype=torch.float32)
        put(f"q2_{tag}_sdpa", torch.stack([o0, o1], dim=1))
    # a q=1 case with three segments and head_dim 64 (Standard decode / stepwise prefill shape)
    g = torch.Generator().manual_seed(9)
    bsz, nh, hd = 3, 4, 64
    q = torch.randn(bsz, nh, hd, generator=g).bfloat16()
    segs, names = [], []
    for i, (cap, per_head) in enumerate(((40, False), (9, True), (300, True))):
        kk = torch.randn(bsz, nh, cap, hd, generator=g).bfloat16()
        vv = torch.randn(bsz, nh, cap, hd, generator=g).bfloat16()
        shape = (bsz, nh) if per_head else (bsz,)
        ln = torch.randint(0, cap + 1, shape, generator=g)
        segs.append(KVSegment(kk, vv, ln))
        put(f"q1_k{i}", kk), put(f"q1_v{i}", vv), put(f"q1_len{i}", ln)
    ek = torch.randn(bsz, nh, hd, generator=g).bfloat16()
    ev = torch.randn(bsz, nh, hd, generator=g).bfloat16()
    put("q1_q", q), put("q1_ek", ek), put("q1_ev", ev)
    put("q1_out", masked_kv_attention(q.float(), [KVSegment(s.k.float(), s.v.float(), s.lengths) for s in segs],
                                      extra_kv=[(ek.float(), ev.float())], attn_dtype=torch.float32))


def visibility_cases():
    # tests/models/reverse_sps/test_forward_efficient.py:130-156: which normal (even) keys a
    # query sees under the odd-persistent rule, straight from the reference's score modifier
    t = 5
    for w in (0, 1, 2):
        mod = window_score_mod_factory(window_size=w)
        vis = np.zeros((2 * t, 2 * t), dtype=np.int64)
        for qi in range(2 * t):
            for ki in range(qi + 1):
                s = mod(torch.tensor(0.0), torch.tensor(0), torch.tensor(0),
                        torch.tensor(qi), torch.tensor(ki))
                vis[qi, ki] = int(torch.isfinite(s))
        put(f"vis_reverse_w{w}", vis)


def kv_update_cases():
    from modeling.tests.models.delayed_state.test_forward_efficient import _make_delayed_state_model
    torch.manual_seed(11)
    w, steps, bsz, max_tokens = 3, 7, 3, 8
    model = _make_delayed_state_model(window_size=w)
    nh = model.config.n_head
    hd = model.config.hidden_size // nh
    state = model._build_decode_state(batch_size=bsz, max_tokens=max_tokens, device=torch.device("cpu"),
                                      attn_dtype=torch.float32)
    seq = []
    for step in range(steps):
        kw, vw = torch.randn(bsz, nh, hd), torch.randn(bsz, nh, hd)
        kr, vr = torch.randn(bsz, nh, hd), torch.randn(bsz, nh, hd)
        active = torch.tensor([True, step % 3 != 1, step < 4])
        model._update_normal_memory_unfused(state, 0, kw, vw, active)
        model._update_predict_memory_unfused(state, 0, kr, vr, active)
        seq.append((kw, vw, kr, vr, active.long()))
    for i, nm in enumerate(("kw", "vw", "kr", "vr", "active")):
        put(f"kvu_{nm}", torch.stack([s[i] for s in seq]))
    put("kvu_window", np.int64(w))
    put("kvu_nw_k", state.normal_window.k[0]), put("kvu_nw_v", state.normal_window.v[0])
    put("kvu_nw_len", state.normal_window.len[0]), put("kvu_nw_pos", state.normal_window.pos[0])
    put("kvu_br_k", state.predict_retained.k[0]), put("kvu_br_v", state.predict_retained.v[0])
    put("kvu_br_len", state.predict_retained.len[0])


def cache_fill_cases():
    """The reference's own hand-over (reverse_sps/inference.py:568-613) on its tiny SPS and
    Delayed-State test models: left padding, a finished earlier document, a one-token document."""
    from modeling.tests.models.delayed_state.test_forward_efficient import _make_delayed_state_model
    from modeling.tests.models.sps.test_dense_only import _make_sps_model
    for tag, make, w in (("ds", lambda: _make_delayed_state_model(window_size=3), 3),
                         ("sps", _make_sps_model, 2)):
        torch.manual_seed(21)
        bsz, t = 4, 9
        model = make()
        nh = model.config.n_head
        hd = model.config.hidden_size // nh
        state = model._build_decode_state(batch_size=bsz, max_tokens=t + 2, device=torch.device("cpu"),
                                          attn_dtype=torch.float32)
        k = torch.randn(bsz, 2 * t, nh, hd).bfloat16().float()
        v = torch.randn(bsz, 2 * t, nh, hd).bfloat16().float()
        mask = torch.zeros(bsz, t, dtype=torch.bool)
        mask[0, :] = True
        mask[1, 4:] = True
        mask[2, -1] = True
        mask[3, 2:4] = True
        model._materialize_prefill_layer_state(state, 0, k, v, mask)
        put(f"fill_{tag}_k", k), put(f"fill_{tag}_v", v), put(f"fill_{tag}_mask", mask.long())
        put(f"fill_{tag}_window", np.int64(w))
        put(f"fill_{tag}_slots", np.array([model._retained_slot_index, model._window_slot_index]))
        put(f"fill_{tag}_br_k", state.predict_retained.k[0]), put(f"fill_{tag}_br_v", state.predict_retained.v[0])
        put(f"fill_{tag}_br_len", state.predict_retained.len[0])
        put(f"fill_{tag}_nw_k", state.normal_window.k[0]), put(f"fill_{tag}_nw_v", state.normal_window.v[0])
        put(f"fill_{tag}_nw_len", state.normal_window.len[0]), put(f"fill_{tag}_nw_pos", state.normal_window.pos[0])


def rope_cases():
    """apply_rotary_emb + the bf16 operand cast, exactly as the attention modules chain them."""
    from modeling.models.model import apply_rotary_emb, precompute_freqs_cis
    g = torch.Generator().manual_seed(31)
    B, N, H, D = 2, 12, 3, 16
    fc = precompute_freqs_cis(D, 40)
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        xq = torch.randn(B, N, H, D, generator=g).to(dt)
        xk = torch.randn(B, N, H, D, generator=g).to(dt)
        pos = torch.arange(N // 2).repeat_interleave(2)                      # doubled sequence: shared positions
        q1, k1 = apply_rotary_emb(xq, xk, freqs_cis=fc[pos])
        per_seq = torch.stack([fc[pos], fc[pos + 7]])                        # [B, N, D/2]: left-padded batches
        q2, k2 = apply_rotary_emb(xq, xk, freqs_cis=per_seq)
        put(f"rope_{tag}_xq", xq), put(f"rope_{tag}_xk", xk)
        put(f"rope_{tag}_q1", q1.to(torch.bfloat16)), put(f"rope_{tag}_k1", k1.to(torch.bfloat16))
        put(f"rope_{tag}_q2", q2.to(torch.bfloat16)), put(f"rope_{tag}_k2", k2.to(torch.bfloat16))
    OUT["rope_freqs"] = torch.view_as_real(fc).numpy()
    put("rope_pos", pos)


def model_cases():
    """Logits and greedy tokens of the reference's own tiny SPS and Reverse-SPS models on CPU fp32
    (sizes of tests/models/sps/test_dense_only.py:13, head_dim 64), weights included."""
    import types
    import modeling.models.sps.core as sps_core
    import modeling.models.reverse_sps.core as rsps_core
    from modeling.models.delayed_state import DelayedStateConfig, DelayedStateModel
    from modeling.models.reverse_sps import ReverseSPSConfig, ReverseSPSModel
    from modeling.models.reverse_sps.inference import ReverseSPSInferenceMixin as Mixin
    from modeling.models.sps import SPSConfig, SPSModel

    def sps_attn(q, k, v, sm_scale, temporary_key_window, warp_specialize=True, documents_idx_BxT=None,
                 persistent_key_window=None):
        assert persistent_key_window is None
        return _sdpa_reference_attention_sps(q.float(), k.float(), v.float(), temporary_key_window,
                                             documents_idx_BxT)

    def rsps_attn(q, k, v, sm_scale, temporary_key_window, warp_specialize=True, documents_idx_BxT=None,
                  persistent_key_window=None):
        # this oracle has no document argument: only single-document rows go through it
        assert persistent_key_window is None
        assert documents_idx_BxT is None or bool((documents_idx_BxT == documents_idx_BxT[:, :1]).all())
        return _reference_persistent_key_window_attention(
            q.float(), k.float(), v.float(), temporary_key_window=temporary_key_window,
            persistent_key_window=2 * q.shape[2], persistent_key_remainder=1)

    sps_core.triton_sps_sliding_attention = sps_attn
    rsps_core.triton_reverse_sps_sliding_attention = rsps_attn
    for tag, cfg_cls, model_cls, w in (("sps", SPSConfig, SPSModel, 2), ("sps_w5", SPSConfig, SPSModel, 5),
                                       ("rsps", ReverseSPSConfig, ReverseSPSModel, 3),
                                       ("ds", DelayedStateConfig, DelayedStateModel, 3)):
        torch.manual_seed(41)
        cfg = cfg_cls(block_size=32, vocab_size=64, n_layer=2, n_head=2, hidden_size=128,
                      intermediate_size=256, dropout=0.0, bias=False, eos_token_id=63, pad_token_id=62,
                      predict_token_id=61, window_size=w, enable_triton_attention=True,
                      warp_specialize=False)
        model = model_cls(cfg).eval()
        # larger weights than the 0.02 init so that logits are not near-ties; bf16-representable
        # so that a bf16 run starts from identical parameters
        with torch.no_grad():
            for prm in model.parameters():
                if prm.dim() >= 2:
                    prm.mul_(6.0)
                prm.copy_(prm.bfloat16().float())
        model._update_normal_memory = types.MethodType(Mixin._update_normal_memory_unfused, model)
        model._update_predict_memory = types.MethodType(Mixin._update_predict_memory_unfused, model)
        for name, t in model.state_dict().items():
            put(f"model_{tag}_w__{name}", t)
        put(f"model_{tag}_dims", np.array([cfg.block_size, cfg.vocab_size, cfg.n_layer, cfg.n_head,
                                            cfg.hidden_size, cfg.intermediate_size, cfg.eos_token_id,
                                            cfg.pad_token_id, cfg.predict_token_id, cfg.window_size]))
        eos, pad = cfg.eos_token_id, cfg.pad_token_id
        g = torch.Generator().manual_seed(43)
        dense_idx = torch.randint(0, 60, (2, 12), generator=g)
        if tag not in ("rsps", "ds"):
            dense_idx[1, 4] = eos
        put(f"model_{tag}_dense_idx", dense_idx)
        put(f"model_{tag}_dense_logits", model(dense_idx))
        put(f"model_{tag}_stepwise_logits", model.forward_efficient(dense_idx))
        padded = torch.randint(0, 60, (3, 10), generator=g)
        padded[0, :3] = pad
        padded[1, 5] = eos
        padded[2, :6] = pad
        padded[2, 7] = eos
        put(f"model_{tag}_padded_idx", padded)
        put(f"model_{tag}_padded_logits", model.forward_efficient(padded))
        seq = padded.clone()
        margins = []
        for _ in range(8):
            z = model.forward_efficient(seq)[:, -1, :].clone()
            z[:, cfg.predict_token_id] = float("-inf")
            z[:, cfg.pad_token_id] = float("-inf")
            top2 = z.topk(2, dim=-1).values
            margins.append(top2[:, 0] - top2[:, 1])
            seq = torch.cat([seq, z.argmax(dim=-1, keepdim=True)], dim=1)
        put(f"model_{tag}_greedy", seq)
        OUT[f"model_{tag}_greedy_margin"] = torch.stack(margins, dim=1).numpy()


def standard_model_cases():
    """The reference's Standard model (full_attention_model.py) on CPU fp32: logits of its
    generation prefill path over left-padded prompts with an EOS inside, and its own greedy
    ``generate`` (cached decode), weights included."""
    from modeling.models.full_attention_model import Model, ModelConfig
    torch.manual_seed(47)
    cfg = ModelConfig(block_size=32, vocab_size=64, n_layer=2, n_head=2, hidden_size=128,
                      intermediate_size=256, dropout=0.0, bias=False, eos_token_id=63, pad_token_id=62)
    model = Model(cfg).eval()
    with torch.no_grad():
        for prm in model.parameters():
            if prm.dim() >= 2:
                prm.mul_(6.0)
            prm.copy_(prm.bfloat16().float())
    for name, t in model.state_dict().items():
        put(f"model_std_w__{name}", t)
    put("model_std_dims", np.array([cfg.block_size, cfg.vocab_size, cfg.n_layer, cfg.n_head, cfg.hidden_size,
                                     cfg.intermediate_size, cfg.eos_token_id, cfg.pad_token_id, -1, 0]))
    g = torch.Generator().manual_seed(53)
    padded = torch.randint(0, 60, (3, 10), generator=g)
    padded[0, :3] = cfg.pad_token_id
    padded[1, 5] = cfg.eos_token_id
    padded[2, :6] = cfg.pad_token_id
    padded[2, 7] = cfg.eos_token_id
    put("model_std_padded_idx", padded)
    hidden, _ = model._forward_generation_hidden_states(padded)
    put("model_std_padded_logits", model.lm_head(hidden))
    out = model.generate(padded, 8, do_sample=False, stop_on_eos=False)
    put("model_std_greedy", out)
    margins = []
    for step in range(8):
        seq = out[:, : padded.shape[1] + step]
        z = model.lm_head(model._forward_generation_hidden_states(seq)[0])[:, -1].clone()
        z[:, cfg.pad_token_id] = float("-inf")
        top2 = z.topk(2, dim=-1).values
        margins.append(top2[:, 0] - top2[:, 1])
    OUT["model_std_greedy_margin"] = torch.stack(margins, dim=1).numpy()
    # a prompt that ends on EOS: the decode cache starts empty (full_attention_model.py:703-705)
    ends = torch.randint(0, 60, (2, 6), generator=g)
    ends[0, -1] = cfg.eos_token_id
    put("model_std_eos_end_idx", ends)
    put("model_std_eos_end_greedy", model.generate(ends, 5, do_sample=False, stop_on_eos=False))


def grad_cases():
    """dQ, dK, dV by autograd through the reference's own SDPA oracles, the way its backward tests
    obtain them (test_sps_attention.py:79-131, test_full_flash_attention.py:126-160)."""
    def grads(fn, q, k, v, g):
        qs = [t.clone().requires_grad_(True) for t in (q, k, v)]
        with torch.enable_grad():
            fn(*qs).backward(g)
        return [t.grad for t in qs]

    # the reference's own backward case and larger packed ones
    for tag, (b, h, n, d, w, mean, seed) in {
        "t16_nodoc": (1, 2, 32, 64, 3, 0, 17), "t16_doc": (1, 2, 32, 64, 3, -1, 17),
        "n200": (2, 2, 200, 64, 7, 30, 3), "n384": (1, 2, 384, 64, 64, 60, 4),
        "n256_d128": (1, 2, 256, 128, 16, 50, 5),
    }.items():
        gen = torch.Generator().manual_seed(1000 + seed + n)
        q, k, v, g = (torch.randn(b, h, n, d, generator=gen).bfloat16().float() for _ in range(4))
        docs = None
        if mean == -1:
            docs = torch.tensor([[0] * 6 + [1] * 8 + [2] * 2]).repeat_interleave(2, dim=1)
        elif mean > 0:
            docs = geometric_docs(b, n // 2, mean, seed)
        dq, dk, dv = grads(lambda a, b_, c: _sdpa_reference_attention_sps(a, b_, c, w, documents_idx_BxT=docs),
                           q, k, v, g)
        name = f"grad_sps_{tag}"
        put(f"{name}_q", q), put(f"{name}_k", k), put(f"{name}_v", v), put(f"{name}_do", g)
        put(f"{name}_w", np.int64(w))
        if docs is not None:
            put(f"{name}_docs", docs)
        put(f"{name}_dq", dq, True), put(f"{name}_dk", dk, True), put(f"{name}_dv", dv, True)
    # Standard model: causal + same document
    gen = torch.Generator().manual_seed(2024)
    q, k, v, g = (torch.randn(2, 2, 200, 64, generator=gen).bfloat16().float() for _ in range(4))
    docs = geometric_docs(2, 200, 40, 6)[:, ::2].contiguous()
    dq, dk, dv = grads(lambda a, b_, c: _pytorch_reference_attention(a, b_, c, 0.125, docs), q, k, v, g)
    put("grad_full_q", q), put("grad_full_k", k), put("grad_full_v", v), put("grad_full_do", g)
    put("grad_full_docs", docs), put("grad_full_dq", dq, True), put("grad_full_dk", dk, True), put("grad_full_dv", dv, True)
    # persistent window, both parities
    for rem in (0, 1):
        gen = torch.Generator().manual_seed(70 + rem)
        q, k, v, g = (torch.randn(1, 2, 96, 64, generator=gen).bfloat16().float() for _ in range(4))
        dq, dk, dv = grads(lambda a, b_, c: _reference_persistent_key_window_attention(
            a, b_, c, persistent_key_window=5, persistent_key_remainder=rem, temporary_key_window=2), q, k, v, g)
        name = f"grad_pkw{rem}"
        put(f"{name}_q", q), put(f"{name}_k", k), put(f"{name}_v", v), put(f"{name}_do", g)
        put(f"{name}_dq", dq, True), put(f"{name}_dk", dk, True), put(f"{name}_dv", dv, True)


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    grad_cases()
    gpath = os.path.join(here, "reference_grad_vectors.npz")
    np.savez_compressed(gpath, **OUT)
    print(f"wrote {gpath}: {len(OUT)} arrays, {os.path.getsize(gpath) / 1e6:.2f} MB")
    OUT.clear()
    if "--grads-only" in sys.argv:
        raise SystemExit(0)
    with torch.no_grad():
        sps_cases()
        persistent_window_cases()
        full_cases()
        decode_cases()
        visibility_cases()
        kv_update_cases()
        cache_fill_cases()
        rope_cases()
        model_cases()
        standard_model_cases()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(path, **OUT)
    print(f"wrote {path}: {len(OUT)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")
