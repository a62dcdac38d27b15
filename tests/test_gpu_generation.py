"""The generation engine and the entry points it adds (decode step with the cache update folded in,
fused q/k/v rotary cast, block glue kernels) against the committed logits and greedy tokens of the
reference's own models, the model-level CPU oracle, and the separate calls they replace.
Needs a B200."""

import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import sps_model_oracle as mo
from oracle import sps_oracle as orc

TAGS = {"sps": "sps", "sps_w5": "sps", "rsps": "reverse_sps", "ds": "delayed_state"}


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


def _golden_model(golden, tag):
    d = [int(x) for x in golden[f"model_{tag}_dims"]]
    fields = dict(block_size=d[0], vocab_size=d[1], n_layer=d[2], n_head=d[3], hidden_size=d[4],
                  intermediate_size=d[5], eos_token_id=d[6], pad_token_id=d[7], predict_token_id=d[8],
                  window_size=d[9])
    prefix = f"model_{tag}_w__"
    weights = {k[len(prefix):]: torch.from_numpy(np.asarray(v)) for k, v in golden.items() if k.startswith(prefix)}
    return weights, fields


def _engine(weights, fields, variant, dtype):
    from sps_b200.generation import SPSDims, SPSGenerator
    return SPSGenerator(weights, SPSDims(**fields), variant=variant, device=_dev(), param_dtype=dtype)


# ----------------------------------------------------------------------------- glue kernels

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_add_rmsnorm_matches_the_reference_ops(dtype):
    from sps_b200 import _lib
    lib, dev = _lib.load(), _dev()
    g = torch.Generator(device=dev).manual_seed(3)
    rows, c, eps = 77, 2048, 1e-6
    x = torch.randn(rows, c, generator=g, device=dev).to(dtype)
    delta = torch.randn(rows, c, generator=g, device=dev).to(dtype)
    w = (1 + 0.1 * torch.randn(c, generator=g, device=dev)).to(dtype)
    # model.py:324-327 then :118-132, op by op in the parameter dtype
    x_ref = x + delta
    xf = x_ref.float()
    y_ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x_ref) * w
    xx, y = x.clone(), torch.empty_like(x)
    code = _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_FP32
    rc = lib.spsattn_add_rmsnorm(xx.data_ptr(), delta.data_ptr(), w.data_ptr(), y.data_ptr(), code, rows, c,
                                 eps, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "add_rmsnorm")
    assert torch.equal(xx, x_ref)                       # the residual add rounds like torch's
    if dtype == torch.float32:
        torch.testing.assert_close(y, y_ref, atol=1e-5, rtol=1e-5)
    else:
        # the sum of squares is accumulated in a different order: at most one bf16 step apart
        torch.testing.assert_close(y.float(), y_ref.float(), atol=0, rtol=2 ** -7)
        assert (y == y_ref).float().mean().item() > 0.99
    # without delta: x untouched
    x2, y2 = x.clone(), torch.empty_like(x)
    rc = lib.spsattn_add_rmsnorm(x2.data_ptr(), None, w.data_ptr(), y2.data_ptr(), code, rows, c, eps,
                                 torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "add_rmsnorm")
    assert torch.equal(x2, x)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu_matches_the_reference_ops(dtype):
    from sps_b200 import _lib
    lib, dev = _lib.load(), _dev()
    g = torch.Generator(device=dev).manual_seed(4)
    rows, inter = 50, 768
    gu = (2 * torch.randn(rows, 2 * inter, generator=g, device=dev)).to(dtype)
    ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]           # model.py:313-314
    y = torch.empty(rows, inter, device=dev, dtype=dtype)
    code = _lib.DTYPE_BF16 if dtype == torch.bfloat16 else _lib.DTYPE_FP32
    _lib.check(lib.spsattn_swiglu(gu.data_ptr(), y.data_ptr(), code, rows, inter,
                                  torch.cuda.current_stream().cuda_stream), "swiglu")
    if dtype == torch.float32:
        torch.testing.assert_close(y, ref, atol=1e-5, rtol=1e-5)
    else:
        torch.testing.assert_close(y.float(), ref.float(), atol=1e-30, rtol=2 ** -7)
        assert (y == ref).float().mean().item() > 0.99


def test_glue_rejects_bad_arguments():
    from sps_b200 import _lib
    lib, dev = _lib.load(), _dev()
    x = torch.zeros(4, 64, device=dev, dtype=torch.bfloat16)
    assert lib.spsattn_add_rmsnorm(x.data_ptr(), None, x.data_ptr(), x.data_ptr(), 1, 4, 64, 1e-6, None) == -1
    assert lib.spsattn_add_rmsnorm(x.data_ptr(), None, x.data_ptr(), x.data_ptr(), 0, 4, 60, 1e-6, None) == -3
    assert lib.spsattn_swiglu(None, x.data_ptr(), 0, 4, 32, None) == -1


# ----------------------------------------------------------------------------- fused rotary cast

@pytest.mark.parametrize("xdt", [torch.bfloat16, torch.float32])
def test_qkv_rope_cast_matches_oracle(xdt):
    from sps_b200 import _lib
    lib, dev = _lib.load(), _dev()
    g = torch.Generator().manual_seed(9)
    B, N, H, D = 3, 10, 4, 64
    c = H * D
    qkv = torch.randn(B, N, 3 * c, generator=g).to(xdt)
    pos = torch.randint(0, 50, (B, N), generator=g)
    fc = mo.freqs_cis(D, 64)[pos]                                         # [B, N, D/2] complex
    q, k, v = qkv.view(B, N, 3, H, D).unbind(2)
    ref = [orc.rope_cast(q, fc), orc.rope_cast(k, fc), orc.rope_cast(v, None)]   # [B, N, H, D] bf16
    x = qkv.to(dev)
    f = torch.view_as_real(fc).contiguous().to(dev)
    out = torch.empty(3, B, N, H, D, device=dev, dtype=torch.bfloat16)
    groups = (_lib.RopeGroup * 3)()
    for gi in range(3):
        groups[gi].out = out[gi].data_ptr()
        groups[gi].stride_b, groups[gi].stride_n, groups[gi].stride_h = N * c, c, D
        groups[gi].rotate = int(gi < 2)
    rc = lib.spsattn_qkv_rope_cast(x.data_ptr(), 0 if xdt == torch.bfloat16 else 2, N * 3 * c, 3 * c, D,
                                   f.data_ptr(), N * (D // 2), groups, 3, _lib.DTYPE_BF16, B, N, H, D,
                                   torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "qkv_rope_cast")
    for gi in range(3):
        assert torch.equal(out[gi].cpu(), ref[gi]), gi


# ----------------------------------------------------------------------------- decode step

def _step_case(seed, S, H, D, w, cap, ring_full):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    t = lambda *s: torch.randn(*s, generator=g).to(bf)
    case = dict(
        q=t(S, 2, H, D), k2=t(2, S, H, D), v2=t(2, S, H, D),
        nw_k=t(S, H, max(w, 1), D), nw_v=t(S, H, max(w, 1), D),
        br_k=t(S, H, cap, D), br_v=t(S, H, cap, D),
        nw_len=torch.full((S,), w, dtype=torch.long) if ring_full else torch.randint(0, w + 1, (S,), generator=g),
        nw_pos=torch.randint(0, max(w, 1), (S,), generator=g),
        br_len=torch.randint(0, cap + 1, (S, H), generator=g),      # cap itself: append out of bounds
        active=(torch.rand(S, generator=g) > 0.3).to(torch.int8))
    case["br_len"][0] = 0                                            # an empty retained cache
    return case


@pytest.mark.parametrize("D,w,ring_full,cap", [(64, 4, True, 37), (64, 4, False, 37), (128, 7, False, 37),
                                                (64, 0, False, 37), (64, 6, True, 333), (128, 5, False, 700)])
def test_decode_step_equals_attention_then_update(D, w, ring_full, cap):
    """spsattn_decode_step == spsattn_decode_fwd followed by spsattn_kv_update: same output
    (fp32 exactly, 16-bit as its rounding), same caches and counters bit for bit.  The larger
    capacities split a (sequence, head) over several blocks, some of them past the live length;
    both calls share one workspace, the second relying on the tickets the first left at zero."""
    import sps_b200
    from sps_b200 import _lib
    lib, dev = _lib.load(), _dev()
    S, H = 9, 3
    shared_ws = {}
    case = {k: v.to(dev) for k, v in _step_case(11 + D + w, S, H, D, w, cap, ring_full).items()}
    ws_slot, ret_slot = 1, 0
    # separate calls on copies
    a = {k: v.clone() for k, v in case.items()}
    segs = ([sps_b200.KVSegment(a["nw_k"], a["nw_v"], a["nw_len"], max_len_cap=min(w, cap))] if w > 0 else [])
    segs.append(sps_b200.KVSegment(a["br_k"], a["br_v"], a["br_len"], max_len_cap=cap))
    out_ref = sps_b200.triton_segmented_q2_attention(
        a["q"], segs, current_normal_k_BxHxD=a["k2"][0], current_normal_v_BxHxD=a["v2"][0],
        current_predict_k_BxHxD=a["k2"][1], current_predict_v_BxHxD=a["v2"][1], attn_dtype=torch.bfloat16)
    sps_b200.fused_sps_kv_update(
        nw_k=a["nw_k"], nw_v=a["nw_v"], nw_len=a["nw_len"], nw_pos=a["nw_pos"], br_k=a["br_k"], br_v=a["br_v"],
        br_len=a["br_len"], k_window_BxHxD=a["k2"][ws_slot], v_window_BxHxD=a["v2"][ws_slot],
        k_retained_BxHxD=a["k2"][ret_slot], v_retained_BxHxD=a["v2"][ret_slot],
        active_mask_B=a["active"], window_tokens=w)
    for out_dtype in (_lib.DTYPE_FP32, _lib.DTYPE_BF16):
        b = {k: v.clone() for k, v in case.items()}
        storage = max(w, 1)
        sarr = (_lib.Segment * 2)()
        n_seg = 0
        if w > 0:
            sg = sarr[n_seg]
            sg.k, sg.v = b["nw_k"].data_ptr(), b["nw_v"].data_ptr()
            sg.seq_offset, sg.seq_stride, sg.head_stride, sg.row_stride = None, H * storage * D, storage * D, D
            sg.lengths, sg.lengths_per_head, sg.max_rows, sg.query_mask = b["nw_len"].data_ptr(), 0, min(w, cap), 3
            n_seg += 1
        sg = sarr[n_seg]
        sg.k, sg.v = b["br_k"].data_ptr(), b["br_v"].data_ptr()
        sg.seq_offset, sg.seq_stride, sg.head_stride, sg.row_stride = None, H * cap * D, cap * D, D
        sg.lengths, sg.lengths_per_head, sg.max_rows, sg.query_mask = b["br_len"].data_ptr(), 1, cap, 3
        n_seg += 1
        ex = (_lib.Extra * 2)()
        ex[0].k, ex[0].v, ex[0].query_mask = b["k2"][0].data_ptr(), b["v2"][0].data_ptr(), 3
        ex[1].k, ex[1].v, ex[1].query_mask = b["k2"][1].data_ptr(), b["v2"][1].data_ptr(), 2
        ap = _lib.KvAppend()
        if w > 0:
            ap.nw_k, ap.nw_v = b["nw_k"].data_ptr(), b["nw_v"].data_ptr()
            ap.nw_len, ap.nw_pos = b["nw_len"].data_ptr(), b["nw_pos"].data_ptr()
        ap.br_k, ap.br_v, ap.br_len = b["br_k"].data_ptr(), b["br_v"].data_ptr(), b["br_len"].data_ptr()
        ap.k_window, ap.v_window = b["k2"][ws_slot].data_ptr(), b["v2"][ws_slot].data_ptr()
        ap.k_retained, ap.v_retained = b["k2"][ret_slot].data_ptr(), b["v2"][ret_slot].data_ptr()
        ap.active = b["active"].data_ptr()
        ap.window_storage, ap.retained_storage, ap.window_tokens = storage, cap, w
        ws_bytes = lib.spsattn_decode_step_workspace_bytes(S, H, D, 2, sarr, n_seg)
        if "ws" not in shared_ws:
            shared_ws["ws"] = torch.zeros(ws_bytes, device=dev, dtype=torch.uint8)   # tickets start at zero
        ws = shared_ws["ws"]
        out = torch.empty(S, 2, H, D, device=dev,
                          dtype=torch.float32 if out_dtype == _lib.DTYPE_FP32 else torch.bfloat16)
        rc = lib.spsattn_decode_step(b["q"].data_ptr(), 2, out.data_ptr(), out_dtype, sarr, n_seg, ex, 2,
                                     C.byref(ap), S, H, D, _lib.DTYPE_BF16, 1.0 / math.sqrt(D), ws.data_ptr(),
                                     ws_bytes, None, torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "decode_step")
        torch.cuda.synchronize()
        tickets = ws[ws_bytes - 256 * ((4 * (S * H + S) + 255) // 256):]
        assert int(tickets.count_nonzero()) == 0                        # left zero for the next call
        if out_dtype == _lib.DTYPE_FP32:
            assert torch.equal(out, out_ref)
        else:
            assert torch.equal(out, out_ref.to(torch.bfloat16))
        for name in ("nw_k", "nw_v", "nw_len", "nw_pos", "br_k", "br_v", "br_len"):
            assert torch.equal(a[name], b[name]), name
    # and the update against the oracle's integer rule
    o = {k: v.cpu().clone() for k, v in case.items()}
    orc.kv_update(o["nw_k"], o["nw_v"], o["nw_len"], o["nw_pos"], o["br_k"], o["br_v"], o["br_len"],
                  o["k2"][ws_slot], o["v2"][ws_slot], o["k2"][ret_slot], o["v2"][ret_slot], o["active"], w)
    for name in ("nw_k", "nw_v", "nw_len", "nw_pos", "br_k", "br_v", "br_len"):
        assert torch.equal(o[name], a[name].cpu()), name


def test_decode_step_rejects_bad_arguments():
    from sps_b200 import _lib
    lib, dev = _lib.load(), _dev()
    q = torch.zeros(2, 2, 2, 64, device=dev, dtype=torch.bfloat16)
    ln = torch.zeros(2, dtype=torch.long, device=dev)
    sarr = (_lib.Segment * 1)()
    sarr[0].k, sarr[0].v, sarr[0].lengths = q.data_ptr(), q.data_ptr(), ln.data_ptr()
    sarr[0].seq_stride, sarr[0].head_stride, sarr[0].row_stride, sarr[0].max_rows = 128, 64, 64, 1
    ws = torch.zeros(1 << 16, device=dev, dtype=torch.uint8)
    args = lambda out_dtype, ap, wsb: (q.data_ptr(), 2, q.data_ptr(), out_dtype, sarr, 1, None, 0, ap, 2, 2, 64,
                                       _lib.DTYPE_BF16, 0.125, ws.data_ptr(), wsb, None, None)
    assert lib.spsattn_decode_step(*args(_lib.DTYPE_FP16, None, 1 << 16)) == -1     # out type != query type
    assert lib.spsattn_decode_step(*args(_lib.DTYPE_BF16, C.byref(_lib.KvAppend()), 1 << 16)) == -1  # empty append
    assert lib.spsattn_decode_step(*args(_lib.DTYPE_BF16, None, 16)) == -4          # workspace too small


# ----------------------------------------------------------------------------- the engine

@pytest.mark.parametrize("tag", list(TAGS))
def test_dense_logits_match_reference_model(golden, tag):
    """forward_logits against the reference's own dense forward (fp32 parameters, bf16 attention
    operands as in sps/core.py:53-55), with the tolerance the reference's tests use for this
    comparison (tests/models/sps/test_dense_only.py:357)."""
    weights, fields = _golden_model(golden, tag)
    eng = _engine(weights, fields, TAGS[tag], torch.float32)
    idx = torch.from_numpy(golden[f"model_{tag}_dense_idx"])
    got = eng.forward_logits(idx).float().cpu()
    ref = torch.from_numpy(golden[f"model_{tag}_dense_logits"])
    torch.testing.assert_close(got, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("tag", list(TAGS))
@pytest.mark.parametrize("split", [0, 7, 8, 10])
def test_prefill_then_decode_matches_reference_stepwise(golden, tag, split):
    """Prefill the first ``split`` columns of left-padded prompts in one batch (0: none, every
    column goes through the decode step, pad columns as inactive rows), decode the rest token by
    token with the given tokens: every logit row against the reference's stepwise decode (fp32
    there; the bf16 attention operands alone move these logits by up to 0.06 in the CPU
    restatement, hence the absolute tolerance)."""
    weights, fields = _golden_model(golden, tag)
    eng = _engine(weights, fields, TAGS[tag], torch.float32)
    idx = torch.from_numpy(golden[f"model_{tag}_padded_idx"]).to(_dev())
    ref = torch.from_numpy(golden[f"model_{tag}_padded_logits"])
    pad = fields["pad_token_id"]
    b, t = idx.shape
    got = {}
    if split == 0:
        state = eng.build_decode_state(b, t)
    else:
        state, logits = eng.prefill(idx[:, :split].clone(), max_new_tokens=t - split + 1)
        got[split - 1] = logits.float().cpu()
    for col in range(split, t):
        active = idx[:, col] != pad
        got[col] = eng.decode_one_token(state, idx[:, col], active).float().cpu()
    for col, z in got.items():
        real = (idx[:, col] != pad).cpu()
        torch.testing.assert_close(z[real], ref[:, col][real], atol=8e-2, rtol=2e-2)
        err = (z[real] - ref[:, col][real]).abs().mean().item()
        assert err < 2e-2, (col, err)


@pytest.mark.parametrize("tag", list(TAGS))
@pytest.mark.parametrize("use_graph", [False, True])
def test_greedy_tokens_match_reference(golden, tag, use_graph):
    """generate() against the reference's greedy continuation; a position is compared only while
    every earlier choice of its row had a top-1 / top-2 gap the operand rounding cannot close."""
    weights, fields = _golden_model(golden, tag)
    eng = _engine(weights, fields, TAGS[tag], torch.float32)
    idx = torch.from_numpy(golden[f"model_{tag}_padded_idx"])
    ref = torch.from_numpy(golden[f"model_{tag}_greedy"])
    margin = torch.from_numpy(golden[f"model_{tag}_greedy_margin"])
    n_new = ref.shape[1] - idx.shape[1]
    out = eng.generate(idx, n_new, stop_on_eos=False, use_graph=use_graph).cpu()
    assert out.shape == ref.shape and torch.equal(out[:, :idx.shape[1]], idx)
    compared = 0
    for r in range(idx.shape[0]):
        for s in range(n_new):
            if float(margin[r, s]) < 0.15:
                break
            assert int(out[r, idx.shape[1] + s]) == int(ref[r, idx.shape[1] + s]), (r, s)
            compared += 1
    assert compared >= 4          # every fixture has enough clear choices to make this a real check


def _random_model(seed, n_layer, n_head, hidden, inter, vocab, block, w):
    fields = dict(block_size=block, vocab_size=vocab, n_layer=n_layer, n_head=n_head, hidden_size=hidden,
                  intermediate_size=inter, eos_token_id=vocab - 1, pad_token_id=vocab - 2,
                  predict_token_id=vocab - 3, window_size=w)
    g = torch.Generator().manual_seed(seed)
    sd = {"transformer.wte.weight": (torch.randn(vocab, hidden, generator=g) * 0.12).bfloat16().float()}
    sd["lm_head.weight"] = sd["transformer.wte.weight"]
    for layer in range(n_layer):
        pre = f"transformer.h.{layer}."
        rnd = lambda *s: (torch.randn(*s, generator=g) * 0.12).bfloat16().float()
        sd[pre + "attention_norm.weight"] = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().float()
        sd[pre + "attn.c_attn.weight"] = rnd(3 * hidden, hidden)
        sd[pre + "attn.c_proj.weight"] = rnd(hidden, hidden)
        sd[pre + "mlp_norm.weight"] = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().float()
        sd[pre + "mlp.gate_proj.weight"] = rnd(inter, hidden)
        sd[pre + "mlp.up_proj.weight"] = rnd(inter, hidden)
        sd[pre + "mlp.down_proj.weight"] = rnd(hidden, inter)
    sd["transformer.output_norm.weight"] = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16().float()
    return sd, fields


@pytest.mark.parametrize("variant,hd", [("sps", 128), ("reverse_sps", 128), ("sps", 32)])
def test_engine_matches_model_oracle_on_a_larger_case(variant, hd):
    """head_dim 128 (and 32, the CUDA-core prefill), window 8 shorter than the documents, left
    padding, an EOS in the prompt: prefill logits, 6 decoded tokens and their logits against the
    pinned CPU oracle of the model."""
    sd, fields = _random_model(5, n_layer=2, n_head=2, hidden=2 * hd, inter=4 * hd, vocab=96, block=128, w=8)
    dims = mo.Dims(**fields)
    g = torch.Generator().manual_seed(6)
    idx = torch.randint(0, 90, (3, 40), generator=g)
    idx[0, :7] = fields["pad_token_id"]
    idx[1, 22] = fields["eos_token_id"]
    idx[2, :33] = fields["pad_token_id"]
    eng = _engine(sd, fields, variant, torch.float32)
    state, logits = eng.prefill(idx, max_new_tokens=7)
    seq = idx.clone()
    for step in range(7):
        pos = mo.left_padded_positions(seq, dims.pad_token_id)
        ref = mo.logits(sd, dims, seq, variant=variant, positions=pos)[:, -1]
        torch.testing.assert_close(logits.float().cpu(), ref, atol=3e-2, rtol=2e-2)
        tok = mo.greedy_token(ref, dims)
        seq = torch.cat([seq, tok[:, None]], dim=1)
        if step < 6:
            logits = eng.decode_one_token(state, tok, torch.ones(3, dtype=torch.bool))
    # caches: every layer holds the current document of every row
    doc = mo.document_idx(seq[:, :-1], dims.eos_token_id, dims.pad_token_id)
    live = ((doc == doc[:, -1:]) & (seq[:, :-1] != dims.pad_token_id)).sum(dim=1)
    assert torch.equal(state.br_len.cpu(), live.view(1, 3, 1).expand(2, 3, 2))
    assert torch.equal(state.nw_len.cpu(), live.clamp(max=8).view(1, 3).expand(2, 3))


def test_engine_at_the_width_of_the_generation_benchmark():
    """The generation benchmark's layer width (hidden 2048, 16 heads x 128, SwiGLU 8192, window 64,
    the reference's N(0, 0.02) initialisation) on two layers, a prompt of 256 tokens with left
    padding in one row and an EOS inside the other: prefill logits and the logits of 8
    teacher-forced decode steps (tokens chosen greedily by the oracle) against the pinned CPU
    oracle of the model.  The 24-layer model of the benchmark is this block repeated."""
    from sps_b200.generation import SPSDims, random_state_dict
    fields = dict(block_size=320, vocab_size=4096, n_layer=2, n_head=16, hidden_size=2048,
                  intermediate_size=8192, eos_token_id=4000, pad_token_id=4095, predict_token_id=4001,
                  window_size=64)
    sd = {k: v.float() for k, v in random_state_dict(SPSDims(**fields), seed=3, device="cpu",
                                                     dtype=torch.float32).items()}
    dims = mo.Dims(**fields)
    g = torch.Generator().manual_seed(12)
    idx = torch.randint(0, 4000, (2, 256), generator=g)
    idx[0, :19] = fields["pad_token_id"]
    idx[1, 101] = fields["eos_token_id"]
    eng = _engine(sd, fields, "sps", torch.float32)
    n_new = 9
    state, logits = eng.prefill(idx, max_new_tokens=n_new)
    seq = idx.clone()
    on = torch.ones(2, dtype=torch.bool)
    for step in range(n_new):
        pos = mo.left_padded_positions(seq, dims.pad_token_id)
        ref = mo.logits(sd, dims, seq, variant="sps", positions=pos)[:, -1]
        err = (logits.float().cpu() - ref).abs()
        assert float(err.max()) <= 3e-2 + 2e-2 * float(ref.abs().max()), (step, float(err.max()))
        assert float(err.mean()) <= 4e-3, (step, float(err.mean()))
        tok = mo.greedy_token(ref, dims)
        seq = torch.cat([seq, tok[:, None]], dim=1)
        if step + 1 < n_new:
            logits = eng.decode_one_token(state, tok, on)
    import sps_b200
    sps_b200.check_device_status()


def test_bf16_parameters_track_the_fp32_run(golden):
    """bf16 parameters (how the reference generates on CUDA): logits stay within bf16 noise of the
    fp32-parameter run and of the reference."""
    weights, fields = _golden_model(golden, "sps_w5")
    idx = torch.from_numpy(golden["model_sps_w5_dense_idx"])
    ref = torch.from_numpy(golden["model_sps_w5_dense_logits"])
    got = _engine(weights, fields, "sps", torch.bfloat16).forward_logits(idx).float().cpu()
    err = (got - ref).abs()
    assert err.max().item() < 0.25 and err.mean().item() < 0.04, (err.max().item(), err.mean().item())


def test_generate_stops_rows_at_eos_and_pads(golden):
    """stop_on_eos: a row that emits EOS is padded afterwards and its caches stop growing
    (utils/generation.py:171-195); forced here by forbidding every token but EOS for the choice."""
    weights, fields = _golden_model(golden, "sps")
    eng = _engine(weights, fields, "sps", torch.float32)
    idx = torch.from_numpy(golden["model_sps_padded_idx"])
    eos, pad = fields["eos_token_id"], fields["pad_token_id"]
    forbidden = torch.tensor([t for t in range(fields["vocab_size"]) if t != eos])
    out = eng.generate(idx, 4, stop_on_eos=True, forbidden_token_ids=forbidden).cpu()
    new = out[:, idx.shape[1]:]
    assert torch.equal(new[:, 0], torch.full((3,), eos)) and bool((new[:, 1:] == pad).all())
    # without stopping, the same constraint keeps emitting EOS
    out2 = eng.generate(idx, 4, stop_on_eos=False, forbidden_token_ids=forbidden).cpu()
    assert bool((out2[:, idx.shape[1]:] == eos).all())


def test_prefill_rejects_what_the_reference_rejects(golden):
    weights, fields = _golden_model(golden, "sps")
    eng = _engine(weights, fields, "sps", torch.float32)
    pad = fields["pad_token_id"]
    with pytest.raises(ValueError):
        eng.prefill(torch.tensor([[5, pad, 7]]), 2)                 # pad after a real token
    with pytest.raises(ValueError):
        eng.prefill(torch.tensor([[pad, pad, pad]]), 2)             # no real token
    with pytest.raises(ValueError):
        eng.prefill(torch.randint(0, 50, (1, 30)), 8)               # beyond block_size 32
    with pytest.raises(NotImplementedError):
        eng.generate(torch.tensor([[5, 6]]), 2, do_sample=True)


def test_bind_generate_replaces_a_reference_style_generate(golden):
    """generator_for / bind_generate read dims, parameters and the variant off a model object with
    the reference's attributes and install a generate() with the reference's signature."""
    import types
    import sps_b200
    weights, fields = _golden_model(golden, "rsps")
    cfg = types.SimpleNamespace(norm_eps=1e-6, **fields)
    model = types.SimpleNamespace(config=cfg, _prediction_slot_index=0,
                                  state_dict=lambda: {k: v.to(_dev()) for k, v in weights.items()})
    eng = sps_b200.bind_generate(model)
    assert eng.variant == "reverse_sps" and eng.param_dtype == torch.float32
    idx = torch.from_numpy(golden["model_rsps_padded_idx"])
    out = model.generate(idx, 3, temperature=1.0, top_k=None, top_p=None, do_sample=False, stop_on_eos=False,
                         forbidden_token_ids=None)
    assert torch.equal(out.cpu(), eng.generate(idx, 3, stop_on_eos=False).cpu())
    with pytest.raises(NotImplementedError):
        model.generate(idx, 3, do_sample=True)


def test_left_padded_batch_matches_unpadded_rows(golden):
    """A row's logits and greedy continuation do not depend on the padding or on the other rows of
    the batch (tests/models/sps/test_dense_only.py:251-285)."""
    weights, fields = _golden_model(golden, "sps_w5")
    eng = _engine(weights, fields, "sps", torch.float32)
    pad, eos = fields["pad_token_id"], fields["eos_token_id"]
    prompts = torch.tensor([[pad, pad, 11, eos, 12, 13], [21, 22, 23, 24, 25, 26]])
    _, batched_logits = eng.prefill(prompts, 4)
    batched_logits = batched_logits.float().cpu()
    batched = eng.generate(prompts, 4, stop_on_eos=False).cpu()
    solo_eng = _engine(weights, fields, "sps", torch.float32)
    for r in range(2):
        first = int((prompts[r] != pad).nonzero()[0])
        single = prompts[r, first:].unsqueeze(0)
        _, z = solo_eng.prefill(single, 4)
        torch.testing.assert_close(z.float().cpu()[0], batched_logits[r], atol=2e-3, rtol=2e-3)
        out = solo_eng.generate(single, 4, stop_on_eos=False).cpu()
        assert torch.equal(batched[r, :first], torch.full((first,), pad))
        assert torch.equal(batched[r, first:], out[0]), r


# ----------------------------------------------------------------------------- Standard model

@pytest.mark.parametrize("split", [0, 7, 10])
def test_standard_model_prefill_then_decode_matches_reference(golden, split):
    """The Standard model (one row per token, cache = current document, q = 1 decode): logits of
    a batched prefill of the first ``split`` columns and of the token-by-token decode of the rest
    against the reference's own prefill path (full_attention_model.py:744-853), fp32 there."""
    weights, fields = _golden_model(golden, "std")
    eng = _engine(weights, fields, "standard", torch.float32)
    idx = torch.from_numpy(golden["model_std_padded_idx"]).to(_dev())
    ref = torch.from_numpy(golden["model_std_padded_logits"])
    pad = fields["pad_token_id"]
    b, t = idx.shape
    got = {}
    if split == 0:
        state = eng.build_decode_state(b, t)
    else:
        state, logits = eng.prefill(idx[:, :split].clone(), max_new_tokens=t - split + 1)
        got[split - 1] = logits.float().cpu()
    for col in range(split, t):
        got[col] = eng.decode_one_token(state, idx[:, col], idx[:, col] != pad).float().cpu()
    for col, z in got.items():
        real = (idx[:, col] != pad).cpu()
        torch.testing.assert_close(z[real], ref[:, col][real], atol=8e-2, rtol=2e-2)
        assert (z[real] - ref[:, col][real]).abs().mean().item() < 2e-2
    full = eng.forward_logits(idx).float().cpu()      # dense path, positions 0..T-1: unpadded row only
    torch.testing.assert_close(full[1], ref[1], atol=8e-2, rtol=2e-2)


@pytest.mark.parametrize("use_graph", [False, True])
def test_standard_model_greedy_tokens_match_reference(golden, use_graph):
    weights, fields = _golden_model(golden, "std")
    eng = _engine(weights, fields, "standard", torch.float32)
    idx = torch.from_numpy(golden["model_std_padded_idx"])
    ref = torch.from_numpy(golden["model_std_greedy"])
    margin = torch.from_numpy(golden["model_std_greedy_margin"])
    n_new = ref.shape[1] - idx.shape[1]
    out = eng.generate(idx, n_new, stop_on_eos=False, use_graph=use_graph).cpu()
    compared = 0
    for r in range(idx.shape[0]):
        for s in range(n_new):
            if float(margin[r, s]) < 0.15:
                break
            assert int(out[r, idx.shape[1] + s]) == int(ref[r, idx.shape[1] + s]), (r, s)
            compared += 1
    assert compared >= 8
    # a prompt that ends on EOS: the cache starts empty, the first new token opens a document
    ends = torch.from_numpy(golden["model_std_eos_end_idx"])
    want = torch.from_numpy(golden["model_std_eos_end_greedy"])
    dims = mo.Dims(**fields)
    _, margins = mo.generate(weights, dims, ends, 5, variant="standard", stop_on_eos=False, return_margins=True)
    got = eng.generate(ends, 5, stop_on_eos=False, use_graph=use_graph).cpu()
    for r in range(2):
        for s in range(5):
            if float(margins[r, s]) < 0.15:
                break
            assert int(got[r, 6 + s]) == int(want[r, 6 + s]), (r, s)


@pytest.mark.parametrize("use_graph", [False, True])
def test_session_keeps_its_step_buffers_across_a_foreign_decode(golden, use_graph):
    """generate(), then a prefill and an eager decode_one_token on a second state (which binds other
    step buffers), then generate() again: the cached session (and its captured graph) must still
    run on the buffers it was recorded on and give the same tokens."""
    weights, fields = _golden_model(golden, "sps")
    eng = _engine(weights, fields, "sps", torch.float32)
    idx = torch.from_numpy(golden["model_sps_padded_idx"])
    n_new = 6
    first = eng.generate(idx, n_new, stop_on_eos=False, use_graph=use_graph).cpu()
    other, logits = eng.prefill(idx[:1, -4:].contiguous(), 3)
    tok = logits.float().argmax(dim=-1)
    eng.decode_one_token(other, tok, torch.ones(1, dtype=torch.bool))
    again = eng.generate(idx, n_new, stop_on_eos=False, use_graph=use_graph).cpu()
    assert torch.equal(first, again)


def test_decode_one_token_refuses_a_step_past_the_caches(golden):
    """The reference raises when processed_tokens reaches the block size (reverse_sps/inference.py:
    384-389); here the bound is kept on the host (longest prompt + steps taken), so the refusal comes
    before any launch and the out-of-range step never runs on the device."""
    weights, fields = _golden_model(golden, "sps")
    eng = _engine(weights, fields, "sps", torch.float32)
    idx = torch.from_numpy(golden["model_sps_padded_idx"])[:1, -4:].contiguous()
    state, logits = eng.prefill(idx, 2)            # caches hold the prompt + 2 tokens
    tok = logits.float().argmax(dim=-1)
    on = torch.ones(1, dtype=torch.bool)
    longest = int((idx != fields["pad_token_id"]).sum())
    assert state.host_tokens == longest and state.max_tokens == longest + 2
    eng.decode_one_token(state, tok, on)
    eng.decode_one_token(state, tok, on)
    with pytest.raises(ValueError, match="Cannot decode another token"):
        eng.decode_one_token(state, tok, on)
    torch.cuda.synchronize()
