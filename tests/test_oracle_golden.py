"""The CPU oracle against the reference's own outputs (tests/golden) and against the
literal known answers the reference's tests hold.  No GPU needed."""

import math

import numpy as np
import pytest
import torch

from oracle import sps_oracle as orc

T = torch.from_numpy


def _close(a, b, atol=2e-5, rtol=1e-4):
    np.testing.assert_allclose(np.asarray(a), np.asarray(b), atol=atol, rtol=rtol)


@pytest.mark.parametrize("tag", ["nodoc", "doc", "n8", "n24", "n200", "n384"])
def test_sps_prefill_matches_reference_oracle(golden, tag):
    g = golden
    p = f"sps_{tag}"
    docs = T(g[p + "_docs"]) if (p + "_docs") in g else None
    out = orc.prefill_attention(T(g[p + "_q"]), T(g[p + "_k"]), T(g[p + "_v"]), 1 / 8.0,
                                persistent_parity=orc.PARITY_EVEN,
                                temporary_window=int(g[p + "_w"]), docs=docs)
    _close(out, g[p + "_out"])


def test_sps_cfg0_matches_reference_oracle(golden):
    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 8, 512, 64, generator=gen) for _ in range(3))
    chk = float(q.double().sum() + 2 * k.double().sum() + 3 * v.double().sum())
    assert abs(chk - float(golden["sps_cfg0_q_checksum"])) < 1e-3, "seeded inputs drifted"
    docs = T(golden["sps_cfg0_docs"])
    out = orc.prefill_attention(q[:, [0, 5]], k[:, [0, 5]], v[:, [0, 5]], 1 / 8.0,
                                temporary_window=64, docs=docs)
    _close(out, golden["sps_cfg0_out_h0h5"])
    sd = orc.prefill_attention_sdpa(q[:, [0, 5]], k[:, [0, 5]], v[:, [0, 5]], 1 / 8.0,
                                    temporary_window=64, docs=docs)
    _close(sd, golden["sps_cfg0_out_h0h5"])


@pytest.mark.parametrize("tag,pw,w", [("pkw", 1, 8), ("pkwL", 5, 2)])
@pytest.mark.parametrize("rem", [0, 1])
def test_persistent_window_matches_reference_oracle(golden, tag, pw, w, rem):
    p = f"{tag}{rem}"
    out = orc.prefill_attention(T(golden[p + "_q"]), T(golden[p + "_k"]), T(golden[p + "_v"]), 1 / 8.0,
                                persistent_parity=rem, temporary_window=w, persistent_window=pw)
    # the reference oracle rounds its output to the input dtype (fp16 / bf16)
    _close(out, golden[p + "_out"], atol=8e-3, rtol=8e-3)


@pytest.mark.parametrize("tag,d", [("full_n128", 64), ("full_n200", 128)])
def test_full_attention_matches_reference_oracle(golden, tag, d):
    q, k, v = (T(golden[f"{tag}_{x}"]) for x in "qkv")
    out = orc.prefill_attention(q, k, v, 1 / math.sqrt(d), persistent_parity=orc.PARITY_NONE,
                                docs=T(golden[tag + "_docs"]))
    _close(out, golden[tag + "_out"])
    out = orc.prefill_attention(q, k, v, 1 / math.sqrt(d), persistent_parity=orc.PARITY_NONE)
    _close(out, golden[tag + "_out_nodoc"])


@pytest.mark.parametrize("tag", ["shared", "empty"])
def test_q2_decode_matches_reference_oracle(golden, tag):
    g = {k[len(f"q2_{tag}_"):]: v for k, v in golden.items() if k.startswith(f"q2_{tag}_")}
    segs = [orc.Segment(T(g["k0"]), T(g["v0"]), T(g["len0"]), int(g["cap0"])),
            orc.Segment(T(g["k1"]), T(g["v1"]), T(g["len1"]), 8)]
    extras = [(T(g["cnk"]), T(g["cnv"]), 0b11), (T(g["cpk"]), T(g["cpv"]), 0b10)]
    out = orc.decode_attention(T(g["q"]), segs, extras)
    _close(out, g["out"])
    _close(out, g["sdpa"], atol=1e-5)


def test_q1_decode_matches_reference_fallback(golden):
    g = golden
    segs = [orc.Segment(T(g[f"q1_k{i}"]), T(g[f"q1_v{i}"]), T(g[f"q1_len{i}"])) for i in range(3)]
    out = orc.decode_attention(T(g["q1_q"]).unsqueeze(1), segs, [(T(g["q1_ek"]), T(g["q1_ev"]), 1)])
    _close(out[:, 0], g["q1_out"], atol=1e-5)


@pytest.mark.parametrize("w", [0, 1, 2])
def test_reverse_visibility_matches_reference_score_mod(golden, w):
    ref = golden[f"vis_reverse_w{w}"].astype(bool)
    vis = orc.visible_mask(10, persistent_parity=orc.PARITY_ODD, temporary_window=w)
    assert np.array_equal(vis, ref)
    # literal known answer (tests/models/reverse_sps/test_forward_efficient.py:130-156)
    for tok in range(5):
        want = list(range(max(0, tok - w), tok + 1))
        for qi in (2 * tok, 2 * tok + 1):
            assert [j // 2 for j in range(0, 10, 2) if vis[qi, j]] == want


def test_sps_rule_known_answers():
    # input queries see the previous <= w predict keys; predict queries see w+1 (self included)
    vis = orc.visible_mask(16, persistent_parity=orc.PARITY_EVEN, temporary_window=2)
    assert [j for j in range(16) if vis[10, j]] == [0, 2, 4, 6, 7, 8, 9, 10]
    assert [j for j in range(16) if vis[11, j]] == [0, 2, 4, 6, 7, 8, 9, 10, 11]
    # closed-form pair count for one document of L tokens: L(L+1) + L + 2*sum(min(t,w))
    L, w = 37, 5
    want = L * (L + 1) + L + 2 * sum(min(t, w) for t in range(L))
    assert orc.count_visible_pairs(None, 2 * L, 1, temporary_window=w) == want


def test_kv_update_matches_reference_eager(golden):
    g = {k[4:]: v for k, v in golden.items() if k.startswith("kvu_")}
    w = int(g["window"])
    steps, B, H, D = g["kw"].shape
    cap = g["br_k"].shape[2]
    nw_k, nw_v = torch.zeros(B, H, w, D), torch.zeros(B, H, w, D)
    br_k, br_v = torch.zeros(B, H, cap, D), torch.zeros(B, H, cap, D)
    nw_len, nw_pos = torch.zeros(B, dtype=torch.long), torch.zeros(B, dtype=torch.long)
    br_len = torch.zeros(B, H, dtype=torch.long)
    for s in range(steps):
        orc.kv_update(nw_k, nw_v, nw_len, nw_pos, br_k, br_v, br_len, T(g["kw"][s]), T(g["vw"][s]),
                      T(g["kr"][s]), T(g["vr"][s]), T(g["active"][s]), w)
    for name, val in (("nw_k", nw_k), ("nw_v", nw_v), ("nw_len", nw_len), ("nw_pos", nw_pos),
                      ("br_k", br_k), ("br_v", br_v), ("br_len", br_len)):
        assert np.array_equal(val.numpy(), g[name]), name


def test_ring_wraps_without_shifting():
    # tests/models/delayed_state/test_forward_efficient.py:280-312: three inserts at w=2
    nw_k, nw_v = torch.zeros(1, 2, 2, 4), torch.zeros(1, 2, 2, 4)
    br_k, br_v = torch.zeros(1, 2, 5, 4), torch.zeros(1, 2, 5, 4)
    nw_len, nw_pos = torch.zeros(1, dtype=torch.long), torch.zeros(1, dtype=torch.long)
    br_len = torch.zeros(1, 2, dtype=torch.long)
    for val in (1.0, 2.0, 3.0):
        kk, vv = torch.full((1, 2, 4), val), torch.full((1, 2, 4), val + 10)
        orc.kv_update(nw_k, nw_v, nw_len, nw_pos, br_k, br_v, br_len, kk, vv, kk, vv,
                      torch.tensor([1]), 2)
    assert int(nw_len[0]) == 2 and int(nw_pos[0]) == 1
    assert nw_k[0, 0, :, 0].tolist() == [3.0, 2.0]
    assert br_len.tolist() == [[3, 3]]


def test_run_starts_and_monotone():
    d = np.array([0, 0, 1, 1, 1, 2, 2])
    assert orc.run_starts(d).tolist() == [0, 0, 2, 2, 2, 5, 5]
    assert orc.is_monotone(d) and not orc.is_monotone(np.array([0, 1, 0]))
    # left-padded ids from the reference's known answer (tests/core/test_document_idx.py:105-115)
    d = np.array([0, 1, 2, 2, 2, 3, 3])
    assert orc.is_monotone(d)
    lo = orc.run_starts(d)
    i, j = np.arange(7)[:, None], np.arange(7)[None, :]
    assert np.array_equal((d[:, None] == d[None, :]) & (j <= i), (j >= lo[:, None]) & (j <= i))


@pytest.mark.parametrize("tag", ["ds", "sps"])
def test_cache_fill_matches_reference_handover(golden, tag):
    g = {k[len(f"fill_{tag}_"):]: v for k, v in golden.items() if k.startswith(f"fill_{tag}_")}
    w = int(g["window"])
    rs, ws = (int(x) for x in g["slots"])
    br_k, br_v = torch.zeros(g["br_k"].shape), torch.zeros(g["br_v"].shape)
    nw_k, nw_v = torch.zeros(g["nw_k"].shape), torch.zeros(g["nw_v"].shape)
    br_len = torch.zeros(g["br_len"].shape, dtype=torch.long)
    nw_len = torch.zeros(g["nw_len"].shape, dtype=torch.long)
    nw_pos = torch.zeros(g["nw_pos"].shape, dtype=torch.long)
    orc.fill_decode_caches(T(g["k"]), T(g["v"]), T(g["mask"]), br_k, br_v, br_len, nw_k, nw_v, nw_len, nw_pos,
                           w, rs, ws)
    for name, val in (("br_k", br_k), ("br_v", br_v), ("br_len", br_len), ("nw_k", nw_k), ("nw_v", nw_v),
                      ("nw_len", nw_len), ("nw_pos", nw_pos)):
        assert np.array_equal(val.numpy(), g[name]), name


@pytest.mark.parametrize("tag,dt", [("f32", torch.float32), ("bf16", torch.bfloat16)])
def test_rope_cast_matches_reference_rotary(golden, tag, dt):
    g = golden
    fc = torch.view_as_complex(T(g["rope_freqs"]).contiguous())
    pos = T(g["rope_pos"])
    xq, xk = T(g[f"rope_{tag}_xq"]).to(dt), T(g[f"rope_{tag}_xk"]).to(dt)
    for name, x, freqs in (("q1", xq, fc[pos]), ("k1", xk, fc[pos]),
                           ("q2", xq, torch.stack([fc[pos], fc[pos + 7]])),
                           ("k2", xk, torch.stack([fc[pos], fc[pos + 7]]))):
        out = orc.rope_cast(x, freqs)
        assert np.array_equal(out.float().numpy(), g[f"rope_{tag}_{name}"]), name
    assert torch.equal(orc.rope_cast(xq, None), xq.to(torch.bfloat16))
