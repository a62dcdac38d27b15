"""The four kernels against each other, the way the reference checks its model paths
(dense forward == stepwise decode, src/modeling/tests/models/sps/test_dense_only.py:338-387):
prefill attention over the doubled sequence must equal, row pair by row pair, the segmented
decode attention over caches that were built by the hand-over kernel and advanced by the cache
update kernel.  Also: the decode step is capturable in a CUDA graph.  Needs a B200."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


@pytest.mark.parametrize("family,rs,ws", [("sps", 0, 1), ("reverse", 1, 0)])
def test_dense_prefill_equals_handover_plus_stepwise_decode(family, rs, ws):
    import sps_b200
    dev, bf = _dev(), torch.bfloat16
    B, H, T, D, w = 3, 2, 45, 64, 4
    t_split = 29                                  # prefill the first 29 tokens, decode the rest
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, 2 * T, H, D, generator=g).to(bf).to(dev) for _ in range(3))   # token-major
    # documents: row 0 one document; row 1 a new document starts at token 11; row 2 at token 20
    docs_T = torch.zeros(B, T, dtype=torch.long)
    docs_T[1, 11:] = 1
    docs_T[2, 20:] = 1
    docs = docs_T.repeat_interleave(2, dim=1).to(dev)
    fn = sps_b200.sps_sliding_attention if family == "sps" else sps_b200.reverse_sps_sliding_attention
    dense = fn(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), 1 / math.sqrt(D), w,
               documents_idx_BxT=docs).transpose(1, 2).float()          # [B, 2T, H, D]

    cap = T + 1
    br_k, br_v = (torch.zeros(B, H, cap, D, device=dev, dtype=bf) for _ in range(2))
    nw_k, nw_v = (torch.zeros(B, H, w, D, device=dev, dtype=bf) for _ in range(2))
    br_len = torch.zeros(B, H, dtype=torch.long, device=dev)
    nw_len, nw_pos = (torch.zeros(B, dtype=torch.long, device=dev) for _ in range(2))
    last_doc = docs_T[:, t_split - 1:t_split]
    mask = (docs_T[:, :t_split] == last_doc).to(dev)
    sps_b200.fill_decode_caches(k[:, :2 * t_split], v[:, :2 * t_split], mask, br_k=br_k, br_v=br_v, br_len=br_len,
                                nw_k=nw_k, nw_v=nw_v, nw_len=nw_len, nw_pos=nw_pos, window_tokens=w,
                                retained_slot=rs, window_slot=ws)
    active = torch.ones(B, dtype=torch.bool, device=dev)
    worst = 0.0
    for t in range(t_split, T):
        for b in range(B):                        # a document start empties the caches of that row
            if t > 0 and int(docs_T[b, t]) != int(docs_T[b, t - 1]):
                br_len[b] = 0
                nw_len[b] = 0
                nw_pos[b] = 0
        pair = q[:, 2 * t:2 * t + 2]              # [B, 2, H, D]
        cur = [k[:, 2 * t], v[:, 2 * t], k[:, 2 * t + 1], v[:, 2 * t + 1]]
        segs = [sps_b200.KVSegment(nw_k, nw_v, nw_len, max_len_cap=w),
                sps_b200.KVSegment(br_k, br_v, br_len, max_len_cap=cap)]
        out = sps_b200.segmented_q2_attention(pair, segs, current_normal_k_BxHxD=cur[0],
                                              current_normal_v_BxHxD=cur[1], current_predict_k_BxHxD=cur[2],
                                              current_predict_v_BxHxD=cur[3], attn_dtype=bf)
        worst = max(worst, float((out - dense[:, 2 * t:2 * t + 2]).abs().max()))
        slot = lambda s: (k[:, 2 * t + s], v[:, 2 * t + s])
        sps_b200.fused_sps_kv_update(nw_k=nw_k, nw_v=nw_v, nw_len=nw_len, nw_pos=nw_pos, br_k=br_k, br_v=br_v,
                                     br_len=br_len, k_window_BxHxD=slot(ws)[0], v_window_BxHxD=slot(ws)[1],
                                     k_retained_BxHxD=slot(rs)[0], v_retained_BxHxD=slot(rs)[1],
                                     active_mask_B=active, window_tokens=w)
    sps_b200.check_device_status()
    assert worst <= 2e-2, worst
    assert br_len[0, 0].item() == T and nw_len.tolist() == [w] * B


def test_decode_step_runs_inside_a_cuda_graph():
    """Attention + cache update of one decode step hold no host synchronisation, so the step can
    be captured once and replayed (device-side lengths and counters advance inside the graph)."""
    import sps_b200
    dev, bf = _dev(), torch.bfloat16
    S, H, D, w, cap, steps = 4, 2, 64, 8, 64, 6
    g = torch.Generator().manual_seed(2)
    rnd = lambda *s: torch.randn(*s, generator=g).to(bf).to(dev)
    feed = [dict(q=rnd(S, 2, H, D), nk=rnd(S, H, D), nv=rnd(S, H, D), pk=rnd(S, H, D), pv=rnd(S, H, D))
            for _ in range(steps)]

    def fresh():
        return dict(br_k=torch.zeros(S, H, cap, D, device=dev, dtype=bf), br_v=torch.zeros(S, H, cap, D, device=dev, dtype=bf),
                    nw_k=torch.zeros(S, H, w, D, device=dev, dtype=bf), nw_v=torch.zeros(S, H, w, D, device=dev, dtype=bf),
                    br_len=torch.zeros(S, H, dtype=torch.long, device=dev), nw_len=torch.zeros(S, dtype=torch.long, device=dev),
                    nw_pos=torch.zeros(S, dtype=torch.long, device=dev))

    active = torch.ones(S, dtype=torch.int8, device=dev)

    def step(c, x):
        segs = [sps_b200.KVSegment(c["nw_k"], c["nw_v"], c["nw_len"], max_len_cap=w),
                sps_b200.KVSegment(c["br_k"], c["br_v"], c["br_len"], max_len_cap=cap)]
        out = sps_b200.segmented_q2_attention(x["q"], segs, current_normal_k_BxHxD=x["nk"], current_normal_v_BxHxD=x["nv"],
                                              current_predict_k_BxHxD=x["pk"], current_predict_v_BxHxD=x["pv"], attn_dtype=bf)
        sps_b200.fused_sps_kv_update(nw_k=c["nw_k"], nw_v=c["nw_v"], nw_len=c["nw_len"], nw_pos=c["nw_pos"],
                                     br_k=c["br_k"], br_v=c["br_v"], br_len=c["br_len"], k_window_BxHxD=x["pk"],
                                     v_window_BxHxD=x["pv"], k_retained_BxHxD=x["nk"], v_retained_BxHxD=x["nv"],
                                     active_mask_B=active, window_tokens=w)
        return out

    eager_c = fresh()
    eager = [step(eager_c, x).clone() for x in feed]

    graph_c = fresh()
    static = {key: torch.empty_like(val) for key, val in feed[0].items()}
    for key in static:
        static[key].copy_(feed[0][key])
    side = torch.cuda.Stream(dev)                  # warm up outside the capture, then reset the state
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(graph_c, static)
    torch.cuda.current_stream().wait_stream(side)
    graph_c2 = fresh()
    for key in graph_c:
        graph_c[key].copy_(graph_c2[key])
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = step(graph_c, static)
    for key in graph_c:                            # the capture itself ran nothing; start from zero state
        graph_c[key].copy_(graph_c2[key])
    for i, x in enumerate(feed):
        for key in static:
            static[key].copy_(x[key])
        graph.replay()
        assert torch.equal(static_out, eager[i]), i
    assert torch.equal(graph_c["br_len"], eager_c["br_len"]) and torch.equal(graph_c["nw_pos"], eager_c["nw_pos"])
