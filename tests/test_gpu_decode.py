"""Parity of the CUDA decode path (segmented attention + KV-cache update, through the C ABI)
against the CPU oracle and the committed reference vectors.  Needs a B200."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import sps_oracle as orc


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


def _c(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(_dev())
    return t if dtype is None else t.to(dtype)


def _close(out, ref, atol=2e-2, mean=2e-3):
    out, ref = out.float().cpu(), torch.as_tensor(ref).float()
    assert out.shape == ref.shape and torch.isfinite(out).all()
    err = (out - ref).abs()
    assert float(err.max()) <= atol and float(err.mean()) <= mean, (float(err.max()), float(err.mean()))


@pytest.mark.parametrize("tag", ["shared", "empty"])
def test_q2_matches_reference_vectors(golden, tag):
    """The reference's own q2 test case (head_dim 16, 3 heads, [B] and [B,H] lengths, caps,
    an empty first segment): test_segmented_q2_attention.py:65-117."""
    import sps_b200
    g = {k[len(f"q2_{tag}_"):]: v for k, v in golden.items() if k.startswith(f"q2_{tag}_")}
    bf = torch.bfloat16
    segs = [sps_b200.KVSegment(_c(g["k0"], bf), _c(g["v0"], bf), _c(g["len0"]), max_len_cap=int(g["cap0"])),
            sps_b200.KVSegment(_c(g["k1"], bf), _c(g["v1"], bf), _c(g["len1"]), max_len_cap=8)]
    out = sps_b200.triton_segmented_q2_attention(
        _c(g["q"], bf), segs, current_normal_k_BxHxD=_c(g["cnk"], bf), current_normal_v_BxHxD=_c(g["cnv"], bf),
        current_predict_k_BxHxD=_c(g["cpk"], bf), current_predict_v_BxHxD=_c(g["cpv"], bf), attn_dtype=bf)
    assert out.dtype == torch.float32 and tuple(out.shape) == g["out"].shape
    _close(out, g["out"], atol=2e-3, mean=2e-4)       # fp32 math on identical bf16 inputs
    _close(out, g["sdpa"], atol=2e-3, mean=2e-4)


def test_q1_matches_reference_fallback(golden):
    import sps_b200
    g, bf = golden, torch.bfloat16
    segs = [sps_b200.KVSegment(_c(g[f"q1_k{i}"], bf), _c(g[f"q1_v{i}"], bf), _c(g[f"q1_len{i}"])) for i in range(3)]
    out = sps_b200.masked_kv_attention(_c(g["q1_q"], bf), segs, extra_kv=[(_c(g["q1_ek"], bf), _c(g["q1_ev"], bf))],
                                       attn_dtype=bf, require_triton=True)
    _close(out, g["q1_out"], atol=2e-3, mean=2e-4)


def _ragged_case(seed, S, H, D, caps, per_head, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(S, 2, H, D, generator=g).to(dtype)
    segs = []
    for cap, ph in zip(caps, per_head):
        k = torch.randn(S, H, cap, D, generator=g).to(dtype)
        v = torch.randn(S, H, cap, D, generator=g).to(dtype)
        ln = torch.randint(0, cap + 1, (S, H) if ph else (S,), generator=g)
        ln.view(-1)[0] = 0
        ln.view(-1)[-1] = cap
        segs.append((k, v, ln))
    cur = [torch.randn(S, H, D, generator=g).to(dtype) for _ in range(4)]
    return q, segs, cur


@pytest.mark.parametrize("D", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_q2_ragged_matches_oracle(D, dtype):
    import sps_b200
    q, segs, cur = _ragged_case(D, 5, 3, D, (64, 1500), (False, True), dtype)
    dev = _dev()
    ksegs = [sps_b200.KVSegment(k.to(dev), v.to(dev), ln.to(dev)) for k, v, ln in segs]
    out = sps_b200.segmented_q2_attention(
        q.to(dev), ksegs, current_normal_k_BxHxD=cur[0].to(dev), current_normal_v_BxHxD=cur[1].to(dev),
        current_predict_k_BxHxD=cur[2].to(dev), current_predict_v_BxHxD=cur[3].to(dev), attn_dtype=dtype)
    ref = orc.decode_attention(q, [orc.Segment(k, v, ln) for k, v, ln in segs],
                               [(cur[0], cur[1], 0b11), (cur[2], cur[3], 0b10)])
    _close(out, ref, atol=3e-3, mean=3e-4)


def test_query_masks_and_packed_layout_match_oracle():
    """The input query skipping the ring (the prose variant of the decode configuration), and a
    packed token-major cache [sum(len), H, D] addressed through the offset table, no copy."""
    import sps_b200
    dev, bf = _dev(), torch.bfloat16
    S, H, D = 6, 4, 64
    q, segs, cur = _ragged_case(11, S, H, D, (64, 900), (False, False))
    (rk, rv, rl), (ck, cv, cl) = segs
    ref = orc.decode_attention(q, [orc.Segment(rk, rv, rl, query_mask=0b10), orc.Segment(ck, cv, cl)],
                               [(cur[0], cur[1], 0b11), (cur[2], cur[3], 0b10)])
    lens = cl.tolist()
    offs = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int64) * H * D
    pk = torch.cat([ck[s, :, :lens[s]].permute(1, 0, 2) for s in range(S)]).contiguous()   # [sum, H, D]
    pv = torch.cat([cv[s, :, :lens[s]].permute(1, 0, 2) for s in range(S)]).contiguous()
    packed = sps_b200.PackedKVSegment(pk.to(dev), pv.to(dev), torch.from_numpy(offs).to(dev), head_stride=D,
                                      row_stride=H * D, lengths=cl.to(dev), max_rows=900)
    ring = sps_b200.KVSegment(rk.to(dev), rv.to(dev), rl.to(dev))
    out = sps_b200.decode_attention(q.to(dev), [ring, packed],
                                    [(cur[0].to(dev), cur[1].to(dev), 0b11), (cur[2].to(dev), cur[3].to(dev), 0b10)],
                                    segment_query_masks=[0b10, 0b11])
    _close(out, ref, atol=3e-3, mean=3e-4)


def test_no_visible_key_gives_zero():
    import sps_b200
    dev, bf = _dev(), torch.bfloat16
    q = torch.randn(2, 1, 2, 64, device=dev).to(bf)
    k = torch.randn(2, 2, 8, 64, device=dev).to(bf)
    seg = sps_b200.KVSegment(k, k, torch.zeros(2, dtype=torch.long, device=dev))
    out = sps_b200.decode_attention(q, [seg], [])
    assert float(out.abs().max()) == 0.0


def test_full_size_decode_properties_and_spot_sequences():
    """The benchmark's decode configuration (128 sequences, lengths U[512,4096], ring 64,
    16 heads x 64): V = 1 gives 1 everywhere, the ring order does not matter, and a sample of
    sequences matches the oracle."""
    import sps_b200
    from sps_b200 import workloads
    wl = workloads.make_decode("cfg2_segmented_decode", _dev())

    def run(ck, cv, rk, rv, cur_v=None, pred_v=None):
        segs = [sps_b200.KVSegment(rk, rv, wl.ring_len, max_len_cap=64),
                sps_b200.KVSegment(ck, cv, wl.cache_len, max_len_cap=4096)]
        return sps_b200.segmented_q2_attention(
            wl.q, segs, current_normal_k_BxHxD=wl.cur_k, current_normal_v_BxHxD=wl.cur_v if cur_v is None else cur_v,
            current_predict_k_BxHxD=wl.pred_k, current_predict_v_BxHxD=wl.pred_v if pred_v is None else pred_v,
            attn_dtype=torch.bfloat16)

    out = run(wl.cache_k, wl.cache_v, wl.ring_k, wl.ring_v)
    one_c, one_r, one_t = torch.ones_like(wl.cache_v), torch.ones_like(wl.ring_v), torch.ones_like(wl.cur_v)
    o1 = run(wl.cache_k, one_c, wl.ring_k, one_r, one_t, one_t)
    assert float((o1 - 1).abs().max()) <= 1e-4
    perm = torch.randperm(64, device=_dev())
    o2 = run(wl.cache_k, wl.cache_v, wl.ring_k[:, :, perm].contiguous(), wl.ring_v[:, :, perm].contiguous())
    assert float((o2 - out).abs().max()) <= 1e-4
    for s in (0, 77, 127):
        sl = slice(s, s + 1)
        ref = orc.decode_attention(
            wl.q[sl].cpu(),
            [orc.Segment(wl.ring_k[sl].cpu(), wl.ring_v[sl].cpu(), wl.ring_len[sl].cpu(), 64),
             orc.Segment(wl.cache_k[sl].cpu(), wl.cache_v[sl].cpu(), wl.cache_len[sl].cpu(), 4096)],
            [(wl.cur_k[sl].cpu(), wl.cur_v[sl].cpu(), 0b11), (wl.pred_k[sl].cpu(), wl.pred_v[sl].cpu(), 0b10)])
        _close(out[sl], ref, atol=2e-3, mean=2e-4)


def test_kv_update_matches_reference_vectors(golden):
    import sps_b200
    dev = _dev()
    g = {k[4:]: v for k, v in golden.items() if k.startswith("kvu_")}
    w = int(g["window"])
    steps, B, H, D = g["kw"].shape
    cap = g["br_k"].shape[2]
    for dtype in (torch.float32, torch.bfloat16):
        nw_k, nw_v = torch.zeros(B, H, w, D, device=dev, dtype=dtype), torch.zeros(B, H, w, D, device=dev, dtype=dtype)
        br_k, br_v = torch.zeros(B, H, cap, D, device=dev, dtype=dtype), torch.zeros(B, H, cap, D, device=dev, dtype=dtype)
        nw_len, nw_pos = torch.zeros(B, dtype=torch.long, device=dev), torch.zeros(B, dtype=torch.long, device=dev)
        br_len = torch.zeros(B, H, dtype=torch.long, device=dev)
        for s in range(steps):
            sps_b200.fused_sps_kv_update(
                nw_k=nw_k, nw_v=nw_v, nw_len=nw_len, nw_pos=nw_pos, br_k=br_k, br_v=br_v, br_len=br_len,
                k_window_BxHxD=_c(g["kw"][s]), v_window_BxHxD=_c(g["vw"][s]), k_retained_BxHxD=_c(g["kr"][s]),
                v_retained_BxHxD=_c(g["vr"][s]), active_mask_B=_c(g["active"][s]).bool(), window_tokens=w)
        for name, val in (("nw_len", nw_len), ("nw_pos", nw_pos), ("br_len", br_len)):
            assert np.array_equal(val.cpu().numpy(), g[name]), name
        for name, val in (("nw_k", nw_k), ("nw_v", nw_v), ("br_k", br_k), ("br_v", br_v)):
            want = torch.from_numpy(g[name]).to(dtype)
            assert torch.equal(val.cpu(), want), name      # copies: bit-exact in the cache dtype


def test_kv_update_bounds_and_window_disabled():
    import sps_b200
    dev = _dev()
    B, H, D, cap = 2, 3, 16, 2
    br_k, br_v = torch.zeros(B, H, cap, D, device=dev), torch.zeros(B, H, cap, D, device=dev)
    br_len = torch.tensor([[0, 1, 2], [2, 0, 1]], device=dev)
    ref_k, ref_v, ref_len = br_k.cpu().clone(), br_v.cpu().clone(), br_len.cpu().clone()
    kk, vv = torch.randn(B, H, D, device=dev), torch.randn(B, H, D, device=dev)
    act = torch.tensor([True, True], device=dev)
    sps_b200.fused_sps_kv_update(nw_k=br_k, nw_v=br_v, nw_len=br_len[:, 0].contiguous(), nw_pos=br_len[:, 0].contiguous(),
                                 br_k=br_k, br_v=br_v, br_len=br_len, k_window_BxHxD=kk, v_window_BxHxD=vv,
                                 k_retained_BxHxD=kk, v_retained_BxHxD=vv, active_mask_B=act, window_tokens=0)
    orc.kv_update(None, None, None, None, ref_k, ref_v, ref_len, None, None, kk.cpu(), vv.cpu(), act.cpu(), 0)
    assert torch.equal(br_len.cpu(), ref_len) and torch.equal(br_k.cpu(), ref_k) and torch.equal(br_v.cpu(), ref_v)


def test_decode_argument_errors():
    import sps_b200
    dev, bf = _dev(), torch.bfloat16
    q = torch.randn(2, 2, 2, 64, device=dev).to(bf)
    k = torch.randn(2, 2, 8, 64, device=dev).to(bf)
    ln = torch.ones(2, dtype=torch.long, device=dev)
    cur = torch.randn(2, 2, 64, device=dev).to(bf)
    kw = dict(current_normal_k_BxHxD=cur, current_normal_v_BxHxD=cur, current_predict_k_BxHxD=cur,
              current_predict_v_BxHxD=cur, attn_dtype=bf)
    with pytest.raises(RuntimeError):
        sps_b200.segmented_q2_attention(q, [sps_b200.KVSegment(k, k, ln)] * 3, **kw)
    with pytest.raises(RuntimeError):
        sps_b200.segmented_q2_attention(q, [sps_b200.KVSegment(k.transpose(1, 2), k.transpose(1, 2), ln)], **kw)
    with pytest.raises(RuntimeError):
        sps_b200.segmented_q2_attention(q.cpu(), [sps_b200.KVSegment(k, k, ln)], **kw)
    with pytest.raises(RuntimeError):
        sps_b200.segmented_q2_attention(q, [sps_b200.KVSegment(k, k, ln.cpu())], **kw)
    with pytest.raises(RuntimeError, match="forward only"):          # no backward behind decode
        sps_b200.segmented_q2_attention(q.clone().requires_grad_(True), [sps_b200.KVSegment(k, k, ln)], **kw)
    with torch.no_grad():
        sps_b200.segmented_q2_attention(q.clone().requires_grad_(True), [sps_b200.KVSegment(k, k, ln)], **kw)


@pytest.mark.parametrize("tag", ["ds", "sps"])
def test_cache_fill_matches_reference_vectors(golden, tag):
    """Prefill -> decode hand-over against the reference's own Python loop
    (reverse_sps/inference.py:568-613), bit-exact: it is a gather of 16-bit rows."""
    import sps_b200
    dev, bf = _dev(), torch.bfloat16
    g = {k[len(f"fill_{tag}_"):]: v for k, v in golden.items() if k.startswith(f"fill_{tag}_")}
    w = int(g["window"])
    rs, ws = (int(x) for x in g["slots"])
    B, H, cap, D = g["br_k"].shape
    canary = 7.0
    br_k, br_v = (torch.full((B, H, cap, D), canary, device=dev, dtype=bf) for _ in range(2))
    nw_k, nw_v = (torch.full(g["nw_k"].shape, canary, device=dev, dtype=bf) for _ in range(2))
    br_len = torch.full((B, H), -5, dtype=torch.long, device=dev)
    nw_len, nw_pos = (torch.full((B,), -5, dtype=torch.long, device=dev) for _ in range(2))
    sps_b200.fill_decode_caches(_c(g["k"], bf), _c(g["v"], bf), _c(g["mask"]).bool(), br_k=br_k, br_v=br_v,
                                br_len=br_len, nw_k=nw_k, nw_v=nw_v, nw_len=nw_len, nw_pos=nw_pos,
                                window_tokens=w, retained_slot=rs, window_slot=ws)
    want_len = g["br_len"]
    for b in range(B):
        n = int(want_len[b, 0])
        assert br_len[b].tolist() == [n] * H
        assert torch.equal(br_k[b, :, :n].float().cpu(), torch.from_numpy(g["br_k"][b, :, :n]))
        assert torch.equal(br_v[b, :, :n].float().cpu(), torch.from_numpy(g["br_v"][b, :, :n]))
        assert float((br_k[b, :, n:].float() - canary).abs().max()) == 0 if n < cap else True   # untouched
        wl = int(g["nw_len"][b])
        assert int(nw_len[b]) == wl and int(nw_pos[b]) == 0
        assert torch.equal(nw_k[b, :, :wl].float().cpu(), torch.from_numpy(g["nw_k"][b, :, :wl]))
        assert torch.equal(nw_v[b, :, :wl].float().cpu(), torch.from_numpy(g["nw_v"][b, :, :wl]))


def test_cache_fill_large_ragged_matches_oracle():
    """Left-padded prompts of different lengths with earlier documents, strided K/V views (slices
    of a fused projection buffer), T not a multiple of the block's chunk, an empty selection."""
    import sps_b200
    dev, bf = _dev(), torch.bfloat16
    B, T, H, D, w = 5, 333, 4, 64, 64
    g = torch.Generator().manual_seed(8)
    qkv = torch.randn(B, 2 * T, 3 * H * D, generator=g).to(bf)
    k, v = (x.view(B, 2 * T, H, D) for x in qkv.split(H * D, dim=2)[1:])
    mask = torch.zeros(B, T, dtype=torch.bool)
    for b, start in enumerate((0, 100, 332, 290)):
        mask[b, start:] = True
    cap = T + 8
    outs = []
    for where in ("cpu", "cuda"):
        br_k, br_v = (torch.zeros(B, H, cap, D, dtype=bf) for _ in range(2))
        nw_k, nw_v = (torch.zeros(B, H, w, D, dtype=bf) for _ in range(2))
        br_len = torch.zeros(B, H, dtype=torch.long)
        nw_len, nw_pos = torch.zeros(B, dtype=torch.long), torch.full((B,), 3, dtype=torch.long)
        if where == "cpu":
            orc.fill_decode_caches(k, v, mask, br_k, br_v, br_len, nw_k, nw_v, nw_len, nw_pos, w, 0, 1)
        else:
            br_k, br_v, nw_k, nw_v, br_len, nw_len, nw_pos = (x.to(dev) for x in (br_k, br_v, nw_k, nw_v, br_len,
                                                                               nw_len, nw_pos))
            kd, vd = (x.view(B, 2 * T, H, D) for x in qkv.to(dev).split(H * D, dim=2)[1:])
            assert not kd.is_contiguous()
            sps_b200.fill_decode_caches(kd, vd, mask.to(dev), br_k=br_k, br_v=br_v, br_len=br_len,
                                        nw_k=nw_k, nw_v=nw_v, nw_len=nw_len, nw_pos=nw_pos, window_tokens=w,
                                        retained_slot=0, window_slot=1)
        outs.append([x.cpu() for x in (br_k, br_v, br_len, nw_k, nw_v, nw_len, nw_pos)])
    for a, b_ in zip(*outs):
        assert torch.equal(a, b_)
