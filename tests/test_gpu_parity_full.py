"""Parity at the benchmark's own sizes, every row: all 8192 rows of several (batch, head) pairs of
the two prefill configurations, all 128 sequences of the decode configuration, and the
reference's long-context regression shapes (src/modeling/tests/attention/triton/
test_full_long_context.py:27-39: a length that is no multiple of 128, where a flat tile walk
would run into the next head).  Needs a B200."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import sps_oracle as orc

MAX_ABS, MEAN_ABS = 2e-2, 2e-3     # bf16 tolerance against the fp32 oracle


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


def _check(out, ref, max_abs=MAX_ABS, mean_abs=MEAN_ABS):
    out = out.float().cpu()
    ref = torch.as_tensor(ref).float()
    assert out.shape == ref.shape
    assert torch.isfinite(out).all()
    err = (out - ref).abs()
    assert float(err.max()) <= max_abs, f"max-abs {float(err.max()):.4g}"
    assert float(err.mean()) <= mean_abs, f"mean-abs {float(err.mean()):.4g}"


def test_s_scale_prefill_every_row_of_four_pairs():
    """[8,12,8192,64], w = 64, packed documents, one launch over the whole batch; all 8192 rows of
    four (batch, head) pairs against the oracle, among them both batch rows with the most
    documents (seven each with seed 0)."""
    import sps_b200
    from sps_b200 import workloads
    wl = workloads.make_prefill("cfg1_s_scale", _dev())
    n_docs = [len(np.unique(wl.docs[b].cpu().numpy())) for b in range(wl.docs.shape[0])]
    busiest = int(np.argmax(n_docs))
    out = sps_b200.sps_sliding_attention(wl.q, wl.k, wl.v, wl.sm_scale, wl.window, documents_idx_BxT=wl.docs)
    sps_b200.check_device_status()
    pairs = {(busiest, 0), (4, 5), (2, 11), (7, 3)}
    assert len(pairs) == 4
    for b, h in sorted(pairs):
        ref = orc.prefill_attention(wl.q[b:b + 1, h:h + 1].cpu(), wl.k[b:b + 1, h:h + 1].cpu(),
                                    wl.v[b:b + 1, h:h + 1].cpu(), wl.sm_scale, temporary_window=wl.window,
                                    docs=wl.docs[b:b + 1].cpu())
        _check(out[b:b + 1, h:h + 1], ref)


def test_full_window_prefill_every_row_of_two_pairs():
    """[4,16,8192,128], w = 4096, one document per row, the full launch; all rows of two pairs."""
    import sps_b200
    from sps_b200 import workloads
    wl = workloads.make_prefill("cfg4_full_window", _dev())
    out = sps_b200.sps_sliding_attention(wl.q, wl.k, wl.v, wl.sm_scale, wl.window)
    sps_b200.check_device_status()
    for b, h in ((0, 0), (3, 13)):
        ref = orc.prefill_attention(wl.q[b:b + 1, h:h + 1].cpu(), wl.k[b:b + 1, h:h + 1].cpu(),
                                    wl.v[b:b + 1, h:h + 1].cpu(), wl.sm_scale, temporary_window=wl.window)
        _check(out[b:b + 1, h:h + 1], ref)


def test_decode_every_sequence():
    """128 sequences, cache lengths U[512,4096], ring 64, 16 heads x 64: every sequence against
    the oracle's padded-SDPA formulation (the reference's fallback, decode_attention.py:637-704),
    32 sequences at a time to bound host memory."""
    import sps_b200
    from sps_b200 import workloads
    wl = workloads.make_decode("cfg2_segmented_decode", _dev())
    segs = [sps_b200.KVSegment(wl.ring_k, wl.ring_v, wl.ring_len, max_len_cap=64),
            sps_b200.KVSegment(wl.cache_k, wl.cache_v, wl.cache_len, max_len_cap=4096)]
    out = sps_b200.segmented_q2_attention(
        wl.q, segs, current_normal_k_BxHxD=wl.cur_k, current_normal_v_BxHxD=wl.cur_v,
        current_predict_k_BxHxD=wl.pred_k, current_predict_v_BxHxD=wl.pred_v, attn_dtype=torch.bfloat16)
    sps_b200.check_device_status()
    S = wl.q.shape[0]
    for s0 in range(0, S, 32):
        sl = slice(s0, s0 + 32)
        ref = orc.decode_attention_batched(
            wl.q[sl].cpu(), wl.cache_k[sl].cpu(), wl.cache_v[sl].cpu(), wl.cache_len[sl].cpu(),
            wl.ring_k[sl].cpu(), wl.ring_v[sl].cpu(), wl.ring_len[sl].cpu(),
            wl.cur_k[sl].cpu(), wl.cur_v[sl].cpu(), wl.pred_k[sl].cpu(), wl.pred_v[sl].cpu())
        err = (out[sl].float().cpu() - ref).abs()
        assert float(err.max()) <= 2e-3 and float(err.mean()) <= 2e-4, (s0, float(err.max()), float(err.mean()))


def _head_boundary_rows(n):
    """Rows next to both ends of a head and around every multiple of 128, plus a coarse sweep."""
    rows = set(range(0, 6)) | set(range(n - 6, n)) | set(range(0, n, 251))
    for m in range(128, n, 128):
        rows |= {m - 1, m}
    rows |= set(range(n - n % 128 - 3, n - n % 128 + 3))
    return np.array(sorted(r for r in rows if 0 <= r < n))


@pytest.mark.parametrize("shape", [(1, 12, 4032, 64), (8, 8, 4032, 64)])
def test_standard_attention_long_context_shapes(shape):
    """The reference's long-context regression shapes for the Standard kernel: T = 4032 is not a
    multiple of 128, so the last tile of a head is ragged; the rows around every head boundary
    (and a sweep in between) of several heads against the oracle."""
    import sps_b200
    B, H, T, D = shape
    g = torch.Generator().manual_seed(4032 + B)
    q, k, v = (torch.randn(B, H, T, D, generator=g).bfloat16() for _ in range(3))
    docs = torch.zeros(B, T, dtype=torch.int64)
    docs[:, 1500:] = 1
    docs[:, 3000:] = 2
    dev = _dev()
    out = sps_b200.full_attention(q.to(dev), k.to(dev), v.to(dev), 1 / math.sqrt(D), False, docs.to(dev))
    sps_b200.check_device_status()
    rows = _head_boundary_rows(T)
    for b, h in {(0, 0), (0, H - 1), (B - 1, H // 2), (B - 1, H - 1)}:
        ref = orc.prefill_attention(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], 1 / math.sqrt(D),
                                    persistent_parity=orc.PARITY_NONE, docs=docs[b:b + 1], rows=rows)
        _check(out[b:b + 1, h:h + 1][:, :, torch.from_numpy(rows).to(dev)], ref)
    # a value that ran over from a neighbouring head would show as a wrong normalisation
    ones = torch.ones_like(v).to(dev)
    o1 = sps_b200.full_attention(q.to(dev), k.to(dev), ones, 1 / math.sqrt(D), False, docs.to(dev))
    assert float((o1.float() - 1).abs().max()) <= 8e-3


@pytest.mark.parametrize("reverse", [False, True])
def test_sps_attention_long_context_doubled_length(reverse):
    """The same length for the SPS kernels: 4032 tokens doubled to N = 8064 rows (63 query tiles
    of 128), three heads, both persistent parities."""
    import sps_b200
    B, H, N, D, w = 2, 3, 8064, 64, 64
    g = torch.Generator().manual_seed(8064 + int(reverse))
    q, k, v = (torch.randn(B, H, N, D, generator=g).bfloat16() for _ in range(3))
    docs = torch.zeros(B, N // 2, dtype=torch.int64)
    docs[0, 700:] = 1
    docs[0, 2900:] = 2
    docs[1, 4000:] = 1
    docs = docs.repeat_interleave(2, dim=1)
    dev = _dev()
    fn = sps_b200.reverse_sps_sliding_attention if reverse else sps_b200.sps_sliding_attention
    out = fn(q.to(dev), k.to(dev), v.to(dev), 1 / math.sqrt(D), w, documents_idx_BxT=docs.to(dev))
    sps_b200.check_device_status()
    rows = _head_boundary_rows(N)
    for b, h in ((0, 0), (0, 2), (1, 1), (1, 2)):
        ref = orc.prefill_attention(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], 1 / math.sqrt(D),
                                    persistent_parity=orc.PARITY_ODD if reverse else orc.PARITY_EVEN,
                                    temporary_window=w, docs=docs[b:b + 1], rows=rows)
        _check(out[b:b + 1, h:h + 1][:, :, torch.from_numpy(rows).to(dev)], ref)
