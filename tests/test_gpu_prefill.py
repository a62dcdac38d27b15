"""Parity of the CUDA prefill path (through the C ABI, via the reference-signature wrappers)
against the CPU oracle and the committed reference vectors.  Needs a B200."""

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


def _cuda(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(_dev()).to(dtype)


@pytest.fixture(params=[0, 2], ids=["tiles64", "persistent128"], autouse=True)
def prefill_kernel(request):
    """Every test of this file runs against both tensor-core kernels that serve head_dim 64: the
    default one (64-key tiles) and the persistent one (128-key tiles, P in tensor memory)."""
    from sps_b200 import _lib
    lib = _lib.load()
    _lib.check(lib.spsattn_debug_prefill_path(request.param), "spsattn_debug_prefill_path")
    yield request.param
    _lib.check(lib.spsattn_debug_prefill_path(0), "spsattn_debug_prefill_path")


@pytest.mark.parametrize("tag", ["nodoc", "doc", "n8", "n24", "n200", "n384"])
def test_sps_matches_reference_vectors(golden, tag):
    import sps_b200
    p = f"sps_{tag}"
    q, k, v = (_cuda(golden[f"{p}_{x}"], torch.bfloat16) for x in "qkv")
    docs = _cuda(golden[p + "_docs"], torch.int64) if (p + "_docs") in golden else None
    with torch.no_grad():
        out = sps_b200.sps_sliding_attention(q, k, v, 1 / 8.0, int(golden[p + "_w"]),
                                             warp_specialize=False, documents_idx_BxT=docs)
    sps_b200.check_device_status()
    _check(out, golden[p + "_out"])


def test_sps_cfg0_shape_matches_reference_vectors(golden):
    import sps_b200
    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 8, 512, 64, generator=gen) for _ in range(3))
    docs = _cuda(golden["sps_cfg0_docs"], torch.int64)
    qb, kb, vb = (x.to(_dev()).bfloat16() for x in (q, k, v))
    out = sps_b200.sps_sliding_attention(qb, kb, vb, 1 / 8.0, 64, documents_idx_BxT=docs)
    sps_b200.check_device_status()
    # against the oracle on the same bf16-rounded inputs (tight) ...
    ref = orc.prefill_attention(qb.float().cpu(), kb.float().cpu(), vb.float().cpu(), 1 / 8.0,
                                temporary_window=64, docs=docs.cpu())
    _check(out, ref)
    # ... and against the reference's fp32 run of the fp32 inputs (input rounding included)
    _check(out[:, [0, 5]], golden["sps_cfg0_out_h0h5"], max_abs=4e-2, mean_abs=4e-3)


@pytest.mark.parametrize("tag,pw,w,dtype", [("pkw", 1, 8, torch.float16), ("pkwL", 5, 2, torch.bfloat16)])
@pytest.mark.parametrize("rem", [0, 1])
def test_persistent_key_window_matches_reference_vectors(golden, tag, pw, w, dtype, rem):
    import sps_b200
    p = f"{tag}{rem}"
    q, k, v = (_cuda(golden[f"{p}_{x}"], dtype) for x in "qkv")
    fn = sps_b200.sps_sliding_attention if rem == 0 else sps_b200.reverse_sps_sliding_attention
    out = fn(q, k, v, 1 / 8.0, w, warp_specialize=False, persistent_key_window=pw)
    sps_b200.check_device_status()
    _check(out, golden[p + "_out"], max_abs=2e-2, mean_abs=4e-3)


@pytest.mark.parametrize("tag,d", [("full_n128", 64), ("full_n200", 128)])
def test_full_attention_matches_reference_vectors(golden, tag, d):
    import sps_b200
    q, k, v = (_cuda(golden[f"{tag}_{x}"], torch.bfloat16) for x in "qkv")
    docs = _cuda(golden[tag + "_docs"], torch.int64)
    out = sps_b200.full_attention(q, k, v, 1 / math.sqrt(d), documents_idx_BxT=docs)
    _check(out, golden[tag + "_out"])
    out = sps_b200.full_attention(q, k, v, 1 / math.sqrt(d), documents_idx_BxT=docs.to(torch.int32))
    _check(out, golden[tag + "_out"])
    out = sps_b200.full_attention(q, k, v, 1 / math.sqrt(d))
    sps_b200.check_device_status()
    _check(out, golden[tag + "_out_nodoc"])


def _random_docs(rng, batch, n, mode):
    if mode == "none":
        return None
    if mode == "mono":
        steps = rng.random((batch, n)) < 0.05
        return np.cumsum(steps, axis=1).astype(np.int64)
    if mode == "per_token":
        steps = rng.random((batch, n // 2)) < 0.1
        return np.repeat(np.cumsum(steps, axis=1), 2, axis=1).astype(np.int64)
    return rng.integers(0, 3, size=(batch, n)).astype(np.int64)    # arbitrary, ids reappear


@pytest.mark.parametrize("parity", [0, 1, -1])
@pytest.mark.parametrize("docs_mode", ["none", "mono", "per_token", "arbitrary"])
def test_mask_is_bit_exact(parity, docs_mode):
    """The visibility the kernels apply (their own interval arithmetic + document pre-pass,
    evaluated on the device) equals the integer rule of the oracle, element for element."""
    from sps_b200 import attention
    rng = np.random.default_rng(abs(parity) * 10 + len(docs_mode))
    for n, w, pw, flags in ((8, 0, None, 0), (64, 3, None, 0), (258, 64, None, 0), (300, 7, 2, 0),
                            (130, 5, -1, 0), (200, 1000, None, 0), (96, 4, None, 1), (514, -1, 0, 0)):
        if parity == -1 and (pw is not None or flags):
            continue
        docs = _random_docs(rng, 2, n, docs_mode)
        for dt in (torch.int64, torch.int32):
            dd = None if docs is None else torch.from_numpy(docs).to(_dev()).to(dt)
            vis = attention.visibility(n, persistent_parity=parity, temporary_window=w,
                                       persistent_window=pw, documents_idx=dd, mask_flags=flags,
                                       batch=2).cpu().numpy()
            for b in range(2):
                want = orc.visible_mask(n, persistent_parity=parity, temporary_window=w,
                                        persistent_window=pw, mask_flags=flags,
                                        docs_row=None if docs is None else docs[b])
                assert np.array_equal(vis[b], want), (n, w, pw, flags, docs_mode, b)


@pytest.mark.parametrize("d", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("parity", [0, 1, -1])
def test_random_shapes_match_oracle(d, parity):
    import sps_b200
    rng = np.random.default_rng(d + parity)
    for n, w, mode in ((136, 9, "mono"), (520, 64, "per_token"), (256, 300, "none"), (200, 3, "arbitrary")):
        g = torch.Generator().manual_seed(n + d)
        q, k, v = (torch.randn(2, 3, n, d, generator=g).bfloat16() for _ in range(3))
        docs = _random_docs(rng, 2, n, mode)
        dd = None if docs is None else torch.from_numpy(docs)
        out = sps_b200.prefill_attention(q.to(_dev()), k.to(_dev()), v.to(_dev()), 1 / math.sqrt(d),
                                         persistent_parity=parity, temporary_window=w,
                                         documents_idx=None if dd is None else dd.to(_dev()))
        sps_b200.check_device_status()
        ref = orc.prefill_attention(q, k, v, 1 / math.sqrt(d), persistent_parity=parity,
                                    temporary_window=w, docs=dd)
        _check(out, ref)


def test_lse_and_flag_mode_match_oracle():
    import sps_b200
    g = torch.Generator().manual_seed(3)
    n, d = 392, 64
    q, k, v = (torch.randn(1, 2, n, d, generator=g).bfloat16() for _ in range(3))
    docs = torch.from_numpy(_random_docs(np.random.default_rng(5), 1, n, "per_token"))
    for flags, w in ((0, 16), (orc.FLAG_PERSISTENT_Q_SKIPS_TEMPORARY, 15)):
        out, lse = sps_b200.prefill_attention(q.to(_dev()), k.to(_dev()), v.to(_dev()), 0.125,
                                              persistent_parity=0, temporary_window=w,
                                              documents_idx=docs.to(_dev()), mask_flags=flags,
                                              return_lse=True)
        ref, ref_lse = orc.prefill_attention(q, k, v, 0.125, temporary_window=w, docs=docs,
                                             mask_flags=flags, return_lse=True)
        _check(out, ref)
        assert float((lse.cpu() - ref_lse).abs().max()) < 2e-2


def test_full_attention_no_cross_document_leakage():
    """NaN-poisoned keys/values of document 2 must not reach document 1
    (src/modeling/tests/attention/triton/test_document_leakage.py:27-72)."""
    import sps_b200
    torch.manual_seed(2024)
    B, H, T, D = 1, 2, 256, 64
    half = T // 2
    q, k, v = (torch.randn(B, H, T, D, device=_dev()).bfloat16() for _ in range(3))
    solo = sps_b200.full_attention(q[:, :, :half], k[:, :, :half], v[:, :, :half], 0.125)
    kp, vp = k.clone(), v.clone()
    kp[:, :, half:] = float("nan")
    vp[:, :, half:] = float("nan")
    docs = torch.zeros(B, T, device=_dev(), dtype=torch.int32)
    docs[:, half:] = 1
    out = sps_b200.full_attention(q, kp, vp, 0.125, documents_idx_BxT=docs)
    doc1 = out[:, :, :half]
    assert torch.isfinite(doc1).all()
    torch.testing.assert_close(doc1.float(), solo.float(), atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("fn_name", ["sps_sliding_attention", "reverse_sps_sliding_attention"])
def test_sliding_attention_no_cross_document_leakage(fn_name):
    """test_document_leakage.py:75-131 (fp16, split on a tile boundary), both parities."""
    import sps_b200
    fn = getattr(sps_b200, fn_name)
    torch.manual_seed(2025)
    B, H, t, D = 1, 2, 128, 64
    two_t, half = 2 * t, t
    q, k, v = (torch.randn(B, H, two_t, D, device=_dev()).half() for _ in range(3))
    solo = fn(q[:, :, :half], k[:, :, :half], v[:, :, :half], 0.125, 4, warp_specialize=False)
    kp, vp = k.clone(), v.clone()
    kp[:, :, half:] = float("nan")
    vp[:, :, half:] = float("nan")
    docs = torch.zeros((B, two_t), device=_dev(), dtype=torch.int64)
    docs[:, half:] = 1
    out = fn(q, kp, vp, 0.125, 4, warp_specialize=False, documents_idx_BxT=docs)
    doc1 = out[:, :, :half]
    assert torch.isfinite(doc1).all()
    torch.testing.assert_close(doc1.float(), solo.float(), atol=3e-2, rtol=3e-2)


def test_full_size_properties_and_spot_rows():
    """At the benchmark's full prefill size ([8,12,8192,64], w=64, packed documents):
    V = 1 gives O = 1 on every row (normalisation, no row without keys), attention is linear
    in V, and a sample of rows matches the oracle evaluated on those rows only."""
    import sps_b200
    from sps_b200 import workloads
    wl = workloads.make_prefill("cfg1_s_scale", _dev())
    ones = torch.ones_like(wl.v)
    o1 = sps_b200.sps_sliding_attention(wl.q, wl.k, ones, wl.sm_scale, wl.window, documents_idx_BxT=wl.docs)
    assert float((o1.float() - 1).abs().max()) <= 8e-3
    out = sps_b200.sps_sliding_attention(wl.q, wl.k, wl.v, wl.sm_scale, wl.window, documents_idx_BxT=wl.docs)
    v2 = torch.randn_like(wl.v)
    oa = sps_b200.sps_sliding_attention(wl.q, wl.k, v2, wl.sm_scale, wl.window, documents_idx_BxT=wl.docs)
    ob = sps_b200.sps_sliding_attention(wl.q, wl.k, (wl.v.float() + v2.float()).bfloat16(), wl.sm_scale,
                                        wl.window, documents_idx_BxT=wl.docs)
    sps_b200.check_device_status()
    lin = (ob.float() - out.float() - oa.float()).abs()
    assert float(lin.max()) <= 6e-2 and float(lin.mean()) <= 4e-3
    rows = np.unique(np.concatenate([np.arange(0, 8192, 397), np.arange(8192 - 130, 8192),
                                     np.random.default_rng(0).integers(0, 8192, 64)]))
    for b, h in ((0, 0), (3, 7), (7, 11)):
        ref = orc.prefill_attention(wl.q[b:b + 1, h:h + 1].cpu(), wl.k[b:b + 1, h:h + 1].cpu(),
                                    wl.v[b:b + 1, h:h + 1].cpu(), wl.sm_scale, temporary_window=wl.window,
                                    docs=wl.docs[b:b + 1].cpu(), rows=rows)
        _check(out[b:b + 1, h:h + 1][:, :, torch.from_numpy(rows).to(out.device)], ref)


def test_prefill_with_documents_replays_from_a_cuda_graph():
    """With document ids the attention kernel is launched as a programmatic dependent of the
    pre-pass.  The pair must survive stream capture: two captured calls, replayed twice, give the
    eager result bit for bit, and back-to-back eager calls on a side stream do too."""
    import sps_b200
    from sps_b200 import workloads
    wl = workloads.make_prefill("cfg1_s_scale", _dev(), batch_slice=slice(0, 2), head_slice=slice(0, 4))
    ref = torch.empty_like(wl.q)
    out = torch.empty_like(wl.q)

    def call(o):
        return sps_b200.prefill_attention(wl.q, wl.k, wl.v, wl.sm_scale, persistent_parity=0,
                                          temporary_window=wl.window, documents_idx=wl.docs, out=o)
    call(ref)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        call(out)
        call(out)
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    out.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        call(out)
        call(out)
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    sps_b200.check_device_status()
    assert torch.equal(out, ref)


def test_full_window_config_spot_rows():
    """[.,.,8192,128], w = 4096, one document: the least sparse mask (head-sharded in the bench)."""
    import sps_b200
    from sps_b200 import workloads
    wl = workloads.make_prefill("cfg4_full_window", _dev(), batch_slice=slice(0, 1), head_slice=slice(0, 2))
    out = sps_b200.sps_sliding_attention(wl.q, wl.k, wl.v, wl.sm_scale, wl.window)
    sps_b200.check_device_status()
    rows = np.unique(np.concatenate([np.arange(0, 8192, 509), np.arange(8192 - 66, 8192)]))
    ref = orc.prefill_attention(wl.q.cpu(), wl.k.cpu(), wl.v.cpu(), wl.sm_scale,
                                temporary_window=wl.window, rows=rows)
    _check(out[:, :, torch.from_numpy(rows).to(out.device)], ref)


def test_argument_errors():
    import sps_b200
    q = torch.randn(1, 1, 7, 64, device=_dev()).bfloat16()
    with pytest.raises(AssertionError):
        sps_b200.sps_sliding_attention(q, q, q, 0.125, 2)           # odd doubled length
    q = torch.randn(1, 1, 8, 48, device=_dev()).bfloat16()
    with pytest.raises(AssertionError):
        sps_b200.sps_sliding_attention(q, q, q, 0.125, 2)           # head_dim
    q = torch.randn(1, 1, 8, 32, device=_dev()).bfloat16().requires_grad_(True)
    with pytest.raises(RuntimeError):
        sps_b200.sps_sliding_attention(q, q, q, 0.125, 2)           # head_dim 32 is forward only
    with pytest.raises(RuntimeError):
        sps_b200.sps_sliding_attention(q.detach().cpu(), q.detach().cpu(), q.detach().cpu(), 0.125, 2)


@pytest.mark.parametrize("d", [64, 128])
def test_token_major_and_fused_projection_views_need_no_copy(d):
    """The layouts the reference's modules actually pass (sps/core.py:45-55): q, k, v as transposed
    views of token-major [B, N, H, D] data, here even as slices of one fused [B, N, 3*H*D]
    projection buffer.  The kernel reads them in place and returns token-major output."""
    import sps_b200
    dev = _dev()
    B, H, N, w = 2, 3, 456, 9
    g = torch.Generator().manual_seed(d)
    qkv = torch.randn(B, N, 3 * H * d, generator=g).bfloat16().to(dev)
    q, k, v = (x.view(B, N, H, d).transpose(1, 2) for x in qkv.split(H * d, dim=2))
    assert not q.is_contiguous()
    docs = torch.from_numpy(_random_docs(np.random.default_rng(1), B, N, "per_token")).to(dev)
    out = sps_b200.sps_sliding_attention(q, k, v, 1 / math.sqrt(d), w, documents_idx_BxT=docs)
    sps_b200.check_device_status()
    assert out.shape == (B, H, N, d)
    assert out.transpose(1, 2).is_contiguous()          # y.transpose(1, 2).contiguous() is free
    ref = orc.prefill_attention(q.cpu(), k.cpu(), v.cpu(), 1 / math.sqrt(d), temporary_window=w, docs=docs.cpu())
    _check(out, ref)
    dense = sps_b200.sps_sliding_attention(q.contiguous(), k.contiguous(), v.contiguous(), 1 / math.sqrt(d), w,
                                           documents_idx_BxT=docs)
    assert torch.equal(dense, out)                      # same kernel, same tiles: bit-identical


def _ulp_close(out, ref):
    """bf16 results of fp32 math: identical up to a rare last-bit flip (products and sums of
    the complex multiply may be fused differently on the two sides)."""
    out, ref = out.float().cpu(), ref.float()
    diff = (out - ref).abs()
    ulp = ref.abs().clamp_min(1e-30) * 2.0 ** -7
    assert bool((diff <= ulp).all()), float((diff / ulp).max())
    assert float((diff > 0).float().mean()) <= 1e-3


@pytest.mark.parametrize("tag,dt", [("f32", torch.float32), ("bf16", torch.bfloat16)])
def test_rope_cast_matches_reference_vectors(golden, tag, dt):
    import sps_b200
    dev = _dev()
    g = golden
    fc = torch.view_as_complex(torch.from_numpy(g["rope_freqs"]).contiguous())
    pos = torch.from_numpy(g["rope_pos"])
    for which in ("q", "k"):
        x = torch.from_numpy(g[f"rope_{tag}_x{which}"]).to(dt).to(dev)
        out = sps_b200.rope_cast(x, fc[pos].to(dev))
        assert out.shape == (x.shape[0], x.shape[2], x.shape[1], x.shape[3]) and out.dtype == torch.bfloat16
        _ulp_close(out.transpose(1, 2), torch.from_numpy(g[f"rope_{tag}_{which}1"]))
        out = sps_b200.rope_cast(x, torch.stack([fc[pos], fc[pos + 7]]).to(dev))
        _ulp_close(out.transpose(1, 2), torch.from_numpy(g[f"rope_{tag}_{which}2"]))


def test_rope_cast_feeds_the_attention_kernel_without_copies():
    """Fused [B, N, 3*H*D] projection -> rope_cast(q), rope_cast(k), v in place -> attention:
    the whole operand path of the reference's attention module (sps/core.py:41-79) with no
    transposing copy, against the oracle."""
    import sps_b200
    dev = _dev()
    B, T, H, D, w = 2, 150, 3, 64, 6
    N = 2 * T
    g = torch.Generator().manual_seed(4)
    qkv = (torch.randn(B, N, 3 * H * D, generator=g) * 0.7).bfloat16().to(dev)
    q, k, v = (x.view(B, N, H, D) for x in qkv.split(H * D, dim=2))
    freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.outer(torch.arange(T).repeat_interleave(2).float(), freqs)
    fc = torch.polar(torch.ones_like(ang), ang).to(dev)
    qr, kr = sps_b200.rope_cast(q, fc), sps_b200.rope_cast(k, fc)
    vr = sps_b200.rope_cast(v, None)
    docs = torch.from_numpy(_random_docs(np.random.default_rng(3), B, N, "per_token")).to(dev)
    out = sps_b200.sps_sliding_attention(qr, kr, vr, 1 / math.sqrt(D), w, documents_idx_BxT=docs)
    out2 = sps_b200.sps_sliding_attention(qr, kr, v.transpose(1, 2), 1 / math.sqrt(D), w, documents_idx_BxT=docs)
    sps_b200.check_device_status()
    assert torch.equal(out, out2)                      # bf16 v is read straight from the fused buffer
    q_ref = orc.rope_cast(q.cpu(), fc.cpu()).transpose(1, 2)
    k_ref = orc.rope_cast(k.cpu(), fc.cpu()).transpose(1, 2)
    _ulp_close(qr, q_ref)
    ref = orc.prefill_attention(qr.cpu(), kr.cpu(), vr.cpu(), 1 / math.sqrt(D), temporary_window=w, docs=docs.cpu())
    _check(out, ref)
