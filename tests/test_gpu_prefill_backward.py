"""Backward of the prefill attention (dQ, dK, dV) through the C ABI against the reference's
gradients (golden vectors from autograd through its SDPA oracles) and the CPU gradient oracle.
Tolerance: the reference's own, atol = rtol = 4e-2 (test_sps_attention.py:129-131), plus a
mean-abs bound that catches a wrong tile without being tripped by bf16 rounding."""

import math

import numpy as np
import pytest
import torch

from oracle import sps_oracle as orc
from tests.golden.loader import load_golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def grads():
    return load_golden(grads=True)


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _run(q, k, v, g, fn, dtype=torch.bfloat16):
    import sps_b200
    dev = torch.device("cuda:0")
    qs = [x.to(dev, dtype).requires_grad_(True) for x in (q, k, v)]
    out = fn(*qs)
    out.backward(g.to(dev, dtype))
    sps_b200.check_device_status(dev)
    return out.detach().float().cpu(), [x.grad.float().cpu() for x in qs]


def _close(got, ref, what):
    for x, r, key in zip(got, ref, ("dq", "dk", "dv")):
        err = (x - r).abs()
        bound = 4e-2 + 4e-2 * r.abs()
        assert bool((err <= bound).all()), (what, key, float(err.max()))
        assert float(err.mean()) <= 4e-3 + 4e-3 * float(r.abs().mean()), (what, key, float(err.mean()))


@pytest.mark.parametrize("tag", ["t16_nodoc", "t16_doc", "n200", "n384", "n256_d128"])
def test_sps_backward_matches_reference_gradients(grads, tag):
    import sps_b200
    name = f"grad_sps_{tag}"
    q, k, v, g = (_t(grads[f"{name}_{x}"]) for x in ("q", "k", "v", "do"))
    docs = _t(grads[f"{name}_docs"]).cuda() if f"{name}_docs" in grads else None
    w = int(grads[f"{name}_w"])
    _, got = _run(q, k, v, g, lambda a, b, c: sps_b200.sps_sliding_attention(
        a, b, c, 1.0 / math.sqrt(q.shape[-1]), w, documents_idx_BxT=docs))
    _close(got, [_t(grads[f"{name}_{x}"]) for x in ("dq", "dk", "dv")], name)


def test_full_backward_matches_reference_gradients(grads):
    import sps_b200
    q, k, v, g = (_t(grads[f"grad_full_{x}"]) for x in ("q", "k", "v", "do"))
    docs = _t(grads["grad_full_docs"]).cuda()
    _, got = _run(q, k, v, g, lambda a, b, c: sps_b200.full_attention(a, b, c, 0.125, documents_idx_BxT=docs))
    _close(got, [_t(grads[f"grad_full_{x}"]) for x in ("dq", "dk", "dv")], "full")


@pytest.mark.parametrize("rem", [0, 1])
def test_persistent_window_backward_matches_reference_gradients(grads, rem):
    import sps_b200
    name = f"grad_pkw{rem}"
    q, k, v, g = (_t(grads[f"{name}_{x}"]) for x in ("q", "k", "v", "do"))
    fn = sps_b200.sps_sliding_attention if rem == 0 else sps_b200.reverse_sps_sliding_attention
    _, got = _run(q, k, v, g, lambda a, b, c: fn(a, b, c, 0.125, 2, persistent_key_window=5))
    _close(got, [_t(grads[f"{name}_{x}"]) for x in ("dq", "dk", "dv")], name)


def _packed_docs(B, T, mean, seed):
    rng = np.random.default_rng(seed)
    rows = []
    for _ in range(B):
        ids, d = [], 0
        while len(ids) < T:
            ids += [d] * int(rng.geometric(1.0 / mean))
            d += 1
        rows.append(ids[:T])
    return torch.tensor(rows).repeat_interleave(2, dim=1)


CASES = [
    # (B, H, N, D, parity, w, pw, docs mean (0 none, -1 non-monotone), dtype)
    (1, 2, 1024, 64, 0, 64, None, 150, torch.bfloat16),
    (2, 1, 1536, 64, 1, 32, None, 300, torch.bfloat16),
    (1, 2, 1000, 64, 0, 5, 40, 0, torch.bfloat16),
    (1, 1, 1024, 128, 0, 64, None, 200, torch.bfloat16),
    (1, 2, 768, 128, -1, 0, None, 100, torch.float16),
    (1, 1, 640, 64, 0, 16, None, -1, torch.bfloat16),
    (1, 1, 2048, 64, 0, 2048, None, 0, torch.bfloat16),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"N{c[2]}D{c[3]}p{c[4]}w{c[5]}docs{c[7]}")
def test_backward_matches_gradient_oracle(case):
    import sps_b200
    B, H, N, D, parity, w, pw, mean, dtype = case
    gen = torch.Generator().manual_seed(N + D + w)
    q, k, v, g = (torch.randn(B, H, N, D, generator=gen).to(dtype).float() for _ in range(4))
    docs = None
    if mean > 0:
        docs = _packed_docs(B, N // 2, mean, N) if parity >= 0 else _packed_docs(B, N, mean, N)[:, ::2].contiguous()
    elif mean < 0:
        docs = torch.randint(0, 3, (B, N // 2), generator=gen).repeat_interleave(2, dim=1)   # ids come back
    scale = 1.0 / math.sqrt(D)
    out, got = _run(q, k, v, g, lambda a, b, c: sps_b200.prefill_attention(
        a, b, c, scale, persistent_parity=parity, temporary_window=w, persistent_window=pw,
        documents_idx=None if docs is None else docs.cuda()), dtype)
    ref_out = orc.prefill_attention(q, k, v, scale, persistent_parity=parity, temporary_window=w,
                                    persistent_window=pw, docs=docs)
    assert float((out - ref_out).abs().max()) <= 2e-2
    ref = orc.prefill_attention_grads(q, k, v, g, scale, persistent_parity=parity, temporary_window=w,
                                      persistent_window=pw, docs=docs)
    _close(got, ref, str(case))


def test_backward_random_shapes_and_masks():
    """Seeded random sweep: lengths that are no multiple of any tile, both parities and the Standard
    rule, windows from 0 to the whole sequence, persistent windows, the skip flag, packed /
    non-monotone / no documents, bf16 and fp16, head_dim 64 and 128."""
    import sps_b200
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(7)
    for case in range(40):
        D = int(rng.choice([64, 128]))
        parity = int(rng.choice([0, 1, -1]))
        N = int(rng.integers(1, 500)) * 2 if parity >= 0 else int(rng.integers(1, 1000))
        B, H = int(rng.integers(1, 3)), int(rng.integers(1, 3))
        w = int(rng.choice([0, 1, 3, 17, 64, 200, N]))
        pw = None if parity < 0 or rng.random() < 0.6 else int(rng.choice([-1, 0, 2, 40]))
        flags = int(rng.random() < 0.2) if parity >= 0 else 0
        kind = str(rng.choice(["none", "mono", "general"]))
        T = N // 2 if parity >= 0 else N
        docs = None
        if kind == "mono":
            docs = _packed_docs(B, T, int(rng.choice([3, 20, 150])), case)[:, ::2].contiguous()
        elif kind == "general":
            docs = torch.from_numpy(rng.integers(0, 3, (B, T)))
        if docs is not None and parity >= 0:
            docs = docs.repeat_interleave(2, dim=1)
        dtype = torch.bfloat16 if rng.random() < 0.8 else torch.float16
        gen = torch.Generator().manual_seed(case)
        q, k, v, g = (torch.randn(B, H, N, D, generator=gen).to(dtype).float() for _ in range(4))
        scale = 1.0 / math.sqrt(D)
        _, got = _run(q, k, v, g, lambda a, b, c: sps_b200.prefill_attention(
            a, b, c, scale, persistent_parity=parity, temporary_window=w, persistent_window=pw,
            documents_idx=None if docs is None else docs.to(dev), mask_flags=flags), dtype)
        ref = orc.prefill_attention_grads(q, k, v, g, scale, persistent_parity=parity, temporary_window=w,
                                          persistent_window=pw, docs=docs, mask_flags=flags)
        for x in got:
            assert bool(torch.isfinite(x).all()), case
        _close(got, ref, (case, D, parity, N, w, pw, flags, kind))


def test_backward_is_linear_in_the_output_gradient():
    """At a multi-tile size: backward(a * g1 + g2) == a * backward(g1) + backward(g2) up to rounding."""
    import sps_b200
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(5)
    B, H, N, D, w = 2, 2, 2048, 64, 64
    q, k, v = (torch.randn(B, H, N, D, generator=gen).bfloat16().to(dev) for _ in range(3))
    docs = _packed_docs(B, N // 2, 400, 9).to(dev)
    o, lse = sps_b200.prefill_attention(q, k, v, 0.125, persistent_parity=0, temporary_window=w,
                                        documents_idx=docs, return_lse=True)
    g1, g2 = (torch.randn(B, H, N, D, generator=gen).bfloat16().to(dev) for _ in range(2))
    bw = lambda g: [x.float() for x in sps_b200.attention.prefill_attention_backward(
        q, k, v, o, lse, g, 0.125, persistent_parity=0, temporary_window=w, documents_idx=docs)]
    a, b, c = bw(g1), bw(g2), bw((2 * g1.float() + g2.float()).bfloat16())
    for x, y, z in zip(a, b, c):
        ref = 2 * x + y
        assert float((z - ref).abs().max()) <= 6e-2 + 3e-2 * float(ref.abs().max())
        assert float((z - ref).abs().mean()) <= 1e-2 * float(ref.abs().mean()) + 1e-3
    sps_b200.check_device_status(dev)


@pytest.mark.parametrize("d", [64, 128])
def test_backward_reads_and_writes_token_major_views_in_place(d):
    """The layouts the reference's modules produce (sps/core.py:45-55): q, k, v as transposed views
    of a fused [B, N, 3*H*D] projection, dO as the transposed view autograd hands back.  Same
    gradients as the dense call, bit for bit, and the q / k / v gradients come back token-major."""
    import sps_b200
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(3 + d)
    B, H, N, w = 2, 2, 640, 24
    qkv = torch.randn(B, N, 3 * H * d, generator=gen).bfloat16().to(dev)
    docs = _packed_docs(B, N // 2, 90, 4).to(dev)
    views = [t.view(B, N, H, d).transpose(1, 2) for t in qkv.split(H * d, dim=2)]
    g_tm = torch.randn(B, N, H, d, generator=gen).bfloat16().to(dev).transpose(1, 2)
    scale = 1.0 / math.sqrt(d)
    o, lse = sps_b200.prefill_attention(*views, scale, persistent_parity=0, temporary_window=w,
                                        documents_idx=docs, return_lse=True)
    bw = sps_b200.attention.prefill_attention_backward
    got = bw(*views, o, lse, g_tm, scale, persistent_parity=0, temporary_window=w, documents_idx=docs)
    dense = [t.contiguous() for t in views]
    want = bw(*dense, o.contiguous(), lse, g_tm.contiguous(), scale, persistent_parity=0, temporary_window=w,
              documents_idx=docs)
    for x, y in zip(got, want):
        assert x.stride(2) > x.stride(1)                 # token-major
        assert torch.equal(x, y)
    # and through autograd down to the fused projection
    leaf = qkv.clone().requires_grad_(True)
    lv = [t.view(B, N, H, d).transpose(1, 2) for t in leaf.split(H * d, dim=2)]
    out = sps_b200.sps_sliding_attention(*lv, scale, w, documents_idx_BxT=docs)
    out.transpose(1, 2).reshape(B, N, H * d).backward(g_tm.transpose(1, 2).reshape(B, N, H * d))
    ref = torch.cat([t.transpose(1, 2).reshape(B, N, H * d) for t in want], dim=2)
    assert torch.equal(leaf.grad, ref)
    sps_b200.check_device_status(dev)


@pytest.mark.parametrize("d", [64, 128])
def test_backward_is_deterministic_for_every_tile_count(d):
    """No atomics anywhere: repeated calls give identical bits.  Lengths chosen so that the number
    of streamed tiles per block takes every residue modulo 4 (at head_dim 128 two warpgroups take
    alternate tiles and the one that owns the last tile writes the result)."""
    import sps_b200
    dev = torch.device("cuda:0")
    bw = sps_b200.attention.prefill_attention_backward
    for n in (128, 192, 320, 448, 684, 1100):
        gen = torch.Generator().manual_seed(n)
        q, k, v, g = (torch.randn(1, 2, n, d, generator=gen).bfloat16().to(dev) for _ in range(4))
        scale = 1.0 / math.sqrt(d)
        o, lse = sps_b200.prefill_attention(q, k, v, scale, persistent_parity=1, temporary_window=200, return_lse=True)
        first = bw(q, k, v, o, lse, g, scale, persistent_parity=1, temporary_window=200)
        for _ in range(6):
            again = bw(q, k, v, o, lse, g, scale, persistent_parity=1, temporary_window=200)
            for x, y in zip(first, again):
                assert torch.equal(x, y), (n, d)
    sps_b200.check_device_status(dev)


def test_backward_needs_a_supported_head_dim():
    import sps_b200
    dev = torch.device("cuda:0")
    q = torch.randn(1, 1, 64, 32, device=dev, dtype=torch.bfloat16, requires_grad=True)
    with pytest.raises(RuntimeError, match="forward only"):
        sps_b200.sps_sliding_attention(q, q, q, 0.2, 4)
