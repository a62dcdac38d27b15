"""The two decode kernels behind spsattn_decode_step — tensor cores (TMA + tcgen05) and CUDA cores —
against each other and against the CPU oracle, on the cases that stress the tile logic of the
tensor-core kernel: lengths on and around tile and chunk borders, empty and full segments,
per-head lengths, one and two queries, query masks, NaN stored past the live length, fp16.
Needs a B200."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import sps_oracle as orc


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


@pytest.fixture
def decode_path():
    """Yields a setter for the kernel choice and restores the automatic choice afterwards."""
    from sps_b200 import _lib
    lib = _lib.load()
    yield lambda p: _lib.check(lib.spsattn_debug_decode_path(p), "decode_path")
    lib.spsattn_debug_decode_path(0)


def _case(seed, S, H, D, nq, caps, lens, dtype, poison=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(S, nq, H, D, generator=g).to(dtype)
    segs = []
    for cap, ln in zip(caps, lens):
        k = torch.randn(S, H, cap, D, generator=g).to(dtype)
        v = torch.randn(S, H, cap, D, generator=g).to(dtype)
        ln = torch.as_tensor(ln, dtype=torch.long)
        if poison:   # whatever sits past the live length must not matter
            full = ln.view(S, -1).expand(S, H) if ln.dim() == 2 else ln.view(S, 1).expand(S, H)
            dead = torch.arange(cap).view(1, 1, cap) >= full.unsqueeze(2)
            k[dead] = float("nan")
            v[dead] = float("nan")
        segs.append((k, v, ln))
    cur = [torch.randn(S, H, D, generator=g).to(dtype) for _ in range(4)]
    return q, segs, cur


def _run(q, segs, cur, nq, masks=None, caps=None):
    import sps_b200
    dev = _dev()
    ksegs = [sps_b200.KVSegment(k.to(dev), v.to(dev), ln.to(dev), max_len_cap=None if caps is None else caps[i])
             for i, (k, v, ln) in enumerate(segs)]
    if nq == 2:
        extras = [(cur[0].to(dev), cur[1].to(dev), 0b11), (cur[2].to(dev), cur[3].to(dev), 0b10)]
    else:
        extras = [(cur[0].to(dev), cur[1].to(dev), 1)]
    return sps_b200.decode_attention(q.to(dev), ksegs, extras, segment_query_masks=masks).cpu()


def _oracle(q, segs, cur, nq, masks=None, caps=None):
    osegs = []
    for i, (k, v, ln) in enumerate(segs):
        sg = orc.Segment(k, v, ln, max_len_cap=None if caps is None else caps[i])
        if masks is not None:
            sg.query_mask = masks[i]
        osegs.append(sg)
    extras = ([(cur[0], cur[1], 0b11), (cur[2], cur[3], 0b10)] if nq == 2 else [(cur[0], cur[1], 1)])
    return orc.decode_attention(q, osegs, extras)


BORDER_LENS = [0, 1, 63, 64, 127, 128, 129, 255, 256, 257, 511, 512, 513, 700]


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("nq", [1, 2])
def test_lengths_around_tile_and_chunk_borders(decode_path, D, nq):
    S, H, cap = len(BORDER_LENS), 2, 700
    ring_lens = [(7 * i) % 9 for i in range(S)]
    q, segs, cur = _case(3 + D + nq, S, H, D, nq, (8, cap), (ring_lens, BORDER_LENS), torch.bfloat16,
                         poison=True)
    ref = _oracle(q, segs, cur, nq)
    outs = {}
    for path in (2, 1):
        decode_path(path)
        outs[path] = _run(q, segs, cur, nq)
        assert torch.isfinite(outs[path]).all()
        err = (outs[path] - ref).abs()
        assert float(err.max()) <= 3e-3 and float(err.mean()) <= 3e-4, (path, float(err.max()))
    # the tensor-core kernel rounds p to bf16 before the second product, the CUDA-core one does not
    assert float((outs[1] - outs[2]).abs().max()) <= 4e-3


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
def test_per_head_lengths_masks_and_caps(decode_path, D, dtype):
    S, H = 6, 3
    g = torch.Generator().manual_seed(17)
    per_head = torch.randint(0, 901, (S, H), generator=g)
    per_head[0] = 0
    per_head[1] = 900
    ring = torch.tensor([0, 64, 64, 13, 1, 64])
    q, segs, cur = _case(29 + D, S, H, D, 2, (64, 900), (ring, per_head), dtype)
    masks, caps = [0b10, 0b11], [48, 777]          # input query skips the ring; caps below the storage
    ref = _oracle(q, segs, cur, 2, masks, caps)
    for path in (2, 1):
        decode_path(path)
        out = _run(q, segs, cur, 2, masks, caps)
        err = (out - ref).abs()
        assert float(err.max()) <= 4e-3 and float(err.mean()) <= 4e-4, (path, float(err.max()))


def test_large_scores_move_the_reference_point(decode_path):
    """Scores that grow along the cache force the lazy reference point of the tensor-core kernel
    to move (its accumulator rows are rescaled in tensor memory)."""
    S, H, D, cap = 2, 2, 64, 640
    q, segs, cur = _case(41, S, H, D, 2, (cap,), ([cap, 500],), torch.bfloat16)
    k, v, ln = segs[0]
    ramp = torch.linspace(0.0, 6.0, cap).view(1, 1, cap, 1)
    k = (k.float() + ramp * q[:, 0].float().unsqueeze(2) / q[:, 0].float().norm(dim=-1, keepdim=True).unsqueeze(2)
         ).to(torch.bfloat16)
    segs = [(k, v, ln)]
    ref = _oracle(q, segs, cur, 2)
    decode_path(2)
    out = _run(q, segs, cur, 2)
    err = (out - ref).abs()
    assert float(err.max()) <= 4e-3, float(err.max())


def test_forcing_the_tensor_core_kernel_where_it_cannot_run_is_an_error(decode_path):
    import sps_b200
    from sps_b200 import _lib
    dev = _dev()
    decode_path(2)
    q = torch.randn(2, 2, 2, 32, device=dev).to(torch.bfloat16)
    k = torch.randn(2, 2, 8, 32, device=dev).to(torch.bfloat16)
    seg = sps_b200.KVSegment(k, k, torch.full((2,), 8, dtype=torch.long, device=dev))
    with pytest.raises(_lib.SpsAttnError):
        sps_b200.decode_attention(q, [seg], [])
    decode_path(0)
    assert float(sps_b200.decode_attention(q, [seg], []).abs().max()) > 0.0
