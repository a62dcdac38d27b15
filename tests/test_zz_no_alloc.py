"""The allocation-free decode entry point (spsattn_decode_fwd_noalloc) against the regular one.

Some hosts cannot allocate device memory where they decode: the serving process has already
handed all of HBM to its own cache arena, or the step loop must avoid cudaMalloc's device-wide
synchronisation, or the binding comes through an FFI with no allocator to pass along.  For them
the library keeps a 16 MiB scratch buffer inside its own image and the caller passes inputs and
outputs only.  This test drives that entry point through the C ABI, twice in a row on different
inputs (the buffer is shared between calls and keeps the previous call's records), compares
each result with spsattn_decode_fwd on a caller-owned workspace, and checks that a problem whose
records would not fit is refused with SPSATTN_ERR_SCRATCH_LIMIT before anything is launched.
The file name sorts last so a failure here cannot hide the other tests in a -x run.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


def _problem(seed, S, H, D, cap, ring):
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(seed)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev).bfloat16()
    t = dict(q=rnd(S, 2, H, D), ck=rnd(S, H, cap, D), cv=rnd(S, H, cap, D), rk=rnd(S, H, ring, D),
             rv=rnd(S, H, ring, D), cur=[rnd(S, H, D) for _ in range(4)],
             cl=torch.randint(0, cap + 1, (S, H), generator=g, device=dev),
             rl=torch.randint(0, ring + 1, (S,), generator=g, device=dev))
    return t


def _tables(t, S, H, D, cap, ring):
    from sps_b200 import _lib
    segs = (_lib.Segment * 2)()
    for i, (k, v, ln, rows, per_head) in enumerate(((t["rk"], t["rv"], t["rl"], ring, 0),
                                                     (t["ck"], t["cv"], t["cl"], cap, 1))):
        segs[i].k, segs[i].v, segs[i].seq_offset = k.data_ptr(), v.data_ptr(), None
        segs[i].seq_stride, segs[i].head_stride, segs[i].row_stride = H * rows * D, rows * D, D
        segs[i].lengths, segs[i].lengths_per_head, segs[i].max_rows = ln.data_ptr(), per_head, rows
        segs[i].query_mask = 0b11
    extras = (_lib.Extra * 2)()
    extras[0].k, extras[0].v, extras[0].query_mask = t["cur"][0].data_ptr(), t["cur"][1].data_ptr(), 0b11
    extras[1].k, extras[1].v, extras[1].query_mask = t["cur"][2].data_ptr(), t["cur"][3].data_ptr(), 0b10
    return segs, extras


def test_noalloc_decode_matches_workspace_decode_twice_in_a_row():
    from sps_b200 import _lib
    lib = _lib.load()
    dev = _dev()
    stream = torch.cuda.current_stream().cuda_stream
    S, H, D, cap, ring = 24, 8, 64, 1500, 64
    for call, seed in enumerate((101, 202)):
        t = _problem(seed, S, H, D, cap, ring)
        segs, extras = _tables(t, S, H, D, cap, ring)
        need = lib.spsattn_decode_workspace_bytes(S, H, D, 2, segs, 2)
        assert need <= _lib.NOALLOC_SCRATCH_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        want = torch.empty((S, 2, H, D), dtype=torch.float32, device=dev)
        got = torch.full((S, 2, H, D), float("nan"), dtype=torch.float32, device=dev)
        scale = 1.0 / D ** 0.5
        rc = lib.spsattn_decode_fwd(t["q"].data_ptr(), 2, want.data_ptr(), segs, 2, extras, 2, S, H, D,
                                    _lib.DTYPE_BF16, scale, ws.data_ptr(), need, None, stream)
        _lib.check(rc, "spsattn_decode_fwd")
        rc = lib.spsattn_decode_fwd_noalloc(t["q"].data_ptr(), 2, got.data_ptr(), segs, 2, extras, 2, S, H, D,
                                            _lib.DTYPE_BF16, scale, None, stream)
        _lib.check(rc, "spsattn_decode_fwd_noalloc")
        torch.cuda.synchronize()
        assert torch.isfinite(got).all(), f"call {call}"
        err = (got - want).abs()
        assert float(err.max()) <= 2e-3 and float(err.mean()) <= 2e-4, (call, float(err.max()))


def test_noalloc_decode_refuses_problems_beyond_its_buffer():
    from sps_b200 import _lib
    lib = _lib.load()
    S, H, D = 512, 16, 64
    segs = (_lib.Segment * 1)()
    segs[0].max_rows = 4096
    assert lib.spsattn_decode_workspace_bytes(S, H, D, 2, segs, 1) > _lib.NOALLOC_SCRATCH_BYTES
    fake = C.c_void_p(4096)
    rc = lib.spsattn_decode_fwd_noalloc(fake, 2, fake, segs, 1, None, 0, S, H, D, _lib.DTYPE_BF16, 0.125,
                                        None, None)
    assert rc == -8
    assert "16 MiB" in lib.spsattn_strerror(rc).decode()
