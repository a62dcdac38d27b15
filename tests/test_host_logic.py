"""Host-side logic that needs no GPU: the C-ABI library loads and exports what the header
declares, argument errors are caught before any launch, the key-tile planner and the workload
arithmetic agree with the oracle's exhaustive counts."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import sps_oracle as orc
from sps_b200 import _lib, workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    header = open(os.path.join(ROOT, "include", "spsattn.h")).read()
    declared = set(re.findall(r"\b(spsattn_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.spsattn_version() >= 1


def test_argument_errors_are_reported_before_any_launch():
    lib = _lib.load()
    err = lambda c: lib.spsattn_strerror(c).decode()
    # null pointers / bad sizes never reach CUDA
    rc = lib.spsattn_prefill_fwd(None, None, None, None, None, None, 0, 0, 0, 1, 1, 8, 64, 0, 0.125,
                                 0, 1, _lib.NO_WINDOW, 0, None, 0, None, None)
    assert rc == -1 and "invalid argument" in err(rc)
    fake = ctypes.c_void_p(4096)
    args = lambda **kw: [fake, fake, fake, fake, None, None, 0, 0, 0, kw.get("B", 1), 1, kw.get("N", 8),
                         kw.get("D", 64), kw.get("dtype", 0), kw.get("scale", 0.125), kw.get("parity", 0), 1,
                         _lib.NO_WINDOW, 0, None, 0, None, None]
    assert lib.spsattn_prefill_fwd(*args(D=48)) == -2
    assert lib.spsattn_prefill_fwd(*args(N=7)) == -5
    assert lib.spsattn_prefill_fwd(*args(scale=0.0)) == -1
    assert lib.spsattn_prefill_fwd(*args(dtype=5)) == -1
    assert lib.spsattn_prefill_fwd(*args(parity=3)) == -1
    bad = ctypes.c_void_p(4100)
    a = args()
    a[0] = bad
    assert lib.spsattn_prefill_fwd(*a) == -3
    assert lib.spsattn_decode_fwd(None, 2, None, None, 0, None, 0, 1, 1, 64, 0, 0.125, None, 0, None, None) == -1
    assert lib.spsattn_decode_fwd(fake, 3, fake, None, 0, None, 0, 1, 1, 64, 0, 0.125, None, 0, None, None) == -1
    assert lib.spsattn_decode_fwd(fake, 2, fake, None, 0, None, 0, 1, 1, 24, 0, 0.125, None, 0, None, None) == -2
    # missing workspace
    assert lib.spsattn_decode_fwd(fake, 2, fake, None, 0, None, 0, 1, 1, 64, 0, 0.125, None, 0, None, None) == -4
    assert lib.spsattn_kv_update(*([None] * 12), 1, 1, 64, 0, 4, 0, 2, None) == -1
    assert "unknown" not in err(-7)
    # the backward entry point: q, k, v, o, d_o, lse, dq, dk, dv, then the forward's arguments
    bargs = lambda **kw: [fake] * 9 + [None, 0, 0, 0, 1, 1, kw.get("N", 8), kw.get("D", 64), kw.get("dtype", 0),
                                        kw.get("scale", 0.125), kw.get("parity", 0), 1, _lib.NO_WINDOW, 0,
                                        kw.get("ws", None), kw.get("ws_bytes", 0), None, None]
    assert lib.spsattn_prefill_bwd(*([None] * 9 + bargs()[9:])) == -1
    assert lib.spsattn_prefill_bwd(*bargs(D=32)) == -2          # backward kernels: head_dim 64 and 128
    assert lib.spsattn_prefill_bwd(*bargs(N=7)) == -5
    assert lib.spsattn_prefill_bwd(*bargs(N=2 * 65536)) == -7
    assert lib.spsattn_prefill_bwd(*bargs(scale=-1.0)) == -1
    assert lib.spsattn_prefill_bwd(*bargs()) == -4               # workspace missing
    assert lib.spsattn_prefill_bwd(*bargs(ws=fake, ws_bytes=16)) == -4


def test_workspace_sizes():
    lib = _lib.load()
    assert lib.spsattn_prefill_workspace_bytes(8, 12, 8192, 64) >= 8 * 8192 * 4 + 8 * 4
    # backward: the forward's pre-pass arrays + delta [B, H, N] fp32 + run ends [B, N] int32
    assert (lib.spsattn_prefill_bwd_workspace_bytes(8, 12, 8192, 64)
            >= lib.spsattn_prefill_workspace_bytes(8, 12, 8192, 64) + 8 * 12 * 8192 * 4 + 8 * 8192 * 4)
    seg = (_lib.Segment * 2)()
    seg[0].max_rows, seg[1].max_rows = 64, 4096
    need = lib.spsattn_decode_workspace_bytes(128, 16, 64, 2, seg, 2)
    chunks = -(-4160 // 512)
    assert need >= 128 * 16 * chunks * 2 * 66 * 4


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libspsattn.so")
    with pytest.raises(_lib.SpsAttnError):
        _lib.load()


def test_cpu_tensors_are_refused():
    import sps_b200
    q = torch.randn(1, 1, 8, 64).bfloat16()
    with pytest.raises(RuntimeError):
        sps_b200.sps_sliding_attention(q, q, q, 0.125, 2)
    with pytest.raises(RuntimeError):
        sps_b200.decode_attention(torch.randn(1, 2, 1, 64).bfloat16(), [], [])


def test_closed_form_pair_counts_match_exhaustive_count():
    docs = workloads.geometric_docs(2, 256, 100, 0)
    assert workloads.useful_pairs(docs, 64) == orc.count_visible_pairs(docs, 512, 2, temporary_window=64) == 80266
    # the prose variant of the rule: input queries skip the predict stream, exclusive window
    want = orc.count_visible_pairs(docs, 512, 2, temporary_window=63,
                                   mask_flags=orc.FLAG_PERSISTENT_Q_SKIPS_TEMPORARY)
    assert workloads.useful_pairs(docs, 64, "baseline_prose") == want == 61432
    docs = workloads.geometric_docs(3, 300, 40, 5)
    assert workloads.useful_pairs(docs, 7) == orc.count_visible_pairs(docs, 600, 3, temporary_window=7)


def test_benchmark_work_figures():
    B, H, T, D, w, mean = workloads.PREFILL_CONFIGS["cfg1_s_scale"]
    pairs = workloads.useful_pairs(workloads.geometric_docs(B, T, mean, 0), w)
    assert pairs == 55671620 and abs(workloads.prefill_flops(pairs, H, D) / 1e9 - 171.02) < 0.01
    B, H, T, D, w, mean = workloads.PREFILL_CONFIGS["cfg4_full_window"]
    assert workloads.useful_pairs(workloads.geometric_docs(B, T, mean, 0), w) == 134234112
    lens = workloads.decode_lengths("cfg2_segmented_decode")
    assert int(lens.sum()) == 299847
    assert abs(workloads.decode_bytes(lens, 64, 16, 64) / 1e6 - 1264.35) < 0.01


def test_shard_slices_cover_everything_once():
    for n, world in ((8, 1), (8, 2), (8, 8), (128, 3), (16, 4), (5, 8)):
        seen = []
        for r in range(world):
            seen += list(range(n)[workloads.shard_slice(n, r, world)])
        assert seen == list(range(n))


def _host_intervals(n, parity, w, pw, flags, docs_row):
    """The kernels' per-row interval rule, restated on the host from csrc/mask.cuh."""
    lo = orc.run_starts(docs_row) if docs_row is not None else np.zeros(n, dtype=np.int64)
    vis = np.zeros((n, n), dtype=bool)
    ks = 1 if parity == -1 else 2
    for i in range(n):
        for p in range(ks):
            if ks == 1:
                kmin, kmax = int(lo[i]), i
            else:
                kmax = (i - p) >> 1
                kmin = (int(lo[i]) - p + 1) >> 1
                ti = i >> 1
                if p == parity:
                    if pw is not None:
                        if pw >= 0:
                            kmin = max(kmin, ti - pw)
                        elif (i & 1) == p:
                            kmin = kmax = ti
                        else:
                            kmin, kmax = 0, -1
                else:
                    kmin = max(kmin, ti - w)
                    if (flags & 1) and (i & 1) == parity:
                        kmin, kmax = 0, -1
            for kt in range(max(kmin, 0), kmax + 1):
                vis[i, ks * kt + p] = True
    return vis


@pytest.mark.parametrize("parity", [0, 1, -1])
def test_interval_rule_equals_reference_rule(parity):
    rng = np.random.default_rng(parity + 3)
    for n, w, pw, flags in ((8, 0, None, 0), (30, 2, None, 0), (64, 5, 1, 0), (40, 3, -1, 0), (50, 4, None, 1),
                            (36, -1, 0, 0), (20, 100, None, 0)):
        if parity == -1 and (pw is not None or flags):
            continue
        for docs in (None, np.cumsum(rng.random(n) < 0.15).astype(np.int64)):
            got = _host_intervals(n, parity, w, pw, flags, docs)
            want = orc.visible_mask(n, persistent_parity=parity, temporary_window=w, persistent_window=pw,
                                    mask_flags=flags, docs_row=docs)
            assert np.array_equal(got, want), (n, w, pw, flags)


def test_generation_workload_helpers():
    """The whole-model generation configuration: dims of the benchmark configuration, the speed
    benchmark's forbidden-id filter, prompt ids below EOS, and the bytes one token step must move."""
    from sps_b200 import workloads
    cfg = workloads.GENERATION_CONFIGS["cfg3_xl_generation"]
    assert (cfg["hidden_size"], cfg["n_layer"], cfg["n_head"], cfg["vocab_size"]) == (2048, 24, 16, 50304)
    assert cfg["hidden_size"] // cfg["n_head"] == 128 and cfg["block_size"] >= cfg["prompt"] + cfg["new_tokens"]
    forb = workloads.generation_forbidden_ids(cfg)
    assert forb == list(range(50257, 50304)) and cfg["pad_token_id"] in forb and cfg["predict_token_id"] in forb
    assert cfg["eos_token_id"] not in forb
    p0, p1 = workloads.generation_prompts(cfg, 4, seed=0), workloads.generation_prompts(cfg, 4, seed=1)
    assert p0.shape == (4, 1024) and p0.max() < cfg["eos_token_id"] and p0.min() >= 0
    assert (p0 != p1).any()                         # ranks draw different prompts
    c, i, L = 2048, 8192, 24
    params = L * (4 * c * c + 3 * c * i) + 50304 * c
    kv = L * 32 * (1152 + 64) * c * 2
    assert workloads.generation_step_bytes(cfg, 32, 1152) == 2.0 * (params + kv)


def test_generator_refuses_to_work_without_cuda_extension_inputs():
    """Host-side argument checks of the generation engine that need no GPU."""
    import pytest as _pytest
    import torch
    from sps_b200.generation import (SPSDims, left_padded_position_ids, _validate_left_padded)
    idx = torch.tensor([[62, 62, 5, 6], [1, 2, 3, 4]])
    assert left_padded_position_ids(idx, 62).tolist() == [[0, 0, 0, 1], [0, 1, 2, 3]]
    _validate_left_padded(idx, 62, "prompts")
    with _pytest.raises(ValueError):
        _validate_left_padded(torch.tensor([[5, 62, 6]]), 62, "prompts")
    with _pytest.raises(ValueError):
        _validate_left_padded(torch.tensor([[62, 62]]), 62, "prompts")
    assert SPSDims(32, 64, 2, 2, 128, 256).head_dim == 64


def _row_interval(n, ks, parity, w, pw, flags, i, lo_i, p):
    """row_interval() of sps_b200/csrc/mask.cuh restated (same arithmetic as _host_intervals)."""
    if i >= n:
        return 0, -1
    if ks == 1:
        return lo_i, i
    kmax, kmin, ti = (i - p) >> 1, (lo_i - p + 1) >> 1, i >> 1
    if p == parity:
        if pw is not None:
            if pw >= 0:
                kmin = max(kmin, ti - pw)
            elif (i & 1) == p:
                kmin = kmax = ti
            else:
                kmin, kmax = 0, -1
    else:
        kmin = max(kmin, ti - w)
        if (flags & 1) and (i & 1) == parity:
            kmin, kmax = 0, -1
    return kmin, kmax


def test_backward_tile_classification_from_first_and_last_row():
    """The dK/dV kernel decides from the first and last row of a 64-row query tile whether the
    tile sees a 128-token key tile at all and whether it sees all of it
    (sps_b200/csrc/prefill_bwd_sm100.cuh).  Against the dense mask: every needed tile is kept,
    none is kept in vain, and a tile called interior is fully visible."""
    rng = np.random.default_rng(0)
    kept = needed = 0
    for _ in range(120):
        parity = int(rng.choice([0, 1, -1]))
        ks = 1 if parity < 0 else 2
        n = int(rng.integers(1, 400)) * ks
        w = min(int(rng.choice([0, 1, 3, 17, 64, 200, n])), n)
        pw = None if parity < 0 or rng.random() < 0.5 else int(rng.choice([-1, 0, 2, 40]))
        flags = int(rng.random() < 0.3) if parity >= 0 else 0
        t = n // ks
        docs = None
        if rng.random() < 0.7:
            ids, d, mean = [], 0, int(rng.choice([3, 20, 150]))
            while len(ids) < t:
                ids += [d] * int(rng.geometric(1.0 / mean))
                d += 1
            docs = np.repeat(np.array(ids[:t]), ks)
        vis = orc.visible_mask(n, persistent_parity=parity, temporary_window=w, persistent_window=pw,
                               docs_row=docs, mask_flags=flags)
        lo = np.zeros(n, dtype=np.int64) if docs is None else orc.run_starts(docs)
        for stream in range(ks):
            filt, only = False, -1                       # stream_row_filter() of mask.cuh
            if ks == 2 and stream == parity and pw is not None and pw < 0:
                filt, only = True, stream
            elif ks == 2 and stream != parity and (flags & 1):
                filt, only = True, 1 - parity
            for x0 in range(0, t, 128):
                keys = [ks * kt + stream for kt in range(x0, min(x0 + 128, t))]
                for q0 in range(0, n, 64):
                    rows = list(range(q0, min(q0 + 64, n)))
                    sub = vis[np.ix_(rows, keys)]
                    t_any = bool(sub.any())
                    t_all = bool(sub.all()) and len(rows) == 64 and len(keys) == 128
                    ra, rb = q0, min(q0 + 63, n - 1)
                    if filt:
                        ra += int((ra & 1) != only)
                        rb -= int((rb & 1) != only)
                    f_any = f_all = False
                    if ra <= rb:
                        kmin_a, kmax_a = _row_interval(n, ks, parity, w, pw, flags, ra, int(lo[ra]), stream)
                        kmin_b, kmax_b = _row_interval(n, ks, parity, w, pw, flags, rb, int(lo[rb]), stream)
                        f_any = kmax_b >= x0 and kmin_a <= x0 + 127
                        f_all = (not filt) and q0 + 63 <= n - 1 and kmin_b <= x0 and kmax_a >= x0 + 127
                    assert f_any or not t_any, (parity, n, w, pw, flags, stream, x0, q0)
                    assert t_all or not f_all, (parity, n, w, pw, flags, stream, x0, q0)
                    kept += f_any
                    needed += t_any
    assert kept == needed and needed > 500


def test_balanced_partition_and_grouped_block_order():
    """Host logic of the multi-GPU split and of the kernels' block order.  The decode split puts
    sequences into bins of nearly equal summed length; the prefill kernels walk (batch, head)
    pairs in groups and, inside a group, the late (heavy) query tiles of every head first: the
    mapping from block number to (pair, tile) must hit every pair and tile exactly once."""
    import numpy as np
    from sps_b200 import workloads
    w = np.array([9, 1, 8, 2, 7, 3, 6, 4, 5, 5])
    bins = workloads.balanced_partition(w, 3)
    assert sorted(i for b in bins for i in b) == list(range(10))
    loads = [int(w[b].sum()) for b in bins]
    assert max(loads) - min(loads) <= 2
    assert workloads.balanced_partition([4.0], 2) == [[0], []]

    def block_to_item(block, n_pairs, n_qtiles, group):       # the kernels' arithmetic restated
        per_group = group * n_qtiles
        grp, in_grp = divmod(block, per_group)
        gsize = min(group, n_pairs - grp * group)
        return grp * group + in_grp % gsize, n_qtiles - 1 - in_grp // gsize

    for n_pairs, n_qtiles, group in ((96, 64, 24), (7, 3, 4), (5, 9, 32), (64, 64, 12), (1, 1, 1)):
        seen = [block_to_item(b, n_pairs, n_qtiles, group) for b in range(n_pairs * n_qtiles)]
        assert sorted(seen) == [(p, t) for p in range(n_pairs) for t in range(n_qtiles)]
        # inside a group the tile number never increases
        first_group = [t for p, t in seen[:min(group, n_pairs) * n_qtiles]]
        assert first_group == sorted(first_group, reverse=True)
