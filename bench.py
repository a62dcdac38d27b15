#!/usr/bin/env python
"""Benchmark of the SPS attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of SPS prefill attention over the s-scale configuration
([8, 12, 8192, 64] bf16, w = 64, packed documents ~ Geometric(mean 1000 tokens)); the headline
metric is useful (unmasked) TFLOP/s.  The same run also times the segmented decode step
(128 sequences, cache lengths U[512, 4096], ring 64, 16 heads x 64) and reports it under
"decode" with its own HBM roofline.  With N > 1 (one process per GPU under torchrun) every rank
runs the full per-GPU workload on its own shard of sequences: no collective on the data path,
weak scaling, time = max over ranks.

`--impl reference` times the reference's CPU formulation of the same math (dense additive
mask + SDPA, restated in oracle/) on the host cores, on a bounded sample of the workload.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PREFILL = "cfg1_s_scale"
DECODE = "cfg2_segmented_decode"
PREFILL_FULL_WINDOW = "cfg4_full_window"
GENERATION = "cfg3_xl_generation"
# DRAM traffic per full-size launch, from ncu captures of a smaller case scaled by the units
# processed (traffic is proportional to batch rows / sequences)
PREFILL_DRAM_BYTES_PER_LAUNCH = 2 * (151.6e6 + 32.6e6)
DECODE_DRAM_BYTES_PER_LAUNCH = 4 * (332.2e6 + 4.9e6)
# head_dim 128 forward: ncu dram bytes of a 4-head launch (quarter of the heads) x4
FULL_WINDOW_DRAM_BYTES_PER_LAUNCH = 4 * (100.7e6 + 15.4e6)
# dK/dV kernel + dQ kernel of one backward call: ncu dram bytes of a 4-row call x2
BACKWARD_DRAM_BYTES_PER_CALL = 2 * (204.8e6 + 76.8e6 + 204.7e6 + 36.4e6)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


_SAMPLER_SRC = r"""
import sys, time
idx, period = int(sys.argv[1]), float(sys.argv[2])
try:
    import pynvml as nv
    nv.nvmlInit()
    h = nv.nvmlDeviceGetHandleByIndex(idx)
    print("MAX %d" % nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM), flush=True)
except Exception as e:
    print("ERR %r" % (e,), flush=True)
    sys.exit(0)
while True:
    try:
        c = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
        r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        sys.stdout.write("%.6f %d %d\n" % (time.time(), c, r))
        sys.stdout.flush()
    except Exception:
        pass
    time.sleep(period)
"""


class ClockSampler:
    """SM clock and throttle reasons through NVML while the timed regions run.  The polling
    loop lives in a child process, so it never competes with the launching thread for the
    interpreter; the parent only notes the wall-clock window of every timed region and keeps the
    samples that fall inside one.  Reading clocks changes no setting of the GPU."""

    _BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.002):
        import subprocess
        import tempfile
        self.windows, self.max_mhz = [], None
        self._out = tempfile.NamedTemporaryFile(mode="w+", suffix=".clk", delete=False)
        try:
            self._proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_SRC, str(index), str(period_s)],
                                          stdout=self._out, stderr=subprocess.DEVNULL)
        except Exception:
            self._proc = None
        t0 = time.time()
        while self._proc is not None and time.time() - t0 < 5.0:        # wait for the first line
            with open(self._out.name) as f:
                head = f.readline()
            if head.startswith("MAX"):
                self.max_mhz = float(head.split()[1])
                break
            if head.startswith("ERR") or self._proc.poll() is not None:
                break
            time.sleep(0.02)

    def begin(self):
        self._t0 = time.time()

    def end(self):
        self.windows.append((self._t0, time.time()))

    def summary(self):
        if self._proc is not None:
            self._proc.terminate()          # our own child, by handle
            try:
                self._proc.wait(timeout=5)
            except Exception:
                pass
        samples, reasons = [], set()
        try:
            with open(self._out.name) as f:
                for line in f:
                    parts = line.split()
                    if len(parts) != 3 or parts[0] in ("MAX", "ERR"):
                        continue
                    t, c, r = float(parts[0]), float(parts[1]), int(parts[2])
                    if any(a <= t <= b for a, b in self.windows):
                        samples.append(c)
                        reasons.update(name for bit, name in self._BITS.items() if r & bit)
            os.unlink(self._out.name)
        except Exception:
            pass
        return {"sm_mhz": float(np.median(samples)) if samples else None, "sm_max_mhz": self.max_mhz,
                "samples": len(samples), "reasons": sorted(reasons),
                "how": "NVML polled every 2 ms by a child process; samples inside the timed regions only"}


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="nccl" if torch.cuda.is_available() else "gloo")
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_over_ranks(x: float, world: int, device) -> list:
    if world == 1:
        return [x]
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [float(o.item()) for o in out]


def timed_steps(fn, steps, warmup, world, device, regions=5, sampler=None):
    """W untimed steps, then `regions` back-to-back timed regions of exactly K steps, each
    bracketed by barrier + synchronize on both sides and timed with CUDA events on the launching
    stream.  The region reported is the median one (by its max over ranks): a single late rank
    in a region of a few milliseconds otherwise decides the figure.  Returns (region ms as max
    over ranks, mean launch ms on this rank, details)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    mine, per_launch = [], []
    for _ in range(regions):
        barrier(world)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        if sampler is not None:
            sampler.begin()
        ev[0].record()
        for i in range(steps):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        if sampler is not None:
            sampler.end()
        barrier(world)
        torch.cuda.synchronize()
        mine.append(ev[0].elapsed_time(ev[-1]))
        per_launch.append(float(np.mean([ev[i].elapsed_time(ev[i + 1]) for i in range(steps)])))
    maxima = [max_over_ranks(m, world, device) for m in mine]
    pick = int(np.argsort(maxima)[len(maxima) // 2])
    details = {"regions_ms_max_over_ranks": maxima, "reported_region": pick,
               "rank_region_ms": gather_over_ranks(mine[pick], world, device)}
    return maxima[pick], per_launch[pick], details


# ------------------------------------------------------------------------------------- ours

def headline_config(world: int) -> dict:
    """The `config` object of the JSON line; both arms print exactly this for the same --gpus."""
    from sps_b200 import workloads
    B, H, T, D, w, _ = workloads.PREFILL_CONFIGS[PREFILL]
    docs = workloads.geometric_docs(B, T, 1000, 0)
    flops = workloads.prefill_flops(workloads.useful_pairs(docs, w), H, D)
    return {
        "workload": f"{PREFILL}: SPS prefill attention [B={B},H={H},2T={2 * T},D={D}] bf16, w={w}, "
                    "documents ~ Geometric(mean 1000 tokens), reference mask rule, per GPU",
        "useful_gflop_per_step_per_gpu": flops / 1e9,
        "l2": f"inputs larger than L2: {4 * B * H * 2 * T * D * 2 / 1e6:.0f} MB of Q/K/V/O per step vs 126 MB",
        "parallelism": f"independent shards x{world}, no collective; every rank runs the configuration's seed-0 "
                       "inputs (weak scaling: identical work per GPU)",
    }


def _prefill_fn(sps_b200, wl, out, docs=True):
    return lambda: sps_b200.prefill_attention(wl.q, wl.k, wl.v, wl.sm_scale, persistent_parity=0,
                                              temporary_window=wl.window,
                                              documents_idx=wl.docs if docs else None, out=out)


def strong_prefill(sps_b200, workloads, name, axis, world, rank, device, steps):
    """The north-star split of one prefill configuration: the fixed total problem cut over the
    ranks by batch rows or by heads (shards are independent, no collective); aggregate rate =
    useful FLOPs of the whole problem / slowest rank's time."""
    B, H = workloads.PREFILL_CONFIGS[name][:2]
    n = B if axis == "batch" else H
    sl = workloads.shard_slice(n, rank, world)
    if sl.stop <= sl.start:
        raise RuntimeError(f"{name}: more ranks than {axis} items")
    kw = {"batch_slice": sl} if axis == "batch" else {"head_slice": sl}
    wl = workloads.make_prefill(name, device, **kw)
    out = torch.empty_like(wl.q)
    region_ms, launch_ms, det = timed_steps(_prefill_fn(sps_b200, wl, out, wl.docs is not None), steps, 3,
                                            world, device, regions=3)
    total = _sum_over_ranks(wl.flops, world, device)
    return {"split": f"{axis} {n} -> {sl.stop - sl.start} per GPU", "useful_tflops": total * steps / (region_ms * 1e-3) / 1e12,
            "ms_per_step": region_ms / steps, "launch_ms_this_rank": launch_ms, "timing": det,
            "note": "strong scaling: the per-GPU launch shrinks with N (at 1 batch row x 12 heads a launch is "
                    "768 blocks = 1.7 waves), so launch latency and the tail show here"}


def reference_triton(device):
    """The reference's own Triton kernels on this GPU, same inputs, CUDA events, after their
    autotune warm-up: the existing Blackwell path the kernels of this repository replace.  Needs
    the reference installed under baseline/_ref and an importable triton; otherwise the reason."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "modeling", "models")):
        return {"unavailable": "unavailable on this box: baseline/_ref holds no install of the reference"}
    try:
        import triton                                                                  # noqa: F401
        if ref_dir not in sys.path:
            sys.path.insert(0, ref_dir)
        from modeling.models.attention.triton_sps_flash_attention import sps_sliding_attention as ref_sps
        from modeling.models.utils.decode_attention import KVSegment as RefSegment
        from modeling.models.utils.decode_attention import triton_segmented_q2_attention as ref_q2
    except Exception as e:
        return {"unavailable": f"unavailable on this box: {e!r}"}
    import sps_b200
    from sps_b200 import workloads
    out = {"triton": triton.__version__, "how": "3 warm-up calls (autotune), then the fastest of 3 rounds of 10 "
                                                 "timed calls, CUDA events; warp_specialize=False as the "
                                                 "reference's configs run it"}

    def time_it(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                r = fn()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / 10)
        return best, r

    for name in (PREFILL, PREFILL_FULL_WINDOW):
        try:
            wl = workloads.make_prefill(name, device)
            ms, o_ref = time_it(lambda: ref_sps(wl.q, wl.k, wl.v, wl.sm_scale, wl.window, False, wl.docs, None))
            o_our = sps_b200.sps_sliding_attention(wl.q, wl.k, wl.v, wl.sm_scale, wl.window, False, wl.docs, None)
            diff = (o_ref.float() - o_our.float()).abs()
            out[name] = {"ms": ms, "useful_tflops": wl.flops / (ms * 1e-3) / 1e12,
                         "max_abs_diff_vs_this_repo": float(diff.max()), "mean_abs_diff_vs_this_repo": float(diff.mean())}
            del wl, o_ref, o_our, diff
        except Exception as e:
            out[name] = {"unavailable": f"unavailable on this box: {e!r}"}
        torch.cuda.empty_cache()
    try:
        dw = workloads.make_decode(DECODE, device)
        mk = lambda cls: [cls(dw.ring_k, dw.ring_v, dw.ring_len, max_len_cap=dw.ring_k.shape[2]),
                          cls(dw.cache_k, dw.cache_v, dw.cache_len, max_len_cap=dw.cache_k.shape[2])]
        kw = dict(current_normal_k_BxHxD=dw.cur_k, current_normal_v_BxHxD=dw.cur_v,
                  current_predict_k_BxHxD=dw.pred_k, current_predict_v_BxHxD=dw.pred_v, attn_dtype=torch.bfloat16)
        rsegs = mk(RefSegment)
        ms, o_ref = time_it(lambda: ref_q2(dw.q, rsegs, **kw))
        o_our = sps_b200.segmented_q2_attention(dw.q, mk(sps_b200.KVSegment), **kw)
        out[DECODE] = {"ms": ms, "gb_per_s": dw.bytes / (ms * 1e-3) / 1e9,
                       "tokens_per_s": dw.q.shape[0] / (ms * 1e-3),
                       "max_abs_diff_vs_this_repo": float((o_ref - o_our).abs().max())}
        del dw, rsegs, o_ref, o_our
    except Exception as e:
        out[DECODE] = {"unavailable": f"unavailable on this box: {e!r}"}
    torch.cuda.empty_cache()
    # the reference's fused cache update (one Triton launch) against this repository's, on cfg2's
    # cache shapes: the same ten updates on two copies of the caches, contents compared bit for bit
    try:
        from modeling.models.utils.decode_attention_fast import fused_sps_kv_update as ref_update
        S, H, D, ring, _, cap = workloads.DECODE_CONFIGS[DECODE]
        g = torch.Generator(device="cpu").manual_seed(0)
        bf = torch.bfloat16

        def caches():
            gg = torch.Generator(device="cpu").manual_seed(1)
            return dict(
                nw_k=torch.zeros(S, H, ring, D, dtype=bf, device=device), nw_v=torch.zeros(S, H, ring, D, dtype=bf, device=device),
                nw_len=torch.full((S,), ring, dtype=torch.int64, device=device),
                nw_pos=torch.randint(0, ring, (S,), generator=gg).to(device),
                br_k=torch.zeros(S, H, cap, D, dtype=bf, device=device), br_v=torch.zeros(S, H, cap, D, dtype=bf, device=device),
                br_len=torch.randint(512, cap - 64, (S, 1), generator=gg).expand(S, H).contiguous().to(device))
        new = [torch.randn(S, H, D, generator=g).to(bf).to(device) for _ in range(4)]
        active = torch.ones(S, dtype=torch.bool, device=device)
        step = dict(k_window_BxHxD=new[0], v_window_BxHxD=new[1], k_retained_BxHxD=new[2], v_retained_BxHxD=new[3],
                    active_mask_B=active, window_tokens=ring)
        timings = {}
        state = {}
        for tag, fn in (("reference", ref_update), ("ours", sps_b200.fused_sps_kv_update)):
            c = caches()
            fn(**c, **step)                       # warm-up (and the Triton compile)
            c = caches()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn(**c, **step)
            e1.record()
            torch.cuda.synchronize()
            timings[tag] = e0.elapsed_time(e1) / 10
            state[tag] = c
        # rows (of D elements) that differ between the two sets of caches, and whether this
        # repository's ring holds the ten new rows in ten consecutive slots from the old position
        # on, which is what the sequential rule (the reference's unfused methods) gives
        diff_rows = {k: int((state["reference"][k] != state["ours"][k]).reshape(S * H, -1, D).any(-1).sum())
                     for k in ("nw_k", "nw_v", "br_k", "br_v")}
        counters_same = all(torch.equal(state["reference"][k], state["ours"][k]) for k in ("nw_len", "nw_pos", "br_len"))
        pos0 = caches()["nw_pos"]
        slots = (pos0[:, None] + torch.arange(10, device=device)[None, :]) % ring
        filled = state["ours"]["nw_k"].float().abs().sum(-1) != 0                      # [S, H, ring]
        want = torch.zeros(S, ring, dtype=torch.bool, device=device).scatter_(1, slots, True)
        out["fused_sps_kv_update"] = {
            "shape": f"[{S},{H},{D}] new rows into ring {ring} and retained cache {cap}, bf16, 10 updates",
            "ms": timings["reference"], "ms_this_repo": timings["ours"],
            "counters_identical": bool(counters_same), "rows_differing": diff_rows,
            "this_repo_ring_matches_sequential_rule": bool((filled == want[:, None, :]).all()),
            "note": "where rows differ, the reference's kernel wrote a ring row to the wrong slot: its programs "
                    "(b, h != 0) read nw_pos while program (b, 0) advances it, with no ordering between them; "
                    "this repository reads the counters of a sequence in one block before anything is written"}
        del state
    except Exception as e:
        out["fused_sps_kv_update"] = {"unavailable": f"unavailable on this box: {e!r}"}
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import sps_b200
    from sps_b200 import workloads

    world, rank, local = dist_setup(args.gpus)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    peaks, peak_kind = load_peaks()
    K, W = args.steps, max(args.warmup, 3)
    # ---------------- prefill (headline): every rank the full configuration on its own shard
    sampler = ClockSampler(local)
    wl = workloads.make_prefill(PREFILL, device, seed=0)
    out = torch.empty_like(wl.q)
    region_ms, launch_ms, det = timed_steps(_prefill_fn(sps_b200, wl, out), K, W, world, device,
                                            regions=5, sampler=sampler)
    clocks = sampler.summary()
    sps_b200.check_device_status(device)
    flops_all = wl.flops if world == 1 else _sum_over_ranks(wl.flops, world, device)
    value = flops_all * K / (region_ms * 1e-3) / 1e12
    achieved = wl.flops / (launch_ms * 1e-3) / 1e12
    peak = float(peaks["bf16_tflops"])
    result = {
        "metric": "sps_prefill_useful_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": region_ms / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(world),
        "clocks": clocks,
        "gpu_launches": 2 * K,      # document pre-pass + attention kernel per step
        "timing": dict(det, note="5 back-to-back regions of K steps, each bracketed by barrier + synchronize; "
                                 "the median region (by its max over ranks) is the one reported"),
        "roofline": {
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "traffic": PREFILL_DRAM_BYTES_PER_LAUNCH,
            "traffic_source": "ncu dram__bytes_read+write of a 4-row launch (half-batch case) x2",
            "peak_source": f"{peak_kind} bf16 burst (kernel timed alone)",
            "launch_ms": launch_ms,
        },
    }
    if world > 1:
        del wl, out
        torch.cuda.empty_cache()
        result["strong"] = strong_prefill(sps_b200, workloads, PREFILL, "batch", world, rank, device, max(3, min(K, 30)))
        wl = workloads.make_prefill(PREFILL, device, seed=0)
        out = torch.empty_like(wl.q)

    # ---------------- end to end through the public API with host buffers
    # Every step copies its Q, K, V and document ids from pinned host memory, calls the public
    # attention function and copies O back.  Two buffer sets and three streams let the upload of
    # step i+1 and the download of step i-1 run beside the kernel of step i (PCIe is full duplex).
    if not args.skip_e2e:
        hq, hk, hv = (x.cpu().pin_memory() for x in (wl.q, wl.k, wl.v))
        hdocs = wl.docs.cpu().pin_memory()
        ho = [torch.empty_like(hq).pin_memory() for _ in range(2)]
        dev_in = [[torch.empty_like(wl.q) for _ in range(3)] + [torch.empty_like(wl.docs)] for _ in range(2)]
        dev_out = [None, None]
        s_in, s_run, s_out = (torch.cuda.Stream(device) for _ in range(3))
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_run = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_steps(n):
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_run[b])          # inputs of step i-2 consumed
                    for dst, src in zip(dev_in[b], (hq, hk, hv, hdocs)):
                        dst.copy_(src, non_blocking=True)
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(ev_in[b])
                    s_run.wait_event(ev_out[b])         # output buffer of step i-2 downloaded
                    dq, dk, dv, dd = dev_in[b]
                    dev_out[b] = sps_b200.sps_sliding_attention(dq, dk, dv, wl.sm_scale, wl.window,
                                                                documents_idx_BxT=dd)
                    ev_run[b].record(s_run)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_run[b])
                    ho[b].copy_(dev_out[b], non_blocking=True)
                    ev_out[b].record(s_out)

        ke = max(4, min(K, 20))
        e2e_steps(4)
        torch.cuda.synchronize()
        barrier(world)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for st in (s_in, s_run, s_out):
            st.wait_event(t0)
        e2e_steps(ke)
        cur = torch.cuda.current_stream()
        for st in (s_in, s_run, s_out):
            done = torch.cuda.Event()
            done.record(st)
            cur.wait_event(done)
        t1.record()
        torch.cuda.synchronize()
        barrier(world)
        e2e_ms = max_over_ranks(t0.elapsed_time(t1), world, device)
        result["e2e"] = {
            "value": flops_all * ke / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": int(3 * hq.numel() * 2 + hdocs.numel() * 8),
            "d2h_bytes_per_step": int(ho[0].numel() * 2), "steps": ke, "ms_per_step": e2e_ms / ke,
            "note": "host-to-device copy of Q, K, V, ids and device-to-host copy of O inside every step; "
                    "PCIe bound (403 MB per step)",
        }
        del hq, hk, hv, ho, dev_in, dev_out

    # ---------------- backward of the same prefill (training path): dQ, dK, dV from dO
    if not args.skip_backward:
        o_b, lse_b = sps_b200.prefill_attention(wl.q, wl.k, wl.v, wl.sm_scale, persistent_parity=0,
                                                temporary_window=wl.window, documents_idx=wl.docs,
                                                return_lse=True)
        d_o = torch.randn(wl.q.shape, device=device, dtype=torch.float32).to(wl.q.dtype)

        def backward_step():
            sps_b200.attention.prefill_attention_backward(
                wl.q, wl.k, wl.v, o_b, lse_b, d_o, wl.sm_scale, persistent_parity=0,
                temporary_window=wl.window, documents_idx=wl.docs)

        kb = max(3, min(K, 30))
        b_region, b_launch, _ = timed_steps(backward_step, kb, 3, world, device, regions=3)
        # five products per visible (query, key) pair against the forward's two
        b_flops = 2.5 * wl.flops
        tb = b_flops / (b_launch * 1e-3) / 1e12
        result["prefill_backward"] = {
            "workload": f"{PREFILL}: dQ, dK, dV of the same batch from dO (pre-passes + dK/dV kernel + "
                        "dQ kernel per step), per GPU",
            "useful_gflop_per_step_per_gpu": b_flops / 1e9, "ms_per_step": b_region / kb,
            "useful_tflops": world * b_flops * kb / (b_region * 1e-3) / 1e12,
            "gpu_launches": 5 * kb,      # document pre-pass, run ends, delta, dK/dV, dQ
            "roofline": {"bound": "tensor", "achieved": tb, "peak": peak, "unit": "TFLOP/s", "frac": tb / peak,
                         "traffic": BACKWARD_DRAM_BYTES_PER_CALL,
                         "traffic_source": "ncu dram__bytes_read+write of the two kernels of a 4-row call "
                                           "(half-batch case) x2",
                         "peak_source": f"{peak_kind} bf16 burst", "launch_ms": b_launch,
                         "note": "useful FLOPs = 2.5 x forward; the two kernels recompute S and dP, so they "
                                 "execute 3.5 x forward"},
        }
        del o_b, lse_b, d_o
        sps_b200.check_device_status(device)

    # ---------------- the least sparse prefill mask: head_dim 128, window = whole document
    if not args.skip_full_window:
        del wl, out
        torch.cuda.empty_cache()
        wf = workloads.make_prefill(PREFILL_FULL_WINDOW, device, seed=0)
        outf = torch.empty_like(wf.q)
        kf = max(3, min(K, 30))
        f_region, f_launch, _ = timed_steps(_prefill_fn(sps_b200, wf, outf, False), kf, 3, world, device, regions=3)
        tf = wf.flops / (f_launch * 1e-3) / 1e12
        result["prefill_full_window"] = {
            "workload": f"{PREFILL_FULL_WINDOW}: [B=4,H=16,2T=8192,D=128] bf16, w=4096, one document per row, per GPU",
            "useful_gflop_per_step_per_gpu": wf.flops / 1e9, "ms_per_step": f_region / kf,
            "useful_tflops": world * wf.flops * kf / (f_region * 1e-3) / 1e12, "gpu_launches": kf,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                         "traffic": FULL_WINDOW_DRAM_BYTES_PER_LAUNCH,
                         "traffic_source": "ncu dram__bytes_read+write of a 4-head launch (quarter-heads case) x4",
                         "peak_source": f"{peak_kind} bf16 burst", "launch_ms": f_launch},
        }
        wl = out = None
        del wf, outf
        torch.cuda.empty_cache()
        if world > 1:
            result["prefill_full_window"]["strong"] = strong_prefill(
                sps_b200, workloads, PREFILL_FULL_WINDOW, "heads", world, rank, device, kf)

    # ---------------- segmented decode step (second half of the metric)
    if not args.skip_decode:
        wl = out = None
        torch.cuda.empty_cache()

        def decode_leg(dw, steps, warm, regions):
            segs = [sps_b200.KVSegment(dw.ring_k, dw.ring_v, dw.ring_len, max_len_cap=dw.ring_k.shape[2]),
                    sps_b200.KVSegment(dw.cache_k, dw.cache_v, dw.cache_len, max_len_cap=dw.cache_k.shape[2])]
            fn = lambda: sps_b200.segmented_q2_attention(
                dw.q, segs, current_normal_k_BxHxD=dw.cur_k, current_normal_v_BxHxD=dw.cur_v,
                current_predict_k_BxHxD=dw.pred_k, current_predict_v_BxHxD=dw.pred_v, attn_dtype=torch.bfloat16)
            return timed_steps(fn, steps, warm, world, device, regions=regions)

        dw = workloads.make_decode(DECODE, device, seed=0)
        d_region, d_launch, _ = decode_leg(dw, K, W, 3)
        S = dw.q.shape[0]
        gbs = dw.bytes / (d_launch * 1e-3) / 1e9
        hbm = float(peaks["hbm_gbs"])
        result["decode"] = {
            "workload": f"{DECODE}: {S} sequences/GPU, cache lengths U[512,4096], ring 64, 16 heads x 64, "
                        "2 queries per sequence, bf16 cache, per layer-step",
            "tokens_per_s": world * S * K / (d_region * 1e-3), "ms_per_step": d_region / K,
            "algorithmic_mb_per_step": dw.bytes / 1e6, "gpu_launches": K,   # one launch per step
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                         "traffic": DECODE_DRAM_BYTES_PER_LAUNCH,
                         "traffic_source": "ncu dram__bytes_read+write of a 32-sequence launch x4",
                         "peak_source": f"{peak_kind} copy bandwidth", "launch_ms": d_launch},
        }
        sps_b200.check_device_status(device)
        if world > 1:
            del dw
            torch.cuda.empty_cache()
            bins = workloads.balanced_partition(workloads.decode_lengths(DECODE), world)
            ds = workloads.make_decode(DECODE, device, seq_index=bins[rank])
            s_region, s_launch, s_det = decode_leg(ds, K, 3, 3)
            result["decode"]["strong"] = {
                "split": f"128 sequences in {world} bins of equal summed cache length (heaviest first into the "
                         f"lightest bin): {len(bins[rank])} sequences on this rank",
                "tokens_per_s": 128 * K / (s_region * 1e-3), "ms_per_step": s_region / K,
                "launch_ms_this_rank": s_launch, "timing": s_det}
            del ds
        elif not args.skip_cpu_baseline:
            result["decode"]["cpu_baseline"] = cpu_baseline_decode(dw, budget_s=8.0)
            del dw

    # ---------------- whole-model greedy generation with the attention path inside
    if not args.skip_generation:
        wl = out = dw = None
        torch.cuda.empty_cache()
        result["generation"] = run_generation(GENERATION, world, rank, device, peaks, peak_kind)
        if world == 1 and not args.skip_cpu_baseline:
            result["generation"]["cpu_baseline"] = cpu_baseline_generation(budget_s=10.0)

    # ---------------- the reference's own Triton kernels on the same GPU (rank 0, one GPU)
    if world == 1 and not args.skip_reference_triton:
        torch.cuda.empty_cache()
        result["reference_triton"] = reference_triton(device)

    # ---------------- CPU baseline beside it (rank 0, single GPU runs only)
    if world == 1 and not args.skip_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(budget_s=12.0)
    if rank == 0:
        emit((result))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_generation(name, world, rank, device, peaks, peak_kind, new_tokens=None, runs_n=3):
    """Prompt prefill + greedy decode of a random-init SPS decoder, data parallel over ranks
    (the batch is split, weights replicated).  Tokens/s as the reference's speed benchmark
    defines them: batch * new_tokens / (prefill + decode), and batch * (new_tokens - 1) / decode."""
    import ctypes as C
    import sps_b200
    from sps_b200 import _lib, workloads
    from sps_b200.generation import SPSDims, SPSGenerator, random_state_dict

    cfg = workloads.GENERATION_CONFIGS[name]
    dims = SPSDims(**{k: cfg[k] for k in ("block_size", "vocab_size", "n_layer", "n_head", "hidden_size",
                                          "intermediate_size", "eos_token_id", "pad_token_id",
                                          "predict_token_id", "window_size")})
    batch = max(1, cfg["batch"] // world)
    eng = SPSGenerator(random_state_dict(dims, seed=0, device=device), dims, variant="sps", device=device)
    prompts = torch.from_numpy(workloads.generation_prompts(cfg, batch, seed=rank)).to(device)
    forbidden = torch.tensor(workloads.generation_forbidden_ids(cfg))
    new = int(new_tokens or cfg["new_tokens"])
    eng.generate(prompts, new, stop_on_eos=False, forbidden_token_ids=forbidden)      # builds and captures
    runs = []
    for _ in range(runs_n):
        torch.cuda.synchronize()
        barrier(world)
        tm = {}
        eng.generate(prompts, new, stop_on_eos=False, forbidden_token_ids=forbidden, timings=tm)
        runs.append(tm)
    sps_b200.check_device_status(device)
    tm = sorted(runs, key=lambda t: t["prefill"] + t["decode"])[len(runs) // 2]        # median run
    total_ms = max_over_ranks(tm["prefill"] + tm["decode"], world, device)
    decode_ms = max_over_ranks(tm["decode"], world, device)
    prefill_ms = max_over_ranks(tm["prefill"], world, device)
    step_ms = tm["decode_steps"] / tm["n_steps"]
    # the attention launches of one token alone (24 x split + merge, no cache update)
    s = eng._step
    scale = 1.0 / (dims.head_dim ** 0.5)
    lib = _lib.load()

    def attention_only():
        for segs, n_seg, extras, _ap in s.layer_args:
            lib.spsattn_decode_step(s.q.data_ptr(), 2, s.y.data_ptr(), _lib.DTYPE_BF16, segs, n_seg, extras, 2,
                                    None, batch, dims.n_head, dims.head_dim, _lib.DTYPE_BF16, scale,
                                    s.ws.data_ptr(), s.ws_bytes, None,
                                    torch.cuda.current_stream().cuda_stream)

    for _ in range(3):
        attention_only()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(10):
        attention_only()
    t1.record()
    torch.cuda.synchronize()
    attn_ms = t0.elapsed_time(t1) / 10
    live = cfg["prompt"] + new / 2.0
    step_bytes = workloads.generation_step_bytes(cfg, batch, live)
    hbm = float(peaks["hbm_gbs"])
    gbs = step_bytes / (step_ms * 1e-3) / 1e9
    return {
        "workload": f"{name}: SPS decoder {dims.n_layer} layers, hidden {dims.hidden_size}, {dims.n_head} heads x "
                    f"{dims.head_dim}, SwiGLU {dims.intermediate_size}, vocabulary {dims.vocab_size}, bf16, random "
                    f"init; batch {batch} per GPU ({batch * world} in all), prompt {cfg['prompt']}, {new} new "
                    f"tokens, greedy, w={dims.window_size}",
        "tokens_per_s": world * batch * new / (total_ms * 1e-3),
        "decode_tokens_per_s": world * batch * (new - 1) / (decode_ms * 1e-3),
        "prefill_ms": prefill_ms, "decode_ms": decode_ms, "ms_per_token_step": step_ms,
        "attention_ms_per_token_step": attn_ms, "attention_share_of_step": attn_ms / step_ms,
        "scaling": "strong (batch split over ranks, weights replicated)",
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                     "traffic": None, "peak_source": f"{peak_kind} copy bandwidth",
                     "bytes_per_step": step_bytes,
                     "note": "whole token step: every parameter once + live K/V of all layers at mid-generation"},
    }


def run_case(args):
    """Small single-kernel cases for profiler captures (a few hundred MB on the device, inputs
    still larger than L2): `prefill-small` = 4 of the 8 batch rows of the s-scale prefill,
    `full-window-small` = 4 of the 16 heads of the full-window prefill (head_dim 128),
    `backward-small` = the backward of those 4 rows, `backward-full-window-small` = the backward
    of the 4-head full-window case, `decode-small` = 32 of the 128 decode sequences, `generation-small` / `generation` = the
    whole-model generation leg alone on a tiny / the full model.  Prints a short JSON line, not
    the benchmark contract line."""
    import sps_b200
    from sps_b200 import workloads
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    if args.case in ("generation-small", "generation"):
        peaks, peak_kind = load_peaks()
        name = "generation_small" if args.case == "generation-small" else GENERATION
        emit(({"case": args.case, **run_generation(name, 1, 0, device, peaks, peak_kind,
                                                              new_tokens=args.new_tokens, runs_n=args.runs)}))
        return
    if args.case == "prefill-small":
        wl = workloads.make_prefill(PREFILL, device, batch_slice=slice(0, 4))
        out = torch.empty_like(wl.q)
        fn = lambda: sps_b200.prefill_attention(wl.q, wl.k, wl.v, wl.sm_scale, persistent_parity=0,
                                                temporary_window=wl.window, documents_idx=wl.docs, out=out)
        work, unit = wl.flops / 1e12, "TFLOP/s"
    elif args.case == "full-window-small":
        wl = workloads.make_prefill(PREFILL_FULL_WINDOW, device, head_slice=slice(0, 4))
        out = torch.empty_like(wl.q)
        fn = lambda: sps_b200.prefill_attention(wl.q, wl.k, wl.v, wl.sm_scale, persistent_parity=0,
                                                temporary_window=wl.window, documents_idx=None, out=out)
        work, unit = wl.flops / 1e12, "TFLOP/s"
    elif args.case in ("backward-small", "backward-full-window-small"):
        if args.case == "backward-small":
            wl = workloads.make_prefill(PREFILL, device, batch_slice=slice(0, 4))
        else:
            wl = workloads.make_prefill(PREFILL_FULL_WINDOW, device, head_slice=slice(0, 4))
        o_b, lse_b = sps_b200.prefill_attention(wl.q, wl.k, wl.v, wl.sm_scale, persistent_parity=0,
                                                temporary_window=wl.window, documents_idx=wl.docs,
                                                return_lse=True)
        d_o = torch.randn(wl.q.shape, device=device, dtype=torch.float32).to(wl.q.dtype)
        fn = lambda: sps_b200.attention.prefill_attention_backward(
            wl.q, wl.k, wl.v, o_b, lse_b, d_o, wl.sm_scale, persistent_parity=0,
            temporary_window=wl.window, documents_idx=wl.docs)
        work, unit = 2.5 * wl.flops / 1e12, "TFLOP/s"
    else:
        dw = workloads.make_decode(DECODE, device, seq_slice=slice(0, 32))
        segs = [sps_b200.KVSegment(dw.ring_k, dw.ring_v, dw.ring_len, max_len_cap=dw.ring_k.shape[2]),
                sps_b200.KVSegment(dw.cache_k, dw.cache_v, dw.cache_len, max_len_cap=dw.cache_k.shape[2])]
        fn = lambda: sps_b200.segmented_q2_attention(
            dw.q, segs, current_normal_k_BxHxD=dw.cur_k, current_normal_v_BxHxD=dw.cur_v,
            current_predict_k_BxHxD=dw.pred_k, current_predict_v_BxHxD=dw.pred_v, attn_dtype=torch.bfloat16)
        work, unit = dw.bytes / 1e9, "GB/s"
    _, launch_ms, _ = timed_steps(fn, args.steps, max(args.warmup, 1), 1, device, regions=1)
    sps_b200.check_device_status(device)
    emit(({"case": args.case, "launch_ms": launch_ms, "work": work,
                      "achieved": work / (launch_ms * 1e-3), "unit": unit}))


def _sum_over_ranks(x, world, device):
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


# -------------------------------------------------------------------------- CPU baseline

def _reference_cpu_modules():
    """The reference's own CPU formulations, when its package is installed under baseline/_ref:
    (its SDPA test oracle for SPS attention, its masked_kv_attention + KVSegment), else None."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "modeling", "models")):
        return None
    try:
        if ref_dir not in sys.path:
            sys.path.insert(0, ref_dir)
        from modeling.models.utils.decode_attention import KVSegment, masked_kv_attention
        from modeling.tests.attention.triton.test_sps_attention import _sdpa_reference_attention_sps
        return _sdpa_reference_attention_sps, masked_kv_attention, KVSegment
    except Exception:
        return None


CPU_SAMPLE_HEADS = 2


def cpu_sample():
    """One bounded sample of the prefill workload on the host: batch row 0, the first two heads,
    full length (2T = 8192), through the dense additive mask + SDPA formulation: the reference's
    own function (src/modeling/tests/attention/triton/test_sps_attention.py:25-74) when its
    package is installed under baseline/_ref, else the restatement in oracle/.  Returns
    (callable, useful FLOPs of one call, kind, description)."""
    from sps_b200 import workloads
    B, H, T, D, w, mean = workloads.PREFILL_CONFIGS[PREFILL]
    n_heads = CPU_SAMPLE_HEADS
    docs = workloads.geometric_docs(B, T, mean, 0)[:1]
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, n_heads, 2 * T, D, generator=g) for _ in range(3))
    flops = workloads.prefill_flops(workloads.useful_pairs(docs, w), n_heads, D)
    dd = torch.from_numpy(docs)
    what = f"{PREFILL} batch row 0, heads 0-{n_heads - 1}, full length {2 * T} per step: dense additive mask + torch SDPA fp32"
    ref = _reference_cpu_modules()
    if ref is not None:
        fn = ref[0]
        return (lambda: fn(q, k, v, w, dd)), flops, "reference", what + " (the reference's _sdpa_reference_attention_sps)"
    from oracle import sps_oracle as orc
    return (lambda: orc.prefill_attention_sdpa(q, k, v, 1.0 / np.sqrt(D), temporary_window=w, docs=dd)), flops, \
        "port", what + " (the reference's CPU formulation restated in oracle/)"


def cpu_baseline(budget_s: float):
    torch.set_num_threads(os.cpu_count() or 1)
    run, flops, kind, what = cpu_sample()
    run()                                   # warm-up
    t0, n = time.perf_counter(), 0
    while True:
        run()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 50:
            break
    dt = (time.perf_counter() - t0) / n
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
            "sample": f"{what}, {n} passes of {dt:.2f} s", "seconds_per_pass": dt}


def cpu_baseline_decode(dw, budget_s: float, n_seq: int = 8):
    """The decode step on the host for the first `n_seq` sequences of the workload: the
    reference's SDPA fallback (masked_kv_attention, src/modeling/models/utils/decode_attention.py:
    637-704), once per query as the reference's callers use it, or its restatement in oracle/.
    GB/s on the same algorithmic bytes as the GPU figure."""
    from sps_b200 import workloads
    torch.set_num_threads(os.cpu_count() or 1)
    sl = slice(0, n_seq)
    t = {n: getattr(dw, n)[sl].cpu() for n in ("q", "cache_k", "cache_v", "cache_len", "ring_k", "ring_v", "ring_len",
                                                "cur_k", "cur_v", "pred_k", "pred_v")}
    H, D, ring = t["q"].shape[2], t["q"].shape[3], t["ring_k"].shape[2]
    nbytes = workloads.decode_bytes(dw.lens_np[sl], ring, H, D)
    ref = _reference_cpu_modules()
    if ref is not None:
        _, mkv, Seg = ref
        f32 = {n: (x.float() if x.is_floating_point() else x) for n, x in t.items()}
        segs = [Seg(f32["ring_k"], f32["ring_v"], f32["ring_len"], max_len_cap=ring),
                Seg(f32["cache_k"], f32["cache_v"], f32["cache_len"], max_len_cap=f32["cache_k"].shape[2])]

        def run():
            mkv(f32["q"][:, 0], segs, extra_kv=[(f32["cur_k"], f32["cur_v"])], attn_dtype=torch.float32)
            mkv(f32["q"][:, 1], segs, extra_kv=[(f32["cur_k"], f32["cur_v"]), (f32["pred_k"], f32["pred_v"])],
                attn_dtype=torch.float32)
        kind, what = "reference", "the reference's masked_kv_attention SDPA fallback, one call per query"
    else:
        from oracle import sps_oracle as orc

        def run():
            orc.decode_attention_batched(t["q"], t["cache_k"], t["cache_v"], t["cache_len"], t["ring_k"], t["ring_v"],
                                         t["ring_len"], t["cur_k"], t["cur_v"], t["pred_k"], t["pred_v"])
        kind, what = "port", "padded K/V + boolean mask + torch SDPA fp32 (the reference's fallback restated in oracle/)"
    run()
    t0, n = time.perf_counter(), 0
    while True:
        run()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 50:
            break
    dt = (time.perf_counter() - t0) / n
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "tokens_per_s": n_seq / dt, "cores": torch.get_num_threads(),
            "kind": kind, "sample": f"{DECODE} sequences 0-{n_seq - 1} of 128 (padded to 4096 rows): {what}, "
                                    f"{n} passes of {dt:.2f} s"}


def cpu_baseline_generation(budget_s: float):
    """Greedy generation of the model-level CPU oracle (oracle/sps_model_oracle.py: dense re-forward
    per token in fp32, the attention oracle inside) on a labelled reduced size: tokens/s."""
    from oracle import sps_model_oracle as mo
    from sps_b200 import workloads
    from sps_b200.generation import SPSDims, random_state_dict
    torch.set_num_threads(os.cpu_count() or 1)
    cfg = workloads.GENERATION_CONFIGS["generation_small"]
    fields = {k: cfg[k] for k in ("block_size", "vocab_size", "n_layer", "n_head", "hidden_size", "intermediate_size",
                                  "eos_token_id", "pad_token_id", "predict_token_id", "window_size")}
    sd = {k: v.float() for k, v in random_state_dict(SPSDims(**fields), seed=0, device="cpu").items()}
    dims = mo.Dims(**fields)
    batch, new = 2, 4
    prompts = torch.from_numpy(workloads.generation_prompts(cfg, batch, 0))
    t0, n = time.perf_counter(), 0
    while True:
        mo.generate(sd, dims, prompts, new, variant="sps", stop_on_eos=False)
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 20:
            break
    dt = (time.perf_counter() - t0) / n
    return {"value": batch * new / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"REDUCED SIZE (generation_small: {fields['n_layer']} layers, hidden {fields['hidden_size']}, "
                      f"{fields['n_head']} heads, prompt {cfg['prompt']}, batch {batch}, {new} new tokens): the model "
                      f"oracle's greedy generation (dense fp32 re-forward per token), {n} passes of {dt:.2f} s; the "
                      "reference's model classes have no CPU path for the fused decode step"}


def run_reference(args):
    """The reference's CPU path for this workload on the host cores: rank 0 only.  Same metric,
    unit and config object as the other arm; every step is the bounded sample of `cpu_sample`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    K, W = max(1, args.steps), max(args.warmup, 3)
    run, flops, kind, what = cpu_sample()
    for _ in range(W):
        run()
    t0 = time.perf_counter()
    for _ in range(K):
        run()
    dt = time.perf_counter() - t0
    value = flops * K / dt / 1e12
    emit(({
        "impl": "reference", "metric": "sps_prefill_useful_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": dt / K * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(world),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": what},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--case", choices=["full", "prefill-small", "full-window-small", "backward-small", "backward-full-window-small", "decode-small", "generation-small", "generation"], default="full")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-decode", action="store_true")
    ap.add_argument("--skip-backward", action="store_true", help="skip the prefill backward section")
    ap.add_argument("--skip-full-window", action="store_true")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-generation", action="store_true")
    ap.add_argument("--skip-reference-triton", action="store_true",
                    help="do not time the reference's Triton kernels (baseline/_ref) beside ours")
    ap.add_argument("--prefill-path", choices=["auto", "tiles64", "persistent128"], default="auto",
                    help="tensor-core prefill kernel at head_dim 64 (auto: the 64-key-tile kernel)")
    ap.add_argument("--decode-path", choices=["auto", "cuda-core", "tensor-core"], default="auto",
                    help="decode kernel behind the decode step (auto: tensor cores at head_dim 64)")
    ap.add_argument("--new-tokens", type=int, default=None, help="generation cases: tokens to generate")
    ap.add_argument("--runs", type=int, default=3, help="generation cases: timed repetitions")
    args = ap.parse_args()
    # stdout carries the JSON line and nothing else: libraries that print there (NCCL's version
    # banner, for one) are sent to stderr by swapping the descriptors for the whole run
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    try:
        _dispatch(args)
    finally:
        sys.stdout.flush()
        os.dup2(json_fd, 1)
        os.close(json_fd)
    for line in _JSON_LINES:
        print(line, flush=True)


_JSON_LINES = []


def emit(obj):
    """Queue one JSON line for stdout (printed after the run, when stdout is ours again)."""
    _JSON_LINES.append(json.dumps(obj))


def _dispatch(args):
    if args.decode_path != "auto" and args.impl == "ours":
        from sps_b200 import _lib
        _lib.check(_lib.load().spsattn_debug_decode_path({"cuda-core": 1, "tensor-core": 2}[args.decode_path]),
                   "spsattn_debug_decode_path")
    if args.prefill_path != "auto" and args.impl == "ours":
        from sps_b200 import _lib
        _lib.check(_lib.load().spsattn_debug_prefill_path({"tiles64": 1, "persistent128": 2}[args.prefill_path]),
                   "spsattn_debug_prefill_path")
    if args.impl == "reference":
        run_reference(args)
    elif args.case != "full":
        run_case(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
