"""Seeded synthetic workloads with the shapes, sizes and value distributions of the benchmark
configurations, and the algorithmic work (useful FLOPs, bytes) each one represents.

The reference measures on tokenised web text and trained checkpoints; neither ships with it, so
these generators stand in: N(0,1) Q/K/V, document lengths ~ Geometric(mean), cache lengths ~
UniformInt.  Pure host logic plus tensor creation; nothing here computes attention.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

# name -> (B, H, T, D, window, mean document length or None for one document per row)
PREFILL_CONFIGS = {
    "cfg0_cpu_shape": (2, 8, 256, 64, 64, 100),
    "cfg1_s_scale": (8, 12, 4096, 64, 64, 1000),
    "cfg4_full_window": (4, 16, 4096, 128, 4096, None),
}
# name -> (S, H, D, ring, len_lo, len_hi)
DECODE_CONFIGS = {
    "cfg2_segmented_decode": (128, 16, 64, 64, 512, 4096),
}
# name -> model dims, batch, prompt length, new tokens.  The shapes of the reference's generation
# benchmark (prompt 1024, greedy, bf16 cache, w = 64; scripts/benchmark/benchmark_generation_speed.py)
# on the decoder the reference implements (RMSNorm, rotary, SwiGLU, tied head).
GENERATION_CONFIGS = {
    "cfg3_xl_generation": dict(block_size=1280, vocab_size=50304, n_layer=24, n_head=16, hidden_size=2048,
                               intermediate_size=8192, eos_token_id=50256, pad_token_id=50303,
                               predict_token_id=50257, window_size=64, batch=32, prompt=1024, new_tokens=256),
    "generation_small": dict(block_size=160, vocab_size=2048, n_layer=2, n_head=4, hidden_size=512,
                             intermediate_size=1024, eos_token_id=2000, pad_token_id=2047,
                             predict_token_id=2001, window_size=16, batch=4, prompt=96, new_tokens=24),
}


def generation_forbidden_ids(cfg: dict) -> list:
    """Token ids the reference's speed benchmark never lets the model emit: everything above EOS,
    the pad and the <predict> id (benchmark_generation_speed.py:204-220)."""
    ids = set(range(cfg["eos_token_id"] + 1, cfg["vocab_size"]))
    ids.update((cfg["pad_token_id"], cfg["predict_token_id"]))
    return sorted(ids)


def generation_prompts(cfg: dict, batch: int, seed: int) -> np.ndarray:
    """[batch, prompt] int64 ids uniform in [0, eos): single-document prompts without special ids."""
    rng = np.random.default_rng(seed)
    return rng.integers(0, cfg["eos_token_id"], size=(batch, cfg["prompt"]), dtype=np.int64)


def generation_step_bytes(cfg: dict, batch: int, live_tokens: float) -> float:
    """Bytes one decode step must read at least: every parameter once (bf16; the embedding table is
    read once as the head) plus the live K/V rows of every layer (retained cache + ring)."""
    c, i, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["n_layer"]
    params = L * (4 * c * c + 3 * c * i) + cfg["vocab_size"] * c
    kv = L * batch * (live_tokens + cfg["window_size"]) * c * 2
    return 2.0 * (params + kv)


def geometric_docs(batch: int, tokens: int, mean: Optional[float], seed: int) -> np.ndarray:
    """Document id per row of the doubled sequence, [batch, 2*tokens] int64: per batch row,
    document lengths ~ Geometric(1/mean) are laid end to end until `tokens` tokens are covered
    (the last one truncated); ids 0,1,2,...; each token's id is repeated for its <predict> row."""
    out = np.zeros((batch, tokens), dtype=np.int64)
    if mean is not None:
        rng = np.random.default_rng(seed)
        for b in range(batch):
            pos, d = 0, 0
            while pos < tokens:
                ln = int(rng.geometric(1.0 / mean))
                out[b, pos:pos + ln] = d
                pos += ln
                d += 1
    return np.repeat(out, 2, axis=1)


def run_lengths(ids_row: np.ndarray) -> np.ndarray:
    """Lengths of the maximal runs of equal ids in a row."""
    change = np.flatnonzero(ids_row[1:] != ids_row[:-1]) + 1
    edges = np.concatenate([[0], change, [len(ids_row)]])
    return np.diff(edges)


def useful_pairs(docs: np.ndarray, window: int, rule: str = "reference") -> int:
    """Visible (query, key) pairs summed over the batch, closed form per document of L tokens.

    reference rule (the kernels' default; input queries also see the <= w previous predict keys,
    window inclusive):      L(L+1) + L + 2 * sum_{t<L} min(t, w)
    'baseline_prose' rule (input queries see input keys only, predict window exclusive):
                             L(L+1) + sum_{t<L} min(t+1, w)
    Valid for ids that are constant per token and non-decreasing along the row.
    """
    total = 0
    for row in docs:
        for rows in run_lengths(row):
            L = int(rows) // 2
            t = np.arange(L, dtype=np.int64)
            if rule == "reference":
                total += L * (L + 1) + L + 2 * int(np.minimum(t, window).sum())
            elif rule == "baseline_prose":
                total += L * (L + 1) + int(np.minimum(t + 1, window).sum())
            else:
                raise ValueError(rule)
    return int(total)


def prefill_flops(pairs: int, heads: int, head_dim: int) -> float:
    """2 FLOP per multiply-add, two contractions (QK^T and PV), per head."""
    return 4.0 * head_dim * heads * pairs


@dataclass
class PrefillWorkload:
    name: str
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    docs: Optional[torch.Tensor]       # [B, 2T] int64 on the same device, or None
    docs_np: np.ndarray
    window: int
    sm_scale: float
    pairs: int                          # visible pairs, reference rule
    flops: float                        # useful FLOPs


def make_prefill(name: str, device, *, seed: int = 0, dtype=torch.bfloat16,
                 batch_slice: Optional[slice] = None, head_slice: Optional[slice] = None) -> PrefillWorkload:
    """Build one prefill configuration.  `batch_slice` / `head_slice` select this rank's shard
    of the full problem (the documents and the values of the shard are those of the full one)."""
    B, H, T, D, w, mean = PREFILL_CONFIGS[name]
    docs_np = geometric_docs(B, T, mean, seed)
    bs = range(B)[batch_slice] if batch_slice is not None else range(B)
    hs = range(H)[head_slice] if head_slice is not None else range(H)
    docs_np = docs_np[list(bs)]
    gen = torch.Generator(device="cpu").manual_seed(seed)
    # one seed per (tensor, batch row, head) so shards see the values of the full problem
    seeds = torch.randint(0, 2**31 - 1, (3, B, H), generator=gen)
    dev = torch.device(device)
    tensors = []
    for t in range(3):
        x = torch.empty((len(bs), len(hs), 2 * T, D), dtype=dtype, device=dev)
        for bi, b in enumerate(bs):
            for hi, h in enumerate(hs):
                g = torch.Generator(device=dev).manual_seed(int(seeds[t, b, h]))
                x[bi, hi] = torch.randn((2 * T, D), generator=g, device=dev, dtype=torch.float32).to(dtype)
        tensors.append(x)
    pairs = useful_pairs(docs_np, w)
    docs = None if mean is None else torch.from_numpy(docs_np).to(dev)
    return PrefillWorkload(name, tensors[0], tensors[1], tensors[2], docs, docs_np, w,
                           1.0 / float(np.sqrt(D)), pairs, prefill_flops(pairs, len(hs), D))


@dataclass
class DecodeWorkload:
    name: str
    q: torch.Tensor                    # [S, 2, H, D]
    cache_k: torch.Tensor              # [S, H, cap, D]
    cache_v: torch.Tensor
    cache_len: torch.Tensor            # [S] int64
    ring_k: torch.Tensor               # [S, H, ring, D]
    ring_v: torch.Tensor
    ring_len: torch.Tensor             # [S] int64
    cur_k: torch.Tensor                # [S, H, D] current input token
    cur_v: torch.Tensor
    pred_k: torch.Tensor               # [S, H, D] current <predict> token
    pred_v: torch.Tensor
    lens_np: np.ndarray
    bytes: float                       # algorithmic bytes of one step


def decode_lengths(name: str, seed: int = 0) -> np.ndarray:
    S, _, _, _, lo, hi = DECODE_CONFIGS[name]
    return np.random.default_rng(seed).integers(lo, hi + 1, size=S).astype(np.int64)


def decode_bytes(lens: np.ndarray, ring: int, heads: int, head_dim: int, nq: int = 2,
                 elem: int = 2) -> float:
    """Bytes one decode step has to move: every live K and V row once (cache + ring), the
    current K/V entries, the queries, and the fp32 output."""
    S = len(lens)
    kv = float((lens.sum() + S * ring)) * heads * head_dim * 2 * elem
    cur = 4.0 * S * heads * head_dim * elem
    qb = float(S) * nq * heads * head_dim * elem
    ob = float(S) * nq * heads * head_dim * 4
    return kv + cur + qb + ob


def make_decode(name: str, device, *, seed: int = 0, dtype=torch.bfloat16,
                seq_slice: Optional[slice] = None, seq_index=None) -> DecodeWorkload:
    """Build the decode configuration, or this rank's shard of it: `seq_slice` (a contiguous
    range) or `seq_index` (any list of sequence numbers, e.g. one bin of `balanced_partition`)."""
    S, H, D, ring, lo, hi = DECODE_CONFIGS[name]
    lens = decode_lengths(name, seed)
    if seq_index is not None:
        sel = np.asarray(sorted(int(i) for i in seq_index), dtype=np.int64)
    else:
        sel = np.arange(S)[seq_slice] if seq_slice is not None else np.arange(S)
    lens = lens[sel]
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed * 7919 + int(sel[0]) + 1)
    n = len(sel)

    def rnd(*shape):
        return torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dtype)

    cache_k, cache_v = torch.empty((n, H, hi, D), dtype=dtype, device=dev), torch.empty((n, H, hi, D), dtype=dtype, device=dev)
    for s in range(n):     # row by row keeps the fp32 staging buffer small
        cache_k[s] = rnd(H, hi, D)
        cache_v[s] = rnd(H, hi, D)
    return DecodeWorkload(
        name, rnd(n, 2, H, D), cache_k, cache_v, torch.from_numpy(lens).to(dev),
        rnd(n, H, ring, D), rnd(n, H, ring, D), torch.full((n,), ring, dtype=torch.int64, device=dev),
        rnd(n, H, D), rnd(n, H, D), rnd(n, H, D), rnd(n, H, D), lens,
        decode_bytes(lens, ring, H, D))


def shard_slice(n_items: int, rank: int, world: int) -> slice:
    """Contiguous shard of `n_items` for `rank` of `world` (sizes differ by at most one)."""
    base, rem = divmod(n_items, world)
    start = rank * base + min(rank, rem)
    return slice(start, start + base + (1 if rank < rem else 0))


def balanced_partition(weights, world: int) -> list:
    """Split items 0..n-1 into `world` bins of nearly equal total weight: heaviest item first,
    each into the lightest bin so far (ties: the lower bin).  Returns the sorted item numbers of
    every bin; used to shard decode sequences by the sum of their cache lengths rather than by
    their count."""
    w = np.asarray(weights, dtype=np.float64)
    bins = [[] for _ in range(world)]
    load = np.zeros(world)
    for i in sorted(range(len(w)), key=lambda i: (-w[i], i)):
        r = int(np.argmin(load))
        bins[r].append(i)
        load[r] += w[i]
    return [sorted(b) for b in bins]
