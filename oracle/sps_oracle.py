"""CPU oracle for the SPS attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy (integer mask / index rules) and CPU torch fp32
(the floating-point attention itself), what the reference computes for

  * SPS / Reverse-SPS / Standard prefill attention over the doubled 2T sequence,
  * the segmented q=2 / q=1 decode attention over length-masked KV segments,
  * the fused decode KV-cache update (ring insert + retained append).

Only tests, the smoke check and the ``cpu_baseline`` / ``--impl reference``
legs of the benchmark may import it.  Nothing in the ``sps_b200`` package does:
the product path is CUDA only and fails loudly without its extension.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the reference's own
PyTorch oracles (imported from the reference checkout) on seeded inputs and
stores inputs and outputs; ``tests/test_oracle_golden.py`` checks every function
here against those fixtures, and against the literal known answers the
reference's tests hold (window visibility lists, ring contents).

Each function cites the reference file:line it follows (paths relative to the
reference project root).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

# persistent-key parity codes shared with the C ABI (include/spsattn.h)
PARITY_EVEN = 0    # SPS: input slot (even row) is the persistent / window-exempt key
PARITY_ODD = 1     # Reverse-SPS, Delayed-State: the odd row is persistent
PARITY_NONE = -1   # Standard model: causal + document mask only

# mask_flags bits shared with the C ABI
FLAG_PERSISTENT_Q_SKIPS_TEMPORARY = 1  # query rows of persistent parity see no temporary keys


# ---------------------------------------------------------------------------
# integer rules (bit-exact targets)
# ---------------------------------------------------------------------------

def visible_mask(
    n_ctx: int,
    *,
    persistent_parity: int = PARITY_EVEN,
    temporary_window: int = 0,
    persistent_window: Optional[int] = None,
    docs_row: Optional[np.ndarray] = None,
    mask_flags: int = 0,
) -> np.ndarray:
    """Boolean [n_ctx, n_ctx] visibility matrix, query row i x key row j.

    Follows src/modeling/models/attention/triton_sps_flash_attention.py:81-111
    (document bias :81-87, temporary window on ``rel > w`` :93-95, persistent
    keys exempt :97-105, self-persistent exception :106-107, causal :109-111),
    src/modeling/models/attention/triton_reverse_sps_flash_attention.py:106-136
    (same rule with the persistent key at odd parity, :123) and
    src/modeling/models/attention/triton_full_flash_attention.py:95-104
    (``PARITY_NONE``: causal and same-document only).  The additive -1e6 biases
    of the reference are treated as hard masks: exp2 of them is exactly 0 in fp32.
    """
    i = np.arange(n_ctx, dtype=np.int64)[:, None]
    j = np.arange(n_ctx, dtype=np.int64)[None, :]
    vis = j <= i
    if docs_row is not None:
        d = np.asarray(docs_row).astype(np.int64).reshape(n_ctx)
        vis &= d[:, None] == d[None, :]
    if persistent_parity != PARITY_NONE:
        rel = i // 2 - j // 2
        k_persistent = (j % 2) == persistent_parity
        temp_ok = rel <= int(temporary_window)
        if mask_flags & FLAG_PERSISTENT_Q_SKIPS_TEMPORARY:
            temp_ok = temp_ok & ((i % 2) != persistent_parity)
        if persistent_window is None:
            pers_ok = np.ones_like(temp_ok)
        else:
            pers_ok = (rel <= int(persistent_window)) | (i == j)
        vis &= np.where(k_persistent, pers_ok, temp_ok)
    return vis


def count_visible_pairs(
    docs: Optional[np.ndarray],
    n_ctx: int,
    batch: int,
    **rule,
) -> int:
    """Number of visible (query, key) pairs summed over the batch rows.

    Useful FLOPs of prefill are 4 * D * H * this count (2 FLOP per MAC, two
    contractions).  Computed exhaustively in key blocks so 8192 x 8192 fits.
    """
    total = 0
    for b in range(batch):
        row = None if docs is None else np.asarray(docs[b])
        total += _count_row(n_ctx, row, **rule)
    return int(total)


def _count_row(n_ctx, docs_row, *, persistent_parity=PARITY_EVEN, temporary_window=0,
               persistent_window=None, mask_flags=0, block=1024) -> int:
    d = None if docs_row is None else np.asarray(docs_row).astype(np.int64)
    total = 0
    for i0 in range(0, n_ctx, block):
        i = np.arange(i0, min(i0 + block, n_ctx), dtype=np.int64)[:, None]
        for j0 in range(0, i0 + block, block):
            j = np.arange(j0, min(j0 + block, n_ctx), dtype=np.int64)[None, :]
            vis = j <= i
            if d is not None:
                vis &= d[i[:, 0]][:, None] == d[j[0]][None, :]
            if persistent_parity != PARITY_NONE:
                rel = i // 2 - j // 2
                kp = (j % 2) == persistent_parity
                t_ok = rel <= int(temporary_window)
                if mask_flags & FLAG_PERSISTENT_Q_SKIPS_TEMPORARY:
                    t_ok = t_ok & ((i % 2) != persistent_parity)
                p_ok = np.ones_like(t_ok) if persistent_window is None else (
                    (rel <= int(persistent_window)) | (i == j))
                vis &= np.where(kp, p_ok, t_ok)
            total += int(vis.sum())
    return total


def run_starts(docs_row: np.ndarray) -> np.ndarray:
    """lo[i] = first row of the maximal run of equal document ids containing row i.

    This is the integer table the CUDA pre-pass writes; for non-decreasing ids
    ``docs[i] == docs[j]`` with ``j <= i`` is equivalent to ``j >= lo[i]``.
    """
    d = np.asarray(docs_row).astype(np.int64)
    n = d.shape[0]
    starts = np.zeros(n, dtype=np.int64)
    if n > 1:
        change = d[1:] != d[:-1]
        starts[1:] = np.where(change, np.arange(1, n), 0)
    return np.maximum.accumulate(starts).astype(np.int32)


def is_monotone(docs_row: np.ndarray) -> bool:
    d = np.asarray(docs_row).astype(np.int64)
    return bool(np.all(d[1:] >= d[:-1]))


def segment_rows(length: int, capacity: int, max_len_cap: Optional[int]) -> int:
    """Number of cache rows [0, n) a decode query scans in one segment.

    Follows src/modeling/models/utils/decode_attention.py:381-390 (scan length =
    storage, or clamp(cap, 1, storage) when a cap is given) combined with the
    kernel's ``offs < len`` validity test (:206-210): rows scanned =
    min(len, scan_len), never negative.
    """
    if capacity == 0:
        return 0
    scan = capacity if max_len_cap is None else max(1, min(capacity, int(max_len_cap)))
    return max(0, min(int(length), scan))


# ---------------------------------------------------------------------------
# prefill attention (fp32)
# ---------------------------------------------------------------------------

def prefill_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: float,
    *,
    persistent_parity: int = PARITY_EVEN,
    temporary_window: int = 0,
    persistent_window: Optional[int] = None,
    docs: Optional[torch.Tensor] = None,
    mask_flags: int = 0,
    rows: Optional[np.ndarray] = None,
    return_lse: bool = False,
):
    """Masked softmax attention in fp32 on CPU, one (batch, head) slice at a time.

    Same math as the reference's test oracle
    src/modeling/tests/attention/triton/test_sps_attention.py:25-74 (additive
    mask then scaled_dot_product_attention) and
    src/modeling/tests/attention/triton/test_full_flash_attention.py:29-59, but
    sliced per (b, h) so the [N, N] score matrix stays small.  ``rows`` restricts
    the queries evaluated (all keys are still considered) for spot checks at
    full size.  Rows with no visible key return 0.
    ``lse`` (optional) is log2(sum exp2(score * scale * log2 e)), the quantity the
    reference kernel stores as M (triton_sps_flash_attention.py:265-267).
    """
    B, H, N, D = q.shape
    qf, kf, vf = q.float(), k.float(), v.float()
    sel = np.arange(N) if rows is None else np.asarray(rows, dtype=np.int64)
    out = torch.zeros((B, H, len(sel), D), dtype=torch.float32)
    lse = torch.zeros((B, H, len(sel)), dtype=torch.float32)
    sel_t = torch.from_numpy(sel)
    for b in range(B):
        drow = None if docs is None else docs[b].cpu().numpy()
        vis = torch.from_numpy(_visible_rows(N, sel, persistent_parity, temporary_window,
                                             persistent_window, drow, mask_flags))
        any_vis = vis.any(dim=1)
        for h in range(H):
            s = (qf[b, h, sel_t] @ kf[b, h].T) * float(sm_scale)
            s = s.masked_fill(~vis, float("-inf"))
            m = s.max(dim=1, keepdim=True).values
            m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
            p = torch.exp(s - m)
            l = p.sum(dim=1, keepdim=True)
            o = (p @ vf[b, h]) / torch.where(l > 0, l, torch.ones_like(l))
            out[b, h] = torch.where(any_vis[:, None], o, torch.zeros_like(o))
            lse[b, h] = ((m + torch.log(torch.where(l > 0, l, torch.ones_like(l))))
                         * 1.4426950408889634).squeeze(1)
    return (out, lse) if return_lse else out


def prefill_attention_grads(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    d_o: torch.Tensor,
    sm_scale: float,
    *,
    persistent_parity: int = PARITY_EVEN,
    temporary_window: int = 0,
    persistent_window: Optional[int] = None,
    docs: Optional[torch.Tensor] = None,
    mask_flags: int = 0,
):
    """dQ, dK, dV of ``prefill_attention`` in fp32 on CPU, one (batch, head) slice at a time.

    The closed form every flash-attention backward uses, and the one the reference's kernels
    implement (src/modeling/models/attention/triton_sps_flash_attention.py:272-488):
    P = softmax(mask(S)), dV = P^T dO, dP = dO V^T, dS = P * (dP - rowsum(dO * O)),
    dQ = dS K * scale, dK = dS^T Q * scale.  The reference's own test obtains the same
    quantities from autograd through its SDPA oracle
    (src/modeling/tests/attention/triton/test_sps_attention.py:79-131); the CPU tests check
    this function against exactly that.
    """
    B, H, N, D = q.shape
    qf, kf, vf, gf = q.float(), k.float(), v.float(), d_o.float()
    dq, dk, dv = torch.zeros_like(qf), torch.zeros_like(kf), torch.zeros_like(vf)
    sel = np.arange(N)
    for b in range(B):
        drow = None if docs is None else docs[b].cpu().numpy()
        vis = torch.from_numpy(_visible_rows(N, sel, persistent_parity, temporary_window,
                                             persistent_window, drow, mask_flags))
        for h in range(H):
            s = (qf[b, h] @ kf[b, h].T) * float(sm_scale)
            s = s.masked_fill(~vis, float("-inf"))
            m = s.max(dim=1, keepdim=True).values
            m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
            p = torch.exp(s - m)
            l = p.sum(dim=1, keepdim=True)
            p = p / torch.where(l > 0, l, torch.ones_like(l))
            o = p @ vf[b, h]
            dv[b, h] = p.T @ gf[b, h]
            dp = gf[b, h] @ vf[b, h].T
            ds = p * (dp - (gf[b, h] * o).sum(dim=1, keepdim=True))
            dq[b, h] = (ds @ kf[b, h]) * float(sm_scale)
            dk[b, h] = (ds.T @ qf[b, h]) * float(sm_scale)
    return dq, dk, dv


def _visible_rows(n, sel, parity, w, pw, drow, flags) -> np.ndarray:
    i = sel.astype(np.int64)[:, None]
    j = np.arange(n, dtype=np.int64)[None, :]
    vis = j <= i
    if drow is not None:
        d = np.asarray(drow).astype(np.int64)
        vis &= d[sel][:, None] == d[None, :]
    if parity != PARITY_NONE:
        rel = i // 2 - j // 2
        kp = (j % 2) == parity
        t_ok = rel <= int(w)
        if flags & FLAG_PERSISTENT_Q_SKIPS_TEMPORARY:
            t_ok = t_ok & ((i % 2) != parity)
        p_ok = np.ones_like(t_ok) if pw is None else ((rel <= int(pw)) | (i == j))
        vis &= np.where(kp, p_ok, t_ok)
    return vis


def prefill_attention_sdpa(q, k, v, sm_scale, *, temporary_window, docs=None):
    """The reference's CPU path for SPS prefill, restated: dense additive mask +
    torch SDPA over the whole [B,H,N,N] problem (test_sps_attention.py:25-74).
    Used as the timed CPU baseline; ``prefill_attention`` is the checker.
    """
    B, H, N, D = q.shape
    add = torch.zeros((B, 1, N, N), dtype=torch.float32)
    for b in range(B):
        drow = None if docs is None else docs[b].cpu().numpy()
        vis = visible_mask(N, persistent_parity=PARITY_EVEN, temporary_window=temporary_window,
                           docs_row=drow)
        add[b, 0] = torch.from_numpy(np.where(vis, 0.0, -np.inf).astype(np.float32))
    return torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float(), v.float(), attn_mask=add, is_causal=False, scale=float(sm_scale))


# ---------------------------------------------------------------------------
# decode attention (fp32)
# ---------------------------------------------------------------------------

@dataclass
class Segment:
    """Host mirror of a KV segment: k, v [S,H,cap,D]; lengths [S] or [S,H]
    (src/modeling/models/utils/decode_attention.py:21-32)."""
    k: torch.Tensor
    v: torch.Tensor
    lengths: torch.Tensor
    max_len_cap: Optional[int] = None
    query_mask: int = 0xFF  # bit i set: query slot i scans this segment


def decode_attention(
    q: torch.Tensor,                       # [S, nq, H, D]
    segments: Sequence[Segment],
    extras: Sequence[tuple],               # (k [S,H,D], v [S,H,D], query_mask)
    sm_scale: Optional[float] = None,
) -> torch.Tensor:
    """Segmented decode attention, fp32 out [S, nq, H, D].

    Follows src/modeling/tests/models/attention/test_segmented_q2_attention.py:25-62
    (per (b,h): concatenate the live rows of every segment, then the current
    keys; slot 0 sees the current normal key, slot 1 both currents) and the
    kernel src/modeling/models/utils/decode_attention.py:267-368 (``out = 0``
    when no key is visible, :363-366).  Scale is 1/sqrt(D) as at :575.
    """
    S, nq, H, D = q.shape
    scale = 1.0 / math.sqrt(D) if sm_scale is None else float(sm_scale)
    out = torch.zeros((S, nq, H, D), dtype=torch.float32)
    for s in range(S):
        for h in range(H):
            for qi in range(nq):
                ks, vs = [], []
                for seg in segments:
                    if not (seg.query_mask >> qi) & 1:
                        continue
                    ln = seg.lengths[s] if seg.lengths.dim() == 1 else seg.lengths[s, h]
                    n = segment_rows(int(ln), int(seg.k.shape[2]), seg.max_len_cap)
                    if n:
                        ks.append(seg.k[s, h, :n].float())
                        vs.append(seg.v[s, h, :n].float())
                for ek, ev, qm in extras:
                    if (qm >> qi) & 1:
                        ks.append(ek[s, h].float().view(1, D))
                        vs.append(ev[s, h].float().view(1, D))
                if not ks:
                    continue
                kk, vv = torch.cat(ks), torch.cat(vs)
                p = torch.softmax((q[s, qi, h].float() @ kk.T) * scale, dim=-1)
                out[s, qi, h] = p @ vv
    return out


def decode_attention_batched(q, seg_k, seg_v, seg_len, ring_k, ring_v, ring_len,
                             cur_k, cur_v, pred_k, pred_v):
    """Vectorised q=2 decode for the timed CPU baseline (same math as
    ``decode_attention`` with segments [ring, retained] and the two current
    keys; padded-SDPA formulation of decode_attention.py:637-704)."""
    S, nq, H, D = q.shape
    cap, rcap = seg_k.shape[2], ring_k.shape[2]
    keys = torch.cat([seg_k.float(), ring_k.float(), cur_k.float().unsqueeze(2),
                      pred_k.float().unsqueeze(2)], dim=2)
    vals = torch.cat([seg_v.float(), ring_v.float(), cur_v.float().unsqueeze(2),
                      pred_v.float().unsqueeze(2)], dim=2)
    pos = torch.arange(cap).view(1, 1, cap)
    sl = seg_len.view(S, -1, 1) if seg_len.dim() == 2 else seg_len.view(S, 1, 1)
    rl = ring_len.view(S, 1, 1)
    valid = torch.cat([(pos < sl).expand(S, H, cap),
                       (torch.arange(rcap).view(1, 1, rcap) < rl).expand(S, H, rcap),
                       torch.ones(S, H, 2, dtype=torch.bool)], dim=2)
    mask = valid.unsqueeze(2).repeat(1, 1, 2, 1)
    mask[:, :, 0, -1] = False          # slot 0 does not see the current predict key
    return torch.nn.functional.scaled_dot_product_attention(
        q.float().permute(0, 2, 1, 3), keys, vals, attn_mask=mask,
        scale=1.0 / math.sqrt(D)).permute(0, 2, 1, 3).contiguous()


# ---------------------------------------------------------------------------
# decode KV-cache update (integer + copies, bit-exact)
# ---------------------------------------------------------------------------

def kv_update(nw_k, nw_v, nw_len, nw_pos, br_k, br_v, br_len,
              k_window, v_window, k_retained, v_retained, active, window_tokens: int) -> None:
    """In-place ring insert + retained append.

    Follows src/modeling/models/utils/decode_attention_fast.py:34-105 (window:
    insert at ``pos`` when full else at ``len``, then ``len += 1`` or
    ``pos = (pos + 1) % window``; retained: store at ``len[b,h]`` when in bounds
    and increment) and :108-136 (window disabled), which equal the eager
    src/modeling/models/reverse_sps/inference.py:137-167 and :240-268.
    """
    B, H, _ = k_retained.shape
    for b in range(B):
        if not bool(active[b]):
            continue
        if window_tokens > 0:
            ln, ps = int(nw_len[b]), int(nw_pos[b])
            full = ln >= window_tokens
            ins = ps if full else ln
            nw_k[b, :, ins] = k_window[b].to(nw_k.dtype)
            nw_v[b, :, ins] = v_window[b].to(nw_v.dtype)
            if full:
                nw_pos[b] = (ps + 1) % window_tokens
            else:
                nw_len[b] = ln + 1
        for h in range(H):
            ln = int(br_len[b, h])
            if ln < br_k.shape[2]:
                br_k[b, h, ln] = k_retained[b, h].to(br_k.dtype)
                br_v[b, h, ln] = v_retained[b, h].to(br_v.dtype)
                br_len[b, h] = ln + 1


def fill_decode_caches(k, v, doc_mask, br_k, br_v, br_len, nw_k, nw_v, nw_len, nw_pos,
                       window_tokens: int, retained_slot: int, window_slot: int) -> None:
    """In-place prefill -> decode hand-over of one layer.

    Follows src/modeling/models/reverse_sps/inference.py:568-613: per batch row, the positions
    selected by ``doc_mask`` are compacted; retained-slot rows fill the retained cache and set its
    lengths; window-slot rows of the last ``window_tokens`` positions fill the ring, ``pos = 0``.
    k, v: [B, 2T, H, D].
    """
    B = k.shape[0]
    for b in range(B):
        pos = torch.nonzero(doc_mask[b].bool()).flatten()
        n = int(pos.numel())
        if n == 0:
            continue
        br_k[b, :, :n] = k[b, 2 * pos + retained_slot].transpose(0, 1).to(br_k.dtype)
        br_v[b, :, :n] = v[b, 2 * pos + retained_slot].transpose(0, 1).to(br_v.dtype)
        br_len[b, :] = n
        if window_tokens > 0:
            wp = pos[-window_tokens:]
            wl = int(wp.numel())
            nw_k[b, :, :wl] = k[b, 2 * wp + window_slot].transpose(0, 1).to(nw_k.dtype)
            nw_v[b, :, :wl] = v[b, 2 * wp + window_slot].transpose(0, 1).to(nw_v.dtype)
            nw_len[b] = wl
            nw_pos[b] = 0


def rope_cast(x: torch.Tensor, freqs_cis: Optional[torch.Tensor], out_dtype=torch.bfloat16) -> torch.Tensor:
    """Rotary embedding of a [B, N, H, D] projection followed by the operand cast.

    Follows src/modeling/models/model.py:201-230 (pairs viewed as complex, multiplied by
    ``freqs_cis`` broadcast over heads, viewed back as real, ``type_as`` the input) and the bf16
    cast of src/modeling/models/sps/core.py:53-55.  ``freqs_cis``: complex64 [N, D/2] or
    [B, N, D/2]; None = cast only.
    """
    if freqs_cis is None:
        return x.to(out_dtype)
    x_ = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    f = freqs_cis.unsqueeze(2) if freqs_cis.dim() == 3 else freqs_cis.view(1, x.shape[1], 1, -1)
    out = torch.view_as_real(x_ * f).flatten(3)
    return out.type_as(x).to(out_dtype)
