"""Segmented decode attention and the decode KV-cache update on sm_100a, behind the
reference's call signatures (src/modeling/models/utils/decode_attention.py and
decode_attention_fast.py).  All compute happens in libspsattn.so; there is no fallback.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
from torch import Tensor

from . import _lib
from .attention import _dtype_code, _forward_only, _status


@dataclass
class KVSegment:
    """A block of keys/values with per-element validity lengths
    (same fields as decode_attention.py:21-32).

    k, v: [B, H, max_T, D]; lengths: [B, H] (per head) or [B]; max_len_cap: optional host cap
    on the rows scanned.
    """
    k: Tensor
    v: Tensor
    lengths: Tensor
    max_len_cap: Optional[int] = None


@dataclass
class PackedKVSegment:
    """A cache that is not a dense [B, H, max_T, D] block: row r of (sequence s, head h) is at
    element offset ``seq_offset[s] + h * head_stride + r * row_stride`` of ``k`` / ``v``.
    ``lengths`` is [S] or [S, H] int64; ``max_rows`` caps the rows scanned (host int).
    """
    k: Tensor
    v: Tensor
    seq_offset: Tensor
    head_stride: int
    row_stride: int
    lengths: Tensor
    max_rows: int


def _segment_scan_len(seg: KVSegment) -> int:
    # decode_attention.py:381-390
    max_t = int(seg.k.size(2))
    if max_t == 0:
        return 0
    if seg.max_len_cap is None:
        return max_t
    cap = int(seg.max_len_cap)
    if cap < 0:
        raise ValueError(f"KVSegment.max_len_cap must be non-negative, got {cap}")
    return max(1, min(max_t, cap))


_step_ws: dict = {}


def _step_workspace(device, stream_handle: int, nbytes: int) -> Tensor:
    """Zeroed workspace of the single-launch decode, one per (device, stream): the kernel leaves its
    completion tickets at zero, and calls on one stream are ordered, so the buffer is cleared only
    when it is (re)allocated.  A buffer of another size starts over: the tickets sit at its end."""
    if torch.cuda.is_current_stream_capturing():
        # memory of a graph's private pool must not outlive the capture in this cache
        return torch.zeros(nbytes, dtype=torch.uint8, device=device)
    key = (device.index, stream_handle)
    ws = _step_ws.get(key)
    if ws is None or ws.numel() != nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _step_ws[key] = ws
    return ws


def _lengths_i64(lengths: Tensor, device) -> Tensor:
    if lengths.device != device:
        raise RuntimeError("Segment lengths must live on the same device as query")
    if lengths.dtype != torch.int64:
        lengths = lengths.to(torch.int64)
    return lengths.contiguous()


def decode_attention(
    q: Tensor,                                   # [S, nq, H, D]
    segments: Sequence,                          # KVSegment | PackedKVSegment, with query masks
    extras: Sequence[tuple],                     # (k [S,H,D], v [S,H,D], query_mask)
    *,
    segment_query_masks: Optional[Sequence[int]] = None,
    sm_scale: Optional[float] = None,
) -> Tensor:
    """nq (1 or 2) queries per (sequence, head) over the live rows of every segment plus the
    extra single-token entries; returns fp32 [S, nq, H, D].  Bit i of a query mask says whether
    query slot i sees that segment / entry."""
    lib = _lib.load()
    if not q.is_cuda:
        raise RuntimeError("CUDA tensors are required for segmented decode attention")
    # decode is the generation path: no backward kernels behind it
    _forward_only(q, *[t for seg in segments for t in (seg.k, seg.v)], *[t for e in extras for t in e[:2]])
    S, nq, H, D = q.shape
    q = q.contiguous()
    dt = _dtype_code(q)
    dev = q.device
    n_seg = len(segments)
    keep = [q]
    seg_arr = (_lib.Segment * max(1, n_seg))()
    for i, seg in enumerate(segments):
        qm = 0xFF if segment_query_masks is None else int(segment_query_masks[i])
        lengths = _lengths_i64(seg.lengths, dev)
        keep.append(lengths)
        st = seg_arr[i]
        if isinstance(seg, PackedKVSegment):
            off = seg.seq_offset.to(torch.int64).contiguous()
            keep.append(off)
            st.k, st.v = seg.k.data_ptr(), seg.v.data_ptr()
            st.seq_offset, st.seq_stride = off.data_ptr(), 0
            st.head_stride, st.row_stride = int(seg.head_stride), int(seg.row_stride)
            st.max_rows = int(seg.max_rows)
            kd = seg.k.dtype
        else:
            if seg.k.dim() != 4 or seg.v.dim() != 4:
                raise RuntimeError("Segment K/V tensors must be rank-4 [B,H,T,D]")
            if seg.k.shape != seg.v.shape:
                raise RuntimeError(f"Segment K/V shapes differ: {tuple(seg.k.shape)} vs {tuple(seg.v.shape)}")
            if seg.k.size(0) != S or seg.k.size(1) != H or seg.k.size(3) != D:
                raise RuntimeError("Segment K/V tensors must match query batch/head/head_dim, got "
                                   f"{tuple(seg.k.shape)} for query {(S, H, D)}")
            if (not seg.k.is_cuda) or (not seg.v.is_cuda):
                raise RuntimeError("Segment K/V tensors must be CUDA tensors")
            if (not seg.k.is_contiguous()) or (not seg.v.is_contiguous()):
                raise RuntimeError("Segment K/V tensors must be contiguous")
            max_t = int(seg.k.size(2))
            st.k, st.v = seg.k.data_ptr(), seg.v.data_ptr()
            st.seq_offset, st.seq_stride = None, H * max_t * D
            st.head_stride, st.row_stride = max_t * D, D
            st.max_rows = _segment_scan_len(seg)
            kd = seg.k.dtype
        if st.max_rows > 0 and kd != q.dtype:
            raise RuntimeError(f"Segment dtype {kd} differs from the attention dtype {q.dtype}")
        st.lengths = lengths.data_ptr()
        st.lengths_per_head = int(lengths.dim() == 2)
        st.query_mask = qm
    ex_arr = (_lib.Extra * max(1, len(extras)))()
    for i, (ek, ev, qm) in enumerate(extras):
        if (not ek.is_cuda) or (not ev.is_cuda):
            raise RuntimeError("Current-token K/V tensors must be CUDA tensors")
        if tuple(ek.shape) != (S, H, D) or tuple(ev.shape) != (S, H, D):
            raise RuntimeError(f"Current-token K/V tensors must have shape {(S, H, D)}, got {tuple(ek.shape)}")
        ek, ev = ek.to(q.dtype).contiguous(), ev.to(q.dtype).contiguous()
        keep += [ek, ev]
        ex_arr[i].k, ex_arr[i].v, ex_arr[i].query_mask = ek.data_ptr(), ev.data_ptr(), int(qm)
    out = torch.empty((S, nq, H, D), device=dev, dtype=torch.float32)
    ws_bytes = lib.spsattn_decode_step_workspace_bytes(S, H, D, nq, seg_arr, n_seg)
    scale = 1.0 / math.sqrt(D) if sm_scale is None else float(sm_scale)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream()
        ws = _step_workspace(dev, stream.cuda_stream, ws_bytes)
        rc = lib.spsattn_decode_step(q.data_ptr(), nq, out.data_ptr(), _lib.DTYPE_FP32, seg_arr, n_seg, ex_arr,
                                     len(extras), None, S, H, D, dt, scale, ws.data_ptr(), ws_bytes,
                                     _status(dev).data_ptr(), stream.cuda_stream)
    _lib.check(rc, "spsattn_decode_step")
    return out


def segmented_q2_attention(
    q_Bx2xHxD: Tensor,
    segments: list,
    *,
    current_normal_k_BxHxD: Tensor,
    current_normal_v_BxHxD: Tensor,
    current_predict_k_BxHxD: Tensor,
    current_predict_v_BxHxD: Tensor,
    attn_dtype: torch.dtype,
) -> Tensor:
    """q=2 segmented decode attention for SPS-family generation (decode_attention.py:483-594).

    Slot 0 attends over the segments plus the current normal key; slot 1 over the same
    segments plus current normal and current predict.  Fail-fast like the reference.
    """
    if not q_Bx2xHxD.is_cuda:
        raise RuntimeError("CUDA tensors are required for SPS-family cached generation attention")
    if len(segments) > 2:
        raise RuntimeError(f"SPS-family q2 attention supports at most 2 segments, got {len(segments)}")
    if q_Bx2xHxD.dim() != 4 or q_Bx2xHxD.shape[1] != 2:
        raise RuntimeError(f"Expected q_Bx2xHxD slot dimension to be 2, got {tuple(q_Bx2xHxD.shape)}")
    head_dim = q_Bx2xHxD.shape[3]
    if head_dim <= 0 or head_dim > 256:
        raise RuntimeError(f"Unsupported SPS-family q2 attention head_dim={head_dim}")
    q = q_Bx2xHxD.to(attn_dtype)
    extras = [(current_normal_k_BxHxD, current_normal_v_BxHxD, 0b11),
              (current_predict_k_BxHxD, current_predict_v_BxHxD, 0b10)]
    return decode_attention(q, segments, extras)


# the name the reference binds (src/modeling/models/reverse_sps/inference.py:354)
triton_segmented_q2_attention = segmented_q2_attention


def segmented_q1_attention(q_BxHxD: Tensor, segments: list, *, extra_kv=None,
                           attn_dtype: torch.dtype) -> Tensor:
    """q=1 variant: up to 3 segments and 2 always-valid extra entries (decode_attention.py:393-480)."""
    if len(segments) > 3:
        raise RuntimeError(f"q1 attention supports at most 3 segments, got {len(segments)}")
    extras = [(ek, ev, 1) for ek, ev in (extra_kv or [])]
    if len(extras) > 2:
        raise RuntimeError(f"q1 attention supports at most 2 extra entries, got {len(extras)}")
    q = q_BxHxD.to(attn_dtype).unsqueeze(1)
    return decode_attention(q, segments, extras)[:, 0]


def masked_kv_attention(q_BxHxD: Tensor, segments: list, *, extra_kv=None, attn_dtype: torch.dtype,
                        check_finite: bool = False, error_context: str = "",
                        prefer_triton: bool = False, require_triton: bool = False) -> Tensor:
    """Attention of one query per (batch, head) over variable-length KV segments
    (decode_attention.py:597-704).  Always runs the CUDA kernel; ``prefer_triton`` /
    ``require_triton`` are accepted for signature compatibility."""
    del prefer_triton, require_triton
    out = segmented_q1_attention(q_BxHxD, segments, extra_kv=extra_kv, attn_dtype=attn_dtype)
    if check_finite and not torch.isfinite(out).all():
        raise RuntimeError(f"Non-finite attention output{error_context}")
    return out


def fused_sps_kv_update(*, nw_k: Tensor, nw_v: Tensor, nw_len: Tensor, nw_pos: Tensor,
                        br_k: Tensor, br_v: Tensor, br_len: Tensor,
                        k_window_BxHxD: Tensor, v_window_BxHxD: Tensor,
                        k_retained_BxHxD: Tensor, v_retained_BxHxD: Tensor,
                        active_mask_B: Tensor, window_tokens: int) -> None:
    """Single-launch in-place KV update for SPS-family decode (decode_attention_fast.py:139-221)."""
    lib = _lib.load()
    B, H, D = k_retained_BxHxD.shape
    assert br_k.shape == br_v.shape and br_k.is_cuda and br_k.is_contiguous() and br_v.is_contiguous()
    assert br_len.shape == (B, H) and br_len.dtype == torch.int64 and br_len.is_contiguous()
    active = active_mask_B if active_mask_B.dtype == torch.int8 else active_mask_B.to(torch.int8)
    active = active.contiguous()
    kr = k_retained_BxHxD.to(br_k.dtype).contiguous()
    vr = v_retained_BxHxD.to(br_v.dtype).contiguous()
    args_w = [None, None, None, None]
    kw = vw = None
    window_storage = 0
    if window_tokens > 0:
        assert nw_k.shape == nw_v.shape, "nw.k/v shape mismatch"
        assert nw_k.size(0) == B and nw_k.size(1) == H and nw_k.is_contiguous() and nw_v.is_contiguous()
        assert nw_len.shape == (B,) and nw_pos.shape == (B,)
        assert nw_len.dtype == torch.int64 and nw_pos.dtype == torch.int64
        window_storage = int(nw_k.size(2))
        kw = k_window_BxHxD.to(nw_k.dtype).contiguous()
        vw = v_window_BxHxD.to(nw_v.dtype).contiguous()
        args_w = [nw_k.data_ptr(), nw_v.data_ptr(), nw_len.data_ptr(), nw_pos.data_ptr()]
    with torch.cuda.device(br_k.device):
        rc = lib.spsattn_kv_update(
            args_w[0], args_w[1], args_w[2], args_w[3], br_k.data_ptr(), br_v.data_ptr(), br_len.data_ptr(),
            None if kw is None else kw.data_ptr(), None if vw is None else vw.data_ptr(),
            kr.data_ptr(), vr.data_ptr(), active.data_ptr(), B, H, D, window_storage,
            int(br_k.size(2)), int(window_tokens), br_k.element_size(),
            torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "spsattn_kv_update")


def fill_decode_caches(k_Bx2TxHxD: Tensor, v_Bx2TxHxD: Tensor, current_doc_mask_BxT: Tensor, *,
                       br_k: Tensor, br_v: Tensor, br_len: Tensor,
                       nw_k: Optional[Tensor] = None, nw_v: Optional[Tensor] = None,
                       nw_len: Optional[Tensor] = None, nw_pos: Optional[Tensor] = None,
                       window_tokens: int = 0, retained_slot: int = 0, window_slot: int = 1) -> None:
    """Fill one layer's decode caches from the prefill K/V in one launch, no host sync
    (what reverse_sps/inference.py:568-613 does with a Python loop over batch rows).

    ``retained_slot`` / ``window_slot``: parity of the doubled-sequence row that feeds the retained
    cache / the ring (SPS: 0 and 1; Reverse-SPS and Delayed-State: 1 and 0).
    """
    lib = _lib.load()
    B, two_t, H, D = k_Bx2TxHxD.shape
    T = two_t // 2
    k = k_Bx2TxHxD.to(br_k.dtype)
    v = v_Bx2TxHxD.to(br_v.dtype)
    if k.stride(3) != 1 or any(s % 8 for s in k.stride()[:3]):
        k = k.contiguous()
    if v.stride() != k.stride():
        v = v.contiguous()
        k = k.contiguous()
    assert br_k.element_size() == 2, "caches hold 16-bit elements"
    assert br_k.is_contiguous() and br_v.is_contiguous() and br_len.is_contiguous()
    assert br_len.dtype == torch.int64 and tuple(br_len.shape) == (B, H)
    mask = current_doc_mask_BxT.to(torch.uint8).contiguous()
    assert tuple(mask.shape) == (B, T)
    ring = [None, None, None, None]
    window_storage = 0
    if window_tokens > 0:
        assert nw_k.is_contiguous() and nw_v.is_contiguous()
        assert nw_len.dtype == torch.int64 and nw_pos.dtype == torch.int64
        window_storage = int(nw_k.size(2))
        ring = [nw_k.data_ptr(), nw_v.data_ptr(), nw_len.data_ptr(), nw_pos.data_ptr()]
    with torch.cuda.device(k.device):
        rc = lib.spsattn_fill_decode_caches(
            k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.stride(2), mask.data_ptr(),
            br_k.data_ptr(), br_v.data_ptr(), br_len.data_ptr(), ring[0], ring[1], ring[2], ring[3],
            B, T, H, D, int(br_k.size(2)), window_storage, int(window_tokens), int(retained_slot),
            int(window_slot), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "spsattn_fill_decode_caches")
