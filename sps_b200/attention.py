"""Prefill attention of the SPS model family on sm_100a, behind the reference's call signatures.

``sps_sliding_attention``, ``reverse_sps_sliding_attention`` and ``full_attention`` take the
same arguments, in the same order and with the same meaning, as the reference's
src/modeling/models/attention/triton_sps_flash_attention.py:725-753,
triton_reverse_sps_flash_attention.py:827-853 and triton_full_flash_attention.py:679-709, so the
model classes can call them unchanged (see ``sps_b200.install``).  For head_dim 64 and 128 they
are differentiable like the reference's ``torch.autograd.Function``s (backward:
triton_sps_flash_attention.py:623-720); the other head dims are forward only.
All compute happens in libspsattn.so (tcgen05 / TMA kernels for head_dim 64 and 128).
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

_SUPPORTED_HEAD_DIMS = (16, 32, 64, 128, 256)   # triton_sps_flash_attention.py:510
_status_words: dict = {}


def _status(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait expires."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[key]


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel reported a failure (a bounded wait that expired)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status(dev)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise _lib.SpsAttnError(f"device reported status {code} (a bounded wait expired)")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    if t.dtype == torch.float16:
        return _lib.DTYPE_FP16
    raise TypeError(f"sps_b200 attention computes in bf16 or fp16, got {t.dtype}")


def _addressable(t: torch.Tensor) -> bool:
    """Rows of D contiguous elements, 16-byte aligned, batch/head/token strides multiples of 8."""
    D = t.shape[-1]
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and
            all(s % 8 == 0 and s >= D for s in t.stride()[:3]))


_BACKWARD_HEAD_DIMS = (64, 128)


def _needs_grad(*tensors) -> bool:
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


def _forward_only(*tensors) -> None:
    if _needs_grad(*tensors):
        raise RuntimeError(
            "this sps_b200 call is forward only: call it under torch.no_grad() / inference_mode(), "
            "or detach the inputs (backward kernels exist for prefill attention with head_dim 64 "
            "and 128 only)")


def _docs_args(documents_idx, B, N, device):
    """(tensor kept alive, pointer, is_int64, batch stride, token stride) of a document-id tensor."""
    if documents_idx is None:
        return None, None, 0, 0, 0
    docs = documents_idx
    assert docs.shape[0] == B and docs.shape[1] == N
    assert docs.is_cuda and docs.device == device
    if docs.dtype not in (torch.int64, torch.int32):
        docs = docs.to(torch.int64)
    sb, st = docs.stride()
    return docs, docs.data_ptr(), int(docs.dtype == torch.int64), sb, st


def prefill_attention_backward(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
    d_o: torch.Tensor, sm_scale: float, *, persistent_parity: int, temporary_window: int = 0,
    persistent_window: Optional[int] = None, documents_idx: Optional[torch.Tensor] = None,
    mask_flags: int = 0,
):
    """dQ, dK, dV of ``prefill_attention`` from dO, the forward output ``o`` and its ``lse``
    (the reference's backward: triton_sps_flash_attention.py:623-720).  head_dim 64 or 128."""
    lib = _lib.load()
    B, H, N, D = q.shape
    if D not in _BACKWARD_HEAD_DIMS:
        raise RuntimeError(f"the backward kernels cover head_dim {_BACKWARD_HEAD_DIMS}, got {D}")
    dt = _dtype_code(q)
    # operands are read where they lie when their rows are addressable (the token-major views of
    # the reference's modules and the gradient autograd hands back for them); the reference copies
    # all five (triton_sps_flash_attention.py:629-633)
    q, k, v, o, d_o = (x if _addressable(x) else x.contiguous() for x in (q, k, v, o, d_o.to(q.dtype)))
    lse = lse.contiguous()
    assert lse.shape == (B, H, N) and lse.dtype == torch.float32
    docs, docs_ptr, docs_i64, sb, st = _docs_args(documents_idx, B, N, q.device)

    def grad_like(x):           # a token-major operand gets a token-major gradient
        if x.stride(2) > x.stride(1):
            return torch.empty((B, N, H, D), dtype=x.dtype, device=x.device).transpose(1, 2)
        return torch.empty((B, H, N, D), dtype=x.dtype, device=x.device)

    dq, dk, dv = grad_like(q), grad_like(k), grad_like(v)
    strides = (C.c_int64 * 24)(*[s_ for t in (q, k, v, o, d_o, dq, dk, dv) for s_ in t.stride()[:3]])
    ws_bytes = lib.spsattn_prefill_bwd_workspace_bytes(B, H, N, D)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    pw = _lib.NO_WINDOW if persistent_window is None else max(-1, min(int(persistent_window), N))
    with torch.cuda.device(q.device):
        rc = lib.spsattn_prefill_bwd_strided(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), strides, docs_ptr, docs_i64, sb, st, B, H, N, D, dt,
            float(sm_scale), int(persistent_parity), max(-1, min(int(temporary_window), N)), pw,
            int(mask_flags), ws.data_ptr(), ws_bytes, _status(q.device).data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "spsattn_prefill_bwd")
    del docs
    return dq, dk, dv


class _PrefillAttention(torch.autograd.Function):
    """Differentiable prefill attention: forward and backward both run in libspsattn.so."""

    @staticmethod
    def forward(ctx, q, k, v, sm_scale, persistent_parity, temporary_window, persistent_window,
                documents_idx, mask_flags):
        o, lse = _prefill_forward(q, k, v, sm_scale, persistent_parity=persistent_parity,
                                  temporary_window=temporary_window, persistent_window=persistent_window,
                                  documents_idx=documents_idx, mask_flags=mask_flags, return_lse=True)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.docs = documents_idx
        ctx.args = (float(sm_scale), int(persistent_parity), int(temporary_window), persistent_window,
                    int(mask_flags))
        return o

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        sm_scale, parity, tw, pw, flags = ctx.args
        dq, dk, dv = prefill_attention_backward(
            q, k, v, o, lse, d_o, sm_scale, persistent_parity=parity, temporary_window=tw,
            persistent_window=pw, documents_idx=ctx.docs, mask_flags=flags)
        return dq, dk, dv, None, None, None, None, None, None


def prefill_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: float,
    *,
    persistent_parity: int,
    temporary_window: int = 0,
    persistent_window: Optional[int] = None,
    documents_idx: Optional[torch.Tensor] = None,
    mask_flags: int = 0,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
):
    """Masked attention over [B, H, N, D] tensors; the general entry the three wrappers share.

    ``persistent_parity``: 0 (SPS), 1 (Reverse-SPS / Delayed-State) or -1 (Standard).
    Returns O (same dtype as q) and, with ``return_lse``, the base-2 log-sum-exp [B, H, N] fp32.
    When an input requires grad (head_dim 64 or 128) the result is differentiable.
    """
    if _needs_grad(q, k, v):
        if q.shape[-1] not in _BACKWARD_HEAD_DIMS or return_lse or out is not None:
            _forward_only(q, k, v)
        return _PrefillAttention.apply(q, k, v, sm_scale, persistent_parity, temporary_window,
                                       persistent_window, documents_idx, mask_flags)
    return _prefill_forward(q, k, v, sm_scale, persistent_parity=persistent_parity,
                            temporary_window=temporary_window, persistent_window=persistent_window,
                            documents_idx=documents_idx, mask_flags=mask_flags, return_lse=return_lse,
                            out=out)


def _prefill_forward(q, k, v, sm_scale, *, persistent_parity, temporary_window=0, persistent_window=None,
                     documents_idx=None, mask_flags=0, return_lse=False, out=None):
    lib = _lib.load()
    if not q.is_cuda:
        raise RuntimeError("sps_b200 attention needs CUDA tensors; there is no CPU path")
    B, H, N, D = q.shape
    assert k.shape == q.shape and v.shape == q.shape, "q, k, v must have the same shape"
    assert k.dtype == q.dtype and v.dtype == q.dtype, "q, k, v must have the same dtype"
    assert D in _SUPPORTED_HEAD_DIMS, f"head_dim must be one of {_SUPPORTED_HEAD_DIMS}"
    if persistent_parity != _lib.PARITY_NONE:
        assert N % 2 == 0, "Expected doubled sequence length (2T)."
    dt = _dtype_code(q)
    # The tensor-core kernel reads any layout whose rows are contiguous (for instance the
    # transposed views of token-major projections the reference's modules pass); only what it
    # cannot address is copied, where the reference copies always
    # (triton_sps_flash_attention.py:504-506).
    strided_ok = D in (64, 128)
    q, k, v = (x if (strided_ok and _addressable(x)) else x.contiguous() for x in (q, k, v))
    docs_ptr, docs_i64, sb, st = None, 0, 0, 0
    if documents_idx is not None:
        docs = documents_idx
        assert docs.shape[0] == B and docs.shape[1] == N
        assert docs.is_cuda and docs.device == q.device
        if docs.dtype not in (torch.int64, torch.int32):
            docs = docs.to(torch.int64)
        docs_ptr, docs_i64 = docs.data_ptr(), int(docs.dtype == torch.int64)
        sb, st = docs.stride()
    if out is not None:
        o = out
    elif strided_ok and q.stride(2) > q.stride(1):
        # token-major input: produce token-major output, so that the caller's
        # y.transpose(1, 2).contiguous() (sps/core.py:79) is free
        o = torch.empty((B, N, H, D), dtype=q.dtype, device=q.device).transpose(1, 2)
    else:
        o = torch.empty((B, H, N, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, N), dtype=torch.float32, device=q.device) if return_lse else None
    ws_bytes = lib.spsattn_prefill_workspace_bytes(B, H, N, D) if documents_idx is not None else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
    pw = _lib.NO_WINDOW if persistent_window is None else max(-1, min(int(persistent_window), N))
    arr = lambda t: (C.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    with torch.cuda.device(q.device):
        rc = lib.spsattn_prefill_fwd_strided(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            None if lse is None else lse.data_ptr(), arr(q), arr(k), arr(v), arr(o),
            docs_ptr, docs_i64, sb, st, B, H, N, D, dt, float(sm_scale), int(persistent_parity),
            max(-1, min(int(temporary_window), N)), pw, int(mask_flags),
            None if ws is None else ws.data_ptr(), ws_bytes,
            _status(q.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "spsattn_prefill_fwd")
    return (o, lse) if return_lse else o


def sps_sliding_attention(q, k, v, sm_scale, temporary_key_window, warp_specialize=True,
                          documents_idx_BxT=None, persistent_key_window=None):
    """SPS variant: the persistent (window-exempt) key is the even / input slot, the <predict>
    slot is windowed.  ``warp_specialize`` is accepted for signature compatibility and ignored.
    """
    del warp_specialize
    return prefill_attention(q, k, v, sm_scale, persistent_parity=_lib.PARITY_EVEN,
                             temporary_window=int(temporary_key_window),
                             persistent_window=persistent_key_window,
                             documents_idx=documents_idx_BxT)


def reverse_sps_sliding_attention(q, k, v, sm_scale, temporary_key_window, warp_specialize=True,
                                  documents_idx_BxT=None, persistent_key_window=None):
    """Reverse-SPS / Delayed-State variant: the persistent key is the odd slot."""
    del warp_specialize
    return prefill_attention(q, k, v, sm_scale, persistent_parity=_lib.PARITY_ODD,
                             temporary_window=int(temporary_key_window),
                             persistent_window=persistent_key_window,
                             documents_idx=documents_idx_BxT)


def full_attention(q, k, v, sm_scale, warp_specialize=True, documents_idx_BxT=None):
    """Standard model: causal attention with an optional same-document mask."""
    del warp_specialize
    return prefill_attention(q, k, v, sm_scale, persistent_parity=_lib.PARITY_NONE,
                             documents_idx=documents_idx_BxT)


def visibility(n_ctx: int, *, persistent_parity: int, temporary_window: int = 0,
               persistent_window: Optional[int] = None, documents_idx: Optional[torch.Tensor] = None,
               mask_flags: int = 0, batch: int = 1, device="cuda") -> torch.Tensor:
    """The boolean mask the kernels apply, evaluated on the device ([B, N, N] bool); test hook."""
    lib = _lib.load()
    dev = torch.device(device)
    B = batch if documents_idx is None else documents_idx.shape[0]
    vis = torch.empty((B, n_ctx, n_ctx), dtype=torch.uint8, device=dev)
    docs_ptr, docs_i64, sb, st, ws, ws_bytes = None, 0, 0, 0, None, 0
    if documents_idx is not None:
        docs = documents_idx.to(dev)
        if docs.dtype not in (torch.int64, torch.int32):
            docs = docs.to(torch.int64)
        docs_ptr, docs_i64 = docs.data_ptr(), int(docs.dtype == torch.int64)
        sb, st = docs.stride()
        ws_bytes = lib.spsattn_prefill_workspace_bytes(B, 1, n_ctx, 64)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    pw = _lib.NO_WINDOW if persistent_window is None else max(-1, min(int(persistent_window), n_ctx))
    with torch.cuda.device(dev):
        rc = lib.spsattn_debug_visibility(
            vis.data_ptr(), docs_ptr, docs_i64, sb, st, B, n_ctx, int(persistent_parity),
            max(-1, min(int(temporary_window), n_ctx)), pw, int(mask_flags),
            None if ws is None else ws.data_ptr(), ws_bytes, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "spsattn_debug_visibility")
    return vis.bool()


_X_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def rope_cast(x_BxNxHxD: torch.Tensor, freqs_cis: Optional[torch.Tensor], *,
              out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Rotary embedding (``freqs_cis`` complex64 [N, D/2] or [B, N, D/2]; None = cast only) and
    cast of one projection in a single pass.  Input: a [B, N, H, D] view (any of bf16 / fp16 /
    fp32, row strides free).  Returns the attention operand as a [B, H, N, D] view of a
    token-major buffer, which the prefill kernel reads in place.  One kernel instead of the
    float / complex / multiply / cast / transpose chain of model.py:201-230 and sps/core.py:45-55.
    """
    lib = _lib.load()
    x = x_BxNxHxD
    if not x.is_cuda:
        raise RuntimeError("rope_cast needs CUDA tensors")
    B, N, H, D = x.shape
    if x.dtype not in _X_DTYPES:
        raise TypeError(f"unsupported projection dtype {x.dtype}")
    align = 4 if x.dtype == torch.float32 else 8
    if x.stride(3) != 1 or any(s % align for s in x.stride()[:3]) or x.data_ptr() % 16:
        x = x.contiguous()
    out = torch.empty((B, N, H, D), dtype=out_dtype, device=x.device)
    f_ptr, f_sb = None, 0
    if freqs_cis is not None:
        f = torch.view_as_real(freqs_cis.to(torch.complex64)).contiguous()    # [.., N, D/2, 2] fp32
        assert f.shape[-3:] == (N, D // 2, 2), f"freqs_cis must be [N, D/2] or [B, N, D/2], got {tuple(freqs_cis.shape)}"
        if f.dim() == 4:
            assert f.shape[0] == B
            f_sb = N * (D // 2)
        f_ptr = f.data_ptr()
    with torch.cuda.device(x.device):
        rc = lib.spsattn_rope_cast(x.data_ptr(), _X_DTYPES[x.dtype], x.stride(0), x.stride(1), x.stride(2),
                                   f_ptr, f_sb, out.data_ptr(), _dtype_code(out), out.stride(0), out.stride(1),
                                   out.stride(2), B, N, H, D, int(freqs_cis is not None),
                                   torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "spsattn_rope_cast")
    return out.transpose(1, 2)
