"""Greedy generation for the SPS model family (SPS, Reverse-SPS, Delayed-State) and the Standard
model with the attention path of this library.

``SPSGenerator`` runs the reference's decoder (RMSNorm, fused q/k/v projection, rotary embedding,
SPS attention, output projection, SwiGLU MLP, tied head) from a state dict with the reference's
parameter names: a batched prompt prefill that also fills the decode caches, then one fixed chain
of launches per generated token, captured once in a CUDA graph and replayed — no host
synchronisation, allocation or Python between tokens.  Reference behaviour being reproduced:

  * prefill    src/modeling/models/reverse_sps/inference.py:615-701 (_prefill_generation_state_batched)
  * one step   src/modeling/models/reverse_sps/inference.py:364-485 (_decode_one_token_step) and
               :487-503 (_advance_decode_state)
  * the loop   src/modeling/models/utils/generation.py:121-197 (generate_with_batched_prefill) with
               greedy sampling, <predict> and pad suppressed (utils/sampling.py:55-83,
               reverse_sps/inference.py:893-902)
  * the model  src/modeling/models/model.py:101-132, :201-230, :304-327; sps/core.py:35-82, :100-131
  * Standard   src/modeling/models/full_attention_model.py:506-740 (one row per token, the cache holds
               the current document, one query per step)

What runs where: the projections and the head are library GEMMs (``torch.mm``); everything else
on the per-token chain is a kernel of libspsattn.so — residual add + RMSNorm, rotary + cast of
the fused projection into the attention operands, the segmented decode attention with the cache
update folded into its merge pass, the SwiGLU gate — plus a handful of small integer torch ops per
token (not per layer) for the token/position bookkeeping.  Parameters are bf16 (as the reference
generates on CUDA) or fp32; the attention operands and caches are bf16 either way.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch
from torch import Tensor

from . import _lib
from .attention import _status, check_device_status, prefill_attention

_VARIANTS = {
    # name: (prediction slot, ring ("window") slot, retained slot, persistent-key parity)
    "sps": (1, 1, 0, _lib.PARITY_EVEN),            # sps/inference.py:8-12
    "reverse_sps": (0, 0, 1, _lib.PARITY_ODD),     # reverse_sps/inference.py:58-62
    "delayed_state": (1, 0, 1, _lib.PARITY_ODD),   # delayed_state/inference.py:8-10: Reverse-SPS caches and
                                                   # attention, logits read at the odd slot
    # Standard model (full_attention_model.py): one row per token, no <predict> slot and no ring;
    # the cache holds the current document (:506-585), causal attention inside a document
    "standard": (0, None, 0, _lib.PARITY_NONE),
}


@dataclass
class SPSDims:
    """The architecture fields of the reference's SPSConfig (reverse_sps/core.py:128-135,
    model.py:330-343)."""
    block_size: int
    vocab_size: int
    n_layer: int
    n_head: int
    hidden_size: int
    intermediate_size: int
    norm_eps: float = 1e-6
    eos_token_id: int = 50256
    pad_token_id: int = 50303
    predict_token_id: int = 50257
    window_size: int = 64

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.n_head


def random_state_dict(dims: SPSDims, *, seed: int = 0, device="cuda",
                      dtype: torch.dtype = torch.bfloat16) -> Dict[str, Tensor]:
    """Random parameters with the reference's names and initialisation (N(0, 0.02); output
    projections N(0, 0.02 / sqrt(2 n_layer)); norms 1; tied head) — reverse_sps/core.py:203-209,
    sps/core.py:127-129."""
    g = torch.Generator(device=device).manual_seed(seed)
    c, i = dims.hidden_size, dims.intermediate_size

    def normal(*shape, std=0.02):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)

    sd = {"transformer.wte.weight": normal(dims.vocab_size, c)}
    sd["lm_head.weight"] = sd["transformer.wte.weight"]
    for layer in range(dims.n_layer):
        pre = f"transformer.h.{layer}."
        sd[pre + "attention_norm.weight"] = torch.ones(c, device=device, dtype=dtype)
        sd[pre + "attn.c_attn.weight"] = normal(3 * c, c)
        sd[pre + "attn.c_proj.weight"] = normal(c, c, std=0.02 / math.sqrt(2 * dims.n_layer))
        sd[pre + "mlp_norm.weight"] = torch.ones(c, device=device, dtype=dtype)
        sd[pre + "mlp.gate_proj.weight"] = normal(i, c)
        sd[pre + "mlp.up_proj.weight"] = normal(i, c)
        sd[pre + "mlp.down_proj.weight"] = normal(c, i)
    sd["transformer.output_norm.weight"] = torch.ones(c, device=device, dtype=dtype)
    return sd


def left_padded_document_idx(idx: Tensor, eos: int, pad: int) -> Tensor:
    """Document ids of left-padded prompts (model.py:67-99)."""
    real = idx != pad
    b, t = idx.shape
    pad_count = (~real).sum(dim=1, keepdim=True)
    eos_real = real & (idx == eos)
    doc = torch.zeros((b, t), dtype=torch.long, device=idx.device)
    if t > 1:
        doc[:, 1:] = torch.cumsum(eos_real[:, :-1].long(), dim=1)
    doc = doc + pad_count
    pad_doc = torch.clamp(torch.cumsum((~real).long(), dim=1) - 1, min=0)
    return torch.where(real, doc, pad_doc)


def left_padded_position_ids(idx: Tensor, pad: int) -> Tensor:
    """model.py:60-64."""
    real = idx != pad
    pos = real.long().cumsum(dim=1) - 1
    return torch.where(real, pos, torch.zeros_like(pos))


def _validate_left_padded(idx: Tensor, pad: int, context: str) -> None:
    """model.py:39-57 (pads only on the left, at least one real token per row)."""
    real = idx != pad
    ever_real = real.cumsum(dim=1) > 0
    if bool(((~real) & ever_real).any()):
        raise ValueError(f"{context} must be left padded only")
    if bool((real.sum(dim=1) == 0).any()):
        raise ValueError(f"{context} must contain at least one real token per row")


class _Weights:
    """Parameters on the device in the layout the chain wants (gate and up concatenated)."""

    def __init__(self, sd: Dict[str, Tensor], dims: SPSDims, device, dtype: torch.dtype):
        def get(name):
            return sd[name].detach().to(device=device, dtype=dtype).contiguous()

        self.wte = get("transformer.wte.weight")
        head = sd.get("lm_head.weight", sd["transformer.wte.weight"])
        self.lm_head = self.wte if head is sd["transformer.wte.weight"] or torch.equal(
            head.to(self.wte.device, self.wte.dtype), self.wte) else get("lm_head.weight")
        self.out_norm = get("transformer.output_norm.weight")
        self.attn_norm, self.c_attn, self.c_proj, self.mlp_norm, self.gate_up, self.down = [], [], [], [], [], []
        for layer in range(dims.n_layer):
            pre = f"transformer.h.{layer}."
            self.attn_norm.append(get(pre + "attention_norm.weight"))
            self.c_attn.append(get(pre + "attn.c_attn.weight"))
            self.c_proj.append(get(pre + "attn.c_proj.weight"))
            self.mlp_norm.append(get(pre + "mlp_norm.weight"))
            self.gate_up.append(torch.cat([get(pre + "mlp.gate_proj.weight"),
                                           get(pre + "mlp.up_proj.weight")], dim=0).contiguous())
            self.down.append(get(pre + "mlp.down_proj.weight"))


@dataclass
class DecodeState:
    """The decode caches of all layers (one allocation each) and the per-row counters
    (reverse_sps/inference.py:30-55, :64-111)."""
    nw_k: Tensor           # [L, B, H, window_storage, D] ring of the windowed slot
    nw_v: Tensor
    nw_len: Tensor         # [L, B] int64
    nw_pos: Tensor         # [L, B] int64
    br_k: Tensor           # [L, B, H, max_tokens, D] retained cache of the persistent slot
    br_v: Tensor
    br_len: Tensor         # [L, B, H] int64
    processed_tokens: Tensor   # [B] int64
    next_doc_start: Tensor     # [B] bool
    max_tokens: int
    # host-side upper bound of processed_tokens (longest prompt + eager steps taken): lets
    # decode_one_token refuse a step past the caches or the rotary table without a device sync
    host_tokens: int = 0


class SPSGenerator:
    """Batched prefill + graph-replayed greedy decode for one model on one GPU."""

    def __init__(self, state_dict: Dict[str, Tensor], dims: SPSDims, *, variant: str = "sps",
                 device="cuda", param_dtype: torch.dtype = torch.bfloat16):
        if variant not in _VARIANTS:
            raise ValueError(f"variant must be one of {sorted(_VARIANTS)}")
        if param_dtype not in (torch.bfloat16, torch.float32):
            raise TypeError("parameters are bf16 or fp32")
        if dims.hidden_size % dims.n_head or dims.head_dim not in (16, 32, 64, 128, 256):
            raise ValueError("head_dim must be one of 16, 32, 64, 128, 256")   # sps/core.py:57-67
        self.lib = _lib.load()
        self.dims = dims
        self.variant = variant
        self.pred_slot, self.window_slot, self.retained_slot, self.parity = _VARIANTS[variant]
        self.n_slot = 1 if variant == "standard" else 2          # rows per token
        self.window_tokens = 0 if variant == "standard" else int(dims.window_size)
        self.device = torch.device(device)
        self.param_dtype = param_dtype
        self.attn_dtype = torch.bfloat16                       # reverse_sps/inference.py:637
        self.glue_dtype = _lib.DTYPE_BF16 if param_dtype == torch.bfloat16 else _lib.DTYPE_FP32
        self.x_dtype_code = 0 if param_dtype == torch.bfloat16 else 2
        self.w = _Weights(state_dict, dims, self.device, param_dtype)
        hd = dims.head_dim
        # model.py:134-160, kept as (cos, sin) pairs: [block_size, hd/2, 2] fp32
        freqs = 1.0 / (10000.0 ** (torch.arange(0, hd, 2)[: hd // 2].float() / hd))
        ang = torch.outer(torch.arange(dims.block_size).float(), freqs)
        self.freqs = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(self.device).contiguous()
        self._step = None
        self._session = None

    # ------------------------------------------------------------------ library calls
    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def _add_rmsnorm(self, x: Tensor, delta: Optional[Tensor], weight: Tensor, y: Optional[Tensor]) -> None:
        rows, c = x.shape
        rc = self.lib.spsattn_add_rmsnorm(x.data_ptr(), None if delta is None else delta.data_ptr(),
                                          weight.data_ptr(), None if y is None else y.data_ptr(),
                                          self.glue_dtype, rows, c, float(self.dims.norm_eps), self._stream())
        _lib.check(rc, "spsattn_add_rmsnorm")

    def _swiglu(self, gate_up: Tensor, y: Tensor) -> None:
        rows = gate_up.shape[0]
        rc = self.lib.spsattn_swiglu(gate_up.data_ptr(), y.data_ptr(), self.glue_dtype, rows,
                                     self.dims.intermediate_size, self._stream())
        _lib.check(rc, "spsattn_swiglu")

    def _mlp(self, layer: int, xn: Tensor, gate_up: Tensor, hidden: Tensor, delta: Tensor) -> None:
        torch.mm(xn, self.w.gate_up[layer].t(), out=gate_up)
        self._swiglu(gate_up, hidden)
        torch.mm(hidden, self.w.down[layer].t(), out=delta)

    # ------------------------------------------------------------------ prefill
    def _prefill_chain(self, idx: Tensor, positions: Tensor, docs2: Tensor,
                       state: Optional[DecodeState], doc_mask: Optional[Tensor]) -> Tensor:
        """Final-norm hidden states [B, 2T, C] of the doubled prompt; fills ``state`` on the way."""
        d = self.dims
        b, t = idx.shape
        ns = self.n_slot
        n, c, h, hd, inter = ns * t, d.hidden_size, d.n_head, d.head_dim, d.intermediate_size
        rows = b * n
        dev, pdt = self.device, self.param_dtype
        idx2 = idx.repeat_interleave(ns, dim=1)
        if ns == 2:
            idx2[:, 1::2] = d.predict_token_id                              # reverse_sps/core.py:261-264
        x = self.w.wte.index_select(0, idx2.reshape(-1))                    # [rows, C] residual stream
        fc = self.freqs[positions.repeat_interleave(ns, dim=1)].contiguous()  # [B, N, hd/2, 2]
        xn = torch.empty_like(x)
        delta = torch.empty_like(x)
        qkv = torch.empty((rows, 3 * c), device=dev, dtype=pdt)
        ops = torch.empty((3, b, n, h, hd), device=dev, dtype=self.attn_dtype)   # q, k, v token-major
        y = torch.empty((b, n, h, hd), device=dev, dtype=self.attn_dtype)
        gate_up = torch.empty((rows, 2 * inter), device=dev, dtype=pdt)
        hidden = torch.empty((rows, inter), device=dev, dtype=pdt)
        groups = (_lib.RopeGroup * 3)()
        for gi in range(3):
            groups[gi].out = ops[gi].data_ptr()
            groups[gi].stride_b, groups[gi].stride_n, groups[gi].stride_h = n * c, c, hd
            groups[gi].rotate = int(gi < 2)
        scale = 1.0 / math.sqrt(hd)
        self._add_rmsnorm(x, None, self.w.attn_norm[0], xn)
        for layer in range(d.n_layer):
            torch.mm(xn, self.w.c_attn[layer].t(), out=qkv)
            rc = self.lib.spsattn_qkv_rope_cast(qkv.data_ptr(), self.x_dtype_code, n * 3 * c, 3 * c, hd,
                                                fc.data_ptr(), n * (hd // 2), groups, 3, _lib.DTYPE_BF16,
                                                b, n, h, hd, self._stream())
            _lib.check(rc, "spsattn_qkv_rope_cast")
            if state is not None:
                self._fill_caches(state, layer, ops[1], ops[2], doc_mask)
            in_place = hd in (64, 128)     # the tensor-core kernel reads and writes token-major rows
            o = prefill_attention(ops[0].transpose(1, 2), ops[1].transpose(1, 2), ops[2].transpose(1, 2),
                                  scale, persistent_parity=self.parity, temporary_window=self.window_tokens,
                                  documents_idx=docs2, out=y.transpose(1, 2) if in_place else None)
            if not in_place:
                y.copy_(o.transpose(1, 2))
            y2 = y.view(rows, c)
            if pdt != self.attn_dtype:
                y2 = y2.to(pdt)                                             # sps/core.py:80
            torch.mm(y2, self.w.c_proj[layer].t(), out=delta)
            self._add_rmsnorm(x, delta, self.w.mlp_norm[layer], xn)
            self._mlp(layer, xn, gate_up, hidden, delta)
            nxt = self.w.attn_norm[layer + 1] if layer + 1 < d.n_layer else self.w.out_norm
            self._add_rmsnorm(x, delta, nxt, xn)
        return xn.view(b, n, c)

    def _fill_caches(self, st: DecodeState, layer: int, k: Tensor, v: Tensor, doc_mask: Tensor) -> None:
        b, n, h, hd = k.shape
        ring = [None] * 4
        if self.window_tokens > 0:
            ring = [st.nw_k[layer].data_ptr(), st.nw_v[layer].data_ptr(), st.nw_len[layer].data_ptr(),
                    st.nw_pos[layer].data_ptr()]
        # the entry point addresses row 2 * token + slot of a doubled sequence; with one row per
        # token (Standard) half the row stride and slot 0 address row `token`
        row_stride = k.stride(1) if self.n_slot == 2 else k.stride(1) // 2
        rc = self.lib.spsattn_fill_decode_caches(
            k.data_ptr(), v.data_ptr(), k.stride(0), row_stride, k.stride(2), doc_mask.data_ptr(),
            st.br_k[layer].data_ptr(), st.br_v[layer].data_ptr(), st.br_len[layer].data_ptr(),
            ring[0], ring[1], ring[2], ring[3], b, n // self.n_slot, h, hd, st.max_tokens, int(st.nw_k.shape[3]),
            self.window_tokens, self.retained_slot, self.window_slot or 0, self._stream())
        _lib.check(rc, "spsattn_fill_decode_caches")

    def build_decode_state(self, batch_size: int, max_tokens: int) -> DecodeState:
        """reverse_sps/inference.py:64-111, one allocation per kind instead of one per layer."""
        d = self.dims
        dev, L, h, hd = self.device, d.n_layer, d.n_head, d.head_dim
        storage = max(self.window_tokens, 1)
        z = lambda *s, dt: torch.zeros(s, device=dev, dtype=dt)
        return DecodeState(
            nw_k=z(L, batch_size, h, storage, hd, dt=self.attn_dtype),
            nw_v=z(L, batch_size, h, storage, hd, dt=self.attn_dtype),
            nw_len=z(L, batch_size, dt=torch.int64), nw_pos=z(L, batch_size, dt=torch.int64),
            br_k=z(L, batch_size, h, max_tokens, hd, dt=self.attn_dtype),
            br_v=z(L, batch_size, h, max_tokens, hd, dt=self.attn_dtype),
            br_len=z(L, batch_size, h, dt=torch.int64),
            processed_tokens=z(batch_size, dt=torch.int64),
            next_doc_start=torch.ones(batch_size, device=dev, dtype=torch.bool),
            max_tokens=int(max_tokens))

    @torch.no_grad()
    def forward_logits(self, idx_BxT: Tensor) -> Tensor:
        """Token logits [B, T, V] of the dense forward (sps/core.py:133-147: positions 0..T-1,
        logits read at the prediction slot)."""
        idx = idx_BxT.to(self.device)
        b, t = idx.shape
        if t > self.dims.block_size:
            raise ValueError(f"Cannot forward sequence of length {self.n_slot * t}, block size is only {self.dims.block_size}")
        docs2 = left_padded_document_idx(idx, self.dims.eos_token_id, self.dims.pad_token_id)
        docs2 = docs2.repeat_interleave(self.n_slot, dim=1).contiguous()
        pos = torch.arange(t, device=self.device).unsqueeze(0).expand(b, -1)
        xn = self._prefill_chain(idx, pos, docs2, None, None)
        pred = xn[:, self.pred_slot::self.n_slot].reshape(b * t, -1)
        return torch.mm(pred, self.w.lm_head.t()).view(b, t, -1)

    @torch.no_grad()
    def prefill(self, idx_BxT: Tensor, max_new_tokens: int, state: Optional[DecodeState] = None):
        """Batched prompt prefill (reverse_sps/inference.py:615-701): returns the decode state and
        the logits [B, V] that predict the first new token.  ``state``: caches of an earlier call
        to fill again, used when their batch size and capacity fit."""
        d = self.dims
        idx = idx_BxT.to(self.device)
        b, t = idx.shape
        _validate_left_padded(idx, d.pad_token_id, f"{self.variant} generation prefill prompts")
        real = idx != d.pad_token_id
        real_lengths = real.sum(dim=1).to(torch.long)
        longest = int(real_lengths.max().item())
        # the .item() above has synchronised: a bounded wait that expired in an earlier kernel
        # shows in the status word now, before its empty outputs are used
        check_device_status(self.device)
        total = longest + int(max_new_tokens)
        if total > d.block_size:
            raise ValueError(f"Cannot generate {max_new_tokens} new tokens from a prompt with "
                             f"{total - int(max_new_tokens)} real tokens when block size is {d.block_size}")
        if state is not None and state.processed_tokens.shape[0] == b and state.max_tokens == total:
            for t_ in (state.nw_len, state.nw_pos, state.br_len):
                t_.zero_()
        else:
            state = self.build_decode_state(b, total)
        docs = left_padded_document_idx(idx, d.eos_token_id, d.pad_token_id)
        docs2 = docs.repeat_interleave(self.n_slot, dim=1).contiguous()
        doc_mask = real & (docs == docs[:, -1:])
        if self.variant == "standard":
            # a prompt that ends on EOS starts decoding with an empty cache
            # (full_attention_model.py:703-705)
            doc_mask = doc_mask & (idx[:, -1:] != d.eos_token_id)
        doc_mask = doc_mask.to(torch.uint8).contiguous()
        pos = left_padded_position_ids(idx, d.pad_token_id)
        xn = self._prefill_chain(idx, pos, docs2, state, doc_mask)
        last = xn[:, self.n_slot * (t - 1) + self.pred_slot]                # [B, C]
        next_logits = torch.mm(last, self.w.lm_head.t())
        state.processed_tokens.copy_(real_lengths)
        state.next_doc_start.copy_(idx[:, -1] == d.eos_token_id)
        state.host_tokens = longest
        return state, next_logits

    # ------------------------------------------------------------------ one decode step
    def _bind_step(self, state: DecodeState) -> None:
        """Static buffers and pre-built argument blocks of the per-token chain for ``state``."""
        d = self.dims
        dev, pdt = self.device, self.param_dtype
        b = state.processed_tokens.shape[0]
        c, h, hd, inter, L = d.hidden_size, d.n_head, d.head_dim, d.intermediate_size, d.n_layer
        s = type("StepBuffers", (), {})()
        s.state = state
        s.b = b
        s.token = torch.zeros(b, device=dev, dtype=torch.long)
        s.active = torch.zeros(b, device=dev, dtype=torch.bool)
        s.active_i8 = torch.zeros(b, device=dev, dtype=torch.int8)
        ns, wt = self.n_slot, self.window_tokens
        s.idx_pair = torch.full((b, ns), max(d.predict_token_id, 0), device=dev, dtype=torch.long)
        s.pos = torch.zeros(b, device=dev, dtype=torch.long)
        s.fc = torch.zeros((b, hd // 2, 2), device=dev, dtype=torch.float32)
        s.x = torch.zeros((ns * b, c), device=dev, dtype=pdt)
        s.xn = torch.zeros_like(s.x)
        s.delta = torch.zeros_like(s.x)
        s.qkv = torch.zeros((ns * b, 3 * c), device=dev, dtype=pdt)
        s.q = torch.zeros((b, ns, h, hd), device=dev, dtype=self.attn_dtype)
        s.k2 = torch.zeros((ns, b, h, hd), device=dev, dtype=self.attn_dtype)
        s.v2 = torch.zeros((ns, b, h, hd), device=dev, dtype=self.attn_dtype)
        s.y = torch.zeros((ns * b, c), device=dev, dtype=self.attn_dtype)
        s.y_param = s.y if pdt == self.attn_dtype else torch.zeros((ns * b, c), device=dev, dtype=pdt)
        s.gate_up = torch.zeros((ns * b, 2 * inter), device=dev, dtype=pdt)
        s.hidden = torch.zeros((ns * b, inter), device=dev, dtype=pdt)
        s.logits = torch.zeros((b, d.vocab_size), device=dev, dtype=pdt)
        s.zero_tok = torch.zeros(b, device=dev, dtype=torch.long)
        # the [B, ns, 3C] projection seen as one row per sequence with 3 * ns head groups:
        # slot 0 q, k, v (, slot 1 q, k, v)
        groups = (_lib.RopeGroup * (3 * ns))()
        hs = h * hd
        for slot in range(ns):
            gq, gk, gv = groups[3 * slot], groups[3 * slot + 1], groups[3 * slot + 2]
            gq.out, gq.stride_b, gq.rotate = s.q.data_ptr() + slot * hs * 2, ns * hs, 1
            gk.out, gk.stride_b, gk.rotate = s.k2[slot].data_ptr(), hs, 1
            gv.out, gv.stride_b, gv.rotate = s.v2[slot].data_ptr(), hs, 0
            for g in (gq, gk, gv):
                g.stride_n, g.stride_h = 0, hd
        s.groups = groups
        storage = int(state.nw_k.shape[3])
        s.layer_args = []
        ws_bytes = 0
        for layer in range(L):
            segs = (_lib.Segment * 2)()
            n_seg = 0
            qm_all = (1 << ns) - 1
            if wt > 0:                                                     # reverse_sps/inference.py:333-342
                sg = segs[n_seg]
                sg.k, sg.v = state.nw_k[layer].data_ptr(), state.nw_v[layer].data_ptr()
                sg.seq_offset, sg.seq_stride = None, h * storage * hd
                sg.head_stride, sg.row_stride = storage * hd, hd
                sg.lengths, sg.lengths_per_head = state.nw_len[layer].data_ptr(), 0
                sg.max_rows, sg.query_mask = max(1, min(wt, state.max_tokens)), qm_all
                n_seg += 1
            sg = segs[n_seg]                                               # :343-350
            sg.k, sg.v = state.br_k[layer].data_ptr(), state.br_v[layer].data_ptr()
            sg.seq_offset, sg.seq_stride = None, h * state.max_tokens * hd
            sg.head_stride, sg.row_stride = state.max_tokens * hd, hd
            sg.lengths, sg.lengths_per_head = state.br_len[layer].data_ptr(), 1
            sg.max_rows, sg.query_mask = state.max_tokens, qm_all
            n_seg += 1
            # the row(s) of this step: every slot sees the input row, only the <predict> slot its own
            # (decode_attention.py:354-361); Standard: the one row (full_attention_model.py:549-563)
            extras = (_lib.Extra * 2)()
            extras[0].k, extras[0].v, extras[0].query_mask = s.k2[0].data_ptr(), s.v2[0].data_ptr(), qm_all
            if ns == 2:
                extras[1].k, extras[1].v, extras[1].query_mask = s.k2[1].data_ptr(), s.v2[1].data_ptr(), 2
            ap = _lib.KvAppend()
            if wt > 0:
                ap.nw_k, ap.nw_v = state.nw_k[layer].data_ptr(), state.nw_v[layer].data_ptr()
                ap.nw_len, ap.nw_pos = state.nw_len[layer].data_ptr(), state.nw_pos[layer].data_ptr()
                ap.k_window, ap.v_window = s.k2[self.window_slot].data_ptr(), s.v2[self.window_slot].data_ptr()
            ap.br_k, ap.br_v = state.br_k[layer].data_ptr(), state.br_v[layer].data_ptr()
            ap.br_len = state.br_len[layer].data_ptr()
            ap.k_retained, ap.v_retained = (s.k2[self.retained_slot].data_ptr(),
                                            s.v2[self.retained_slot].data_ptr())
            ap.active = s.active_i8.data_ptr()
            ap.window_storage, ap.retained_storage = storage, state.max_tokens
            ap.window_tokens = wt
            s.layer_args.append((segs, n_seg, extras, ap))
            ws_bytes = max(ws_bytes, self.lib.spsattn_decode_step_workspace_bytes(b, h, hd, ns, segs, n_seg))
        s.ws = torch.zeros(ws_bytes, device=dev, dtype=torch.uint8)
        s.ws_bytes = ws_bytes
        self._step = s

    def _step_body(self) -> None:
        """One token for every row: reads ``token`` / ``active`` of the bound buffers, leaves the
        prediction logits in ``logits`` and the caches and counters advanced.  No host sync."""
        s, d, st = self._step, self.dims, self._step.state
        b, c, h, hd, ns = s.b, d.hidden_size, d.n_head, d.head_dim, self.n_slot
        stream = self._stream()
        torch.where(s.active, s.token, s.zero_tok, out=s.idx_pair[:, 0])     # inference.py:391-398
        torch.where(s.active, st.processed_tokens, s.zero_tok, out=s.pos)    # :399-403
        s.active_i8.copy_(s.active)
        torch.index_select(self.freqs, 0, s.pos, out=s.fc)
        # a row that starts a document forgets its caches, in every layer (:113-122, :408-409)
        reset = st.next_doc_start & s.active
        st.nw_len.masked_fill_(reset.unsqueeze(0), 0)
        st.nw_pos.masked_fill_(reset.unsqueeze(0), 0)
        st.br_len.masked_fill_(reset.view(1, b, 1), 0)
        torch.index_select(self.w.wte, 0, s.idx_pair.view(-1), out=s.x)
        self._add_rmsnorm(s.x, None, self.w.attn_norm[0], s.xn)
        scale = 1.0 / math.sqrt(hd)
        for layer in range(d.n_layer):
            segs, n_seg, extras, ap = s.layer_args[layer]
            torch.mm(s.xn, self.w.c_attn[layer].t(), out=s.qkv)
            rc = self.lib.spsattn_qkv_rope_cast(s.qkv.data_ptr(), self.x_dtype_code, 3 * ns * c, 0, hd,
                                                s.fc.data_ptr(), hd // 2, s.groups, 3 * ns, _lib.DTYPE_BF16,
                                                b, 1, h, hd, stream)
            _lib.check(rc, "spsattn_qkv_rope_cast")
            rc = self.lib.spsattn_decode_step(s.q.data_ptr(), ns, s.y.data_ptr(), _lib.DTYPE_BF16, segs, n_seg,
                                              extras, ns, C.byref(ap), b, h, hd, _lib.DTYPE_BF16, scale,
                                              s.ws.data_ptr(), s.ws_bytes, _status(self.device).data_ptr(),
                                              stream)
            _lib.check(rc, "spsattn_decode_step")
            if s.y_param is not s.y:
                s.y_param.copy_(s.y)                                        # inference.py:479-483
            torch.mm(s.y_param, self.w.c_proj[layer].t(), out=s.delta)
            self._add_rmsnorm(s.x, s.delta, self.w.mlp_norm[layer], s.xn)
            self._mlp(layer, s.xn, s.gate_up, s.hidden, s.delta)
            nxt = self.w.attn_norm[layer + 1] if layer + 1 < d.n_layer else self.w.out_norm
            self._add_rmsnorm(s.x, s.delta, nxt, s.xn)
        pred = s.xn.view(b, ns, c)[:, self.pred_slot]
        torch.mm(pred, self.w.lm_head.t(), out=s.logits)
        # _advance_decode_state (:487-503)
        st.processed_tokens.add_(s.active.to(torch.long))
        torch.where(s.active, s.token == d.eos_token_id, st.next_doc_start, out=st.next_doc_start)

    @torch.no_grad()
    def decode_one_token(self, state: DecodeState, token_B: Tensor, active_B: Tensor) -> Tensor:
        """Eager form of one step (decode + advance): logits [B, V], zeros for inactive rows as
        the reference returns them (inference.py:485).  Raises ValueError, like the reference
        (inference.py:384-389), when a row could already hold as many tokens as the rotary table
        or the caches take: past that point the position lookup would read out of range and the
        cache append would be dropped."""
        limit = min(self.dims.block_size, state.max_tokens)
        if state.host_tokens >= limit:
            raise ValueError(f"Cannot decode another token: up to {state.host_tokens} tokens are processed "
                             f"and the block size / cache capacity is {limit}")
        state.host_tokens += 1
        if self._step is None or self._step.state is not state:
            self._bind_step(state)
        s = self._step
        s.token.copy_(token_B.to(self.device))
        s.active.copy_(active_B.to(self.device, torch.bool))
        self._step_body()
        return torch.where(s.active.unsqueeze(1), s.logits, torch.zeros_like(s.logits))

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, idx_BxT: Tensor, max_new_tokens: int, *, stop_on_eos: bool = True,
                 forbidden_token_ids: Optional[Tensor] = None, do_sample: bool = False,
                 use_graph: bool = True, timings: Optional[dict] = None) -> Tensor:
        """Greedy generation: [B, T + max_new_tokens], pad after a row has emitted EOS when
        ``stop_on_eos`` (utils/generation.py:121-197).  The caches, the step buffers and the
        captured graph are kept for the next call with the same batch size, cache capacity and
        sampling options, which then pays neither allocation nor capture.  ``timings`` (optional
        dict) receives CUDA-event times in ms: ``prefill``, ``decode`` (everything after it) and
        ``decode_steps`` (the ``n_steps`` per-token steps alone)."""
        if do_sample:
            raise NotImplementedError("only greedy decoding is implemented")
        if max_new_tokens < 0:
            raise ValueError(f"max_new_tokens must be non-negative, got {max_new_tokens}")
        d = self.dims
        idx = idx_BxT.to(self.device)
        if max_new_tokens == 0:
            return idx.clone()
        b = idx.shape[0]
        # inference.py:893-902; the Standard model suppresses pad only (full_attention_model.py:494-499)
        sup = [d.pad_token_id] + ([d.predict_token_id] if self.n_slot == 2 else [])
        if forbidden_token_ids is not None:
            sup += [int(x) for x in forbidden_token_ids.reshape(-1).tolist()]
        sup = tuple(sorted(set(sup)))
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        g = self._session
        reuse = g is not None and g.state.processed_tokens.shape[0] == b
        state, next_logits = self.prefill(idx, max_new_tokens, state=g.state if reuse else None)
        ev[1].record()
        key = (b, state.max_tokens, int(max_new_tokens), bool(stop_on_eos), sup, bool(use_graph))
        if g is None or g.state is not state or g.key != key:
            g = self._new_session(state, key)
        # the captured graph reads and writes the step buffers it was recorded on: the session owns
        # them, and they are bound again if a decode_one_token on another state replaced them
        self._step = g.step
        s = self._step
        g.next_logits.copy_(next_logits)
        g.generated.fill_(d.pad_token_id)
        g.finished.fill_(False)
        g.step_idx.zero_()
        n_steps = max_new_tokens - 1          # the last token is sampled without a further decode
        if n_steps > 0 and use_graph and g.graph is None:
            # warm-up with every row marked finished: the chain runs, nothing is sampled or stored
            g.finished.fill_(True)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._token_body(g)
            torch.cuda.current_stream(self.device).wait_stream(side)
            g.finished.fill_(False)
            g.step_idx.zero_()
            g.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g.graph):          # capture records, it does not execute
                self._token_body(g)
        ev[2].record()
        for _ in range(n_steps):
            if use_graph:
                g.graph.replay()
            else:
                self._token_body(g)
        ev[3].record()
        self._sample(g)
        ev[4].record()
        state.host_tokens += n_steps
        if timings is not None:
            torch.cuda.synchronize(self.device)
            check_device_status(self.device)
            timings["prefill"] = ev[0].elapsed_time(ev[1])
            timings["decode"] = ev[1].elapsed_time(ev[4])        # includes binding and capture, if any
            timings["decode_steps"] = ev[2].elapsed_time(ev[3])  # the n_steps token steps alone
            timings["n_steps"] = n_steps
        return torch.cat([idx, g.generated.to(idx.dtype)], dim=1)

    def _new_session(self, state: DecodeState, key):
        d, dev = self.dims, self.device
        b, max_new = key[0], key[2]
        if self._step is None or self._step.state is not state:
            self._bind_step(state)
        g = type("GenerationSession", (), {})()
        g.state, g.key, g.graph = state, key, None
        g.step = self._step
        g.stop_on_eos = key[3]
        g.suppressed = torch.tensor(list(key[4]), device=dev, dtype=torch.long)
        g.generated = torch.full((b, max_new), d.pad_token_id, device=dev, dtype=torch.long)
        g.finished = torch.zeros(b, device=dev, dtype=torch.bool)
        g.step_idx = torch.zeros((1, 1), device=dev, dtype=torch.long)
        g.pad_tok = torch.full((b,), d.pad_token_id, device=dev, dtype=torch.long)
        g.next_logits = torch.zeros((b, d.vocab_size), device=dev, dtype=self.param_dtype)
        self._session = g
        return g

    def _sample(self, g):
        """utils/generation.py:171-181 with greedy sampling (utils/sampling.py:55-83)."""
        live = ~g.finished
        z = g.next_logits.float()
        z.index_fill_(1, g.suppressed, float("-inf"))
        tok = torch.where(live, z.argmax(dim=-1), g.pad_tok)
        g.generated.scatter_(1, g.step_idx.expand(tok.shape[0], 1), tok.view(-1, 1))
        newly = live & (tok == self.dims.eos_token_id) if g.stop_on_eos else torch.zeros_like(live)
        return tok, live & ~newly, newly

    def _token_body(self, g) -> None:
        """Sample one token per row, run the decode step on it, keep its logits for the next
        (utils/generation.py:171-195); reads and writes only buffers of the session."""
        s = self._step
        tok, decode_active, newly = self._sample(g)
        s.token.copy_(tok)
        s.active.copy_(decode_active)
        self._step_body()
        torch.where(decode_active.unsqueeze(1), s.logits, g.next_logits, out=g.next_logits)
        g.finished.logical_or_(newly)
        g.step_idx.add_(1)


def generator_for(model, *, param_dtype: Optional[torch.dtype] = None) -> SPSGenerator:
    """Build the engine from an instance of the reference's SPSModel / ReverseSPSModel /
    DelayedStateModel: its ``config`` supplies the dimensions, its ``state_dict()`` the parameters,
    its slot indices (sps/inference.py:8-12, reverse_sps/inference.py:58-62) the variant."""
    cfg = model.config
    is_standard = not hasattr(cfg, "predict_token_id")      # full_attention_model.ModelConfig
    dims = SPSDims(block_size=int(cfg.block_size), vocab_size=int(cfg.vocab_size), n_layer=int(cfg.n_layer),
                   n_head=int(cfg.n_head), hidden_size=int(cfg.hidden_size),
                   intermediate_size=int(cfg.intermediate_size), norm_eps=float(cfg.norm_eps),
                   eos_token_id=int(cfg.eos_token_id), pad_token_id=int(cfg.pad_token_id),
                   predict_token_id=-1 if is_standard else int(cfg.predict_token_id),
                   window_size=0 if is_standard else int(cfg.window_size))
    if is_standard:
        variant = "standard"
    else:
        slots = (int(getattr(model, "_prediction_slot_index", 0)), int(getattr(model, "_window_slot_index", 0)),
                 int(getattr(model, "_retained_slot_index", 1)))
        variant = next((name for name, v in _VARIANTS.items() if v[:3] == slots), None)
        if variant is None:
            raise ValueError(f"unknown slot assignment {slots}")
    sd = model.state_dict()
    first = next(iter(sd.values()))
    if param_dtype is None:
        param_dtype = torch.bfloat16 if first.dtype == torch.bfloat16 else torch.float32
    device = first.device if first.is_cuda else torch.device("cuda")
    return SPSGenerator(sd, dims, variant=variant, device=device, param_dtype=param_dtype)


def bind_generate(model, *, param_dtype: Optional[torch.dtype] = None) -> SPSGenerator:
    """Replace ``model.generate`` (reverse_sps/inference.py:904-951) by the engine, keeping its
    signature; sampling other than greedy raises instead of falling back.  Returns the engine."""
    engine = generator_for(model, param_dtype=param_dtype)

    def generate(idx_BxT, max_new_tokens, *, temperature=1.0, top_k=None, top_p=None, do_sample=False,
                 stop_on_eos=True, forbidden_token_ids=None):
        del temperature, top_k, top_p
        return engine.generate(idx_BxT, max_new_tokens, stop_on_eos=stop_on_eos,
                               forbidden_token_ids=forbidden_token_ids, do_sample=do_sample)

    model.generate = generate
    return engine
