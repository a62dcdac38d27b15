"""CPU oracle for the SPS decoder around the attention path.  TEST INFRASTRUCTURE ONLY.

Restates, in CPU torch fp32, what the reference's SPS-family model computes from token ids to
logits, so that the generation engine (``sps_b200.generation``) can be checked end to end:

  * document ids and positions of left-padded prompts
        src/modeling/models/model.py:60-64 (positions), :67-99 (document ids)
  * the decoder block: RMSNorm, fused q/k/v projection, rotary embedding, the masked attention
    over the doubled sequence, output projection, SwiGLU MLP
        src/modeling/models/model.py:101-132, :201-230, :304-327
        src/modeling/models/sps/core.py:35-82, src/modeling/models/reverse_sps/core.py:56-99
  * which slot carries the prediction (SPS: odd rows; Reverse-SPS / Delayed-State: even rows)
        src/modeling/models/sps/core.py:146 / src/modeling/models/reverse_sps/core.py:276,
        src/modeling/models/sps/inference.py:8-12
  * greedy generation with the <predict> and pad ids suppressed
        src/modeling/models/utils/generation.py:121-197, utils/sampling.py:9-85

Generation is computed by re-running the dense forward over the tokens so far; the reference's
tests establish that its cached decode equals that (tests/models/sps/test_dense_only.py:226-249,
:339-384).  The attention itself is ``sps_oracle.prefill_attention``.

Parity status: PINNED by ``tests/golden/`` (logits of the reference's own ``forward``,
``forward_efficient`` and greedy tokens on tiny models; ``tests/test_oracle_golden.py``).

Only tests, the smoke check and the benchmark's CPU baseline may import this module.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Sequence

import torch

from . import sps_oracle


@dataclass
class Dims:
    """Same fields as the reference's SPSConfig / ReverseSPSConfig (reverse_sps/core.py:128-135,
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


# (prediction slot, persistent-key parity) per model family
VARIANTS = {"sps": (1, sps_oracle.PARITY_EVEN), "reverse_sps": (0, sps_oracle.PARITY_ODD),
            "delayed_state": (1, sps_oracle.PARITY_ODD),   # delayed_state/inference.py:8-10, core.py:49
            # Standard model: no <predict> rows, causal attention inside a document
            # (full_attention_model.py:77-122, :744-853)
            "standard": (0, sps_oracle.PARITY_NONE)}


def document_idx(idx: torch.Tensor, eos: int, pad: int) -> torch.Tensor:
    """model.py:67-99: EOS ends a document; every left-pad token is a document of its own,
    numbered below the real ones."""
    real = idx != pad
    b, t = idx.shape
    pad_count = (~real).sum(dim=1, keepdim=True)
    eos_real = real & (idx == eos)
    doc = torch.zeros((b, t), dtype=torch.long)
    if t > 1:
        doc[:, 1:] = torch.cumsum(eos_real[:, :-1].long(), dim=1)
    doc = doc + pad_count
    pad_doc = torch.clamp(torch.cumsum((~real).long(), dim=1) - 1, min=0)
    return torch.where(real, doc, pad_doc)


def left_padded_positions(idx: torch.Tensor, pad: int) -> torch.Tensor:
    """model.py:60-64: consecutive positions for real tokens, 0 at pads."""
    real = idx != pad
    pos = real.long().cumsum(dim=1) - 1
    return torch.where(real, pos, torch.zeros_like(pos))


def freqs_cis(head_dim: int, end: int, theta: float = 10000.0) -> torch.Tensor:
    """model.py:134-160."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    ang = torch.outer(torch.arange(end).float(), freqs)
    return torch.polar(torch.ones_like(ang), ang)


def _rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x: torch.Tensor, fc: torch.Tensor) -> torch.Tensor:
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    return torch.view_as_real(xc * fc.unsqueeze(2)).flatten(3)


def hidden_states(weights: Dict[str, torch.Tensor], dims: Dims, idx: torch.Tensor, *,
                  variant: str = "sps", positions: Optional[torch.Tensor] = None,
                  operand_dtype: torch.dtype = torch.bfloat16,
                  round_output: bool = True) -> torch.Tensor:
    """Final-norm hidden states [B, 2T, C] of the doubled sequence (reverse_sps/core.py:234-259).
    ``positions`` [B, T]: token positions (default arange(T), as the dense forward uses);
    ``operand_dtype``: rounding applied to q, k, v before attention (sps/core.py:53-55);
    ``round_output``: also round the attention output to it, as a kernel that returns that
    type does."""
    _, parity = VARIANTS[variant]
    w = {k: v.float() for k, v in weights.items()}
    b, t = idx.shape
    nh, c = dims.n_head, dims.hidden_size
    hd = c // nh
    rep = 1 if variant == "standard" else 2     # rows per token
    docs2 = document_idx(idx, dims.eos_token_id, dims.pad_token_id).repeat_interleave(rep, dim=1)
    pos = torch.arange(t).unsqueeze(0).expand(b, -1) if positions is None else positions
    fc = freqs_cis(hd, dims.block_size)[pos.repeat_interleave(rep, dim=1)]     # [B, rep*T, hd/2]
    idx2 = idx.repeat_interleave(rep, dim=1)
    if rep == 2:
        idx2[:, 1::2] = dims.predict_token_id
    n_rows = idx2.shape[1]
    x = w["transformer.wte.weight"][idx2]
    for layer in range(dims.n_layer):
        pre = f"transformer.h.{layer}."
        xn = _rmsnorm(x, w[pre + "attention_norm.weight"], dims.norm_eps)
        q, k, v = (xn @ w[pre + "attn.c_attn.weight"].T).split(c, dim=2)
        q = _rope(q.view(b, n_rows, nh, hd), fc).to(operand_dtype).float().transpose(1, 2)
        k = _rope(k.view(b, n_rows, nh, hd), fc).to(operand_dtype).float().transpose(1, 2)
        v = v.view(b, n_rows, nh, hd).to(operand_dtype).float().transpose(1, 2)
        y = sps_oracle.prefill_attention(q, k, v, 1.0 / math.sqrt(hd), persistent_parity=parity,
                                         temporary_window=dims.window_size, docs=docs2)
        if round_output:
            y = y.to(operand_dtype).float()
        y = y.transpose(1, 2).reshape(b, n_rows, c)
        x = x + y @ w[pre + "attn.c_proj.weight"].T
        xn = _rmsnorm(x, w[pre + "mlp_norm.weight"], dims.norm_eps)
        gate = torch.nn.functional.silu(xn @ w[pre + "mlp.gate_proj.weight"].T)
        x = x + (gate * (xn @ w[pre + "mlp.up_proj.weight"].T)) @ w[pre + "mlp.down_proj.weight"].T
    return _rmsnorm(x, w["transformer.output_norm.weight"], dims.norm_eps)


def logits(weights, dims: Dims, idx: torch.Tensor, *, variant: str = "sps",
           positions: Optional[torch.Tensor] = None,
           operand_dtype: torch.dtype = torch.bfloat16, round_output: bool = True) -> torch.Tensor:
    """Token logits [B, T, V] read at the prediction slot (sps/core.py:146)."""
    slot, _ = VARIANTS[variant]
    x = hidden_states(weights, dims, idx, variant=variant, positions=positions,
                      operand_dtype=operand_dtype, round_output=round_output)
    rep = 1 if variant == "standard" else 2
    return x[:, slot::rep] @ weights["lm_head.weight"].float().T


def greedy_token(logits_BxV: torch.Tensor, dims: Dims,
                 forbidden: Optional[Sequence[int]] = None) -> torch.Tensor:
    """utils/sampling.py:55-83 with do_sample=False: argmax with <predict>, pad and the caller's
    forbidden ids suppressed (reverse_sps/inference.py:893-902)."""
    z = logits_BxV.float().clone()
    if dims.predict_token_id is not None and dims.predict_token_id >= 0:
        z[:, dims.predict_token_id] = float("-inf")
    z[:, dims.pad_token_id] = float("-inf")
    if forbidden is not None and len(forbidden):
        z[:, torch.as_tensor(list(forbidden), dtype=torch.long)] = float("-inf")
    return z.argmax(dim=-1)


def generate(weights, dims: Dims, idx: torch.Tensor, max_new_tokens: int, *, variant: str = "sps",
             stop_on_eos: bool = True, forbidden: Optional[Sequence[int]] = None,
             operand_dtype: torch.dtype = torch.bfloat16, return_margins: bool = False):
    """Greedy generation (utils/generation.py:121-197): [B, T + max_new_tokens], pad after a row
    has emitted EOS.  ``return_margins`` adds the top-1 minus top-2 logit gap of every sampled
    token [B, max_new_tokens] (inf for finished rows), so that a reduced-precision run can be
    compared only where the choice is not a near-tie."""
    b = idx.shape[0]
    seq = idx.clone()
    out = torch.full((b, max_new_tokens), dims.pad_token_id, dtype=idx.dtype)
    margins = torch.full((b, max_new_tokens), float("inf"))
    finished = torch.zeros(b, dtype=torch.bool)
    for step in range(max_new_tokens):
        if bool(finished.all()):
            break
        pos = left_padded_positions(seq, dims.pad_token_id)
        # pads appended to finished rows sit after real tokens; their rows are never read
        lg = logits(weights, dims, seq, variant=variant, positions=pos, operand_dtype=operand_dtype)
        last_real = (seq != dims.pad_token_id).long().cumsum(1).argmax(dim=1)
        z = lg[torch.arange(b), last_real]
        tok = greedy_token(z, dims, forbidden)
        zz = z.float().clone()
        if dims.predict_token_id is not None and dims.predict_token_id >= 0:
            zz[:, dims.predict_token_id] = float("-inf")
        zz[:, dims.pad_token_id] = float("-inf")
        if forbidden is not None and len(forbidden):
            zz[:, torch.as_tensor(list(forbidden), dtype=torch.long)] = float("-inf")
        top2 = zz.topk(2, dim=-1).values
        live = ~finished
        out[live, step] = tok[live]
        margins[live, step] = (top2[:, 0] - top2[:, 1])[live]
        nxt = torch.where(live, tok, torch.full_like(tok, dims.pad_token_id))
        seq = torch.cat([seq, nxt[:, None]], dim=1)
        if stop_on_eos:
            finished = finished | (live & (tok == dims.eos_token_id))
    full = torch.cat([idx, out], dim=1)
    return (full, margins) if return_margins else full
