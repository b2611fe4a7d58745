"""Plain PyTorch statements of every op in this package.

They are the numerical oracle for the CUDA kernels and the execution path on CPU
(gloo ranks, unit tests). Semantics follow the eager model code of the reference
(attention: oslo/models/gptj/modeling_gptj.py:151-191, rotary :49-77; causal softmax:
oslo/fused_kernels/includes/fused_triang_softmax.h:134-251; padded softmax:
includes/fused_softmax.h:111-229; n-gram ban: fused_ngram_repeat_block.cu:18-49).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor


def gelu_tanh(x: Tensor) -> Tensor:
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, reversed: bool = False,
           activation: Optional[str] = None) -> Tensor:
    """``x @ W.T`` (``nn.Linear`` layout) or ``x @ W`` when ``reversed`` (Conv1D ``[in, out]`` layout)."""
    y = torch.matmul(x, weight if reversed else weight.t())
    if bias is not None:
        y = y + bias
    if activation in ("gelu", "gelu_new", "gelu_tanh", "gelu_pytorch_tanh"):
        y = gelu_tanh(y)
    elif activation is not None:
        raise ValueError(f"unsupported fused activation {activation!r}")
    return y


def layer_norm(x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float) -> Tensor:
    return F.layer_norm(x, (x.size(-1),), weight, bias, eps)


def bias_gelu(x: Tensor, bias: Optional[Tensor]) -> Tensor:
    return gelu_tanh(x if bias is None else x + bias)


def bias_dropout_residual(x: Tensor, bias: Optional[Tensor], residual: Optional[Tensor], p: float,
                          training: bool) -> Tensor:
    y = x if bias is None else x + bias
    y = F.dropout(y, p=p, training=training)
    return y if residual is None else y + residual


def rotary_tables(positions: Tensor, rotary_dim: int, base: float = 10000.0) -> Tuple[Tensor, Tensor]:
    """sin/cos of shape ``[..., rotary_dim // 2]`` in fp32 for integer ``positions``."""
    inv = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, device=positions.device, dtype=torch.float32) / rotary_dim))
    ang = positions.to(torch.float32).unsqueeze(-1) * inv
    return torch.sin(ang), torch.cos(ang)


def rotary_interleaved(x: Tensor, positions: Tensor, rotary_dim: int, base: float = 10000.0) -> Tensor:
    """GPT-J rotary embedding: pairs ``(x[2i], x[2i+1])`` of the first ``rotary_dim`` dims are rotated.

    ``x``: ``[B, S, heads, head_dim]``; ``positions``: ``[B, S]`` (or ``[S]``).
    """
    if positions.dim() == 1:
        positions = positions.unsqueeze(0).expand(x.size(0), -1)
    sin, cos = rotary_tables(positions, rotary_dim, base)  # [B, S, r/2]
    sin, cos = sin.unsqueeze(2), cos.unsqueeze(2)
    xr = x[..., :rotary_dim].to(torch.float32)
    x1, x2 = xr[..., 0::2], xr[..., 1::2]
    o1 = x1 * cos - x2 * sin
    o2 = x2 * cos + x1 * sin
    rot = torch.stack((o1, o2), dim=-1).flatten(-2)
    return torch.cat((rot.to(x.dtype), x[..., rotary_dim:]), dim=-1)


def attention_mask_bias(sq: int, sk: int, device, causal: bool, window: Optional[int]) -> Optional[Tensor]:
    """Boolean ``[sq, sk]`` keep-mask. Query ``i`` sits at absolute position ``sk - sq + i``."""
    if not causal and window is None:
        return None
    qpos = torch.arange(sk - sq, sk, device=device).unsqueeze(1)
    kpos = torch.arange(sk, device=device).unsqueeze(0)
    keep = torch.ones(sq, sk, dtype=torch.bool, device=device)
    if causal:
        keep &= kpos <= qpos
    if window is not None:
        keep &= kpos > qpos - window
    return keep


def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, window: Optional[int] = None,
              scale: Optional[float] = None, key_padding_mask: Optional[Tensor] = None,
              dropout_p: float = 0.0, training: bool = False, return_probs: bool = False):
    """Softmax attention on ``[B, heads, S, D]`` tensors, fp32 scores.

    ``key_padding_mask``: ``[B, Sk]`` with 1 = keep, 0 = padded key. ``window`` keeps keys
    ``q_pos - window < k_pos <= q_pos`` (GPT-Neo local attention).
    """
    sq, sk = q.size(-2), k.size(-2)
    if scale is None:
        scale = 1.0 / math.sqrt(q.size(-1))
    s = torch.matmul(q.to(torch.float32), k.to(torch.float32).transpose(-1, -2)) * scale
    keep = attention_mask_bias(sq, sk, q.device, causal, window)
    neg = torch.finfo(torch.float32).min
    if keep is not None:
        s = s.masked_fill(~keep, neg)
    if key_padding_mask is not None:
        s = s.masked_fill(~key_padding_mask.to(torch.bool)[:, None, None, :], neg)
    p = torch.softmax(s, dim=-1)
    if dropout_p > 0.0 and training:
        p = F.dropout(p, dropout_p, True)
    out = torch.matmul(p, v.to(torch.float32)).to(q.dtype)
    return (out, p) if return_probs else out


def scaled_upper_triang_masked_softmax(x: Tensor, scale: float) -> Tensor:
    """Causal softmax of ``scale * x`` on ``[batches, S, S]``; entries above the diagonal are exactly 0."""
    s = x.size(-1)
    keep = torch.ones(s, s, dtype=torch.bool, device=x.device).tril()
    y = (x.to(torch.float32) * scale).masked_fill(~keep, float("-inf"))
    return torch.softmax(y, dim=-1).to(x.dtype)


def scaled_masked_softmax(x: Tensor, mask: Tensor, scale: float) -> Tensor:
    """Softmax of ``scale * x`` on ``[b, heads, sq, sk]`` where ``mask`` (1 = masked) replaces by -10000."""
    y = x.to(torch.float32) * scale
    y = y.masked_fill(mask.to(torch.bool), -10000.0)
    return torch.softmax(y, dim=-1).to(x.dtype)


def softmax_backward(y: Tensor, dy: Tensor, scale: float) -> Tensor:
    yf, gf = y.to(torch.float32), dy.to(torch.float32)
    t = yf * gf
    return (scale * (t - yf * t.sum(-1, keepdim=True))).to(y.dtype)


def cross_entropy(logits: Tensor, labels: Tensor, ignore_index: int = -100) -> Tensor:
    """Mean token cross-entropy in fp32 over ``[N, V]`` logits."""
    return F.cross_entropy(logits.to(torch.float32), labels, ignore_index=ignore_index)


def adam_step(p32: Tensor, g: Tensor, m: Tensor, v: Tensor, step: int, lr: float, beta1: float, beta2: float,
              eps: float, weight_decay: float, grad_scale: float = 1.0, p_lp: Optional[Tensor] = None) -> None:
    """In-place AdamW on fp32 master weights; optionally refreshes a low-precision copy."""
    gf = g.to(torch.float32) * grad_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    if weight_decay != 0.0:
        p32.mul_(1 - lr * weight_decay)
    denom = (v / bc2).sqrt_().add_(eps)
    p32.addcdiv_(m / bc1, denom, value=-lr)
    if p_lp is not None:
        p_lp.copy_(p32)


def banned_ngram_tokens(tokens: Tensor, n: int):
    """For each row, tokens that would complete an n-gram already present in that row."""
    out = []
    rows = tokens.tolist()
    for row in rows:
        banned = set()
        if len(row) + 1 >= n:
            tail = tuple(row[len(row) - n + 1:]) if n > 1 else ()
            for i in range(len(row) - n + 1):
                if tuple(row[i:i + n - 1]) == tail:
                    banned.add(row[i + n - 1])
        out.append(sorted(banned))
    return out


def ban_repeated_ngrams(tokens: Tensor, lprobs: Tensor, n: int) -> Tensor:
    """Set ``lprobs[row, tok] = -inf`` for every token that would repeat an n-gram of ``tokens[row]``."""
    if n <= 0:
        return lprobs
    for r, banned in enumerate(banned_ngram_tokens(tokens, n)):
        if banned:
            lprobs[r, banned] = float("-inf")
    return lprobs
