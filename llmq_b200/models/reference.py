"""fp32 PyTorch-autograd oracle of the decoder and of AdamW.

Independent of the hand-written forward/backward in ``llama.py``: plain tensor algebra on the same fused
weight layout (qkv_w, up_w = [up; gate], half-split RoPE, optional QKV bias, tied or untied head), loss
normalised by the number of positions, ``-100`` targets ignored, optional z-loss.  Used by the tests as
ground truth (the reference repository checks itself against HF transformers in the same way,
src/binding/python/tests/torch_reference.py).
"""
from __future__ import annotations

import math
from typing import Dict

import torch
import torch.nn.functional as F

from ..config import TransformerConfig


def rope_ref(x: torch.Tensor, theta: float) -> torch.Tensor:
    """x: (B, T, H, HS); rotates pairs (d, d + HS/2)."""
    B, T, H, HS = x.shape
    d = torch.arange(HS // 2, dtype=torch.float64)
    inv = theta ** (-2.0 * d / HS)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().to(x.dtype)[None, :, None, :], ang.sin().to(x.dtype)[None, :, None, :]
    x1, x2 = x[..., : HS // 2], x[..., HS // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


def rmsnorm_ref(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def forward_ref(cfg: TransformerConfig, params: Dict[str, torch.Tensor], tokens: torch.Tensor):
    """params uses checkpoint names (``layers.N.qkv_w`` ...).  Returns logits (B, T, V)."""
    B, T = tokens.shape
    Hq, Hkv, HS, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_size, cfg.intermediate_size
    x = params["embed"][tokens.long()]
    for l in range(cfg.num_hidden_layers):
        p = lambda n: params[f"layers.{l}.{n}"]
        h = rmsnorm_ref(x, p("ln1_w"), cfg.rms_norm_eps)
        qkv = h @ p("qkv_w").t()
        if cfg.use_qkv_bias:
            qkv = qkv + p("qkv_b")
        qkv = qkv.view(B, T, Hq + 2 * Hkv, HS)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        q, k = rope_ref(q, cfg.rope_theta), rope_ref(k, cfg.rope_theta)
        rep = Hq // Hkv
        k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
        s = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(HS)
        mask = torch.ones(T, T, dtype=torch.bool).tril()
        s = s.masked_fill(~mask, float("-inf"))
        att = torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), v).reshape(B, T, Hq * HS)
        x = x + att @ p("o_w").t()
        h = rmsnorm_ref(x, p("ln2_w"), cfg.rms_norm_eps)
        ug = h @ p("up_w").t()
        up, gate = ug[..., :D], ug[..., D:]
        x = x + (up * F.silu(gate)) @ p("down_w").t()
    x = rmsnorm_ref(x, params["lnf_w"], cfg.rms_norm_eps)
    head = params["embed"] if cfg.tie_word_embeddings else params["lm_head"]
    return x @ head.t()


def loss_ref(cfg, params, tokens, targets, z_loss: float = 0.0, positions: int | None = None):
    """Sum of token losses divided by ``positions`` (default B*T); z-loss adds z * lse^2 / 2 per token."""
    logits = forward_ref(cfg, params, tokens)
    B, T, V = logits.shape
    tg = targets.long().reshape(-1)
    lg = logits.reshape(-1, V)
    lse = torch.logsumexp(lg, -1)
    valid = tg != -100
    picked = lg.gather(1, tg.clamp_min(0)[:, None])[:, 0]
    per_tok = torch.where(valid, lse - picked, torch.zeros_like(lse))
    n = positions or (B * T)
    ce = per_tok.sum() / n
    z = (torch.where(valid, 0.5 * z_loss * lse * lse, torch.zeros_like(lse))).sum() / n
    return ce + z, ce


def adamw_ref(p, g, m, v, lr, beta1, beta2, step, eps, wd):
    """Bias-corrected AdamW in fp32, decoupled weight decay scaled by the learning rate."""
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    p = p - lr * (mh / (vh.sqrt() + eps) + wd * p)
    return p, m, v
