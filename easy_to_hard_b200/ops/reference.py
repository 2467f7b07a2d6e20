"""Plain PyTorch restatements of every fused op.

They are the oracle the CUDA kernels are tested against and the code path used on CPU
(gloo plumbing tests, data-only tooling). They follow the numerics of the reference model:
bf16 tensors between ops, fp32 inside norm / softmax / RoPE / losses
(models/model.py:363-412, train_sft.py:98-115 of the reference).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return y * weight.to(x.dtype)


def precompute_freqs_cis(seq_len: int, n_elem: int, base: float = 10000.0,
                         dtype=torch.bfloat16, device=None) -> torch.Tensor:
    """[seq_len, n_elem/2, 2] (cos, sin) table; the reference stores it in bf16
    (models/model.py:389-397)."""
    freqs = 1.0 / (base ** (torch.arange(0, n_elem, 2, device=device)[: n_elem // 2].float()
                            / n_elem))
    t = torch.arange(seq_len, device=device)
    ang = torch.outer(t, freqs)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(dtype)


def apply_rotary_emb(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair RoPE. x [B, S, H, D]; freqs_cis [S, D/2, 2]."""
    xs = x.float().reshape(*x.shape[:-1], -1, 2)
    fc = freqs_cis.view(1, xs.size(1), 1, xs.size(3), 2).float()
    out = torch.stack([xs[..., 0] * fc[..., 0] - xs[..., 1] * fc[..., 1],
                       xs[..., 1] * fc[..., 0] + xs[..., 0] * fc[..., 1]], -1)
    return out.flatten(3).type_as(x)


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    return F.silu(g) * u


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor],
              causal: bool = False) -> torch.Tensor:
    """q [B,H,Sq,D], k/v [B,Hkv,Sk,D] -> [B,H,Sq,D]; softmax in fp32."""
    H, Hkv = q.size(1), k.size(1)
    if H != Hkv:
        k = k.repeat_interleave(H // Hkv, dim=1)
        v = v.repeat_interleave(H // Hkv, dim=1)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) / math.sqrt(q.size(-1))
    if causal:
        Sq, Sk = q.size(2), k.size(2)
        cm = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril(Sk - Sq)
        s = s.masked_fill(~cm, float("-inf"))
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v.float()).to(q.dtype)


def logits_to_probs(logits: torch.Tensor, temperature: float = 1.0,
                    top_k: Optional[int] = None) -> torch.Tensor:
    logits = logits / max(temperature, 1e-5)
    if top_k is not None:
        v, _ = torch.topk(logits, min(top_k, logits.size(-1)), dim=-1)
        pivot = v[..., -1:].contiguous()
        logits = torch.where(logits < pivot, torch.full_like(logits, float("-inf")), logits)
    return torch.softmax(logits, dim=-1)


def sample_from_probs(probs: torch.Tensor, generator=None) -> torch.Tensor:
    """argmax(p / q), q ~ Exp(1): a multinomial draw without a host synchronisation."""
    q = torch.empty_like(probs).exponential_(1.0, generator=generator)
    return torch.argmax(probs / q, dim=-1, keepdim=True).to(torch.int32)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
           generator=None):
    """logits [B, V] fp32 -> (token [B,1] int32, probs [B,V]); temperature 0 = greedy."""
    logits = logits.float()
    if temperature <= 0:
        idx = torch.argmax(logits, dim=-1, keepdim=True).to(torch.int32)
        return idx, torch.softmax(logits, -1)
    probs = logits_to_probs(logits, temperature, top_k)
    return sample_from_probs(probs, generator), probs


def cross_entropy_logprobs(logits: torch.Tensor, targets: torch.Tensor,
                           ignore_index: int = -100, temperature: float = 1.0):
    """Per-token log-prob of `targets` and entropy, fp32. logits [N, V], targets [N]."""
    lf = logits.float() / temperature
    lse = torch.logsumexp(lf, dim=-1)
    safe = targets.clamp_min(0)
    tgt = lf.gather(-1, safe.unsqueeze(-1)).squeeze(-1)
    logp = tgt - lse
    p = torch.softmax(lf, dim=-1)
    ent = lse - (p * lf).sum(-1)
    valid = targets != ignore_index
    return torch.where(valid, logp, torch.zeros_like(logp)), ent, valid


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step):
    """The memory-efficient AdamW update of the reference
    (training_utils/memory_efficient_adam.py:61-104), in place."""
    if weight_decay != 0:
        p.mul_(1 - lr * weight_decay)
    gg = g.to(m.dtype)
    m.mul_(beta1).add_(gg, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gg, gg, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m.to(p.dtype), denom.to(p.dtype), value=-lr / bc1)
