"""LM head + log-softmax / cross-entropy / log-prob gather / entropy without materialising the
full ``[tokens, vocab]`` logits: the head GEMM runs chunk by chunk (fp32 logits of a few
thousand tokens at a time), the CUDA kernels of ``csrc/loss.cu`` reduce each chunk to four
numbers per token, and the backward recomputes the chunk, turns it into bf16 ``dlogits`` and
feeds the data-gradient GEMM. With a vocabulary-parallel head each rank does this on its shard
and the per-token statistics are combined over the tensor-parallel group.

CPU tensors take the PyTorch restatement (``reference.cross_entropy_logprobs``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib, gemm, reference

CHUNK_TOKENS = 4096


def _combine_stats(stats: torch.Tensor, group, world: int):
    """stats [N, 4] = (m, s, tgt, u) per shard -> (lse, target logit, entropy) of the full row."""
    m, s, tgt, u = stats.unbind(-1)
    if world > 1:
        gm = m.clone()
        dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=group)
        w = torch.exp(m - gm)
        packed = torch.stack([s * w, tgt, u * w], dim=0)
        dist.all_reduce(packed, group=group)
        s, tgt, u = packed[0], packed[1], packed[2]
        m = gm
    lse = m + torch.log(s)
    ent = lse - u / s
    return lse, tgt, ent


def ce_stats(logits: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
             vocab_start: int = 0) -> torch.Tensor:
    """Per-row (max, sum-exp, target logit, sum p*x) of an fp32 logits (shard) [N, V]."""
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    N, V = logits.shape
    stats = torch.empty(N, 4, dtype=torch.float32, device=logits.device)
    tg = targets.to(torch.int64).contiguous()
    rc = _lib.lib().e2h_ce_stats(logits.data_ptr(), logits.stride(0), N, V, tg.data_ptr(),
                                 vocab_start, 1.0 / temperature, stats.data_ptr(), _lib.stream())
    _lib.check(rc, "ce_stats")
    return stats


def ce_grad(logits, targets, lse, ent, g_lp, g_ent, temperature: float = 1.0,
            vocab_start: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    N, V = logits.shape
    if out is None:
        out = torch.empty(N, V, dtype=torch.bfloat16, device=logits.device)
    tg = targets.to(torch.int64).contiguous()
    rc = _lib.lib().e2h_ce_grad(logits.data_ptr(), logits.stride(0), N, V, tg.data_ptr(),
                                vocab_start, 1.0 / temperature, lse.data_ptr(), _lib.ptr(ent),
                                _lib.ptr(g_lp), _lib.ptr(g_ent), out.data_ptr(), out.stride(0),
                                _lib.stream())
    _lib.check(rc, "ce_grad")
    return out


class _LinearLogprobs(torch.autograd.Function):
    """(log p(target), entropy) per token of softmax(hidden @ W^T / temperature)."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, ignore_index, temperature, vocab_start, group,
                world, weight_requires_grad):
        N = hidden.shape[0]
        logp = torch.empty(N, dtype=torch.float32, device=hidden.device)
        ent = torch.empty_like(logp)
        lse = torch.empty_like(logp)
        safe = targets.clamp_min(0)
        for a in range(0, N, CHUNK_TOKENS):
            b = min(N, a + CHUNK_TOKENS)
            logits = gemm.linear(hidden[a:b], weight, out_dtype=torch.float32)
            st = ce_stats(logits, safe[a:b], temperature, vocab_start)
            L, tgt, H = _combine_stats(st, group, world)
            lse[a:b], ent[a:b], logp[a:b] = L, H, tgt - L
        valid = targets != ignore_index
        logp = torch.where(valid, logp, torch.zeros_like(logp))
        ctx.save_for_backward(hidden, weight, safe, lse, ent, valid)
        ctx.cfg = (temperature, vocab_start, group, world, weight_requires_grad)
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        hidden, weight, safe, lse, ent, valid = ctx.saved_tensors
        temperature, vocab_start, group, world, w_grad = ctx.cfg
        N = hidden.shape[0]
        g_lp = torch.where(valid, g_logp.float(), torch.zeros_like(lse)).contiguous()
        g_en = g_ent.float().contiguous() if g_ent is not None else None
        if g_en is not None and not bool((g_en != 0).any()):
            g_en = None
        dh = torch.empty_like(hidden)
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device) if w_grad \
            else None
        for a in range(0, N, CHUNK_TOKENS):
            b = min(N, a + CHUNK_TOKENS)
            logits = gemm.linear(hidden[a:b], weight, out_dtype=torch.float32)
            dl = ce_grad(logits, safe[a:b], lse[a:b], ent[a:b], g_lp[a:b],
                         None if g_en is None else g_en[a:b], temperature, vocab_start)
            gemm.linear_dgrad(dl, weight, out=dh[a:b])
            if dw is not None:
                gemm.linear_wgrad(dl, hidden[a:b].contiguous(), out=dw, accumulate=a > 0)
        if world > 1:   # the hidden states are replicated: sum the shards' contributions
            dist.all_reduce(dh, group=group)
        return (dh, None if dw is None else dw.to(weight.dtype), None, None, None, None, None,
                None, None)


def linear_logprobs(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                    ignore_index: int = -100, temperature: float = 1.0, vocab_start: int = 0,
                    group=None, world: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """hidden [N, dim], weight [V(/tp), dim], targets [N] -> (logp [N], entropy [N]) fp32.
    ``logp`` is 0 where ``targets == ignore_index``."""
    if not hidden.is_cuda:
        logits = hidden.float() @ weight.float().t()
        if world > 1:
            from ..parallel import collectives as coll
            logits = coll.gather_last_dim(logits)
        lp, ent, _ = reference.cross_entropy_logprobs(logits, targets, ignore_index, temperature)
        return lp, ent
    return _LinearLogprobs.apply(hidden.contiguous(), weight, targets, ignore_index,
                                 float(temperature), int(vocab_start), group, int(world),
                                 bool(weight.requires_grad))


def linear_cross_entropy(hidden, weight, targets, ignore_index: int = -100, **kw) -> torch.Tensor:
    """Mean token cross-entropy over the non-ignored targets (the SFT loss)."""
    logp, _ = linear_logprobs(hidden, weight, targets, ignore_index, **kw)
    n = (targets != ignore_index).sum().clamp_min(1)
    return -logp.sum() / n
