"""One transformer block as an explicit forward / backward over the sm_100a kernels.

The reference trains through ``torch.utils.checkpoint`` around ``TransformerBlock``
(models/model.py:233-243): only the block input is kept and the block is re-run in the
backward pass. ``block_forward`` / ``block_backward`` are that recomputation written out as a
fixed sequence of fused kernels (tcgen05 GEMMs with residual / SwiGLU epilogues, flash
attention forward and backward, RMSNorm, RoPE), with the tensor-parallel collectives at the
same places as ``parallel.collectives``:

    x ── rmsnorm ─[gather]─ wqkv ─ rope ─ flash ─ wo ─[reduce]─ (+x) = h
    h ── rmsnorm ─[gather]─ w1,w3 ─ swiglu ─ w2 ─[reduce]─ (+h) = out

Activations are token-major ``[B*S, features]`` bf16. Weight gradients are written straight
into caller-provided buffers (bf16 ``[out, in]`` views of a flat gradient buffer), which is what
lets the sharded-data-parallel wrapper reduce-scatter a whole block's gradients in one go.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import flash, functional as Fn, gemm
from ..parallel import groups


@dataclass
class BlockShape:
    B: int
    S: int
    n_head: int      # local (per tensor-parallel rank) query heads
    n_kv: int        # local kv heads
    head_dim: int
    eps: float
    tp: int = 1
    sequence_parallel: bool = False


def _tp_all_reduce(t: torch.Tensor, shape: BlockShape) -> torch.Tensor:
    if shape.tp > 1:
        dist.all_reduce(t, group=groups.get_model_parallel_group())
    return t


def _sp_gather(t: torch.Tensor, shape: BlockShape) -> torch.Tensor:
    """[T/tp, F] -> [T, F] along tokens (sequence parallel)."""
    out = torch.empty(t.shape[0] * shape.tp, t.shape[1], dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=groups.get_model_parallel_group())
    return out


def _sp_reduce_scatter(t: torch.Tensor, shape: BlockShape) -> torch.Tensor:
    out = torch.empty(t.shape[0] // shape.tp, t.shape[1], dtype=t.dtype, device=t.device)
    dist.reduce_scatter_tensor(out, t.contiguous(), group=groups.get_model_parallel_group())
    return out


_ROW_REDUCE: Dict[tuple, object] = {}
_SP_SYNC: Dict[tuple, object] = {}
_P2P_REDUCE = {"enabled": None}

# call sites of the sequence-parallel collectives of one block (parallel.symm.SequenceParallelSync)
_PT_ENTRY, _PT_WO, _PT_W2, _PT_DY, _PT_DXN2, _PT_DH, _PT_DXN1 = range(7)


def _sp_sync(T: int, dim: int):
    """Symmetric buffers of the fused sequence-parallel collectives for T tokens per
    tensor-parallel group, one set per shape, created by every rank of the group at the same
    point of its first forward."""
    key = (T, dim)
    sp = _SP_SYNC.get(key)
    if sp is None:
        from ..parallel.symm import SequenceParallelSync
        sp = SequenceParallelSync(T, dim, 8, groups.get_model_parallel_group())
        _SP_SYNC[key] = sp
    return sp


def _row_parallel_sp(sync, point: int, x_in: torch.Tensor, w: torch.Tensor, T: int):
    """Row-parallel GEMM into the next partial slot of ``sync``; its last CTA raises the flag of
    ``point`` on every rank. Returns the slot for the consuming collective."""
    slot, part = sync.next_partial(T)
    gemm.linear(x_in, w, out=part, signal=sync.signal_ptrs(point),
                ticket=sync.gemm_ticket[point:point + 1])
    return slot


def p2p_reduce_enabled(group=None) -> bool:
    """The fused collectives over peer memory are used when symmetric memory is available and
    every rank of ``group`` (default: the tensor-parallel group) is on this host; groups that
    span hosts, and ``E2H_TP_REDUCE=nccl``, take the NCCL collectives. Collective on first use
    per group."""
    if _P2P_REDUCE["enabled"] is None:
        import os
        _P2P_REDUCE["enabled"] = os.environ.get("E2H_TP_REDUCE", "p2p") != "nccl"
    if not _P2P_REDUCE["enabled"]:
        return False
    from ..parallel.symm import peer_memory_usable
    return peer_memory_usable(group if group is not None else groups.get_model_parallel_group())


def _row_reduce(T: int, dim: int):
    """Symmetric partial-sum buffers for T tokens (two alternating slots), one set per shape.
    Every rank of the tensor-parallel group creates it at the same point of its first forward."""
    key = (T, dim)
    rp = _ROW_REDUCE.get(key)
    if rp is None:
        from ..ops import _lib
        from ..parallel.symm import RowParallelReduce
        rp = RowParallelReduce(T, dim, groups.get_model_parallel_group(), dtype=torch.bfloat16)
        # training ranks drift apart (data loading, first-use initialisation) by seconds
        from ..parallel.symm import peer_wait_ms
        _lib.check(_lib.lib().e2h_set_flag_wait_ms(peer_wait_ms()), "set_flag_wait_ms")
        _ROW_REDUCE[key] = rp
    return rp


def _row_parallel_fused(x_in: torch.Tensor, w: torch.Tensor, residual: torch.Tensor,
                        norm_w: Optional[torch.Tensor], eps: float):
    """residual + sum over ranks of (x_in @ w^T), and optionally its RMSNorm, without NCCL: the
    GEMM writes this rank's fp32 partial into symmetric memory and raises a flag on every peer
    when its grid has finished; the consumer kernel waits (bounded) for all flags and sums the
    partials straight out of the peers' memory. The partials are bf16 (the GEMM's TMA-store
    epilogue writes them), summed in fp32."""
    T, dim = residual.shape
    rp = _row_reduce(T, dim)
    s = rp.slot()
    gemm.linear(x_in, w, out=rp.partial_out(s, T), signal=rp.signal_ptrs(s),
                ticket=rp.gemm_ticket[s:s + 1])
    h = torch.empty_like(residual)
    xn = torch.empty_like(residual) if norm_w is not None else None
    Fn.reduce_residual_norm_bf16(residual, norm_w, eps, partials=rp.partial_ptrs(s), h_out=h,
                                 x_out=xn, flags=rp.flags(s), use_count=rp.use_count[s:s + 1],
                                 ticket=rp.norm_ticket[s:s + 1])
    return h, xn


def block_forward(x: torch.Tensor, w: Dict[str, torch.Tensor], freqs: torch.Tensor,
                  pos: torch.Tensor, shape: BlockShape, keep: bool = False):
    """x [T, dim] (T = B*S, or B*S/tp rows under sequence parallelism). ``w`` holds bf16
    ``wqkv, wo, w1, w3, w2`` and the two norm weights. Returns ``out`` and, with ``keep``, the
    intermediates the backward needs."""
    H, Hkv, D = shape.n_head, shape.n_kv, shape.head_dim
    sp = shape.sequence_parallel and shape.tp > 1
    fused_sp = sp and p2p_reduce_enabled()
    if fused_sp:
        # rmsnorm of this rank's rows and the all-gather in one kernel over peer memory
        T = x.shape[0] * shape.tp
        sync = _sp_sync(T, x.shape[1])
        xn1f = sync.gather(_PT_ENTRY, x, T, w["attention_norm"], shape.eps)
        if keep:
            xn1f = xn1f.clone()      # the gather buffer is reused by the next collective
    else:
        xn1 = Fn.rmsnorm(x, w["attention_norm"], shape.eps)
        xn1f = _sp_gather(xn1, shape) if sp else xn1
    T = xn1f.shape[0]
    qkv = gemm.linear(xn1f, w["wqkv"])
    Fn.rope(qkv, freqs, pos, H + Hkv, D, out=qkv)          # q and k heads, in place
    q = qkv[:, : H * D].view(shape.B, shape.S, H, D)
    k = qkv[:, H * D: (H + Hkv) * D].view(shape.B, shape.S, Hkv, D)
    v = qkv[:, (H + Hkv) * D:].view(shape.B, shape.S, Hkv, D)
    o, lse = flash.flash_fwd(q, k, v, None, return_lse=True)
    o2 = o.view(T, H * D)
    fused_reduce = shape.tp > 1 and not sp and p2p_reduce_enabled()
    xn2f = None
    if shape.tp == 1:
        h = gemm.linear_residual(o2, w["wo"], x)
        xn2 = Fn.rmsnorm(h, w["ffn_norm"], shape.eps)
    elif fused_sp:
        # reduce-scatter + residual + RMSNorm + all-gather as the consumer of the wo GEMM
        slot = _row_parallel_sp(sync, _PT_WO, o2, w["wo"], T)
        h, xn2f = sync.reduce_norm_gather(_PT_WO, slot, x, w["ffn_norm"], shape.eps, T)
        if keep:
            xn2f = xn2f.clone()
    elif fused_reduce:
        h, xn2 = _row_parallel_fused(o2, w["wo"], x, w["ffn_norm"], shape.eps)
    else:
        part = gemm.linear(o2, w["wo"])
        part = _sp_reduce_scatter(part, shape) if sp else _tp_all_reduce(part, shape)
        h = part.add_(x)
        xn2 = Fn.rmsnorm(h, w["ffn_norm"], shape.eps)
    if xn2f is None:
        xn2f = _sp_gather(xn2, shape) if sp else xn2
    g, u = gemm.linear_dual(xn2f, w["w1"], w["w3"])
    act = Fn.swiglu(g, u)
    if shape.tp == 1:
        out = gemm.linear_residual(act, w["w2"], h)
    elif fused_sp:
        slot = _row_parallel_sp(sync, _PT_W2, act, w["w2"], T)
        out = sync.reduce(_PT_W2, slot, h, T)
    elif fused_reduce:
        out, _ = _row_parallel_fused(act, w["w2"], h, None, shape.eps)
    else:
        part = gemm.linear(act, w["w2"])
        part = _sp_reduce_scatter(part, shape) if sp else _tp_all_reduce(part, shape)
        out = part.add_(h)
    if not keep:
        return out, None
    return out, dict(xn1f=xn1f, qkv=qkv, q=q, k=k, v=v, o=o, lse=lse, h=h, xn2f=xn2f, g=g, u=u,
                     act=act)


def block_backward(dy: torch.Tensor, x: torch.Tensor, w: Dict[str, torch.Tensor],
                   grads: Dict[str, torch.Tensor], freqs: torch.Tensor, pos: torch.Tensor,
                   shape: BlockShape, accumulate: bool = False,
                   saved: Optional[Dict[str, torch.Tensor]] = None) -> torch.Tensor:
    """Back-propagate ``dy`` through the block. The intermediates come from ``saved`` (what
    ``block_forward(..., keep=True)`` returned for the same input; ``act`` may be left out and is
    then rebuilt from ``g`` and ``u``) or, without it, from re-running the block on its input
    ``x``. Weight gradients go to ``grads[name]`` (``[out, in]`` bf16 or fp32; added to when
    ``accumulate``). Returns dx."""
    H, Hkv, D = shape.n_head, shape.n_kv, shape.head_dim
    sp = shape.sequence_parallel and shape.tp > 1
    if saved is None:
        _, a = block_forward(x, w, freqs, pos, shape, keep=True)
    else:
        a = dict(saved)
        if "act" not in a:
            a["act"] = Fn.swiglu(a["g"], a["u"])
    T = a["xn1f"].shape[0]

    def wgrad(name, d_out, inp):
        gemm.linear_wgrad(d_out, inp, out=grads[name], accumulate=accumulate)

    fused_sp = sp and p2p_reduce_enabled()
    sync = _sp_sync(T, x.shape[1]) if fused_sp else None

    def dgrad_reduce(point, make_partial):
        """Sum of the ranks' input-gradient partials: all-reduce (tensor parallel) or
        reduce-scatter to this rank's rows (sequence parallel, fused: the dgrad GEMMs write
        into a symmetric partial slot and the consumer kernel pulls this rank's rows)."""
        if fused_sp:
            slot, part = sync.next_partial(T)
            make_partial(part, sync.signal_ptrs(point), sync.gemm_ticket[point:point + 1])
            return sync.reduce(point, slot, None, T)
        part = make_partial(None, None, None)
        if shape.tp > 1:
            part = _sp_reduce_scatter(part, shape) if sp else _tp_all_reduce(part, shape)
        return part

    # ---- feed-forward: out = h + w2(act) ----
    if fused_sp:
        dyf = sync.gather(_PT_DY, dy.contiguous(), T)
    else:
        dyf = _sp_gather(dy, shape) if sp else dy
    d_act = gemm.linear_dgrad(dyf, w["w2"])
    wgrad("w2", dyf, a["act"])
    dg, du = Fn.swiglu_bwd(a["g"], a["u"], d_act)

    def d_xn2_partial(out, signal, ticket):
        out = gemm.linear_dgrad(dg, w["w1"], out=out)
        kw = dict(signal=signal, ticket=ticket) if signal else {}
        gemm.gemm(w["w3"], du, epi=gemm.EPI_RESIDUAL, out=out, aux=out, a_mn_major=True, **kw)
        return out

    d_xn2 = dgrad_reduce(_PT_DXN2, d_xn2_partial)
    wgrad("w1", dg, a["xn2f"])
    wgrad("w3", du, a["xn2f"])
    dh = Fn.rmsnorm_bwd(a["h"], d_xn2, w["ffn_norm"], shape.eps, dres=dy)
    # ---- attention: h = x + wo(o) ----
    if fused_sp:
        dhf = sync.gather(_PT_DH, dh, T)
    else:
        dhf = _sp_gather(dh, shape) if sp else dh
    d_o = gemm.linear_dgrad(dhf, w["wo"])
    wgrad("wo", dhf, a["o"].view(T, H * D))
    dqkv = torch.empty_like(a["qkv"])   # dq | dk | dv written in place by the attention backward
    flash.flash_bwd(a["q"], a["k"], a["v"], a["o"], d_o.view(shape.B, shape.S, H, D), a["lse"],
                    dq=dqkv[:, : H * D].view(shape.B, shape.S, H, D),
                    dk=dqkv[:, H * D: (H + Hkv) * D].view(shape.B, shape.S, Hkv, D),
                    dv=dqkv[:, (H + Hkv) * D:].view(shape.B, shape.S, Hkv, D))
    Fn.rope(dqkv, freqs, pos, H + Hkv, D, inverse=True, out=dqkv)
    def d_xn1_partial(out, signal, ticket):
        kw = dict(signal=signal, ticket=ticket) if signal else {}
        return gemm.linear_dgrad(dqkv, w["wqkv"], out=out, **kw)

    d_xn1 = dgrad_reduce(_PT_DXN1, d_xn1_partial)
    wgrad("wqkv", dqkv, a["xn1f"])
    return Fn.rmsnorm_bwd(x, d_xn1, w["attention_norm"], shape.eps, dres=dh)


def dense_weight(linear) -> torch.Tensor:
    """The [out, in] weight of a linear module as the GEMM kernels read it. An int8 weight-only
    module (``weight`` int8 + per-row ``scales``) is dequantised to bf16 on the fly: one extra
    pass over the weight, which scoring passes over thousands of tokens do not notice."""
    w = linear.weight
    if w.dtype == torch.int8 and hasattr(linear, "scales"):
        return (w.to(torch.bfloat16) * linear.scales.to(torch.bfloat16)[:, None]).contiguous()
    return w


def block_weights(blk) -> Dict[str, torch.Tensor]:
    a, f = blk.attention, blk.feed_forward
    return dict(wqkv=dense_weight(a.wqkv), wo=dense_weight(a.wo), w1=dense_weight(f.w1),
                w3=dense_weight(f.w3), w2=dense_weight(f.w2),
                attention_norm=blk.attention_norm.weight, ffn_norm=blk.ffn_norm.weight)


def can_fuse(model, idx: torch.Tensor) -> bool:
    """The cache-less fused forward applies to a CUDA model whose norms are bf16 and whose
    linears are plain bf16 or int8 weight-only modules."""
    if not idx.is_cuda or not len(model.layers):
        return False
    blk = model.layers[0]
    if blk.attention_norm.weight.dtype != torch.bfloat16:
        return False
    for lin in (blk.attention.wqkv, blk.attention.wo, blk.feed_forward.w1, blk.feed_forward.w3,
                blk.feed_forward.w2):
        w = getattr(lin, "weight", None)
        if not isinstance(w, torch.Tensor) or w.dim() != 2:
            return False
        if not (w.dtype == torch.bfloat16 or (w.dtype == torch.int8 and hasattr(lin, "scales"))):
            return False
    return True


@torch.no_grad()
def transformer_hidden(model, idx: torch.Tensor, final_norm: bool = True) -> torch.Tensor:
    """Fully-causal forward of the whole stack without a KV cache (scoring, log-probs of given
    sequences): token ids [B, S] -> final-norm hidden states [B, S, dim] bf16 (the residual
    stream before the final norm with ``final_norm=False``, for heads that fuse the norm). Right
    padding is harmless under the causal mask; the caller ignores padded positions."""
    B, S = idx.shape
    if model.freqs_cis is None or model.max_seq_length < S or model.max_batch_size < B:
        model.setup_caches(B, S, kv_cache=False)
    att = model.layers[0].attention
    shape = BlockShape(B, S, att.n_head, att.n_local_heads, att.head_dim, model.config.norm_eps,
                       tp=getattr(att, "tp_size", 1), sequence_parallel=False)
    pos = torch.arange(S, device=idx.device, dtype=torch.int32).repeat(B)
    x = model.embed(idx).to(torch.bfloat16).reshape(B * S, -1)
    for blk in model.layers:
        x, _ = block_forward(x, block_weights(blk), model.freqs_cis, pos, shape)
    if final_norm:
        x = Fn.rmsnorm(x, model.norm.weight.to(torch.bfloat16), model.config.norm_eps)
    return x.view(B, S, -1)
