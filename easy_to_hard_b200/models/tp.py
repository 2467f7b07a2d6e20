"""Tensor / sequence / vocab parallel sharding of a ``Transformer`` and the parallel losses.

Public surface of the reference's ``models/tp.py``: process-group helpers (re-exported from
``parallel.groups``), ``apply_tp``, ``apply_reward_head_tp``, ``clip_grad_norm_``,
``vocab_parallel_cross_entropy``, ``compute_vocab_parallel_logprobs``.

Sharding rules (models/tp.py:122-286 of the reference): ``wqkv`` is column-sharded separately
inside its q, k and v row segments so every rank owns whole heads; ``wo`` and ``w2`` are
row-sharded; ``w1``/``w3`` column-sharded; weight-only quantized linears shard their packed weight
and their scales consistently. Collectives are not hooks: ``apply_tp`` only sets ``tp_size`` /
``sequence_parallel`` on the modules and the forward code calls ``parallel.collectives``.

The vocab-parallel path (sharded embedding + LM head, sharded cross-entropy, sharded sampling) is
live here; in the reference it is unreachable because ``Transformer.vocab_parallel`` is forced to
False (models/model.py:170).
"""
from __future__ import annotations

import math
from typing import List, Optional, Union

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..parallel import collectives as coll
from ..parallel.groups import (  # noqa: F401  (re-exported API)
    barrier, get_data_parallel_group, get_data_parallel_rank, get_data_parallel_src_rank,
    get_data_parallel_world_size, get_model_parallel_group, get_model_parallel_rank,
    get_model_parallel_src_rank, get_model_parallel_world_size, initialize_model_parallel,
    maybe_init_dist, model_parallel_is_initialized, destroy_model_parallel)
from ..parallel import groups


def _shard(x: torch.Tensor, dim: int, world: int, rank: int) -> torch.Tensor:
    assert x.size(dim) % world == 0, f"dim {dim} of size {x.size(dim)} not divisible by {world}"
    return torch.tensor_split(x, world, dim=dim)[rank].contiguous()


def _shard_segments(x: torch.Tensor, dim: int, splits: List[int], world: int, rank: int):
    return torch.cat([_shard(seg, dim, world, rank) for seg in x.split(splits, dim=dim)], dim=dim)


def _set_weight(mod: nn.Module, name: str, value: torch.Tensor, requires_grad: bool) -> None:
    old = getattr(mod, name)
    if isinstance(old, nn.Parameter):
        setattr(mod, name, nn.Parameter(value, requires_grad=requires_grad))
    else:
        mod.register_buffer(name, value)


def shard_linear(linear: nn.Module, style: str, weight_splits: Optional[List[int]] = None,
                 requires_grad: bool = False, world: Optional[int] = None,
                 rank: Optional[int] = None) -> None:
    """Shard one (possibly weight-only-quantized) linear in place. ``style`` is "colwise"
    (split output features) or "rowwise" (split input features)."""
    from .quantize import WeightOnlyInt4Linear

    world = groups.get_model_parallel_world_size() if world is None else world
    rank = groups.get_model_parallel_rank() if rank is None else rank
    dim, attr = {"colwise": (0, "out_features"), "rowwise": (1, "in_features")}[style]
    assert getattr(linear, attr) % world == 0
    is_int4 = isinstance(linear, WeightOnlyInt4Linear)

    def cut(t, d, splits=None):
        if splits:
            return _shard_segments(t, d, splits, world, rank)
        return _shard(t, d, world, rank)

    if is_int4:
        # packed weight [N/8, K/(ikt*16), 32, ikt/2]; scales_and_zeros [K/g, N, 2]
        w_splits = [s // 8 for s in weight_splits] if weight_splits else None
        weight = cut(linear.weight, dim, w_splits)
        linear.register_buffer("scales_and_zeros",
                               cut(linear.scales_and_zeros, 1 - dim, weight_splits))
    else:
        weight = cut(linear.weight, dim, weight_splits)
    if hasattr(linear, "scales") and style == "colwise":
        linear.register_buffer("scales", cut(linear.scales, 0, weight_splits))
    _set_weight(linear, "weight", weight, requires_grad)
    setattr(linear, attr, getattr(linear, attr) // world)


def pad_int4_ffn_for_tp(ffn: nn.Module, world: int) -> bool:
    """Widen the intermediate dimension of a weight-only int4 feed-forward so that ``w2``'s packed
    K tiles and (scale, zero) groups divide evenly over ``world`` ranks. The reference asserts
    divisibility instead (models/tp.py:143-145, 171-181), which rules out int4 at TP 4 and 8
    for the 7B / 13B FFN widths (11008 = 86 groups of 128). The added features carry code 0 with
    scale 0 and zero 0, i.e. weights that dequantise to exactly 0: ``w1`` / ``w3`` produce 0 for
    them, ``silu(0) * 0 = 0``, and ``w2`` multiplies that by 0, so the function of the layer is
    unchanged. This is an extension of this framework, applied to the in-memory model only; the
    checkpoint format is not touched. Returns True when anything was padded."""
    from .quantize import WeightOnlyInt4Linear
    w1, w2, w3 = ffn.w1, ffn.w2, ffn.w3
    if not all(isinstance(m, WeightOnlyInt4Linear) for m in (w1, w2, w3)):
        return False
    unit = math.lcm(w2.inner_k_tiles * 16, w2.groupsize, 8) * world
    k_old = w2.in_features
    k_new = -(-k_old // unit) * unit
    if k_new == k_old:
        return False
    assert w1.out_features == w3.out_features and w1.out_features <= k_old
    for m in (w1, w3):     # more output features: rows of the packed weight, columns of the qparams
        n_new = k_new - (k_old - m.out_features)
        m.register_buffer("weight", F.pad(m.weight, (0, 0, 0, 0, 0, 0, 0, n_new // 8 - m.weight.shape[0])))
        m.register_buffer("scales_and_zeros",
                          F.pad(m.scales_and_zeros, (0, 0, 0, n_new - m.scales_and_zeros.shape[1])))
        m.out_features = n_new
    kt = w2.inner_k_tiles * 16
    w2.register_buffer("weight", F.pad(w2.weight, (0, 0, 0, 0, 0, k_new // kt - w2.weight.shape[1])))
    w2.register_buffer("scales_and_zeros",
                       F.pad(w2.scales_and_zeros,
                             (0, 0, 0, 0, 0, k_new // w2.groupsize - w2.scales_and_zeros.shape[0])))
    if getattr(w2, "padding", False):
        # the checkpoint's own padding already added zero inputs after origin_in_features
        w2.origin_in_features = k_new - (k_old - w2.origin_in_features)
    w2.in_features = k_new
    return True


def apply_tp(model, requires_grad: bool = False, sequence_parallel: bool = False,
             world: Optional[int] = None, rank: Optional[int] = None, group=None) -> None:
    """Shard ``model`` over the tensor-parallel group in place. ``world`` / ``rank`` / ``group``
    name another group than the job's tensor-parallel one (the rollout copy of a PPO policy that
    generates at a wider tensor-parallel degree than it trains at); the model then carries
    ``tp_group`` / ``tp_rank`` for the decode engine."""
    explicit = world is not None
    world = groups.get_model_parallel_world_size() if world is None else world
    if world <= 1:
        return
    rank = groups.get_model_parallel_rank() if rank is None else rank
    if explicit:
        model.tp_group, model.tp_rank = group, rank
    cfg = model.config
    assert cfg.n_head % world == 0 and cfg.n_local_heads % world == 0
    model.tp_size = world
    model.sequence_parallel = bool(sequence_parallel)
    for blk in model.layers:
        att, ffn = blk.attention, blk.feed_forward
        kv = att.n_local_heads * att.head_dim
        shard_linear(att.wqkv, "colwise", [att.n_head * att.head_dim, kv, kv], requires_grad,
                     world, rank)
        shard_linear(att.wo, "rowwise", None, requires_grad, world, rank)
        att.n_head //= world
        att.n_local_heads //= world
        att.dim //= world
        pad_int4_ffn_for_tp(ffn, world)
        for name, style in (("w1", "colwise"), ("w3", "colwise"), ("w2", "rowwise")):
            shard_linear(getattr(ffn, name), style, None, requires_grad, world, rank)
        for m in (att, ffn):
            m.tp_size, m.sequence_parallel = world, bool(sequence_parallel)
    if model.vocab_parallel:
        assert cfg.vocab_size % world == 0, "vocab-parallel needs vocab divisible by tp"
        emb = model.tok_embeddings
        _set_weight(emb, "weight", _shard(emb.weight, 0, world, rank), False)
        per = cfg.vocab_size // world
        if hasattr(emb, "vocab_start_index"):
            emb.vocab_start_index, emb.vocab_end_index = None, None  # handled by model.embed
        emb.num_embeddings = per
        shard_linear(model.output, "colwise", None, requires_grad, world, rank)
    # the KV cache and attention shapes follow the per-rank head count
    cfg.n_head //= world
    cfg.n_local_heads //= world
    cfg.dim //= world


def apply_reward_head_tp(model: nn.Module, requires_grad: bool = False) -> None:
    """Row-shard the ``[2, dim]`` reward head; its input is split on the last dim and the
    partial scores are summed over the group (models/tp.py:289-294 of the reference)."""
    world = groups.get_model_parallel_world_size()
    if world <= 1:
        return
    shard_linear(model.output, "rowwise", None, requires_grad)
    model.output.tp_row_parallel = True


def reward_head_forward(head: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """Apply a (possibly row-sharded) reward head to replicated hidden states."""
    if getattr(head, "tp_row_parallel", False):
        x = coll.split_last_dim(x)
        return coll.reduce_from_tp(torch.nn.functional.linear(x, head.weight))
    return torch.nn.functional.linear(x, head.weight)


@torch.no_grad()
def clip_grad_norm_(module_or_params, max_norm: Union[float, int],
                    norm_type: Union[float, int] = 2.0, process_group=None) -> torch.Tensor:
    """Global gradient-norm clipping over parameters that are all sharded (tensor-parallel
    and/or data-parallel shards), so the per-rank partial norms add up over the WORLD group
    (models/tp.py:780-885 of the reference; replicated tensors are frozen buffers there, and
    here too). Sharded-optimizer wrappers expose ``grad_shards()`` for their flat shards."""
    if hasattr(module_or_params, "grad_shards"):
        grads = list(module_or_params.grad_shards())
    else:
        params = (module_or_params.parameters() if isinstance(module_or_params, nn.Module)
                  else module_or_params)
        grads = [p.grad for p in params if p.grad is not None]
    max_norm, norm_type = float(max_norm), float(norm_type)
    dev = grads[0].device if grads else torch.device(
        "cuda" if torch.cuda.is_available() else "cpu")
    if norm_type == math.inf:
        total = torch.stack([g.detach().abs().max().float() for g in grads]).max() if grads \
            else torch.zeros((), device=dev)
        if dist.is_initialized():
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=process_group)
    else:
        total = torch.zeros((), device=dev, dtype=torch.float32)
        for g in grads:
            total += torch.linalg.vector_norm(g.detach().float(), norm_type) ** norm_type
        if dist.is_initialized():
            dist.all_reduce(total, group=process_group)
        total = total ** (1.0 / norm_type)
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for g in grads:
        g.mul_(coef.to(g.device, g.dtype))
    return total


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """-log softmax(logits)[target] with the vocabulary dimension sharded over the TP group.
    One fused exchange of (max, target-logit, sum-exp) per token instead of the reference's
    three separate all-reduces (models/tp.py:888-969)."""

    @staticmethod
    def forward(ctx, logits_shard: torch.Tensor, target: torch.Tensor):
        group = groups.get_model_parallel_group()
        world = groups.get_model_parallel_world_size()
        lf = logits_shard.float()
        per = lf.shape[-1]
        start = groups.get_model_parallel_rank() * per
        local_max = lf.max(dim=-1).values
        gmax = local_max.clone()
        if world > 1:
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
        shifted = lf - gmax.unsqueeze(-1)
        outside = (target < start) | (target >= start + per)
        local_t = (target - start).masked_fill(outside, 0)
        picked = shifted.gather(-1, local_t.unsqueeze(-1)).squeeze(-1).masked_fill(outside, 0.0)
        exp = shifted.exp()
        packed = torch.stack([picked, exp.sum(-1)], dim=0)
        if world > 1:
            dist.all_reduce(packed, group=group)
        picked, sumexp = packed[0], packed[1]
        loss = torch.log(sumexp) - picked
        exp.div_(sumexp.unsqueeze(-1))
        ctx.save_for_backward(exp, outside, local_t)
        ctx.in_dtype = logits_shard.dtype
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        softmax, outside, local_t = ctx.saved_tensors
        grad = softmax.clone()
        g2 = grad.view(-1, grad.shape[-1])
        rows = torch.arange(g2.shape[0], device=g2.device)
        g2[rows, local_t.view(-1)] -= (~outside).view(-1).float()
        grad.mul_(grad_out.unsqueeze(-1))
        return grad.to(ctx.in_dtype), None


def vocab_parallel_cross_entropy(vocab_parallel_logits: torch.Tensor,
                                 target: torch.Tensor) -> torch.Tensor:
    return _VocabParallelCrossEntropy.apply(vocab_parallel_logits, target)


def compute_vocab_parallel_logprobs(logits: torch.Tensor, labels: torch.Tensor,
                                    ignore_index: int, reduction: str = "none") -> torch.Tensor:
    """Per-token log-probs of ``labels`` (0 where ignored) from vocab-sharded logits."""
    ignore = labels == ignore_index
    scores = -vocab_parallel_cross_entropy(logits, labels.masked_fill(ignore, 0))
    scores = scores.masked_fill(ignore, 0.0)
    if reduction == "none":
        return scores
    if reduction == "mean":
        return scores.sum() / (ignore.numel() - ignore.sum()).clamp_min(1)
    if reduction == "sum":
        return scores.sum()
    raise ValueError(f"Invalid reduction: {reduction}")


def get_sharding_rank_info():
    return dict(tp_rank=get_model_parallel_rank(), tp_size=get_model_parallel_world_size(),
                dp_rank=get_data_parallel_rank(), dp_size=get_data_parallel_world_size())
