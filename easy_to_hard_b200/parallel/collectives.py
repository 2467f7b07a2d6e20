"""Explicit tensor- and sequence-parallel region boundaries as autograd functions.

The reference attaches these as module hooks (models/tp.py:297-405, 593-777). Here the model code
calls them directly:

* ``enter_parallel_region(x, sp)``  -- before a column-parallel linear.
    tensor parallel: identity forward, all-reduce of the gradient backward;
    sequence parallel: all-gather along dim 0 forward, reduce-scatter backward.
* ``exit_parallel_region(y, sp)``   -- after a row-parallel linear.
    tensor parallel: all-reduce forward, identity backward;
    sequence parallel: reduce-scatter along dim 0 forward, all-gather backward.

As in the reference, "sequence parallel" shards dim 0 of ``[B, S, D]``: every trainer first
gathers the batch over the tensor-parallel group, so dim 0 holds ``tp`` ranks' samples and each
rank keeps its own between the parallel regions. All functions are no-ops for a group of one.
On CUDA these are the NCCL form of the collectives; the hot paths use the peer-memory kernels
instead where they exist (``parallel.symm`` with ``ops/csrc/tp_reduce.cu``, ``ops/csrc/comm.cu``
and the fused consumers in ``ops/csrc/norm_embed.cu``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import groups


def _tp():
    return groups.get_model_parallel_group(), groups.get_model_parallel_world_size()


def _all_reduce(x: torch.Tensor) -> torch.Tensor:
    group, n = _tp()
    if n == 1:
        return x
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    return x


def _gather_dim0(x: torch.Tensor) -> torch.Tensor:
    group, n = _tp()
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] * n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def _reduce_scatter_dim0(x: torch.Tensor) -> torch.Tensor:
    group, n = _tp()
    if n == 1:
        return x
    assert x.shape[0] % n == 0, "dim 0 must be divisible by the tensor-parallel size"
    x = x.contiguous()
    out = torch.empty((x.shape[0] // n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.device.type == "cpu":  # gloo has no reduce_scatter
        dist.all_reduce(x, group=group)
        out.copy_(x.chunk(n, dim=0)[groups.get_model_parallel_rank()])
    else:
        dist.reduce_scatter_tensor(out, x, group=group)
    return out


def _split_dim0(x: torch.Tensor) -> torch.Tensor:
    _, n = _tp()
    if n == 1:
        return x
    assert x.shape[0] % n == 0
    return x.chunk(n, dim=0)[groups.get_model_parallel_rank()].contiguous()


def _gather_last_dim(x: torch.Tensor) -> torch.Tensor:
    group, n = _tp()
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


def _split_last_dim(x: torch.Tensor) -> torch.Tensor:
    _, n = _tp()
    if n == 1:
        return x
    return x.chunk(n, dim=-1)[groups.get_model_parallel_rank()].contiguous()


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g.clone())


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _all_reduce(x.clone())

    @staticmethod
    def backward(ctx, g):
        return g


class _GatherFromSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tensor_parallel_output_grad):
        ctx.tp_grad = tensor_parallel_output_grad
        return _gather_dim0(x)

    @staticmethod
    def backward(ctx, g):
        # When the consumer is tensor-parallel every rank holds a *partial* gradient, so the
        # backward is a reduce-scatter; when it is replicated (the LM head) a split is enough.
        if ctx.tp_grad:
            return _reduce_scatter_dim0(g), None
        return _split_dim0(g), None


class _ReduceScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _reduce_scatter_dim0(x)

    @staticmethod
    def backward(ctx, g):
        return _gather_dim0(g)


class _ScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _split_dim0(x)

    @staticmethod
    def backward(ctx, g):
        return _gather_dim0(g)


class _SplitLastDim(torch.autograd.Function):
    """Forward: keep this rank's slice of the last dim; backward: all-gather the slices."""

    @staticmethod
    def forward(ctx, x):
        return _split_last_dim(x)

    @staticmethod
    def backward(ctx, g):
        return _gather_last_dim(g)


class _GatherLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _gather_last_dim(x)

    @staticmethod
    def backward(ctx, g):
        return _split_last_dim(g)


def enter_parallel_region(x, sequence_parallel: bool = False):
    if groups.get_model_parallel_world_size() == 1:
        return x
    if sequence_parallel:
        return _GatherFromSP.apply(x, True)
    return _CopyToTP.apply(x) if x.requires_grad else x


def exit_parallel_region(y, sequence_parallel: bool = False):
    if groups.get_model_parallel_world_size() == 1:
        return y
    if sequence_parallel:
        return _ReduceScatterToSP.apply(y)
    return _ReduceFromTP.apply(y)


def scatter_to_sequence_parallel(x):
    return _ScatterToSP.apply(x)


def gather_from_sequence_parallel(x, tensor_parallel_output_grad: bool = True):
    return _GatherFromSP.apply(x, tensor_parallel_output_grad)


def split_last_dim(x):
    return _SplitLastDim.apply(x)


def gather_last_dim(x):
    return _GatherLastDim.apply(x)


def reduce_from_tp(x):
    return _ReduceFromTP.apply(x)


def copy_to_tp(x):
    return _CopyToTP.apply(x)


def vocab_parallel_embedding(idx: torch.Tensor, weight_shard: torch.Tensor) -> torch.Tensor:
    """Embedding lookup with the table sharded over the vocabulary: masked local lookup, then a
    sum over the tensor-parallel group (models/tp.py:85-119 of the reference)."""
    n = groups.get_model_parallel_world_size()
    rows = weight_shard.shape[0]
    start = groups.get_model_parallel_rank() * rows
    outside = (idx < start) | (idx >= start + rows)
    local = (idx - start).masked_fill(outside, 0)
    out = torch.nn.functional.embedding(local, weight_shard)
    out = out.masked_fill(outside.unsqueeze(-1), 0.0)
    return _all_reduce(out) if n > 1 else out
