"""Optimizer / schedule / sharded-model factories used by every trainer
(reference: training_utils/trainer_utils.py:37-151)."""
from __future__ import annotations

import math
from functools import partial

import torch
from torch.optim.lr_scheduler import LambdaLR

from ..parallel import groups
from .memory_efficient_adam import MemoryEfficientAdamW


def create_optimizer(args, model: torch.nn.Module, optimizer_cpu_offload: bool = False,
                     model_cpu_offload: bool = False):
    """Memory-efficient AdamW over the trainable parameters (or, for a sharded-data-parallel
    model, over its flat fp32 master shards)."""
    if hasattr(model, "optimizer_parameters"):
        params = list(model.optimizer_parameters())
    else:
        params = [p for p in model.parameters() if p.requires_grad]
    kw = dict(lr=args.learning_rate, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
              weight_decay=args.weight_decay)
    if model_cpu_offload:
        return torch.optim.AdamW(params, **kw)
    dev = torch.device("cpu") if optimizer_cpu_offload or not torch.cuda.is_available() \
        else torch.device("cuda")
    return MemoryEfficientAdamW(params, optim_dtype=args.optim_dtype, optim_device=dev, **kw)


def create_fsdp_model_for_finetune(args, model: torch.nn.Module, bf16_all_reduce_upper_bound=16):
    """Shard ``model`` over the data-parallel group (ZeRO-3 style): one flat parameter per
    transformer block, gathered in ``compute_dtype`` around its use, gradients reduce-scattered
    (in fp32 once the group has >= ``bf16_all_reduce_upper_bound`` ranks, as in the reference's
    MixedPrecision policy, trainer_utils.py:70-99)."""
    from ..parallel.fsdp import ShardedDataParallel
    dp = groups.get_data_parallel_world_size()
    reduce_dtype = torch.float32 if dp >= bf16_all_reduce_upper_bound else args.compute_dtype
    return ShardedDataParallel(model, process_group=groups.get_data_parallel_group(),
                               param_dtype=args.param_dtype, compute_dtype=args.compute_dtype,
                               reduce_dtype=reduce_dtype,
                               keep_params=bool(getattr(args, "slow_cross_node_comm", False)))


def _cosine_with_warmup(step: int, *, warmup: int, total: int, warmup_start_ratio: float,
                        eta_min_ratio: float) -> float:
    if step < warmup:
        return warmup_start_ratio + (1.0 - warmup_start_ratio) * step / max(1, warmup)
    progress = (step - warmup) / max(1, total - warmup)
    half_cos = max(0.0, 0.5 * (1.0 + math.cos(math.pi * progress)))
    return eta_min_ratio + (1.0 - eta_min_ratio) * half_cos


def get_cosine_schedule_with_warmup(optimizer, warmup_epochs: int, max_epochs: int,
                                    warmup_start_ratio: float = 0.0, eta_min_ratio: float = 0.0,
                                    last_epoch: int = -1):
    """Linear warm-up from ``warmup_start_ratio`` to 1 over ``warmup_epochs`` steps, then half a
    cosine down to ``eta_min_ratio`` at ``max_epochs`` (both ratios are fractions of the base
    learning rate)."""
    assert 0.0 <= warmup_start_ratio <= 1.0 and 0.0 <= eta_min_ratio <= 1.0
    fn = partial(_cosine_with_warmup, warmup=warmup_epochs, total=max_epochs,
                 warmup_start_ratio=warmup_start_ratio, eta_min_ratio=eta_min_ratio)
    return LambdaLR(optimizer, fn, last_epoch)
