"""The loop shared by the supervised entry points (SFT, pointwise / pairwise reward modelling,
DPO). The reference repeats this loop in each script (train_sft.py:123-422,
train_rm_pointwise.py:123-446, train_rm_pairwise.py:157-476, train_rl_dpo.py); here each script
only supplies a ``Task``: how to load its model and data, which batch tensors it consumes, how
they are prepared and what the loss is.

The model is always wrapped in the sharded-data-parallel engine (a data-parallel group of one
included): that wrapper runs the fused sm_100a block kernels with fp32 master weights and bf16
compute copies. ``--compile`` is accepted and ignored.
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, DistributedSampler

from ..models.model import set_global_compile_mode
from ..models.tokenizer_utils import AcceleraTokenizer
from ..parallel import groups
from ..parallel.health import HealthMonitor, guarded_step
from ..training import TrainStepper, gather_tp_batch
from ..utils.checkpoint_utils import checkpoint_hook, get_latest_checkpoint_path, load_checkpoint
from ..utils.trainer_utils import (create_fsdp_model_for_finetune, create_optimizer,
                                   get_cosine_schedule_with_warmup)
from .common_utils import manual_seed

try:
    import wandb
except ImportError:  # optional
    wandb = None


@dataclass
class Task:
    name: str
    load_model: Callable            # (args, checkpoint_path, init_path, device, use_tp) -> model
    make_data_module: Callable      # (tokenizer, args) -> {train_dataset, data_collator, ...}
    batch_keys: Sequence[str]       # collated tensors handed to prepare / loss_fn, in order
    loss_fn: Callable               # (model, *tensors) -> loss | (loss, metrics)
    prepare: Optional[Callable] = None   # (tensors, tokenizer) -> tensors, before TP pooling
    max_grad_norm: float = 1.0
    log_every: int = 5
    metric_keys: Sequence[str] = field(default_factory=tuple)
    init_from_resume: bool = False  # skip the warm-start checkpoint when resuming (RM trainers)
    print_keys: Sequence[str] = ("input_ids",)
    # (args, checkpoint_path, init_path, device, use_tp) -> loss_fn, for losses that need more
    # state than the trained model (DPO's frozen reference policy)
    make_loss: Optional[Callable] = None


def _log(rank0: bool, *a):
    if rank0:
        print(*a, flush=True)


def run(args, task: Task) -> Dict:
    """Train ``task`` under ``args``; returns the last logged record (for tests)."""
    checkpoint_path = Path(args.checkpoint_path)
    assert checkpoint_path.is_file(), checkpoint_path
    init_path = args.sft_checkpoint_path
    if init_path is not None:
        assert Path(init_path).is_dir(), init_path
    tokenizer_path = checkpoint_path.parent / "tokenizer.model"
    if not tokenizer_path.is_file():
        tokenizer_path = checkpoint_path.parent
    set_global_compile_mode(args.compile)

    device_id = groups.maybe_init_dist(timeout_s=args.dist_timeout_s)
    use_tp = device_id is not None
    rank0 = (not use_tp) or dist.get_rank() == 0
    if use_tp:
        groups.initialize_model_parallel(args.tensor_parallel_size or dist.get_world_size())
        dist.barrier()
    elif not groups.model_parallel_is_initialized():
        groups.initialize_model_parallel(1)
    world = dist.get_world_size() if use_tp else 1
    device = "cuda" if torch.cuda.is_available() else "cpu"

    if args.report_to == "wandb" and wandb is not None and rank0:
        wandb.init(name=args.wandb_name, project=args.wandb_project, entity=args.wandb_entity,
                   resume="allow")
        wandb.config.update(vars(args))

    resume_path, resume_epoch, resume_global_step = None, 0, 0
    if args.resume_from_checkpoint:
        resume_path, resume_epoch, resume_global_step = get_latest_checkpoint_path(args.save_dir)
    if resume_path is not None and task.init_from_resume:
        init_path = None

    _log(rank0, "Loading model ...")
    t0 = time.time()
    model = task.load_model(args, checkpoint_path, init_path, device, use_tp)
    if use_tp:
        dist.barrier()
    _log(rank0, f"Time to load model: {time.time() - t0:.02f} seconds")

    tokenizer = AcceleraTokenizer(tokenizer_path)
    data_module = task.make_data_module(tokenizer=tokenizer, args=args)
    train_dataset, collator = data_module["train_dataset"], data_module["data_collator"]
    size = sum(p.numel() * p.element_size()
               for p in itertools.chain(model.parameters(), model.buffers()))
    _log(rank0, f"Model size: {size / 1e6:.02f} MB")
    manual_seed(args.seed)

    sampler = DistributedSampler(train_dataset, shuffle=True, drop_last=True) if use_tp else None
    loader = DataLoader(train_dataset, batch_size=args.per_device_train_batch_size,
                        shuffle=sampler is None, sampler=sampler, num_workers=0,
                        pin_memory=torch.cuda.is_available(), collate_fn=collator)
    if args.print_training_examples and rank0:
        for batch in itertools.islice(loader, 16):
            for k in task.print_keys:
                row = batch[k][0]
                row = row.reshape(-1, row.shape[-1])[0] if row.dim() > 1 else row
                print(f"{k}:", tokenizer.decode(row.tolist(), skip_special_tokens=False))

    trainable_param_names = [n for n, p in model.named_parameters() if p.requires_grad]
    model = create_fsdp_model_for_finetune(args, model)
    model.train()
    use_fsdp = True
    _log(rank0, f"Sharded data parallel over {groups.get_data_parallel_world_size()} rank(s), "
                f"tensor parallel over {groups.get_model_parallel_world_size()}")

    optimizer = create_optimizer(args, model=model,
                                 optimizer_cpu_offload=args.optimizer_cpu_offload,
                                 model_cpu_offload=False)
    scheduler = get_cosine_schedule_with_warmup(
        optimizer, warmup_epochs=len(loader) * args.warmup_ratio,
        max_epochs=len(loader) * args.num_train_epochs, warmup_start_ratio=0.0,
        eta_min_ratio=args.lr_eta_min / args.learning_rate)
    if resume_path is not None:
        _log(rank0, f"Resuming from checkpoint: {resume_path} (epoch {resume_epoch}, "
                    f"global step {resume_global_step})")
        load_checkpoint(resume_path, model, optimizer, scheduler, use_fsdp=use_fsdp)
    else:
        resume_global_step = 0

    micro = args.micro_train_batch_size or args.per_device_train_batch_size
    assert args.per_device_train_batch_size % micro == 0, (
        f"per_device_train_batch_size ({args.per_device_train_batch_size}) must be divisible by "
        f"micro_train_batch_size ({micro})")
    _log(rank0, f"Batch size per GPU for training: {args.per_device_train_batch_size}\n",
         f"Micro batch size for training: {micro}\n",
         f"Gradient accumulation steps: {args.per_device_train_batch_size // micro}\n")
    # after pooling, a tensor-parallel group holds the concatenation of its ranks' batches
    micro_global = micro * groups.get_model_parallel_world_size()

    loss_fn = (task.make_loss(args, checkpoint_path, init_path, device, use_tp)
               if task.make_loss is not None else task.loss_fn)
    stepper = TrainStepper(model, optimizer, scheduler, loss_fn, task.max_grad_norm)
    monitor = HealthMonitor(dist.get_rank(), world).start() if use_tp else None
    epoch_length = len(loader)
    record: Dict = {}
    if not args.do_train:
        return record
    _log(rank0, "Starting training ...")
    t0 = time.time()
    from ..utils.tracing import StepProfiler
    profiler = StepProfiler(getattr(args, "profile", None))   # --profile: trace of a few steps
    try:
        for epoch in range(args.num_train_epochs):
            if sampler is not None:
                sampler.set_epoch(epoch)
            for it, batch in enumerate(loader):
                global_step = epoch * epoch_length + it
                if global_step < resume_global_step:
                    continue
                tensors = tuple(batch[k].to(device=device, non_blocking=True)
                                for k in task.batch_keys)
                if task.prepare is not None:
                    tensors = task.prepare(tensors, tokenizer)
                tensors = gather_tp_batch(tensors, use_tp)
                profiler.step()
                loss, grad_norm = guarded_step(monitor, stepper.step, *tensors,
                                               micro_batch_size=micro_global)
                if it % task.log_every == 0:
                    vals = [loss.detach().float().reshape(1)]
                    for k in task.metric_keys:
                        vals.append(torch.as_tensor(stepper.metrics[k], dtype=torch.float32,
                                                    device=loss.device).reshape(1))
                    packed = torch.cat(vals)
                    if use_tp:
                        dist.all_reduce(packed)
                    packed = (packed / world).tolist()
                    record = {"loss": packed[0]}
                    record.update({k: v for k, v in zip(task.metric_keys, packed[1:])})
                    record.update({"learning_rate": scheduler.get_last_lr()[0], "epoch": epoch,
                                   "step": it, "grad_norm": float(grad_norm)})
                    if rank0:
                        if args.report_to == "wandb" and wandb is not None:
                            wandb.log(record, step=global_step)
                        else:
                            print(record, flush=True)
                checkpoint_hook(args, model, optimizer, scheduler, epoch, global_step,
                                epoch_length, use_fsdp=use_fsdp,
                                trainable_param_names=trainable_param_names)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        epoch = args.num_train_epochs
        checkpoint_hook(args, model, optimizer, scheduler, epoch, epoch * epoch_length,
                        epoch_length, use_fsdp=use_fsdp,
                        trainable_param_names=trainable_param_names)
    finally:
        profiler.close()
        if monitor is not None:
            monitor.stop()
    _log(rank0, f"Time to train: {time.time() - t0:.02f} seconds")
    return record
