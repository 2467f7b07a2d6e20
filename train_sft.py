"""Supervised fine-tuning entry point (same flags, data formats and checkpoint files as the
reference's ``train_sft.py``).

    torchrun --standalone --nproc_per_node=8 train_sft.py --do_train \
        --checkpoint_path ckpts/llemma-7b-32016/model.pth --source_max_len 768 \
        --target_max_len 768 --total_max_len 768 --per_device_train_batch_size 16 \
        --micro_train_batch_size 8 --learning_rate 2e-5 --num_train_epochs 3 \
        --dataset data/train.json --dataset_format metamath --save_strategy epoch \
        --save_dir ckpts/sft --tensor_parallel_size 1 --param_dtype fp32 --optim_dtype fp32

Differences from the reference loop (train_sft.py:123-422), all behind the same flags:
the model is always wrapped in the sharded-data-parallel engine (a group of one rank included),
because that wrapper is what runs the fused sm_100a block kernels with fp32 master weights and
bf16 compute copies; the loss is the fused LM-head cross-entropy; gradient clipping keeps its
coefficient on the device; ``--compile`` is accepted and ignored (there is no tracing compiler
in the hot path).
"""
from __future__ import annotations

import itertools
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, DistributedSampler

from easy_to_hard_b200.data_utils.data_utils_sft import make_sft_data_module
from easy_to_hard_b200.models.model import set_global_compile_mode
from easy_to_hard_b200.models.tokenizer_utils import AcceleraTokenizer
from easy_to_hard_b200.models.tp import (get_data_parallel_rank, get_data_parallel_world_size,
                                         get_model_parallel_group, initialize_model_parallel,
                                         maybe_init_dist)
from easy_to_hard_b200.trainers.common_utils import manual_seed
from easy_to_hard_b200.training import (IGNORE_INDEX, SFTStepper, model_forward_with_loss,
                                        prepare_batch)
from easy_to_hard_b200.utils.arguments import Arguments as TrainingArguments
from easy_to_hard_b200.utils.checkpoint_utils import (checkpoint_hook, get_latest_checkpoint_path,
                                                      load_checkpoint, load_model_from_from_ckpt)
from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser
from easy_to_hard_b200.utils.trainer_utils import (create_fsdp_model_for_finetune,
                                                   create_optimizer,
                                                   get_cosine_schedule_with_warmup)

try:
    import wandb
except ImportError:  # optional
    wandb = None

__all__ = ["main", "model_forward_with_loss", "prepare_batch", "IGNORE_INDEX"]


def _log(rank0: bool, *a):
    if rank0:
        print(*a, flush=True)


def main(args: TrainingArguments) -> None:
    checkpoint_path = Path(args.checkpoint_path)
    assert checkpoint_path.is_file(), checkpoint_path
    sft_checkpoint_path = args.sft_checkpoint_path
    if sft_checkpoint_path is not None:
        assert Path(sft_checkpoint_path).is_dir(), sft_checkpoint_path
    tokenizer_path = checkpoint_path.parent / "tokenizer.model"
    if not tokenizer_path.is_file():
        tokenizer_path = checkpoint_path.parent
    set_global_compile_mode(args.compile)

    device_id = maybe_init_dist()
    use_tp = device_id is not None
    rank0 = (not use_tp) or dist.get_rank() == 0
    if use_tp:
        initialize_model_parallel(args.tensor_parallel_size or dist.get_world_size())
        dist.barrier()
    world = dist.get_world_size() if use_tp else 1
    device = "cuda" if torch.cuda.is_available() else "cpu"

    if args.report_to == "wandb" and wandb is not None and rank0:
        wandb.init(name=args.wandb_name, project=args.wandb_project, entity=args.wandb_entity,
                   resume="allow")
        wandb.config.update(vars(args))

    _log(rank0, "Loading model ...")
    t0 = time.time()
    model = load_model_from_from_ckpt(checkpoint_path, sft_checkpoint_path, device,
                                      args.param_dtype, use_tp, requires_grad=True,
                                      sequence_parallel=args.sequence_parallel,
                                      vocab_parallel=args.vocab_parallel)
    _log(rank0, f"Time to load model: {time.time() - t0:.02f} seconds")

    tokenizer = AcceleraTokenizer(tokenizer_path)
    data_module = make_sft_data_module(tokenizer=tokenizer, args=args)
    train_dataset, data_collator = data_module["train_dataset"], data_module["data_collator"]
    size = sum(p.numel() * p.element_size()
               for p in itertools.chain(model.parameters(), model.buffers()))
    _log(rank0, f"Model size: {size / 1e6:.02f} MB")
    manual_seed(args.seed)

    sampler = DistributedSampler(train_dataset, shuffle=True, drop_last=True) if use_tp else None
    train_loader = DataLoader(train_dataset, batch_size=args.per_device_train_batch_size,
                              shuffle=sampler is None, sampler=sampler, num_workers=0,
                              pin_memory=torch.cuda.is_available(), collate_fn=data_collator)

    if args.print_training_examples and rank0:
        for batch in itertools.islice(train_loader, 16):
            print("Input:", tokenizer.decode(batch["input_ids"][0].tolist(),
                                             skip_special_tokens=False))
            print("Target:", tokenizer.decode(batch["labels"][0].tolist(),
                                              skip_special_tokens=False))

    trainable_param_names = [n for n, p in model.named_parameters() if p.requires_grad]
    model = create_fsdp_model_for_finetune(args, model)
    model.train()
    use_fsdp = True
    _log(rank0, f"Sharded data parallel over {get_data_parallel_world_size()} rank(s)")

    optimizer = create_optimizer(args, model=model,
                                 optimizer_cpu_offload=args.optimizer_cpu_offload,
                                 model_cpu_offload=False)
    scheduler = get_cosine_schedule_with_warmup(
        optimizer, warmup_epochs=len(train_loader) * args.warmup_ratio,
        max_epochs=len(train_loader) * args.num_train_epochs, warmup_start_ratio=0.0,
        eta_min_ratio=args.lr_eta_min / args.learning_rate)

    resume_global_step = 0
    if args.resume_from_checkpoint:
        path, resume_epoch, resume_global_step = get_latest_checkpoint_path(args.save_dir)
        if path is not None:
            _log(rank0, f"Resuming from checkpoint: {path} (epoch {resume_epoch}, "
                        f"global step {resume_global_step})")
            load_checkpoint(path, model, optimizer, scheduler, use_fsdp=use_fsdp)
        else:
            resume_global_step = 0

    micro = args.micro_train_batch_size or args.per_device_train_batch_size
    assert args.per_device_train_batch_size % micro == 0, (
        f"per_device_train_batch_size ({args.per_device_train_batch_size}) must be divisible by "
        f"micro_train_batch_size ({micro})")
    _log(rank0, f"Batch size per GPU for training: {args.per_device_train_batch_size}\n",
         f"Micro batch size for training: {micro}\n",
         f"Gradient accumulation steps: {args.per_device_train_batch_size // micro}\n")
    # after prepare_batch a tensor-parallel group holds the concatenation of its ranks' batches
    from easy_to_hard_b200.parallel import groups
    micro_global = micro * groups.get_model_parallel_world_size()

    stepper = SFTStepper(model, optimizer, scheduler, max_grad_norm=1.0)
    epoch_length = len(train_loader)
    if not args.do_train:
        return
    _log(rank0, "Starting training ...")
    t0 = time.time()
    for epoch in range(args.num_train_epochs):
        if sampler is not None:
            sampler.set_epoch(epoch)
        for it, batch in enumerate(train_loader):
            global_step = epoch * epoch_length + it
            if global_step < resume_global_step:
                continue
            input_ids = batch["input_ids"].to(device=device, non_blocking=True)
            labels = batch["labels"].to(device=device, non_blocking=True)
            input_ids, labels = prepare_batch(input_ids, labels, tokenizer.pad_id,
                                              tokenizer.unk_id, use_tp,
                                              get_model_parallel_group() if use_tp else None)
            loss, grad_norm = stepper.step(input_ids, labels, micro_global)
            if it % 5 == 0:
                avg = loss.detach().clone().float()
                if use_tp:
                    dist.all_reduce(avg)
                record = {"loss": avg.item() / world,
                          "learning_rate": scheduler.get_last_lr()[0], "epoch": epoch,
                          "step": it, "grad_norm": float(grad_norm)}
                if rank0:
                    if args.report_to == "wandb" and wandb is not None:
                        wandb.log(record, step=global_step)
                    else:
                        print(record, flush=True)
            checkpoint_hook(args, model, optimizer, scheduler, epoch, global_step, epoch_length,
                            use_fsdp=use_fsdp, trainable_param_names=trainable_param_names)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    epoch = args.num_train_epochs
    checkpoint_hook(args, model, optimizer, scheduler, epoch, epoch * epoch_length, epoch_length,
                    use_fsdp=use_fsdp, trainable_param_names=trainable_param_names)
    _log(rank0, f"Time to train: {time.time() - t0:.02f} seconds")


if __name__ == "__main__":
    parser = HfArgumentParser((TrainingArguments,))
    main(parser.parse_args_into_dataclasses()[0])
