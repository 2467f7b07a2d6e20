"""Pointwise (process) reward-model training entry point: same flags, data formats and
checkpoint files as the reference's ``train_rm_pointwise.py``.

    torchrun --standalone --nproc_per_node=8 train_rm_pointwise.py --do_train \
        --checkpoint_path ckpts/llemma-7b-32016/model.pth --sft_checkpoint_path ckpts/sft \
        --total_max_len 1024 --per_device_train_batch_size 8 --micro_train_batch_size 4 \
        --learning_rate 2e-5 --num_train_epochs 2 --dataset data/prm_train.json \
        --dataset_format prm-v2 --save_strategy epoch --save_dir ckpts/prm \
        --tensor_parallel_size 2 --param_dtype fp32 --optim_dtype fp32

The model is the policy backbone with a 2-row head whose mean is the per-token reward; the loss
is weighted BCE at the step-delimiter positions (train_rm_pointwise.py:78-112 of the reference).
When resuming, the warm start from the SFT checkpoint is skipped (same file, 183-198).
"""
from __future__ import annotations

from easy_to_hard_b200.data_utils.data_utils_rm_pointwise import (
    make_pointwise_reward_modeling_data_module)
from easy_to_hard_b200.trainers import supervised
from easy_to_hard_b200.training import IGNORE_INDEX, pointwise_reward_loss
from easy_to_hard_b200.utils.arguments import Arguments as TrainingArguments
from easy_to_hard_b200.utils.checkpoint_utils import load_reward_model_from_sft_ckpt
from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser

model_forward_with_loss = pointwise_reward_loss


def _load(args, checkpoint_path, sft_checkpoint_path, device, use_tp):
    return load_reward_model_from_sft_ckpt(checkpoint_path, sft_checkpoint_path, device,
                                           args.param_dtype, use_tp, requires_grad=True,
                                           sequence_parallel=args.sequence_parallel)


def _prepare(tensors, tokenizer):
    input_ids, labels, weights = tensors
    labels = labels.masked_fill(labels == tokenizer.pad_id, IGNORE_INDEX)
    if tokenizer.pad_id < 0:
        input_ids = input_ids.masked_fill(input_ids == tokenizer.pad_id, tokenizer.unk_id)
    return input_ids, labels, weights


TASK = supervised.Task(name="rm_pointwise", load_model=_load,
                       make_data_module=make_pointwise_reward_modeling_data_module,
                       batch_keys=("input_ids", "labels", "weights"),
                       loss_fn=pointwise_reward_loss, prepare=_prepare, max_grad_norm=1.0,
                       log_every=5, init_from_resume=True)


def main(args: TrainingArguments):
    return supervised.run(args, TASK)


if __name__ == "__main__":
    parser = HfArgumentParser((TrainingArguments,))
    main(parser.parse_args_into_dataclasses()[0])
