"""Pairwise (outcome) reward-model training entry point: same flags, data formats and checkpoint
files as the reference's ``train_rm_pairwise.py``.

    torchrun --standalone --nproc_per_node=8 train_rm_pairwise.py --do_train \
        --checkpoint_path ckpts/llemma-7b-32016/model.pth --sft_checkpoint_path ckpts/sft \
        --total_max_len 1024 --per_device_train_batch_size 8 --micro_train_batch_size 4 \
        --learning_rate 1e-5 --num_train_epochs 1 --dataset data/pairs.json \
        --save_strategy epoch --save_dir ckpts/orm --tensor_parallel_size 2

Each example holds two candidate sequences and a ``choice``; the loss is BCE on the reward
difference at the last non-pad token, gradients are clipped to 5.0 and loss / accuracy are
logged every step (train_rm_pairwise.py:80-128, 398, 407-440 of the reference).
"""
from __future__ import annotations

from easy_to_hard_b200.data_utils.data_utils_rm_pairwise import (
    make_pairwise_reward_modeling_data_module)
from easy_to_hard_b200.trainers import supervised
from easy_to_hard_b200.training import pairwise_reward_loss, reward_modeling_metrics
from easy_to_hard_b200.utils.arguments import Arguments as TrainingArguments
from easy_to_hard_b200.utils.checkpoint_utils import load_reward_model_from_sft_ckpt
from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser

model_forward_with_loss = pairwise_reward_loss
compute_reward_modeling_metrics = reward_modeling_metrics


def _load(args, checkpoint_path, sft_checkpoint_path, device, use_tp):
    return load_reward_model_from_sft_ckpt(checkpoint_path, sft_checkpoint_path, device,
                                           args.param_dtype, use_tp, requires_grad=True,
                                           sequence_parallel=args.sequence_parallel)


def _prepare(tensors, tokenizer):
    input_ids, choice = tensors
    if tokenizer.pad_id < 0:
        input_ids = input_ids.masked_fill(input_ids == tokenizer.pad_id, tokenizer.unk_id)
    return input_ids, choice


TASK = supervised.Task(name="rm_pairwise", load_model=_load,
                       make_data_module=make_pairwise_reward_modeling_data_module,
                       batch_keys=("input_ids", "choice"), loss_fn=pairwise_reward_loss,
                       prepare=_prepare, max_grad_norm=5.0, log_every=1,
                       metric_keys=("accuracy",), init_from_resume=True)


def main(args: TrainingArguments):
    return supervised.run(args, TASK)


if __name__ == "__main__":
    parser = HfArgumentParser((TrainingArguments,))
    main(parser.parse_args_into_dataclasses()[0])
