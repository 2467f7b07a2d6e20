"""Supervised fine-tuning entry point (same flags, data formats and checkpoint files as the
reference's ``train_sft.py``).

    torchrun --standalone --nproc_per_node=8 train_sft.py --do_train \
        --checkpoint_path ckpts/llemma-7b-32016/model.pth --source_max_len 768 \
        --target_max_len 768 --total_max_len 768 --per_device_train_batch_size 16 \
        --micro_train_batch_size 8 --learning_rate 2e-5 --num_train_epochs 3 \
        --dataset data/train.json --dataset_format metamath --save_strategy epoch \
        --save_dir ckpts/sft --tensor_parallel_size 1 --param_dtype fp32 --optim_dtype fp32

The loop itself lives in ``easy_to_hard_b200.trainers.supervised``; this script supplies the SFT
task: policy loader, SFT data module, next-token cross-entropy on the response tokens
(train_sft.py:72-116 of the reference) through the fused LM-head loss.
"""
from __future__ import annotations

from easy_to_hard_b200.data_utils.data_utils_sft import make_sft_data_module
from easy_to_hard_b200.trainers import supervised
from easy_to_hard_b200.training import IGNORE_INDEX, model_forward_with_loss, prepare_batch
from easy_to_hard_b200.utils.arguments import Arguments as TrainingArguments
from easy_to_hard_b200.utils.checkpoint_utils import load_model_from_from_ckpt
from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser

__all__ = ["main", "model_forward_with_loss", "prepare_batch", "IGNORE_INDEX"]


def _load(args, checkpoint_path, sft_checkpoint_path, device, use_tp):
    return load_model_from_from_ckpt(checkpoint_path, sft_checkpoint_path, device,
                                     args.param_dtype, use_tp, requires_grad=True,
                                     sequence_parallel=args.sequence_parallel,
                                     vocab_parallel=args.vocab_parallel)


def _prepare(tensors, tokenizer):
    input_ids, labels = tensors
    return prepare_batch(input_ids, labels, tokenizer.pad_id, tokenizer.unk_id, use_tp=False)


TASK = supervised.Task(name="sft", load_model=_load, make_data_module=make_sft_data_module,
                       batch_keys=("input_ids", "labels"), loss_fn=model_forward_with_loss,
                       prepare=_prepare, max_grad_norm=1.0, log_every=5,
                       print_keys=("input_ids", "labels"))


def main(args: TrainingArguments):
    return supervised.run(args, TASK)


if __name__ == "__main__":
    parser = HfArgumentParser((TrainingArguments,))
    main(parser.parse_args_into_dataclasses()[0])
