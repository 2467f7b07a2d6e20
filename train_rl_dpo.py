"""Direct preference optimisation entry point: same flags, data formats and checkpoint files as
the reference's ``train_rl_dpo.py``.

    torchrun --standalone --nproc_per_node=8 train_rl_dpo.py --do_train \
        --checkpoint_path ckpts/llemma-7b-32016/model.pth --sft_checkpoint_path ckpts/sft \
        --source_max_len 256 --target_max_len 768 --total_max_len 1024 \
        --per_device_train_batch_size 8 --micro_train_batch_size 2 --learning_rate 2e-6 \
        --dpo_beta 0.1 --dpo_variant dpo --dataset data/pairs.json --save_dir ckpts/dpo

The trained policy runs on the sharded fused engine; the frozen reference policy is a plain bf16
copy (tensor-parallel where the policy is) scored without gradients on the same fused kernels.
Loss variants ``dpo`` (optionally label-smoothed), ``ipo``, ``rpo`` and their ``average`` forms
follow train_rl_dpo.py:77-196 of the reference; gradient clipping at 1.0 and per-step logging of
loss and the three accuracies follow its loop (lines 455-560).
"""
from __future__ import annotations

import torch

from easy_to_hard_b200.data_utils.data_utils_dpo import make_dpo_data_module
from easy_to_hard_b200.trainers import supervised
from easy_to_hard_b200.training import IGNORE_INDEX, dpo_loss
from easy_to_hard_b200.utils.arguments import Arguments as TrainingArguments
from easy_to_hard_b200.utils.checkpoint_utils import load_model_from_from_ckpt
from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser

model_forward_with_loss = dpo_loss


def _load(args, checkpoint_path, sft_checkpoint_path, device, use_tp):
    return load_model_from_from_ckpt(checkpoint_path, sft_checkpoint_path, device,
                                     args.param_dtype, use_tp, requires_grad=True)


def _make_loss(args, checkpoint_path, sft_checkpoint_path, device, use_tp):
    ref_dtype = args.compute_dtype if torch.device(device).type == "cuda" else args.param_dtype
    ref_model = load_model_from_from_ckpt(checkpoint_path, sft_checkpoint_path, device, ref_dtype,
                                          use_tp, requires_grad=False)
    ref_model.eval()

    def loss_fn(model, input_ids_w, labels_w, input_ids_l, labels_l, win_rate_w, win_rate_l):
        return dpo_loss(model, ref_model, input_ids_w, labels_w, input_ids_l, labels_l,
                        win_rate_w, win_rate_l, beta=args.dpo_beta,
                        label_smoothing=args.dpo_label_smoothing, variant=args.dpo_variant)
    return loss_fn


def _prepare(tensors, tokenizer):
    ids_w, lab_w, ids_l, lab_l, wr_w, wr_l = tensors
    pad, unk = tokenizer.pad_id, tokenizer.unk_id
    lab_w = lab_w.masked_fill(lab_w == pad, IGNORE_INDEX)
    lab_l = lab_l.masked_fill(lab_l == pad, IGNORE_INDEX)
    if pad < 0:
        ids_w = ids_w.masked_fill(ids_w == pad, unk)
        ids_l = ids_l.masked_fill(ids_l == pad, unk)
    return ids_w, lab_w, ids_l, lab_l, wr_w, wr_l


TASK = supervised.Task(name="dpo", load_model=_load, make_data_module=make_dpo_data_module,
                       batch_keys=("input_ids_w", "labels_w", "input_ids_l", "labels_l",
                                   "win_rate_w", "win_rate_l"),
                       loss_fn=None, make_loss=_make_loss, prepare=_prepare, max_grad_norm=1.0,
                       log_every=1,
                       metric_keys=("accuracy", "accuracy_policy", "accuracy_reference"),
                       init_from_resume=True, print_keys=("input_ids_w",))


def main(args: TrainingArguments):
    return supervised.run(args, TASK)


if __name__ == "__main__":
    parser = HfArgumentParser((TrainingArguments,))
    main(parser.parse_args_into_dataclasses()[0])
