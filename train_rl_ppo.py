"""PPO entry point: same flags, data formats and checkpoint files as the reference's
``train_rl_ppo.py``.

    torchrun --standalone --nproc_per_node=8 train_rl_ppo.py --do_train \
        --base_checkpoint_path ckpts/llemma-7b-32016/model.pth \
        --policy_checkpoint_path ckpts/sft --reward_checkpoint_path ckpts/prm \
        --source_max_len 256 --target_max_len 512 --rollout_batch_size 512 \
        --step_batch_size 64 --rollout_per_device_batch_size 64 --step_per_device_batch_size 8 \
        --noptepochs 2 --kl_coef 0.01 --gamma 1.0 --lam 0.95 --cliprange 0.2 \
        --temperature 1.0 --ref_policy_model_bits 8 --reward_model_bits 8 \
        --dataset data/ppo_train.json --save_dir ckpts/ppo --tensor_parallel_size 2

Builds the five models (``trainers.ppo_trainer.make_models``), the query data module and the
math-specific reward shaping callbacks, then runs ``PPOTrainer.train`` (train_rl_ppo.py:59-137
of the reference). When ``--resume_from_checkpoint`` is set and ``save_dir`` holds a
``policy_*`` checkpoint, training continues from it.
"""
from __future__ import annotations

from pathlib import Path

import torch
import torch.distributed as dist

from easy_to_hard_b200.data_utils.data_utils_ppo import make_rl_data_module
from easy_to_hard_b200.math_utils.math_rl_utils import (math_stop_token_penalty,
                                                        post_process_math_prm_scores,
                                                        post_process_math_rollouts,
                                                        shape_math_process_rewards)
from easy_to_hard_b200.models.tokenizer_utils import AcceleraTokenizer
from easy_to_hard_b200.parallel import groups
from easy_to_hard_b200.trainers.common_utils import manual_seed
from easy_to_hard_b200.trainers.ppo_trainer import PPOTrainer, make_models
from easy_to_hard_b200.utils.arguments import Arguments as TrainingArguments
from easy_to_hard_b200.utils.checkpoint_utils import get_latest_checkpoint_path
from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser

try:
    import wandb
except ImportError:  # optional
    wandb = None


def main(args: TrainingArguments):
    base = Path(args.base_checkpoint_path)
    tokenizer_path = base.parent / "tokenizer.model"
    if not tokenizer_path.is_file():
        tokenizer_path = base.parent
    device_id = groups.maybe_init_dist(timeout_s=args.dist_timeout_s)
    use_tp = device_id is not None
    if use_tp:
        groups.initialize_model_parallel(args.tensor_parallel_size or dist.get_world_size())
        if args.rollout_tensor_parallel_size:
            groups.initialize_rollout_parallel(args.rollout_tensor_parallel_size)
        dist.barrier()
    elif not groups.model_parallel_is_initialized():
        groups.initialize_model_parallel(1)
    rank0 = device_id in (None, 0)

    checkpoint, _, _ = get_latest_checkpoint_path(args.save_dir, prefix="policy_")
    checkpoint_dir = Path(checkpoint).parent if checkpoint is not None else None
    if use_tp:
        dist.barrier()
    if args.report_to == "wandb" and wandb is not None and rank0:
        wandb.init(name=args.wandb_name, project=args.wandb_project, entity=args.wandb_entity,
                   resume="allow")
        wandb.config.update(vars(args))
    if rank0:
        print("Training from scratch." if checkpoint_dir is None
              else f"Loading from checkpoint: {checkpoint_dir}", flush=True)

    tokenizer = AcceleraTokenizer(tokenizer_path)
    tokenizer.pad_id = tokenizer.unk_id
    manual_seed(args.seed)
    data_module = make_rl_data_module(tokenizer, args)
    if rank0:
        for i in range(min(3, len(data_module["train_dataset"]))):
            print(tokenizer.decode(data_module["train_dataset"][i]["queries"],
                                   skip_special_tokens=True))
            print("=" * 20)
    resume = checkpoint_dir if args.resume_from_checkpoint else None
    models = make_models(tokenizer, args, use_tp=use_tp, resume_from_checkpoint=resume)
    trainer = PPOTrainer(args=args, **data_module, **models, tokenizer=tokenizer,
                         fn_shape_process_rewards=shape_math_process_rewards,
                         fn_post_process_prm_rewards=post_process_math_prm_scores,
                         fn_post_process_rollouts=post_process_math_rollouts,
                         fn_stop_token_penalty=math_stop_token_penalty)
    return trainer.train(resume_training_ckpt=resume)


if __name__ == "__main__":
    parser = HfArgumentParser((TrainingArguments,))
    main(parser.parse_args_into_dataclasses()[0])
