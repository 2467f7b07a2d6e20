"""Command-line configuration shared by every trainer.

One flat dataclass, as in the reference (arguments.py:18-645), parsed by ``HfArgumentParser``:
the same flag names and defaults, so the reference's launch lines (examples/README.md) work
unchanged. The fields are declared from a table; ``__post_init__`` turns the dtype strings into
``torch.dtype`` and, for PPO (``--base_checkpoint_path`` given), derives
``rollout_accumulation_steps`` and ``gradient_accumulation_steps`` from the batch arithmetic.
Flags that no code path of the reference reads (``profile``, ``do_predict``, ``num_train_steps``,
``dpo_pm_*``, ``minimal_reasoning_steps``, ``truncate_on_negative_step``) are accepted too;
``profile`` is honoured here (a torch.profiler trace of the first steps).
"""
from __future__ import annotations

import dataclasses
import logging
import os
from pathlib import Path
from typing import Optional

import torch

logger = logging.getLogger(__name__)

_DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}

# (name, type, default, help)
_FIELDS = [
    ('do_train', bool, False, 'whether to run training'),
    ('do_eval', bool, False, 'whether to run eval on the dev set'),
    ('do_test', bool, False, 'whether to run eval on the test set'),
    ('do_predict', bool, False, 'whether to run predictions on the test set'),
    ('source_max_len', int, 1024, 'maximum length of source sequence'),
    ('target_max_len', int, 256, 'maximum length of target sequence'),
    ('total_max_len', int, None, 'maximum length of total sequence'),
    ('dataset', str, 'alpaca', 'which dataset to finetune on'),
    ('eval_dataset', Optional[str], None, 'which dataset to evaluate on'),
    ('test_dataset', Optional[str], None, 'which dataset to test on'),
    ('dataset_format', str, None, 'which dataset format is used'),
    ('add_eos_to_target', bool, False, 'whether to add an EOS token to the target'),
    ('add_eos_to_marked_target', bool, False, 'whether to add an EOS token to the marked target'),
    ('eval_dataset_size', Optional[int], None, 'number of examples to use for evaluation'),
    ('max_eval_samples', Optional[int], None, 'maximum number of samples to evaluate'),
    ('eval_size', int, 0, 'number of examples to use for evaluation'),
    ('num_train_epochs', int, 1, 'number of training epochs'),
    ('learning_rate', float, 0.0001, 'learning rate'),
    ('lr_eta_min', float, 0.0, 'learning rate min in schedule'),
    ('per_device_train_batch_size', int, 4, 'batch size per GPU for training'),
    ('per_device_eval_batch_size', int, None, 'batch size per GPU for evaluation'),
    ('micro_train_batch_size', Optional[int], None, 'micro batch size for training'),
    ('num_train_steps', Optional[int], None, 'number of training steps'),
    ('max_train_samples', Optional[int], None, 'maximum number of samples to train on'),
    ('train_on_source', bool, False, 'whether to train on source'),
    ('train_on_every_token', bool, False, 'whether to train on every token for reward modeling'),
    ('warmup_ratio', float, 0.2, 'linear warmup ratio for learning rate scheduler'),
    ('tensor_parallel_size', Optional[int], None, 'tensor parallel size'),
    ('vocab_parallel', bool, False, 'whether to use vocabulary parallelism'),
    ('sequence_parallel', bool, False, 'whether to use sequence parallelism for activations'),
    ('adam_beta1', float, 0.9, 'adam beta1'),
    ('adam_beta2', float, 0.999, 'adam beta2'),
    ('adam_eps', float, 1e-08, 'adam epsilon'),
    ('weight_decay', float, 0.0, 'weight decay'),
    ('optimizer_cpu_offload', bool, False, 'whether to offload optimizer states to CPU during fine-tuning'),
    ('reward_head_init_scheme', str, 'zeros', 'whether to initialize the reward head with zeros'),
    ('process_reward_with_answer', bool, False, 'whether to apply process reward with answer'),
    ('dpo_variant', str, 'dpo', 'which variant of DPO to use'),
    ('dpo_beta', float, 0.1, 'beta for DPO'),
    ('dpo_label_smoothing', float, 0.0, 'label smoothing for DPO'),
    ('dpo_pm_checkpoint_path', Optional[Path], None, 'path to the preference model checkpoint to load'),
    ('dpo_pm_total_max_len', Optional[int], None, 'maximum length of total sequence for preference model'),
    ('param_dtype', str, 'bf16', 'parameter datatype for mixed precision training'),
    ('compute_dtype', str, 'bf16', 'reduce operation datatype for mixed precision training'),
    ('optim_dtype', Optional[str], None, 'optimizer state datatype for mixed precision training'),
    ('checkpoint_path', Optional[Path], None, 'path to the checkpoint to load'),
    ('sft_checkpoint_path', Optional[Path], None, 'path to the sft checkpoint to load'),
    ('rm_checkpoint_path', Optional[Path], None, 'path to the reward model checkpoint to load'),
    ('save_strategy', str, 'no', 'the checkpoint save strategy to use'),
    ('save_dir', Optional[Path], None, 'directory to save checkpoints to'),
    ('save_steps', Optional[int], None, 'save checkpoint every X steps'),
    ('eval_steps', Optional[int], None, 'evaluate every X steps'),
    ('resume_from_checkpoint', bool, False, 'whether to resume from checkpoint'),
    ('save_total_limit', int, 1, 'maximum number of checkpoints to save'),
    ('save_only_model', bool, False, 'whether to only save the model'),
    ('report_to', str, 'none', 'to use wandb or something else for reporting'),
    ('wandb_name', Optional[str], None, 'name of the wandb run'),
    ('wandb_project', Optional[str], None, 'name of the wandb project'),
    ('wandb_entity', Optional[str], None, 'name of the wandb entity'),
    ('compile', bool, False, 'compile the model forward function'),
    ('profile', Optional[Path], None, 'profile the model forward function and save the results to the given path'),
    ('seed', int, 42, 'random seed'),
    ('print_training_examples', bool, False, 'whether to print training examples'),
    ('temperature', float, 1.0, 'temperature for rollout in PPO'),
    ('gradient_accumulation_steps', Optional[int], None, 'how many gradients to accumulate before to perform an optimizer step'),
    ('rollout_accumulation_steps', Optional[int], None, 'how many rollouts to accumulate before PPO update'),
    ('noptepochs', int, 2, 'number of epochs in a single PPO update'),
    ('max_grad_norm', float, 1.0, 'maximum gradient norm for clipping'),
    ('policy_model_fsdp', bool, False, 'whether to use Fully Sharded Data Parallelism for policy'),
    ('policy_model_cpu_offload', bool, False, 'whether to offload policy (params, grads, optim_states) to CPU'),
    ('policy_optimizer_cpu_offload', bool, False, 'whether to offload policy optimizer states to CPU'),
    ('value_model_fsdp', bool, False, 'whether to use Fully Sharded Data Parallelism for value'),
    ('value_model_cpu_offload', bool, False, 'whether to offload value (params, grads, optim_states) to CPU'),
    ('value_optimizer_cpu_offload', bool, False, 'whether to offload value optimizer states to CPU'),
    ('reward_model_fsdp', bool, False, 'whether to use Fully Sharded Data Parallelism for reward'),
    ('reward_model_cpu_offload', bool, False, 'whether to offload reward (params, grads, optim_states) to CPU'),
    ('reward_model_bits', int, 16, 'number of bits for reward model quantization'),
    ('ref_policy_model_fsdp', bool, False, 'whether to use Fully Sharded Data Parallelism for ref policy'),
    ('ref_policy_model_cpu_offload', bool, False, 'whether to offload ref policy (params, grads, optim_states) to CPU'),
    ('ref_policy_model_bits', int, 16, 'number of bits for ref policy model quantization'),
    ('ppo_warmup_steps', int, 5, 'number of warmup steps for PPO'),
    ('rollout_batch_size', int, 32, 'batch size for rollouts'),
    ('rollout_per_device_batch_size', int, 1, 'per device batch size for rollouts'),
    ('reward_model_per_device_batch_size', int, None, 'reward model per device batch size'),
    ('step_batch_size', int, 32, 'batch size for gradient updates'),
    ('step_per_device_batch_size', int, 1, 'per device batch size for gradient updates'),
    ('penalize_no_stop_token', bool, False, 'whether to penalize sequences that do not contain stop_token'),
    ('penalty_reward_value', float, -1.0, 'reward assigned to sequences that are truncated, e.g., due to outputting incomplete sentences for given context window'),
    ('relative_stop_token_penalty', bool, False, 'whether to penalize sequences that do not contain stop_token with a relative penalty based on the original reward'),
    ('maxent_normalization', str, 'full', 'normalization for maxent regularization'),
    ('maxent_coef', float, 0.0, 'maxent coef'),
    ('ent_reg_coef', float, 0.0, 'ent reg coef'),
    ('kl_coef', float, 0.2, 'kl coef'),
    ('kl_approximator', str, 'k1', 'kl approximator'),
    ('whiten_rewards', bool, True, 'whiten rewards'),
    ('whitening_async_stats', str, 'per_gpu', 'how to sync statistics for advantage whitening'),
    ('vf_coef', float, 0.1, 'vf coef'),
    ('cliprange', float, 0.2, 'cliprange'),
    ('cliprange_value', float, 0.2, 'cliprange value'),
    ('gamma', float, 1.0, 'gamma'),
    ('lam', float, 1.0, 'lam'),
    ('stop_token', Optional[str], None, 'token to stop generation with'),
    ('min_seq_len', int, 0, 'minimum sequence length for reward modeling'),
    ('min_seq_len_coef', float, 0.0, 'coefficient for penalizing too short sequences'),
    ('base_checkpoint_path', Path, Path('Undefined'), 'path to the policy base model to load'),
    ('reward_base_checkpoint_path', Optional[Path], None, 'path to the reward base model to load'),
    ('value_base_checkpoint_path', Optional[Path], None, 'path to the value base model to load'),
    ('policy_checkpoint_path', Path, Path('Undefined'), 'path to the sft model to load'),
    ('reward_checkpoint_path', Path, Path('Undefined'), 'path to the reward model to load'),
    ('value_checkpoint_path', Optional[Path], None, 'path to the value model to load'),
    ('init_value_with_reward', bool, True, 'initialize the value model with the reward model'),
    ('outcome_reward', bool, False, 'whether to use outcome reward'),
    ('easy_outcome_reward', bool, False, 'whether to use outcome reward on easy problems'),
    ('fsdp_consolidate_cpu_offload', bool, False, 'whether to offload FSDP consolidation to CPU'),
    ('apply_process_reward', bool, False, 'whether to apply process reward in PPO'),
    ('apply_terminal_process_reward', bool, False, 'whether to apply aggregated process reward in PPO'),
    ('process_reward_upper_bound', float, 1.0, 'upper bound for process reward'),
    ('process_reward_scale', float, 1.0, 'scale for process reward'),
    ('process_reward_scheme', str, 'min', 'how to compute process reward'),
    ('minimal_reasoning_steps', Optional[int], None, 'number of minimal reasoning steps'),
    ('truncate_on_negative_step', bool, False, 'whether to truncate on negative step'),
    ('slow_cross_node_comm', bool, False, 'whether to optimize for cross-node communication'),
]
# extensions of this framework (not flags of the reference)
_FIELDS += [
    ("rollout_top_k", int, 50, "top-k used when sampling PPO rollouts (hard-coded to 50 upstream)"),
    ("rollout_tensor_parallel_size", Optional[int], None,
     "tensor-parallel degree of the rollout engine when it differs from training"),
    ("dist_timeout_s", float, 1800.0, "process-group timeout; a hung peer ends the job with an error"),
]


def _post_init(self) -> None:
    for key in ("param_dtype", "compute_dtype"):
        val = getattr(self, key)
        if isinstance(val, str):
            if val not in _DTYPES:
                raise ValueError(f"Unknown {key}: {val}")
            setattr(self, key, _DTYPES[val])
    if self.optim_dtype is None:
        self.optim_dtype = self.param_dtype
    elif isinstance(self.optim_dtype, str):
        if self.optim_dtype not in _DTYPES:
            raise ValueError(f"Unknown optim_dtype: {self.optim_dtype}")
        self.optim_dtype = _DTYPES[self.optim_dtype]
    if Path(self.base_checkpoint_path).name == "Undefined":
        return
    # PPO batch arithmetic
    world = int(os.environ.get("WORLD_SIZE", 1))
    quiet = int(os.environ.get("LOCAL_RANK", 0)) != 0
    for total, per in (("rollout_batch_size", "rollout_per_device_batch_size"),
                       ("step_batch_size", "step_per_device_batch_size")):
        t, p = getattr(self, total), getattr(self, per)
        if t < p * world or t % (p * world) != 0:
            raise AssertionError(
                f"{total}={t} must be a positive multiple of {per} * world_size = {p * world}")
    self.rollout_accumulation_steps = (
        self.rollout_batch_size // self.rollout_per_device_batch_size // world)
    self.gradient_accumulation_steps = (
        self.step_batch_size // self.step_per_device_batch_size // world)
    if not quiet:
        logger.warning(
            "PPO batches: rollout %d = %d/device x %d ranks x %d accumulation; "
            "step %d = %d/device x %d ranks x %d accumulation",
            self.rollout_batch_size, self.rollout_per_device_batch_size, world,
            self.rollout_accumulation_steps, self.step_batch_size,
            self.step_per_device_batch_size, world, self.gradient_accumulation_steps)


Arguments = dataclasses.make_dataclass(
    "Arguments",
    [(n, t, dataclasses.field(default=d, metadata={"help": h})) for n, t, d, h in _FIELDS],
    namespace={"__post_init__": _post_init, "__module__": __name__},
)
Arguments.__doc__ = "All flags of train_sft / train_rm_* / train_rl_* (see module docstring)."
