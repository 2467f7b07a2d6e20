"""Rollout-based RL training loop shared by the PPO trainer (reference: trainers/rl_trainer.py).

One step = sample ``rollout_accumulation_steps`` query batches, roll them out with the current
policy, (optionally) evaluate and save, then run ``noptepochs`` passes of policy and value
updates over the fixed rollouts, step the schedulers, record statistics and update the KL
controller -- the order of rl_trainer.py:285-332 of the reference.

Policy and value networks are ``parallel.fsdp.ShardedDataParallel`` models (fp32 master shards,
bf16 compute copies, fused block kernels); gradient accumulation simply leaves the
reduce-scattered gradients in the shards until the optimizer step, so the reference's
``no_sync`` bookkeeping has no counterpart.
"""
from __future__ import annotations

import abc
import gc
import logging
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, Dataset, DistributedSampler, TensorDataset

from ..models import tp as tp_mod
from ..parallel import groups
from ..parallel.fsdp import ShardedDataParallel
from ..training import GradClipper
from ..utils import trainer_utils
from . import common_utils as utils

logger = logging.getLogger(__name__)

FIRST_STEP_IDX = 1


class KLController(abc.ABC):
    value: float

    def step(self, *args, **kwargs):
        pass


class FixedKLController(KLController):
    def __init__(self, kl_coef: float):
        self.value = kl_coef


class RLTrainer:
    def __init__(self, args, train_dataset: Dataset, data_collator: Callable, tokenizer, policy,
                 eval_dataset: Optional[Dataset] = None, test_dataset: Optional[Dataset] = None,
                 value_model=None, ref_policy=None, reward_model=None, policy_optimizer=None,
                 value_optimizer=None, policy_lr_scheduler=None, value_lr_scheduler=None,
                 reward_tokenizer=None, unwrapped_policy=None):
        self.args = args
        self.train_dataset, self.eval_dataset, self.test_dataset = (train_dataset, eval_dataset,
                                                                    test_dataset)
        self.data_collator = data_collator
        self.policy, self.value_model = policy, value_model
        self.ref_policy, self.reward_model = ref_policy, reward_model
        self.unwrapped_policy = unwrapped_policy
        self.tokenizer = tokenizer
        self.reward_tokenizer = reward_tokenizer if reward_tokenizer is not None else tokenizer
        self.policy_optimizer, self.value_optimizer = policy_optimizer, value_optimizer
        self.policy_lr_scheduler, self.value_lr_scheduler = (policy_lr_scheduler,
                                                             value_lr_scheduler)
        self.kl_ctl = FixedKLController(kl_coef=args.kl_coef)
        self.log_history: List[Dict] = []
        self.best_metrics: Optional[Dict] = None
        self._clippers: Dict[int, GradClipper] = {}

    # ------------------------------------------------------------------ to be provided
    @abc.abstractmethod
    def rollout(self, queries_data) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    @abc.abstractmethod
    def compute_policy_loss(self, rollouts: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, Dict]:
        raise NotImplementedError

    @abc.abstractmethod
    def compute_value_loss(self, rollouts: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, Dict]:
        raise NotImplementedError

    @abc.abstractmethod
    def record_step_stats(self, train_stats, rollouts, step_idx, **kwargs):
        raise NotImplementedError

    @abc.abstractmethod
    def evaluate(self, step_idx: int, temperature: float = 0.0):
        raise NotImplementedError

    @abc.abstractmethod
    def save_model(self, step_idx: int, metrics: Optional[Dict] = None):
        raise NotImplementedError

    @abc.abstractmethod
    def resume_training(self, checkpoint_dir: str) -> int:
        raise NotImplementedError

    # ------------------------------------------------------------------ optimisation
    def _clip_and_step(self, model, optimizer) -> torch.Tensor:
        """Finish the backward of a sharded model, clip the global gradient norm (coefficient
        kept on the device when the fused optimizer can consume it) and step."""
        max_norm = self.args.max_grad_norm
        sharded = isinstance(model, ShardedDataParallel)
        if sharded:
            model.finish_backward()
        fused = (sharded and hasattr(optimizer, "clip_coef") and max_norm is not None
                 and next(iter(model.parameters())).is_cuda)
        if fused:
            clipper = self._clippers.setdefault(id(model), GradClipper(
                next(iter(model.parameters())).device))
            grad_norm = clipper(list(model.grad_shards()), max_norm).clone()
            optimizer.clip_coef = clipper.coef
        else:
            grad_norm = tp_mod.clip_grad_norm_(model, max_norm if max_norm is not None
                                               else float("inf"))
        optimizer.step()
        if sharded:
            model.after_optimizer_step(lp_written=hasattr(optimizer, "clip_coef"))
        model.zero_grad()
        return grad_norm.detach().reshape(())

    def step_with_rollouts(self, rollouts: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """``noptepochs`` passes over fixed rollouts: policy minibatches, then value minibatches
        (rl_trainer.py:175-283 of the reference)."""
        loader = self.get_rollouts_dataloader(rollouts)
        accumulate = max(1, self.args.gradient_accumulation_steps)
        scale = 1.0 / accumulate
        stats_policy, stats_value = [], []
        gc.collect()
        policy_net = self.policy.base_model
        value_net = self.value_model.base_model if self.value_model is not None else None
        policy_net.zero_grad()
        for _ in range(self.args.noptepochs):
            for batch_idx, batch in enumerate(loader, 1):
                loss, stats = self.compute_policy_loss(batch)
                (loss * scale).backward()
                if batch_idx % accumulate == 0:
                    stats = dict(stats)
                    stats["loss/grad_norm_policy"] = self._clip_and_step(policy_net,
                                                                         self.policy_optimizer)
                    stats_policy.append(stats)
            if value_net is not None:
                value_net.zero_grad()
                for batch_idx, batch in enumerate(loader, 1):
                    loss, stats = self.compute_value_loss(batch)
                    (loss * scale).backward()
                    if batch_idx % accumulate == 0:
                        stats = dict(stats)
                        stats["loss/grad_norm_value"] = self._clip_and_step(value_net,
                                                                            self.value_optimizer)
                        stats_value.append(stats)
        out = {}
        if stats_policy:
            out.update(utils.merge_dict(stats_policy, torch.stack))
        if stats_value:
            out.update(utils.merge_dict(stats_value, torch.stack))
        return out

    def step(self, train_dataloader, step_idx: int) -> Dict:
        queries_batches = [next(train_dataloader)
                           for _ in range(self.args.rollout_accumulation_steps)]
        rollouts = self.rollout(queries_batches)
        eval_stats = None
        if self.args.eval_steps is not None and step_idx % self.args.eval_steps == 0:
            eval_stats = self.evaluate(step_idx)
        if self.args.save_steps and step_idx % self.args.save_steps == 0:
            if self.args.save_strategy == "steps":
                self.save_model(step_idx=step_idx)
            elif self.args.save_strategy != "no":
                assert self.args.save_steps % self.args.eval_steps == 0
                assert eval_stats is not None and self.args.save_strategy in eval_stats
                metric = self.args.save_strategy
                if self.best_metrics is None or eval_stats[metric] > self.best_metrics[metric]:
                    self.best_metrics = eval_stats
                    self.save_model(step_idx=step_idx, metrics=eval_stats)
        train_stats = self.step_with_rollouts(rollouts)
        if self.policy_lr_scheduler is not None:
            self.policy_lr_scheduler.step()
        if self.value_lr_scheduler is not None:
            self.value_lr_scheduler.step()
        stats = self.record_step_stats(rollouts=rollouts, train_stats=train_stats,
                                       step_idx=step_idx, kl_coef=self.kl_ctl.value)
        self.kl_ctl.step(stats["objective/kl_sum_seq"])
        return stats

    def create_optimizer_and_scheduler(self, num_training_steps: int) -> None:
        a = self.args
        self.policy_optimizer = trainer_utils.create_optimizer(
            a, model=self.policy.base_model, optimizer_cpu_offload=a.policy_optimizer_cpu_offload,
            model_cpu_offload=a.policy_model_cpu_offload)
        self.policy_lr_scheduler = trainer_utils.get_cosine_schedule_with_warmup(
            self.policy_optimizer, warmup_epochs=a.ppo_warmup_steps, max_epochs=num_training_steps,
            warmup_start_ratio=0.0, eta_min_ratio=0.01)
        if self.value_model is not None:
            self.value_optimizer = trainer_utils.create_optimizer(
                a, model=self.value_model.base_model,
                optimizer_cpu_offload=a.value_optimizer_cpu_offload,
                model_cpu_offload=a.value_model_cpu_offload)
            self.value_lr_scheduler = trainer_utils.get_cosine_schedule_with_warmup(
                self.value_optimizer, warmup_epochs=a.ppo_warmup_steps,
                max_epochs=num_training_steps, warmup_start_ratio=0.0, eta_min_ratio=0.01)

    def train(self, resume_training_ckpt: Optional[str] = None) -> List[Dict]:
        total_epochs = self.args.num_train_epochs
        total_episodes = len(self.train_dataset) * total_epochs
        total_steps = total_episodes // self.args.rollout_batch_size
        if self.is_main_process:
            logger.warning("***Training starts***\nTotal epochs: %s => Total episodes: %s => "
                           "Total steps: %s", total_epochs, total_episodes, total_steps)
        self.create_optimizer_and_scheduler(total_steps)
        skipping_steps = 0
        if resume_training_ckpt is not None:
            skipping_steps = self.resume_training(resume_training_ckpt)
            if self.is_main_process:
                print(f"Resuming training from {resume_training_ckpt} at step {skipping_steps}.")
        loader = self.get_train_dataloader()
        for step_idx in range(FIRST_STEP_IDX, total_steps + FIRST_STEP_IDX):
            if step_idx < skipping_steps:
                for _ in range(self.args.rollout_accumulation_steps):
                    next(loader)
                continue
            self.log_history.append(self.step(loader, step_idx))
        return self.log_history

    # ------------------------------------------------------------------ data
    def get_train_dataloader(self):
        sampler = None
        if dist.is_initialized():
            sampler = DistributedSampler(self.train_dataset, shuffle=True, drop_last=True)
        loader = DataLoader(self.train_dataset,
                            batch_size=self.args.rollout_per_device_batch_size,
                            shuffle=sampler is None, drop_last=True, sampler=sampler,
                            collate_fn=self.data_collator)
        if self.is_main_process:
            logger.warning("Train dataset size: %d", len(self.train_dataset))
        return utils.InfiniteLoader(loader)

    def get_rollouts_dataloader(self, rollouts: Dict[str, torch.Tensor], drop_last: bool = True,
                                keys: Optional[Sequence[str]] = None):
        """Minibatches of ``step_per_device_batch_size * tp`` rollouts, in order (every rank of a
        tensor-parallel group must see the same rows, so no shuffling)."""
        keys = tuple(k for k, v in rollouts.items() if torch.is_tensor(v)) if keys is None \
            else tuple(keys)

        def collate(instances):
            return {k: torch.stack([inst[i] for inst in instances]) for i, k in enumerate(keys)}
        bs = self.args.step_per_device_batch_size * groups.get_model_parallel_world_size()
        return DataLoader(TensorDataset(*[rollouts[k] for k in keys]), batch_size=bs,
                          collate_fn=collate, shuffle=False, drop_last=drop_last)

    @property
    def is_main_process(self) -> bool:
        return not dist.is_initialized() or dist.get_rank() == 0

    @property
    def device(self) -> torch.device:
        return next(iter(self.policy.parameters())).device

    @staticmethod
    @torch.no_grad()
    def prepare_tp_batch(input_ids: Union[torch.Tensor, Dict[str, torch.Tensor]],
                         labels: Optional[torch.Tensor] = None, use_tp: Optional[bool] = None,
                         sync_group=None):
        """Concatenate the batches of the ranks of a tensor-parallel group along dim 0 so that
        every rank of the group holds the same rows (rl_trainer.py:502-563 of the reference)."""
        if use_tp is None:
            use_tp = dist.is_initialized() and groups.get_model_parallel_world_size() > 1
        if not use_tp:
            return (input_ids, labels) if labels is not None else input_ids
        group = sync_group if sync_group is not None else groups.get_model_parallel_group()
        n = dist.get_world_size(group)

        def gather(t):
            t = t.contiguous()
            out = torch.empty((t.shape[0] * n, *t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t, group=group)
            return out
        if isinstance(input_ids, dict):
            assert labels is None
            return {k: gather(v) for k, v in input_ids.items()}
        if not torch.is_tensor(input_ids):
            raise ValueError(f"Unsupported input_ids type: {type(input_ids)} for TP")
        out = gather(input_ids)
        return (out, gather(labels)) if labels is not None else out


def truncate_after_eos(completions: torch.Tensor, eos_token_id: int) -> List[List[int]]:
    out = completions.tolist()
    for i, row in enumerate(out):
        if eos_token_id in row:
            out[i] = row[: row.index(eos_token_id)]
    return out


def truncate_after_eos_padded(completions: torch.Tensor, eos_token_id: int,
                              pad_token_id: int) -> torch.Tensor:
    """Everything from the first EOS on (the EOS included) becomes padding."""
    is_eos = completions == eos_token_id
    after = is_eos.cumsum(dim=1) > 0
    return completions.masked_fill(after, pad_token_id)
