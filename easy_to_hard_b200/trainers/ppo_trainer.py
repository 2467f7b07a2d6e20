"""PPO trainer (reference: trainers/ppo_trainer.py).

Rollout (ppo_trainer.py:238-674 of the reference): sync the rollout copy of the policy from the
sharded training policy, generate responses on the CUDA-graph decode engine, grade them on the
CPU, then score the fixed sequences with the policy (log-probs, entropies), the value model, the
frozen reference policy and the frozen reward model, shape the rewards (KL penalty, process
rewards, stop-token penalty), and compute GAE advantages with batch-wide whitening.

Update (ppo_trainer.py:676-831): clipped policy-gradient loss on the ratio of new to old
log-probs, clipped value loss, both through the sharded fused engine.

What differs from the reference by design:
* the rollout copy is refreshed block by block, device to device, from the all-gathered bf16
  shards of the training policy (no full fp32 state dict, no CPU hop);
* every scoring pass runs the fused cache-less forward and the fused LM-head log-prob kernel,
  so no ``[batch, tokens, vocab]`` logits exist at any point;
* the GAE recursion is one kernel launch (``e2h_gae``) instead of a Python loop over time.
"""
from __future__ import annotations

import gc
import json
import os
from itertools import chain
from pathlib import Path
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models import rl_model
from ..models.model import Transformer, set_global_compile_mode
from ..models.reward_model import RewardModel, apply_reward_modeling_head
from ..models.tp import apply_reward_head_tp
from ..ops import _lib
from ..parallel import groups
from ..parallel.fsdp import ShardedDataParallel
from ..utils.checkpoint_utils import (checkpoint_hook, get_latest_checkpoint_path,
                                      load_checkpoint, load_model_from_from_ckpt,
                                      load_reward_model_from_ckpt)
from ..utils.trainer_utils import create_fsdp_model_for_finetune
from . import common_utils
from .rl_trainer import RLTrainer, truncate_after_eos, truncate_after_eos_padded

try:
    import wandb
except ImportError:  # optional
    wandb = None


def rank0_print(*args):
    if int(os.environ.get("LOCAL_RANK", 0)) == 0:
        print(*args, flush=True)


# ----------------------------------------------------------------------------- numerics helpers

def whiten(values: torch.Tensor, shift_mean: bool = True, epsilon: float = 1e-8,
           async_stats: str = "full_batch") -> torch.Tensor:
    """(values - mean) / (std + eps), statistics over the whole job (``full_batch``: gathered
    over all ranks), this rank (``per_gpu``) or each row (``none``); without ``shift_mean`` the
    mean is added back (ppo_trainer.py:1566-1606 of the reference)."""
    assert async_stats in ("full_batch", "per_gpu", "none")
    if async_stats == "none":
        mean = values.mean(dim=-1, keepdim=True)
        std = values.std(dim=-1, unbiased=False, keepdim=True)
    else:
        if async_stats == "full_batch" and dist.is_initialized() and dist.get_world_size() > 1:
            # sum, sum of squares and count are enough: no need to gather the values
            s = torch.stack([values.sum().double(), (values.double() ** 2).sum(),
                             torch.tensor(float(values.numel()), dtype=torch.float64,
                                          device=values.device)])
            dist.all_reduce(s)
            mean = (s[0] / s[2]).to(values.dtype)
            var = (s[1] / s[2] - (s[0] / s[2]) ** 2).clamp_min(0.0)
            std = var.sqrt().to(values.dtype)
        else:
            mean, std = values.mean(), values.std(unbiased=False)
    out = (values - mean) / (std + epsilon)
    return out if shift_mean else out + mean


def gae(rewards: torch.Tensor, values: torch.Tensor, gamma: float, lam: float
        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Generalised advantage estimation over [B, T] (value after the last step is 0). Returns
    (advantages, returns). One kernel launch on CUDA, a reversed scan elsewhere."""
    B, T = rewards.shape
    rewards, values = rewards.float().contiguous(), values.float().contiguous()
    adv = torch.empty_like(rewards)
    if rewards.is_cuda:
        ret = torch.empty_like(rewards)
        _lib.check(_lib.lib().e2h_gae(rewards.data_ptr(), values.data_ptr(), adv.data_ptr(),
                                      ret.data_ptr(), B, T, float(gamma), float(lam),
                                      _lib.stream()), "gae")
        return adv, ret
    last = torch.zeros(B, dtype=rewards.dtype, device=rewards.device)
    for t in reversed(range(T)):
        nxt = values[:, t + 1] if t < T - 1 else 0.0
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = delta + gamma * lam * last
        adv[:, t] = last
    return adv, adv + values


def truncate_after_stop_token(response: str, stop_token: Optional[str] = None,
                              additional_stop_token: Optional[List[str]] = None) -> str:
    if stop_token is None:
        return response
    for token in (additional_stop_token or ["<s>", "</s>"]) + [stop_token]:
        parts = response.split(token)
        if len(parts) > 1:
            response = parts[0] + token
    return response


def vanilla_stop_token_penalty(text_responses: List[str], stop_token: Optional[str],
                               eos_token: str) -> List[float]:
    if stop_token is not None:
        stop = stop_token.replace(r"\n", "\n").replace(r"\\", "\\")
    else:
        stop = eos_token
    return [0.0 if stop in t else 1.0 for t in text_responses]


def vanilla_post_process_rollouts(text_responses: List[str], **kwargs) -> Dict[str, List[float]]:
    del kwargs
    return {"symbolic_rewards": [0.0] * len(text_responses),
            "outcome_accuracy": [0.0] * len(text_responses)}


def _as_tensor_dict(d: Dict, device) -> Dict:
    """Lists of numbers from the CPU graders become tensors; strings stay as they are."""
    out = {}
    for k, v in d.items():
        if isinstance(v, list) and v and isinstance(v[0], (int, float)):
            out[k] = torch.tensor(v, device=device)
        else:
            out[k] = v
    return out


# ----------------------------------------------------------------------------- trainer

class PPOTrainer(RLTrainer):
    def __init__(self, args, train_dataset, data_collator, policy, value_model, ref_policy,
                 reward_model, tokenizer, eval_dataset=None, test_dataset=None,
                 policy_optimizer=None, policy_lr_scheduler=None, value_optimizer=None,
                 value_lr_scheduler=None, reward_tokenizer=None, unwrapped_policy=None,
                 fn_shape_process_rewards: Optional[Callable] = None,
                 fn_post_process_prm_rewards: Optional[Callable] = None,
                 fn_post_process_rollouts: Optional[Callable] = None,
                 fn_stop_token_penalty: Optional[Callable] = None):
        if reward_tokenizer is not None:
            raise NotImplementedError("Seperate reward tokenizer is not supported yet.")
        super().__init__(args=args, train_dataset=train_dataset, eval_dataset=eval_dataset,
                         test_dataset=test_dataset, data_collator=data_collator, policy=policy,
                         value_model=value_model, ref_policy=ref_policy,
                         reward_model=reward_model, tokenizer=tokenizer,
                         policy_optimizer=policy_optimizer,
                         policy_lr_scheduler=policy_lr_scheduler,
                         value_optimizer=value_optimizer, value_lr_scheduler=value_lr_scheduler,
                         reward_tokenizer=reward_tokenizer, unwrapped_policy=unwrapped_policy)
        self._shape_process_rewards = fn_shape_process_rewards
        self._post_process_prm_rewards = fn_post_process_prm_rewards
        self._post_process_rollouts = fn_post_process_rollouts or vanilla_post_process_rollouts
        self._stop_token_penalty = fn_stop_token_penalty or vanilla_stop_token_penalty

    # ------------------------------------------------------------------ reward shaping
    def _shape_reward(self, rewards, responses, logprobs, ref_logprobs, reg_entropies,
                      terminal_reward: bool = True) -> Dict[str, torch.Tensor]:
        """Per-token rewards = -kl_coef * KL estimate (+ entropy bonus), with the sequence
        reward added at the last response token (or per token for process rewards)."""
        a = self.args
        if a.kl_approximator == "k1":
            kl = torch.clamp(logprobs - ref_logprobs, min=0.0)
        elif a.kl_approximator == "k2":
            kl = logprobs - ref_logprobs
        elif a.kl_approximator == "k3":
            log_r = ref_logprobs - logprobs
            kl = torch.exp(log_r) - 1.0 - log_r
        elif a.kl_approximator == "maxent":
            kl = logprobs
        else:
            raise ValueError(f"Unknown KL approximator: {a.kl_approximator}")
        non_score = -self.kl_ctl.value * kl
        if a.maxent_coef > 0:
            non_score = non_score + a.maxent_coef * reg_entropies
        shaped = non_score.clone()
        terminal = (responses != self.tokenizer.pad_id).sum(dim=1) - 1
        if a.min_seq_len > 0 and a.min_seq_len_coef > 0:
            rewards = rewards - torch.clamp(a.min_seq_len - terminal, min=0.0).float() \
                * a.min_seq_len_coef
        if terminal_reward:
            shaped[torch.arange(rewards.size(0), device=responses.device), terminal] += rewards
        else:
            shaped = shaped + rewards
        return dict(shaped_rewards=shaped, non_score_rewards=non_score, kl=kl)

    def _estimate_advantage(self, rewards: torch.Tensor, values: torch.Tensor) -> Dict:
        a = self.args
        if a.whiten_rewards:
            rewards = whiten(rewards, shift_mean=False, async_stats=a.whitening_async_stats)
        else:
            rewards = rewards * 50.0
        tlen = a.target_max_len
        adv, ret = gae(rewards[:, :tlen], values[:, :tlen], a.gamma, a.lam)
        adv = whiten(adv, shift_mean=True, async_stats=a.whitening_async_stats)
        return dict(returns=ret, advantages=adv)

    def post_terminating_reward(self, reward_outputs: Dict[str, torch.Tensor],
                                responses: torch.Tensor, stop_token_penalty: List[float]) -> Dict:
        """Bad reward for sequences that did not stop properly."""
        if not self.args.penalize_no_stop_token:
            return reward_outputs
        pen = torch.tensor(stop_token_penalty, device=responses.device)
        rewards = reward_outputs["rewards"]
        if self.args.relative_stop_token_penalty:
            rewards = rewards + pen * self.args.penalty_reward_value
        else:
            rewards = rewards.masked_fill(pen > 0.0, self.args.penalty_reward_value)
        reward_outputs["rewards"] = rewards
        return reward_outputs

    # ------------------------------------------------------------------ rollout
    @torch.no_grad()
    def sync_rollout_policy(self) -> None:
        """Refresh the bf16 rollout copy from the training policy's shards, block by block on
        the device (all-gather of the bf16 shards, then a strided copy into the rollout model's
        tensors). Replaces the reference's full-state-dict round trip (ppo_trainer.py:260-311)."""
        if self.unwrapped_policy is None:
            return
        src = self.policy.base_model
        dst = self.unwrapped_policy.base_model
        if getattr(dst, "tp_group", None) is not None or getattr(self, "_relayout", None):
            # rollout layout differs from the training layout: every rollout rank pulls the rows
            # and columns it owns from the training shards over peer memory
            if getattr(self, "_relayout", None) is None:
                from ..parallel.relayout import RolloutRelayout
                assert isinstance(src, ShardedDataParallel), \
                    "a separate rollout TP degree needs the sharded training wrapper"
                src.expose_shards(None)
                self._relayout = RolloutRelayout(src, dst, groups.get_model_parallel_world_size(),
                                                 groups.get_rollout_parallel()[2])
            self._relayout.run()
            return
        if not isinstance(src, ShardedDataParallel):
            sd = {k: v for k, v in src.state_dict().items() if "kv_cache" not in k}
            dst.load_state_dict(sd, strict=False)
            return
        dst_params = dict(dst.named_parameters())
        dst_params.update(dict(dst.named_buffers()))
        for unit in src._all_units():
            buf = torch.empty(unit.padded, dtype=unit.shard_lp.dtype, device=unit.shard_lp.device)
            full = buf[: unit.padded]
            if unit.world > 1:
                dist.all_gather_into_tensor(full, unit.shard_lp, group=unit.group)
            else:
                full.copy_(unit.shard_lp)
            for name, o, n, shp in zip(unit.names, unit.offsets, unit.numels, unit.shapes):
                dst_params[name].data.copy_(full[o:o + n].view(shp))
        # the decode engine reads the rollout model's own tensors (updated in place above), so
        # its captured graphs see the new weights without any refresh

    def _rollout_is_wider(self) -> bool:
        actor = self.unwrapped_policy
        return actor is not None and getattr(actor.base_model, "tp_group", None) is not None

    def _respond(self, actor, queries, masks, temperature):
        """Responses to ``queries`` (identical on the ranks of a training tensor-parallel group).
        With a wider rollout group the neighbouring training groups pool their queries, the
        rollout engine generates for all of them at once, and every training group takes its
        rows back."""
        if not self._rollout_is_wider():
            return actor.respond(queries, masks, temperature=temperature)["responses"]
        group, ranks, size, rank = groups.get_rollout_parallel()
        tp = groups.get_model_parallel_world_size()
        n = queries.shape[0]

        def pool(t):
            every = torch.empty((size * n, *t.shape[1:]), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(every, t.contiguous(), group=group)
            return every.view(size // tp, tp, n, *t.shape[1:])[:, 0].reshape(-1, *t.shape[1:])
        with groups.model_parallel_as(group, ranks, size, rank):
            out = actor.respond(pool(queries), pool(masks), temperature=temperature)["responses"]
        mine = rank // tp
        return out[mine * n:(mine + 1) * n].contiguous()

    @staticmethod
    def sub_batched_outputs(model, rollouts_batch: Dict[str, torch.Tensor],
                            batch_size_per_device: int, sub_batch_size: Optional[int] = None,
                            **kwargs):
        if sub_batch_size is None or sub_batch_size >= batch_size_per_device:
            return model(**rollouts_batch, **kwargs)
        assert batch_size_per_device % sub_batch_size == 0
        outs = []
        for i in range(batch_size_per_device // sub_batch_size):
            sub = {k: v[i * sub_batch_size:(i + 1) * sub_batch_size]
                   for k, v in rollouts_batch.items()}
            outs.append(model(**sub, **kwargs))
        if isinstance(outs[0], dict):
            return common_utils.merge_dict(outs, merge_fn=torch.cat)
        return torch.cat(outs, dim=0)

    @torch.no_grad()
    def rollout(self, queries_data) -> Dict[str, torch.Tensor]:
        a, tok, dev = self.args, self.tokenizer, self.device
        for m in (self.policy, self.value_model, self.ref_policy, self.reward_model):
            m.eval()
        gc.collect()
        self.sync_rollout_policy()
        actor = self.unwrapped_policy if self.unwrapped_policy is not None else self.policy
        actor.eval()
        sub = a.reward_model_per_device_batch_size
        rollouts: List[Dict] = []
        # ---- 1. generate and grade
        for batch in queries_data:
            queries, masks, answers = common_utils.unpack_dict(
                common_utils.prepare_inputs(batch, device=dev),
                keys=("queries", "query_attn_masks", "answers"))
            queries = self.prepare_tp_batch(queries)
            masks = self.prepare_tp_batch(masks)
            answers = self.prepare_tp_batch(answers)
            responses = self._respond(actor, queries, masks, a.temperature)
            rb = {"queries": queries, "query_attn_masks": masks}
            text_queries = tok.batch_decode(queries, skip_special_tokens=True)
            text_responses = [truncate_after_stop_token(t, tok.eos_token)
                              for t in tok.batch_decode(responses, skip_special_tokens=False)]
            outcome = self._post_process_rollouts(
                text_responses, answer_gt_levels=answers, tokenizer=tok, stop_token=a.stop_token,
                outcome_reward=a.outcome_reward, easy_outcome_reward=a.easy_outcome_reward,
                device=dev)
            rb.update(_as_tensor_dict(outcome, dev))
            rb["stop_token_penalty"] = self._stop_token_penalty(text_responses, a.stop_token,
                                                                tok.eos_token)
            rb["text_queries"], rb["text_responses"] = text_queries, text_responses
            rb["responses"] = truncate_after_eos_padded(responses, tok.eos_id, tok.pad_id)
            rollouts.append(rb)
        # ---- 2. score with policy, value model, reference policy
        for rb in rollouts:
            seqs = {k: rb[k] for k in ("queries", "query_attn_masks", "responses")}
            n = rb["responses"].shape[0]
            scorer = self.policy if self._rollout_is_wider() else actor
            pol = self.sub_batched_outputs(scorer, seqs, n, sub, temperature=a.temperature)
            rb["logprobs"] = pol["logprobs"].float()
            rb["entropies"] = pol["entropies"].float()
            reg, regw = pol["reg_entropies"].float(), pol["reg_entropies_weight"].float()
            if a.maxent_normalization == "full":
                rb["reg_entropies"] = reg / regw.sum(dim=-1, keepdim=True)
            elif a.maxent_normalization == "none":
                rb["reg_entropies"] = reg
            elif a.maxent_normalization == "merged":
                rb["reg_entropies"] = reg.sum(dim=-1) / regw.sum(dim=-1)
            else:
                raise ValueError(f"Unknown maxent_normalization: {a.maxent_normalization}")
            rb["values"] = self.sub_batched_outputs(self.value_model, seqs, n, sub)["values"].float()
            ref = self.sub_batched_outputs(self.ref_policy, seqs, n, sub,
                                           temperature=a.temperature)
            rb["ref_logprobs"] = ref["logprobs"].float()
            rb["ref_entropies"] = ref["entropies"].float()
        # ---- 3. reward model, shaping
        for rb in rollouts:
            if a.maxent_normalization == "merged":
                rb["symbolic_rewards"] = rb["symbolic_rewards"] + rb["reg_entropies"] * a.maxent_coef
                rb["reg_entropies"] = torch.zeros_like(rb["reg_entropies"]).unsqueeze(-1)
            penalty = rb.pop("stop_token_penalty")
            text_queries, text_responses = rb.pop("text_queries"), rb.pop("text_responses")
            sequences = torch.cat((rb["queries"], rb["responses"]), dim=1)
            padded, shifts = rl_model.prepare_right_pad_sequences(sequences,
                                                                  pad_token_id=tok.pad_id)
            rewards = self.sub_batched_outputs(self.reward_model, {"idx": padded},
                                               rb["responses"].size(0), sub)
            responses = rb["responses"]
            if a.apply_process_reward or a.apply_terminal_process_reward:
                assert not (a.apply_process_reward and a.apply_terminal_process_reward), \
                    "Cannot use both apply_process_reward and apply_terminal_process_reward."
                rewards = rl_model.restore_from_right_pad_sequences(rewards, shifts).float()
                scores = self._post_process_prm_rewards(sequences, rewards, text_queries,
                                                        text_responses, tok)
                shaped_process, aggregated, responses = self._shape_process_rewards(
                    rb["symbolic_rewards"], rb["queries"], rb["responses"], tok, dev, scores,
                    penalty, a.penalty_reward_value, a.penalize_no_stop_token,
                    a.relative_stop_token_penalty, a.process_reward_scheme,
                    a.process_reward_upper_bound, a.apply_process_reward,
                    a.apply_terminal_process_reward, a.process_reward_scale)
            else:
                shaped_process = None
                aggregated = self.post_terminating_reward(
                    {"rewards": rewards.float()[..., -1]}, responses=rb["responses"],
                    stop_token_penalty=penalty)["rewards"]
            rb["responses"], rb["rewards"] = responses, aggregated
            rb.update(self._shape_reward(
                rewards=shaped_process if a.apply_process_reward else aggregated,
                responses=rb["responses"], logprobs=rb["logprobs"],
                ref_logprobs=rb["ref_logprobs"], reg_entropies=rb["reg_entropies"],
                terminal_reward=not a.apply_process_reward))
        merged = common_utils.merge_dict(
            [{k: v for k, v in rb.items() if torch.is_tensor(v)} for rb in rollouts],
            merge_fn=torch.cat)
        merged.update(self._estimate_advantage(merged["shaped_rewards"].to(dev),
                                               merged["values"].to(dev)))
        return merged

    # ------------------------------------------------------------------ losses
    def compute_policy_loss(self, rollouts: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, Dict]:
        a = self.args
        old_logprob, advantages, queries, masks, responses = common_utils.prepare_inputs(
            common_utils.unpack_dict(rollouts, keys=("logprobs", "advantages", "queries",
                                                     "query_attn_masks", "responses")),
            device=self.device)
        self.policy.train()
        out = self.policy(queries, masks, responses, temperature=a.temperature)
        logprob = out["logprobs"].float()
        advantages, old_logprob = advantages.float(), old_logprob.float()
        ratio = torch.exp(logprob - old_logprob)
        pg1 = -advantages * ratio
        pg2 = -advantages * torch.clamp(ratio, min=1.0 - a.cliprange, max=1.0 + a.cliprange)
        pg_loss = torch.maximum(pg1, pg2).mean()
        clipfrac = (pg2 > pg1).float().mean()
        entropy = out["entropies"].mean()
        reg_entropies = out["reg_entropies"].sum(dim=-1).mean()
        approxkl = 0.5 * ((logprob - old_logprob) ** 2.0).mean()
        if a.ent_reg_coef > 0.0:
            pg_loss = pg_loss - a.ent_reg_coef * reg_entropies
        stats = dict(loss=dict(policy=pg_loss),
                     policy=dict(entropy=entropy, reg_entropy=reg_entropies, approxkl=approxkl,
                                 clipfrac=clipfrac))
        return pg_loss, common_utils.flatten_dict(stats, sep="/",
                                                  postprocess_fn=lambda x: x.detach())

    def compute_value_loss(self, rollouts: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, Dict]:
        a = self.args
        values, returns, queries, masks, responses = common_utils.prepare_inputs(
            common_utils.unpack_dict(rollouts, keys=("values", "returns", "queries",
                                                     "query_attn_masks", "responses")),
            device=self.device)
        self.value_model.train()
        vpred = self.value_model(queries, masks, responses)["values"].float()
        returns, values = returns.float(), values.float()
        clipped = torch.clamp(vpred, min=values - a.cliprange_value,
                              max=values + a.cliprange_value)
        l1, l2 = (vpred - returns) ** 2.0, (clipped - returns) ** 2.0
        vf_loss = 0.5 * torch.maximum(l1, l2).mean()
        loss = a.vf_coef * vf_loss
        stats = dict(loss=dict(value=vf_loss),
                     val=dict(vpred=vpred.mean(), error=((vpred - returns) ** 2).mean(),
                              clipfrac=(l2 > l1).float().mean(), mean=values.mean(),
                              var=values.var(unbiased=False)),
                     returns=dict(mean=returns.mean(), var=returns.var(unbiased=False)))
        return loss, common_utils.flatten_dict(stats, sep="/",
                                               postprocess_fn=lambda x: x.detach())

    # ------------------------------------------------------------------ bookkeeping
    @torch.no_grad()
    def record_step_stats(self, train_stats, rollouts, step_idx, **kwargs):
        kl = rollouts["kl"]
        stats = {
            "objective/kl_coef": kwargs["kl_coef"],
            "objective/kl_sum_seq": kl.sum(dim=1).mean(dim=0),
            "objective/kl_avg_seq": kl.mean(),
            "objective/shaped_rewards": rollouts["shaped_rewards"].sum(dim=1).mean(dim=0),
            "objective/non_score_rewards": rollouts["non_score_rewards"].sum(dim=1).mean(dim=0),
            "objective/rewards": rollouts["rewards"].mean(dim=0),
            "objective/outcome_accuracy": rollouts["outcome_accuracy"].float().mean(dim=0),
            "objective/lr": self.policy_optimizer.param_groups[0]["lr"],
            "objective/entropies": rollouts["entropies"].mean(),
            "objective/ref_entropies": rollouts["ref_entropies"].mean(),
        }
        for level in range(9):
            if f"level_{level}_counts" in rollouts:
                vec = torch.stack([rollouts[f"level_{level}_counts"].sum().float(),
                                   rollouts[f"level_{level}_accuracy"].sum().float()]
                                  ).to(self.device)
                if dist.is_initialized():
                    dist.all_reduce(vec)
                train_stats[f"outcome_accuracy/level_{level}"] = (vec[1] / (vec[0] + 1e-8)).cpu()
        for k, v in train_stats.items():
            stats[f"ppo/{k}"] = v.float().mean(dim=0) if v.dim() > 0 else v
        stats = {k: (v.item() if torch.is_tensor(v) else v) for k, v in stats.items()}
        if self.is_main_process:
            if self.args.report_to == "wandb" and wandb is not None:
                wandb.log(stats, step=step_idx)
            else:
                print(f"Step {step_idx}: {stats}", flush=True)
            if self.args.save_dir is not None:
                tok = self.tokenizer
                records = [
                    {"queries": q, "responses": r, "rewards": str(w)}
                    for q, r, w in zip(
                        tok.batch_decode(truncate_after_eos(rollouts["queries"], tok.eos_id),
                                         skip_special_tokens=False),
                        tok.batch_decode(truncate_after_eos(rollouts["responses"], tok.eos_id),
                                         skip_special_tokens=False),
                        rollouts["rewards"].tolist())]
                log_dir = os.path.join(self.args.save_dir, "rollouts")
                os.makedirs(log_dir, exist_ok=True)
                with open(os.path.join(log_dir, f"step_{step_idx}.json"), "w",
                          encoding="utf-8") as f:
                    json.dump(records, f, indent=4)
        return stats

    @torch.no_grad()
    def resume_training(self, checkpoint_dir) -> int:
        policy_ckpt, epoch, step = get_latest_checkpoint_path(checkpoint_dir, prefix="policy_")
        value_ckpt, _, global_step = get_latest_checkpoint_path(checkpoint_dir, prefix="value_")
        rank0_print(f"Resuming policy from checkpoint: {policy_ckpt}")
        rank0_print(f"Resuming value from checkpoint: {value_ckpt}")
        rank0_print(f"Resuming (epoch {epoch}, global step {step})")
        resumed = load_checkpoint(policy_ckpt, model=self.policy.base_model,
                                  optimizer=self.policy_optimizer,
                                  scheduler=self.policy_lr_scheduler, use_fsdp=True)
        if resumed and "metrics" in resumed:
            self.best_metrics = resumed["metrics"]
        if value_ckpt is not None:
            load_checkpoint(value_ckpt, model=self.value_model.base_model,
                            optimizer=self.value_optimizer, scheduler=self.value_lr_scheduler,
                            use_fsdp=True)
        else:
            global_step = step
        return global_step

    @torch.no_grad()
    def save_model(self, step_idx: int, metrics: Optional[Dict[str, float]] = None):
        checkpoint_hook(args=self.args, model=self.policy.base_model,
                        optimizer=self.policy_optimizer, scheduler=self.policy_lr_scheduler,
                        epoch=None, global_step=step_idx, epoch_length=None, use_fsdp=True,
                        prefix="policy_", metrics=metrics)
        if not self.args.save_only_model:
            checkpoint_hook(args=self.args, model=self.value_model.base_model,
                            optimizer=self.value_optimizer, scheduler=self.value_lr_scheduler,
                            epoch=None, global_step=step_idx, epoch_length=None, use_fsdp=True,
                            prefix="value_", metrics=metrics)

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def evaluate(self, step_idx: int, temperature: float = 0.0) -> Dict:
        """Generate for the eval / test queries (sharded over the data-parallel ranks), grade
        the answers, write the generations to ``save_dir/{evaluate,test}/`` and return the
        per-level and overall accuracies (ppo_trainer.py:994-1265 of the reference)."""
        stats = {}
        for ds, prefix in ((self.eval_dataset, "evaluate"), (self.test_dataset, "test")):
            if ds is None:
                continue
            out = self._evaluate(step_idx, ds.queries, ds.query_attn_masks, ds.answers,
                                 temperature=temperature, eval_prefix=prefix)
            stats.update(out or {})
        return stats

    def _evaluate(self, step_idx, query_data, mask_data, answer_data, temperature, eval_prefix):
        if any(x is None for x in (query_data, mask_data, answer_data)):
            rank0_print("No evaluation data, skipping evaluation.")
            return None
        a, tok, dev = self.args, self.tokenizer, self.device
        dp_rank, dp_size = groups.get_data_parallel_rank(), groups.get_data_parallel_world_size()
        tp_rank, tp_size = groups.get_model_parallel_rank(), groups.get_model_parallel_world_size()
        per_rank = 1 + (len(query_data) - 1) // dp_size
        lo, hi = per_rank * dp_rank, min(per_rank * (dp_rank + 1), len(query_data))
        query_data, mask_data, answer_data = (query_data[lo:hi], mask_data[lo:hi],
                                              answer_data[lo:hi])
        n_mine = len(query_data)
        assert a.per_device_eval_batch_size == a.rollout_per_device_batch_size, \
            "per_device_eval_batch_size should be equal to rollout_per_device_batch_size for now."
        bs = a.per_device_eval_batch_size * tp_size
        query_data, mask_data, answer_data = common_utils.pad_inputs_on_batch(
            (query_data, mask_data, answer_data), per_device_batch_size=bs)
        self.sync_rollout_policy()
        actor = (self.unwrapped_policy if self.unwrapped_policy is not None else self.policy).eval()
        batches = []
        for s in range(0, query_data.size(0), bs):
            queries, masks, answers = common_utils.prepare_inputs(
                (query_data[s:s + bs], mask_data[s:s + bs], answer_data[s:s + bs]), device=dev)
            responses = self._respond(actor, queries, masks, temperature)
            text_queries = tok.batch_decode(queries, skip_special_tokens=True)
            text_responses = [truncate_after_stop_token(t, tok.eos_token)
                              for t in tok.batch_decode(responses, skip_special_tokens=False)]
            rec = {"text_queries": text_queries, "text_responses": text_responses}
            rec.update(_as_tensor_dict(self._post_process_rollouts(text_responses, answers),
                                       "cpu"))
            batches.append({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in rec.items()})

        def merge(items):
            return list(chain(*items)) if isinstance(items[0], list) else torch.cat(items, dim=0)
        merged = {k: v[:n_mine] for k, v in
                  common_utils.merge_dict(batches, merge_fn=merge).items()}
        results = [{"text_query": q, "text_response": r}
                   for q, r in zip(merged["text_queries"], merged["text_responses"])]
        if tp_rank == 0 and a.save_dir is not None:
            log_dir = os.path.join(a.save_dir, eval_prefix)
            os.makedirs(log_dir, exist_ok=True)
            with open(os.path.join(log_dir, f"eval_results_{step_idx}_rank_{dp_rank}.json"), "w",
                      encoding="utf-8") as f:
                json.dump(results, f, indent=4)
        rank0_print(f"End evaluation at step: {step_idx}. Processed {len(results)} examples")

        def reduce_pair(counts, acc):
            vec = torch.stack([torch.as_tensor(counts, dtype=torch.float32),
                               torch.as_tensor(acc, dtype=torch.float32)]).to(dev)
            if dist.is_initialized():
                dist.all_reduce(vec)
            return vec.cpu()
        stats, tot_c, tot_a = {}, 0.0, 0.0
        for level in range(9):
            if f"level_{level}_counts" in merged:
                c = merged[f"level_{level}_counts"].sum().item()
                acc = merged[f"level_{level}_accuracy"].sum().item()
                tot_c, tot_a = tot_c + c, tot_a + acc
                vec = reduce_pair(c, acc)
                stats[f"{eval_prefix}/accuracy_level_{level}"] = (vec[1] / (vec[0] + 1e-8)).item()
                stats[f"{eval_prefix}/counts_level_{level}"] = (vec[0] / tp_size).item()
        vec = reduce_pair(tot_c, tot_a)
        stats[f"{eval_prefix}/accuracy_overall"] = (vec[1] / (vec[0] + 1e-8)).item()
        stats[f"{eval_prefix}/counts_overall"] = (vec[0] / tp_size).item()
        if self.is_main_process:
            if a.report_to == "wandb" and wandb is not None:
                wandb.log(stats, step=step_idx)
            else:
                print(f"Step {step_idx} (Eval): {stats}", flush=True)
        return stats


# ----------------------------------------------------------------------------- model factory

def make_models(tokenizer, args, use_tp: bool = True,
                resume_from_checkpoint: Optional[str] = None) -> dict:
    """The five models of a PPO run (ppo_trainer.py:1303-1563 of the reference): trainable policy
    and value model on the sharded fused engine, a bf16 rollout copy of the policy for the
    decode engine, and the frozen reference policy and reward model (bf16 or int8 weight-only,
    per ``ref_policy_model_bits`` / ``reward_model_bits``)."""
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    use_tp = use_tp and dist.is_initialized()
    rank0_print("Resuming from checkpoint: ", [resume_from_checkpoint])
    set_global_compile_mode(False)
    frozen_dtype = args.compute_dtype if device.type == "cuda" else args.param_dtype

    def finish(model, trainable: bool, bits: int):
        model = model.train() if trainable else model.eval()
        backbone = model.backbone_model if isinstance(model, RewardModel) else model
        bs = max(args.rollout_per_device_batch_size, args.step_per_device_batch_size) \
            * groups.get_model_parallel_world_size()
        seq = min(backbone.config.block_size, args.source_max_len + args.target_max_len + 8)
        backbone.setup_caches(max_batch_size=bs, max_seq_length=seq, kv_cache=False)
        assert not (trainable and bits < 16), "Cannot train with int8 or int4."
        if bits < 16:
            assert bits == 8, "Only int8 is supported."
            rank0_print("Quantizing model ...")
            from ..models.quantize import WeightOnlyInt8QuantHandler
            model = WeightOnlyInt8QuantHandler(model).convert_for_runtime_on_the_fly()
            model = model.to(device=device).eval()
        if trainable:
            model = create_fsdp_model_for_finetune(args, model)
            model.train()
        return model

    def generative(trainable, base_path, resume_path=None, bits=16, tp_override=None):
        m = load_model_from_from_ckpt(
            checkpoint_path=base_path, sft_checkpoint_path=resume_path, device=device,
            precision=args.param_dtype if trainable else frozen_dtype, use_tp=use_tp,
            requires_grad=trainable, skip_init=False, vocab_parallel=args.vocab_parallel,
            sequence_parallel=args.sequence_parallel and trainable, tp_override=tp_override)
        return finish(m, trainable, bits)

    def reward(trainable, base_path, resume_path=None, backbone_only=False, bits=16):
        m = load_reward_model_from_ckpt(
            checkpoint_path=base_path, rm_checkpoint_path=resume_path, device=device,
            precision=args.param_dtype if trainable else frozen_dtype, use_tp=use_tp,
            requires_grad=trainable, skip_init=False, vocab_parallel=args.vocab_parallel,
            sequence_parallel=args.sequence_parallel and trainable)
        if backbone_only:
            m = m.backbone_model
        return finish(m, trainable, bits)

    fresh = resume_from_checkpoint is None
    rank0_print("### Creating the reference policy ...")
    ref_policy = rl_model.make_policy_with_base_model(
        args, generative(False, args.base_checkpoint_path, args.policy_checkpoint_path,
                         bits=args.ref_policy_model_bits), tokenizer)
    rank0_print("### Creating the policy ...")
    policy = rl_model.make_policy_with_base_model(
        args, generative(True, args.base_checkpoint_path,
                         args.policy_checkpoint_path if fresh else None), tokenizer)
    rank0_print("### Creating the rollout copy of the policy ...")
    # generation may run at a wider tensor-parallel degree than training
    # (--rollout_tensor_parallel_size): the copy is then sharded over the rollout group
    rollout = groups.get_rollout_parallel()
    override = rollout if (use_tp and rollout[2] != groups.get_model_parallel_world_size()) \
        else None
    unwrapped_policy = rl_model.make_policy_with_base_model(
        args, generative(False, args.base_checkpoint_path, None, tp_override=override), tokenizer)
    rank0_print("### Creating the value model ...")
    if args.init_value_with_reward:
        base = (args.value_base_checkpoint_path or args.reward_base_checkpoint_path
                or args.base_checkpoint_path)
        resume = (args.value_checkpoint_path or args.reward_checkpoint_path) if fresh else None
        value_model = rl_model.make_value_with_base_model(
            args, reward(True, base, resume, backbone_only=True), tokenizer)
    else:
        base = args.value_base_checkpoint_path or args.base_checkpoint_path
        resume = (args.value_checkpoint_path or args.policy_checkpoint_path) if fresh else None
        m = load_model_from_from_ckpt(
            checkpoint_path=base, sft_checkpoint_path=resume, device=device,
            precision=args.param_dtype, use_tp=use_tp, requires_grad=True,
            vocab_parallel=args.vocab_parallel, sequence_parallel=args.sequence_parallel)
        apply_reward_modeling_head(m, requires_grad=True)
        if use_tp:
            apply_reward_head_tp(m, requires_grad=True)
        value_model = rl_model.make_value_with_base_model(args, finish(m, True, 16), tokenizer)
    rank0_print("### Creating the reward model ...")
    reward_model = reward(False, args.reward_base_checkpoint_path or args.base_checkpoint_path,
                          args.reward_checkpoint_path, bits=args.reward_model_bits)
    return dict(policy=policy, value_model=value_model, ref_policy=ref_policy,
                reward_model=reward_model, unwrapped_policy=unwrapped_policy)
