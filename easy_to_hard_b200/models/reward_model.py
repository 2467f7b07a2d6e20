"""Reward / value model: a ``Transformer`` backbone whose LM head is replaced by a 2-row head;
the reward of a token is the mean of the two head outputs (models/reward_model.py:60-133 of the
reference; two rows instead of one work around a PyTorch scalar-output issue upstream, and the
2 x dim shape is part of the checkpoint contract, so it is kept).

``RewardModel.forward(idx, eos_pos)`` runs the backbone fully causal from position 0 and returns
per-token rewards ``[B, T]`` or, with ``eos_pos``, the reward at that position ``[B]``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from . import tp as tp_mod
from .model import ModelArgs, Transformer


def unpack_dict(d: Dict, keys, return_type=tuple):
    vals = [d[k] for k in keys]
    return return_type(vals) if return_type in (tuple, list) else {k: d[k] for k in keys}


def batch_select(input: Tensor, index: Tensor) -> Tensor:
    """out[b, j] = input[b, index[b, j]]."""
    return torch.gather(input, 1, index.long())


@dataclass
class RewardArgs:
    backbone_args: ModelArgs

    @classmethod
    def from_name(cls, name: str) -> "RewardArgs":
        return cls(backbone_args=ModelArgs.from_name(name))


class RewardModel(nn.Module):
    def __init__(self, config: RewardArgs, **kwargs) -> None:
        super().__init__()
        self.config = config
        self.backbone_model = Transformer(config.backbone_args, **kwargs)

    @classmethod
    def from_name(cls, name: str, **kwargs) -> "RewardModel":
        return cls(RewardArgs.from_name(name), **kwargs)

    def token_rewards(self, hidden: Tensor) -> Tensor:
        """Final-norm hidden states [B, T, dim] -> per-token reward [B, T] (fp32)."""
        head = self.backbone_model.output
        return tp_mod.reward_head_forward(head, hidden).float().mean(dim=-1)

    def _fused_rewards(self, idx: Tensor, eos_pos: Optional[Tensor]) -> Optional[Tensor]:
        """Scoring on CUDA without autograd: the fused block stack, then ONE kernel for the final
        norm, the 2-row head, the mean and the gather at ``eos_pos`` (only those rows are
        normalised and multiplied). A head sharded over its input dimension contributes fp32
        partial dots that are summed over the tensor-parallel group before the rounding."""
        from . import fused_block
        from ..ops import functional as Fn
        bb = self.backbone_model
        head = bb.output
        w = getattr(head, "weight", None)
        if (torch.is_grad_enabled() or not idx.is_cuda or not isinstance(w, Tensor)
                or w.dtype != torch.bfloat16 or w.shape[0] != 2 or not fused_block.can_fuse(bb, idx)):
            return None
        B, S = idx.shape
        hidden = fused_block.transformer_hidden(bb, idx, final_norm=False).view(B * S, -1)
        index = None
        if eos_pos is not None:
            index = (torch.arange(B, device=idx.device) * S + eos_pos.to(idx.device).long()).int()
        sharded = getattr(head, "tp_row_parallel", False)
        k0 = tp_mod.groups.get_model_parallel_rank() * w.shape[1] if sharded else 0
        reward, dots, _ = Fn.reward_head(hidden, bb.norm.weight, w, bb.config.norm_eps,
                                         index=index, k0=k0, finalize=not sharded)
        if sharded:
            dots = tp_mod.coll.reduce_from_tp(dots)
            reward = dots.to(torch.bfloat16).float().mean(dim=-1)
        return reward if eos_pos is not None else reward.view(B, S)

    def forward(self, idx: Tensor, eos_pos: Optional[Tensor] = None) -> Tensor:
        bb = self.backbone_model
        fused = self._fused_rewards(idx, eos_pos)
        if fused is not None:
            return fused
        if bb.freqs_cis is None or bb.max_seq_length < idx.size(-1) \
                or bb.max_batch_size < idx.size(0):
            bb.setup_caches(idx.size(0), idx.size(-1), kv_cache=False)
        pos = torch.arange(idx.size(-1), device=idx.device)
        hidden = bb(idx, input_pos=pos, fully_causal=True, return_hidden=True)
        hidden = hidden.to(bb.output.weight.dtype)
        rewards = self.token_rewards(hidden)
        if eos_pos is not None:
            rewards = batch_select(rewards, eos_pos.unsqueeze(-1)).squeeze(-1)
        return rewards


def apply_reward_modeling_head(transformer: Transformer, requires_grad: bool = False,
                               init_sceheme: str = "zeros") -> None:
    """Swap ``transformer.output`` for a trainable ``[2, dim]`` head (the keyword keeps the
    reference's spelling). ``semantic`` seeds the rows from the LM-head rows of the tokens "2"
    and "1" of the LLaMA vocabulary (ids 29906 / 29896)."""
    out = transformer.output
    old = out.weight
    head = torch.zeros(2, old.shape[1], dtype=old.dtype, device=old.device)
    if init_sceheme == "zeros":
        pass
    elif init_sceheme == "semantic":
        head[0] = old[29906]
        head[1] = -old[29896]
    elif init_sceheme == "random":
        g = torch.Generator(device=head.device).manual_seed(42)
        nn.init.kaiming_uniform_(head, a=math.sqrt(5), generator=g)
        head = head * math.sqrt(2.0)
    else:
        raise ValueError(f"Unknown init_scheme: {init_sceheme}")
    if "weight" in out._buffers:
        del out._buffers["weight"]
    out.weight = nn.Parameter(head, requires_grad=requires_grad)
    out.out_features = 2


def compute_pairwise_reward_modeling_loss(model, inputs, return_outputs: bool = False):
    """BCE on reward differences of candidate pairs. ``input_ids`` [B, C, L], ``eos_pos``
    [B, C], ``index_0`` / ``index_1`` / ``choice`` [B, P] (choice = 1 when index_1 wins)."""
    input_ids, eos_pos, index_0, index_1, choice = unpack_dict(
        inputs, ("input_ids", "eos_pos", "index_0", "index_1", "choice"))
    B, C, L = input_ids.shape
    rewards = model(input_ids.reshape(B * C, L), eos_pos=eos_pos.reshape(B * C)).view(B, C)
    logits = batch_select(rewards, index_1) - batch_select(rewards, index_0)
    loss = F.binary_cross_entropy_with_logits(logits, choice.to(logits.dtype))
    return (loss, dict(logits=logits)) if return_outputs else loss


def compute_pairwise_reward_modeling_metrics(predictions, label_ids) -> Dict:
    logits = torch.as_tensor(predictions).squeeze(-1)
    labels = torch.as_tensor(label_ids[-1]).squeeze(-1)
    return dict(accuracy=(logits >= 0.0).long().eq(labels).float().mean().item(),
                label_positive_rate=(labels == 1).float().mean().item())
