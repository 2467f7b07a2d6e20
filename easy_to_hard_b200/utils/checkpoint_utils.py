"""Checkpoint save / load / resume and tensor-parallel resharding.

File-format contract of the reference (checkpoint_utils.py:51-636), kept bit-compatible:

* base weights: ``<dir>/<model-name>/model.pth`` -- flat gpt-fast state dict, the directory name
  selects the architecture;
* training checkpoints: one file per tensor-parallel rank, written by data-parallel rank 0,
  ``{prefix}epoch_{E}_step_{S}_rank_{tp}.pt`` or ``{prefix}step_{S}_rank_{tp}.pt`` holding
  ``{"model": trainable params (TP-sharded, DP-unsharded), "optimizer": full state keyed by
  parameter name, "scheduler", "epoch", "global_step", "metrics"}``; ``save_only_model`` keeps
  just ``model`` in the compute dtype; ``{prefix}last_checkpoint`` names the newest file with a
  ``_rank*`` wildcard; the oldest files beyond ``save_total_limit`` are removed;
* ``load_inference_checkpoint`` merges (checkpoint TP > current TP) or splits (checkpoint TP <
  current TP) the shards: ``wqkv`` per q/k/v segment along dim 0, ``wo`` / ``w2`` /
  ``output.weight`` along dim 1, norms and embeddings replicated, everything else along dim 0.

The sharded-data-parallel wrapper of this framework (``parallel.fsdp.ShardedDataParallel``)
provides the DP-unsharded views itself (``full_state_dict`` / ``full_optim_state_dict``), so no
re-implementation of PyTorch-private FSDP routines is needed (the reference carries 700 lines of
those in training_utils/fsdp_utils.py).
"""
from __future__ import annotations

import glob
import os
import re
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.model import Transformer
from ..models.tp import (apply_reward_head_tp, apply_tp, get_data_parallel_rank,
                         get_model_parallel_rank, get_model_parallel_world_size)


def rank0_print(*args, **kwargs):
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*args, **kwargs)


def _is_sharded(model) -> bool:
    return hasattr(model, "full_state_dict") and hasattr(model, "full_optim_state_dict")


def get_trainable_state_dict(model, optimizer, scheduler, use_fsdp: bool = False,
                             trainable_param_names: Optional[list] = None,
                             save_only_model: bool = False,
                             compute_dtype: torch.dtype = torch.bfloat16) -> Optional[dict]:
    """State to persist, or None on ranks that do not write (data-parallel rank > 0)."""
    sched_sd = scheduler.state_dict() if scheduler is not None else None
    if use_fsdp or _is_sharded(model):
        model_sd = model.full_state_dict(rank0_only=True)
        if save_only_model:
            optim_sd = None
            if model_sd is not None:
                model_sd = {k: v.to(compute_dtype) for k, v in model_sd.items()}
        else:
            optim_sd = model.full_optim_state_dict(optimizer, rank0_only=True)
        names = trainable_param_names
    else:
        model_sd = model.state_dict()
        optim_sd = None if (save_only_model or optimizer is None) else optimizer.state_dict()
        names = [n for n, p in model.named_parameters() if p.requires_grad]
        if save_only_model:
            model_sd = {k: v.to(compute_dtype) if v.is_floating_point() else v
                        for k, v in model_sd.items()}
    if get_data_parallel_rank() != 0:
        return None
    if names is not None:
        missing = [n for n in names if n not in model_sd]
        if missing:
            rank0_print(f"Missing {len(missing)} parameters in model state dict:", *missing)
            raise ValueError("Missing parameters in model state dict")
        model_sd = {n: model_sd[n] for n in model_sd if n in set(names)}
    return {"model": model_sd, "optimizer": optim_sd, "scheduler": sched_sd}


def _step_of(filename: str) -> int:
    m = re.search(r"step_(\d+)", filename)
    if not m:
        raise ValueError(f"Invalid checkpoint filename: {filename}")
    return int(m.group(1))


def save_checkpoint(checkpoint_path: str, model, optimizer, scheduler, epoch: int,
                    global_step: int, rank: int, save_only_model: bool, save_total_limit: int,
                    use_fsdp: bool = False, trainable_param_names: Optional[list] = None,
                    prefix: str = "", metrics: Optional[dict] = None,
                    compute_dtype: torch.dtype = torch.bfloat16) -> None:
    """``rank`` is the tensor-parallel rank: every TP rank writes its own shard file."""
    state = get_trainable_state_dict(model, optimizer, scheduler, use_fsdp,
                                     trainable_param_names, save_only_model, compute_dtype)
    if state is not None:
        if save_only_model:
            state = {"model": state["model"]}
        state["epoch"] = epoch or -1
        state["global_step"] = global_step
        if metrics is not None:
            state["metrics"] = metrics
        tmp = checkpoint_path + ".tmp"
        torch.save(state, tmp)
        os.replace(tmp, checkpoint_path)  # a crash never leaves a truncated checkpoint behind
    if dist.is_initialized():
        dist.barrier()
    if state is None:
        return
    save_dir = os.path.dirname(checkpoint_path)
    if rank == 0:
        with open(os.path.join(save_dir, f"{prefix}last_checkpoint"), "w") as fh:
            fh.write(os.path.basename(checkpoint_path).replace("_rank_0", "_rank*"))
    if save_total_limit is not None:
        mine = sorted(glob.glob(os.path.join(save_dir, f"{prefix}*_rank_{rank}.pt")),
                      key=_step_of)
        while len(mine) > save_total_limit:
            victim = mine.pop(0)
            rank0_print(f"Removing {victim.replace('_rank_0', '_rank*')}")
            os.remove(victim)


class CheckpointError(RuntimeError):
    """A checkpoint shard is missing or unreadable (truncated, corrupt)."""


def read_checkpoint_file(path: str, **load_kwargs):
    """``torch.load`` with errors a user can act on: which shard is missing, or which file is
    damaged. Training writes each shard to a temporary name and renames it, so a damaged file
    means the storage lost data after the write, not that a save was interrupted."""
    if not os.path.isfile(path):
        raise CheckpointError(f"checkpoint shard {path} does not exist (every tensor-parallel "
                              "rank reads its own *_rank_<k>.pt)")
    try:
        return torch.load(path, **load_kwargs)
    except Exception as e:  # noqa: BLE001 -- zip / pickle / EOF errors of a damaged file
        raise CheckpointError(f"checkpoint shard {path} cannot be read ({type(e).__name__}: "
                              f"{str(e)[:200]}); the file is truncated or corrupt") from e


def _checkpoint_tp_size(checkpoint_path: str, load_rank: int) -> Tuple[str, int]:
    pattern = checkpoint_path.replace(f"_rank_{load_rank}", "_rank_*")
    return pattern, len(glob.glob(pattern))


def load_checkpoint(checkpoint_path: str, model, optimizer=None, scheduler=None,
                    use_fsdp: bool = False) -> dict:
    """Resume training state. The tensor-parallel degree must match the checkpoint's."""
    load_rank, world = get_model_parallel_rank(), get_model_parallel_world_size()
    _, ckpt_world = _checkpoint_tp_size(checkpoint_path, load_rank)
    if ckpt_world != world:
        raise ValueError("The model parallel setting of resuming training does not match the "
                         f"current setting: {ckpt_world} (train) vs {world} (resume)")
    state = read_checkpoint_file(checkpoint_path, map_location="cpu", mmap=True,
                                 weights_only=False)
    if use_fsdp or _is_sharded(model):
        model.load_full_state_dict(state["model"], strict=False)
        if optimizer is not None and state.get("optimizer") is not None:
            model.load_full_optim_state_dict(state["optimizer"], optimizer)
    else:
        model.load_state_dict(state["model"], strict=False)
        if optimizer is not None and state.get("optimizer") is not None:
            optimizer.load_state_dict(state["optimizer"])
    if scheduler is not None:
        if state.get("scheduler") is not None:
            scheduler.load_state_dict(state["scheduler"])
        else:
            scheduler.step(state["global_step"])
    out = {"epoch": state["epoch"], "global_step": state["global_step"]}
    if "metrics" in state:
        out["metrics"] = state["metrics"]
    return out


# ----------------------------------------------------------------------------- TP resharding

_HEADS_BY_HIDDEN = {4096: (32, 32), 5120: (40, 40), 6656: (52, 52), 8192: (64, 8)}


def _qkv_heads(weight: torch.Tensor, heads: Optional[Tuple[int, int]]) -> Tuple[int, int]:
    """(query heads, kv heads) of the full model: given, or -- like the reference
    (checkpoint_utils.py:397-408) -- inferred from the hidden size."""
    if heads is not None:
        return heads
    hidden = weight.size(1)
    if hidden not in _HEADS_BY_HIDDEN:
        raise ValueError(f"cannot infer head counts for hidden size {hidden}; pass heads=")
    return _HEADS_BY_HIDDEN[hidden]


def _shard_axis(key: str) -> Optional[int]:
    if "wo" in key or "w2" in key or "output.weight" in key:
        return 1
    if "norm" in key or "tok_embeddings" in key:
        return None
    return 0


def merge_tp_checkpoint(all_state_dict: List[Dict[str, torch.Tensor]],
                        heads: Optional[Tuple[int, int]] = None) -> Dict[str, torch.Tensor]:
    """Concatenate the shards of consecutive tensor-parallel ranks into one (larger) shard."""
    merged = {}
    for key in list(all_state_dict[0].keys()):
        parts = [sd[key] for sd in all_state_dict]
        if "wqkv" in key:
            # q : k : v row ratio is n_head : n_kv : n_kv in every shard
            nh, nkv = _qkv_heads(parts[0], heads)
            unit = parts[0].size(0) // (nh + 2 * nkv)
            splits = [unit * nh, unit * nkv, unit * nkv]
            segs = [p.split(splits, dim=0) for p in parts]
            merged[key] = torch.cat([torch.cat([s[i] for s in segs], dim=0) for i in range(3)],
                                    dim=0)
        else:
            axis = _shard_axis(key)
            merged[key] = parts[0] if axis is None else torch.cat(parts, dim=axis)
        for sd in all_state_dict:
            del sd[key]
    return merged


def split_tp_checkpoint(full_state_dict: Dict[str, torch.Tensor], split_factor: int,
                        split_idx: int,
                        heads: Optional[Tuple[int, int]] = None) -> Dict[str, torch.Tensor]:
    """Cut shard ``split_idx`` of ``split_factor`` out of a (larger) shard."""
    out = {}
    for key in list(full_state_dict.keys()):
        w = full_state_dict[key]
        if "wqkv" in key:
            nh, nkv = _qkv_heads(w, heads)
            unit = w.size(0) // (nh + 2 * nkv)
            segs = w.split([unit * nh, unit * nkv, unit * nkv], dim=0)
            out[key] = torch.cat([torch.tensor_split(s, split_factor, dim=0)[split_idx]
                                  for s in segs], dim=0)
        else:
            axis = _shard_axis(key)
            out[key] = w if axis is None else torch.tensor_split(w, split_factor,
                                                                 dim=axis)[split_idx]
        del full_state_dict[key]
    return out


def load_inference_checkpoint(checkpoint_path: str, model: torch.nn.Module):
    """Load the ``model`` part of a training checkpoint into ``model``, resharding when the
    checkpoint was written with a different tensor-parallel degree."""
    if not dist.is_initialized():
        state = read_checkpoint_file(checkpoint_path, map_location="cpu",
                                     weights_only=False)["model"]
    else:
        rank, world = get_model_parallel_rank(), get_model_parallel_world_size()
        if f"_rank_{rank}" not in checkpoint_path:
            raise ValueError(f"Invalid checkpoint path: {checkpoint_path} for rank {rank}")
        pattern, ckpt_world = _checkpoint_tp_size(checkpoint_path, rank)
        assert ckpt_world > 0, f"No checkpoint found: '{pattern}'"

        def read(i):
            sd = read_checkpoint_file(pattern.replace("*", str(i)), map_location="cpu",
                                      mmap=True, weights_only=False)["model"]
            return {k: v.cpu() for k, v in sd.items()}

        if ckpt_world == world:
            state = read(rank)
        elif ckpt_world > world:
            assert ckpt_world % world == 0
            f = ckpt_world // world
            state = merge_tp_checkpoint([read(rank * f + i) for i in range(f)])
        else:
            assert world % ckpt_world == 0
            f = world // ckpt_world
            state = split_tp_checkpoint(read(rank // f), f, rank % f)
    if state and all(k.startswith("module.") for k in state):
        state = {k[len("module."):]: v for k, v in state.items()}
    own = model.state_dict()
    for key in list(state.keys()):
        if key in own and own[key].size() != state[key].size():
            rank0_print("Warning: removing", key, "from checkpoint.")
            del state[key]
    model.load_state_dict(state, strict=False)
    return None, None


# ----------------------------------------------------------------------------- paths / hook

def get_checkpoint_path(checkpoint_dir: str, epoch: Optional[int], global_step: int,
                        tp_rank: int, prefix: str) -> str:
    if epoch is None:
        return f"{checkpoint_dir}/{prefix}step_{global_step}_rank_{tp_rank}.pt"
    return f"{checkpoint_dir}/{prefix}epoch_{epoch}_step_{global_step}_rank_{tp_rank}.pt"


def get_latest_checkpoint_path(checkpoint_dir, prefix: Optional[str] = None):
    """(path for this TP rank or None, epoch or None, global_step)."""
    prefix = prefix or ""
    if checkpoint_dir is None:
        return None, 0, 0
    marker = os.path.join(str(checkpoint_dir), f"{prefix}last_checkpoint")
    if not os.path.exists(marker):
        return None, 0, 0
    with open(marker) as fh:
        name = fh.read().strip().split("/")[-1]
    rank = get_model_parallel_rank() if dist.is_initialized() else 0
    path = os.path.join(str(checkpoint_dir), name).replace("_rank*", f"_rank_{rank}")
    epoch = None
    if "epoch_" in name:
        m = re.search(r"epoch_(\d+)", name)
        if not m:
            raise ValueError(f"Invalid checkpoint filename: {name}")
        epoch = int(m.group(1))
    return path, epoch, _step_of(name)


def checkpoint_hook(args, model, optimizer, scheduler, epoch: int, global_step: int,
                    epoch_length: int, use_fsdp: bool = False,
                    trainable_param_names: Optional[list] = None, prefix: str = "",
                    metrics: Optional[dict] = None) -> None:
    """Save according to ``args.save_strategy``: ``no`` | ``epoch`` | ``steps`` | a metric name
    (the caller passes ``metrics`` when a new best value was reached)."""
    if args.save_strategy == "no":
        return
    rank = get_model_parallel_rank() if dist.is_initialized() else 0
    os.makedirs(args.save_dir, exist_ok=True)
    if args.save_strategy == "epoch":
        due = global_step != 0 and global_step % epoch_length == 0
    elif args.save_strategy == "steps":
        due = global_step != 0 and global_step % args.save_steps == 0
    elif metrics is not None:
        due = True
    else:
        raise ValueError(f"Invalid save strategy: {args.save_strategy}")
    if not due:
        return
    path = get_checkpoint_path(str(args.save_dir), epoch, global_step, rank, prefix)
    save_checkpoint(path, model, optimizer, scheduler, epoch, global_step, rank,
                    args.save_only_model, args.save_total_limit, use_fsdp, trainable_param_names,
                    prefix, metrics, args.compute_dtype)


# ----------------------------------------------------------------------------- model loaders

def _refuse_quantised(path: Path) -> None:
    for tag in ("int8", "int4"):
        if tag in str(path):
            raise NotImplementedError(f"{tag} quantization cannot be used for finetuning!")


def _load_base(model: torch.nn.Module, checkpoint_path: Path) -> None:
    sd = torch.load(str(checkpoint_path), mmap=True, weights_only=True)
    model.load_state_dict(sd, assign=True)


def load_model_from_from_ckpt(checkpoint_path: Path, sft_checkpoint_path: Optional[Path],
                              device, precision: torch.dtype, use_tp: bool, requires_grad: bool,
                              skip_init: bool = False, sequence_parallel: bool = False,
                              vocab_parallel: bool = False, tp_override=None):
    """Policy / SFT model: meta build from the directory name, mmap load, TP sharding, optional
    warm start from the latest fine-tuned checkpoint (with TP resharding). ``tp_override``
    = (group, ranks, size, rank) shards over that group instead of the job's tensor-parallel
    one (the rollout copy of a PPO policy, ``parallel.groups.get_rollout_parallel``)."""
    checkpoint_path = Path(checkpoint_path)
    _refuse_quantised(checkpoint_path)
    with torch.device("meta"):
        model = Transformer.from_name(checkpoint_path.parent.name, freeze_tok_embeddings=True,
                                      freeze_output=True, freeze_norm=True,
                                      vocab_parallel=vocab_parallel)
    _load_base(model, checkpoint_path)
    if use_tp and tp_override is not None:
        g, _, size, rank = tp_override
        rank0_print(f"Applying tensor parallel ({size} ranks, rollout group) to model ...")
        apply_tp(model, requires_grad=requires_grad, sequence_parallel=False, world=size,
                 rank=rank, group=g)
        skip_init = True      # fine-tuned shards follow the training layout; weights are synced
    elif use_tp:
        rank0_print("Applying tensor parallel to model ...")
        apply_tp(model, requires_grad=requires_grad, sequence_parallel=sequence_parallel)
    if not skip_init:
        path, _, _ = get_latest_checkpoint_path(sft_checkpoint_path)
        if path is not None:
            rank0_print(f"Loading sft model from {path.replace('_rank_0', '_rank_*')} ...")
            load_inference_checkpoint(path, model)
        else:
            rank0_print("Warning: no sft checkpoint found, using base checkpoint.")
    model.requires_grad_(requires_grad)
    return model.to(device=device, dtype=precision).train(requires_grad)


def _build_reward_model(checkpoint_path: Path, vocab_parallel: bool):
    from ..models.reward_model import RewardModel
    with torch.device("meta"):
        model = RewardModel.from_name(checkpoint_path.parent.name, freeze_tok_embeddings=True,
                                      freeze_norm=True, vocab_parallel=vocab_parallel)
    _load_base(model.backbone_model, checkpoint_path)
    return model


def load_reward_model_from_ckpt(checkpoint_path: Path, rm_checkpoint_path: Optional[Path], device,
                                precision: torch.dtype, use_tp: bool, requires_grad: bool,
                                skip_init: bool = False, sequence_parallel: bool = False,
                                vocab_parallel: bool = False):
    """Reward / value model: backbone from the base checkpoint, 2-row head, head TP, then the
    latest reward-model checkpoint on top."""
    from ..models.reward_model import apply_reward_modeling_head
    checkpoint_path = Path(checkpoint_path)
    _refuse_quantised(checkpoint_path)
    model = _build_reward_model(checkpoint_path, vocab_parallel)
    if use_tp:
        apply_tp(model.backbone_model, requires_grad=requires_grad,
                 sequence_parallel=sequence_parallel)
    apply_reward_modeling_head(model.backbone_model, requires_grad=requires_grad)
    if use_tp:
        apply_reward_head_tp(model.backbone_model, requires_grad=requires_grad)
    if not skip_init:
        path, _, _ = get_latest_checkpoint_path(rm_checkpoint_path)
        if path is not None:
            rank0_print(f"Loading reward model from {path.replace('_rank_0', '_rank_*')} ...")
            load_inference_checkpoint(path, model)
        else:
            rank0_print("Warning: no rm checkpoint found, using base checkpoint.")
    model.requires_grad_(requires_grad)
    return model.to(device=device, dtype=precision).train(requires_grad)


def load_reward_model_from_sft_ckpt(checkpoint_path: Path, sft_checkpoint_path: Optional[Path],
                                    device, precision: torch.dtype, use_tp: bool,
                                    requires_grad: bool, reward_head_init_scheme: str = "zeros",
                                    sequence_parallel: bool = False,
                                    vocab_parallel: bool = False):
    """Reward model initialised from an SFT policy: backbone weights from the SFT checkpoint,
    then a fresh reward head (``zeros`` | ``semantic`` | ``random``)."""
    from ..models.reward_model import apply_reward_modeling_head
    checkpoint_path = Path(checkpoint_path)
    _refuse_quantised(checkpoint_path)
    model = _build_reward_model(checkpoint_path, vocab_parallel)
    if use_tp:
        apply_tp(model.backbone_model, requires_grad=True, sequence_parallel=sequence_parallel)
    path, _, _ = get_latest_checkpoint_path(sft_checkpoint_path)
    if path is not None:
        rank0_print("Loading sft model ...")
        load_inference_checkpoint(path, model.backbone_model)
    apply_reward_modeling_head(model.backbone_model, requires_grad=requires_grad,
                               init_sceheme=reward_head_init_scheme)
    if use_tp:
        apply_reward_head_tp(model.backbone_model, requires_grad=requires_grad)
    model.requires_grad_(requires_grad)
    return model.to(device=device, dtype=precision).train(requires_grad)
