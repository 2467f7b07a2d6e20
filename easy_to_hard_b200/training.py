"""Supervised fine-tuning step shared by ``train_sft.py``, the benchmark and the smoke test.

Mirrors the reference loop (train_sft.py:72-116 loss, 330-362 micro-batching / clip / step,
425-449 batch preparation) on top of the sharded-data-parallel wrapper: next-token
cross-entropy over the non-ignored labels, gradient accumulation over micro batches, global
gradient-norm clipping to 1.0, AdamW, cosine schedule.

On CUDA the LM head and the loss are fused (``ops.loss.linear_cross_entropy``: no ``[tokens,
vocab]`` logits are kept), the clip coefficient stays on the device (the AdamW kernel applies
it), and the optimizer writes the bf16 compute copy of every shard as it updates the fp32
master.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .models import tp
from .ops import _lib, loss as loss_ops
from .parallel import groups
from .parallel.fsdp import ShardedDataParallel

IGNORE_INDEX = -100


def model_forward_with_loss(model, input_ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy of ``labels[:, 1:]`` under the model's prediction at ``[:, :-1]``."""
    B, S = input_ids.shape
    backbone = getattr(model, "backbone", model)
    if isinstance(model, ShardedDataParallel):
        hidden = model.hidden_states(input_ids)
    else:
        model.setup_caches(max_batch_size=B, max_seq_length=S, kv_cache=False)
        hidden = model(input_ids, torch.arange(S, device=input_ids.device), fully_causal=True,
                       return_hidden=True)
    w = backbone.output.weight
    # shift by moving the labels: position t is scored against token t+1, the last one is ignored
    tgt = torch.full_like(labels, IGNORE_INDEX)
    tgt[:, :-1] = labels[:, 1:]
    vp = backbone.vocab_parallel and backbone.tp_size > 1
    if hidden.is_cuda and hidden.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        kw = {}
        if vp:
            kw = dict(vocab_start=groups.get_model_parallel_rank() * w.shape[0],
                      group=groups.get_model_parallel_group(), world=backbone.tp_size)
        return loss_ops.linear_cross_entropy(hidden.reshape(B * S, -1), w, tgt.reshape(-1),
                                             IGNORE_INDEX, **kw)
    if vp:   # replicated hidden states feed a sharded head: the backward sums the shards
        from .parallel import collectives as coll
        hidden = coll.copy_to_tp(hidden)
    logits = F.linear(hidden.float(), w.float())
    if vp:
        return -tp.compute_vocab_parallel_logprobs(logits.view(B * S, -1), tgt.view(-1),
                                                   ignore_index=IGNORE_INDEX, reduction="mean")
    return F.cross_entropy(logits.view(B * S, -1), tgt.view(-1).long(),
                           ignore_index=IGNORE_INDEX, reduction="mean")


def gather_tp_batch(tensors, use_tp: bool, sync_group=None):
    """Make a batch identical on every rank of a tensor-parallel group by concatenating the
    ranks' batches along dim 0 (train_sft.py:436-447 of the reference)."""
    if not (use_tp and groups.get_model_parallel_world_size() > 1):
        return tuple(tensors)
    n = groups.get_model_parallel_world_size()
    group = sync_group if sync_group is not None else groups.get_model_parallel_group()
    out = []
    for t in tensors:
        t = t.contiguous()
        full = torch.empty((t.shape[0] * n, *t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(full, t, group=group)
        out.append(full)
    return tuple(out)


def prepare_batch(input_ids: torch.Tensor, labels: torch.Tensor, pad_id: int, unk_id: int,
                  use_tp: bool, sync_group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mask padded labels, replace a negative pad id in the inputs, pool the batch over the
    tensor-parallel group (train_sft.py:425-449 of the reference)."""
    labels = labels.masked_fill(labels == pad_id, IGNORE_INDEX)
    if pad_id < 0:
        input_ids = input_ids.masked_fill(input_ids == pad_id, unk_id)
    return gather_tp_batch((input_ids, labels), use_tp, sync_group)


class GradClipper:
    """Global L2 gradient-norm clipping whose coefficient never leaves the device: per-shard
    squared norms are accumulated by a reduction kernel, summed over all ranks (every trainable
    tensor is sharded over both the tensor- and the data-parallel group), turned into
    ``min(1, max_norm / (norm + 1e-6))`` by a one-thread kernel and consumed by the AdamW kernel."""

    def __init__(self, device):
        self.acc = torch.zeros(1, dtype=torch.float32, device=device)
        self.coef = torch.ones(1, dtype=torch.float32, device=device)
        self.norm = torch.zeros(1, dtype=torch.float32, device=device)

    def __call__(self, grads, max_norm: float) -> torch.Tensor:
        self.acc.zero_()
        lib = _lib.lib()
        for g in grads:
            code = {torch.float32: 0, torch.bfloat16: 1}[g.dtype]
            _lib.check(lib.e2h_sqnorm(g.data_ptr(), g.numel(), code, self.acc.data_ptr(),
                                      _lib.stream()), "sqnorm")
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self.acc)
        _lib.check(lib.e2h_clip_coef(self.acc.data_ptr(), float(max_norm), self.coef.data_ptr(),
                                     self.norm.data_ptr(), _lib.stream()), "clip_coef")
        return self.norm


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait (a peer's flag, a pipeline barrier) ran out during the step:
    what the kernels computed afterwards is not to be trusted."""


class TrainStepper:
    """zero_grad -> micro-batch forward/backward -> clip -> optimizer -> scheduler, for any
    ``loss_fn(model, *tensors)`` returning a loss or ``(loss, metrics)``."""

    def __init__(self, model, optimizer, scheduler=None, loss_fn=None, max_grad_norm: float = 1.0):
        self.model, self.optimizer, self.scheduler = model, optimizer, scheduler
        self.loss_fn = loss_fn or model_forward_with_loss
        self.max_grad_norm = max_grad_norm
        self.sharded = isinstance(model, ShardedDataParallel)
        dev = next(iter(model.parameters())).device
        self.clipper = GradClipper(dev) if (dev.type == "cuda" and self.sharded
                                            and hasattr(optimizer, "clip_coef")) else None
        self.metrics = None

    def step(self, *tensors: torch.Tensor, micro_batch_size: Optional[int] = None):
        """``tensors`` share dim 0 (the batch). Returns (loss of the last micro batch, gradient
        norm before clipping); both stay on the device. Metrics of the last micro batch, if the
        loss function returns any, are left in ``self.metrics``."""
        model = self.model
        model.zero_grad()
        n = tensors[0].shape[0]
        mb = micro_batch_size or n
        scale = 1.0 / (-(-n // mb))
        loss = None
        nvtx = torch.cuda.nvtx if torch.cuda.is_available() else None
        for a in range(0, n, mb):
            if nvtx:
                nvtx.range_push("forward_backward")
            out = self.loss_fn(model, *[t[a:a + mb] for t in tensors])
            if isinstance(out, tuple):
                loss, self.metrics = out
            else:
                loss = out
            (loss * scale).backward()
            if nvtx:
                nvtx.range_pop()
        if nvtx:
            nvtx.range_push("clip_and_optimizer")
        if self.sharded:
            model.finish_backward()
        self.check_device_status()
        if self.clipper is not None:
            grad_norm = self.clipper(list(model.grad_shards()), self.max_grad_norm)
            self.optimizer.clip_coef = self.clipper.coef
        else:
            grad_norm = tp.clip_grad_norm_(model, self.max_grad_norm)
        self.optimizer.step()
        if self.sharded:
            model.after_optimizer_step(lp_written=hasattr(self.optimizer, "clip_coef"))
        if self.scheduler is not None:
            self.scheduler.step()
        if nvtx:
            nvtx.range_pop()
        return loss.detach(), grad_norm


    def check_device_status(self) -> None:
        """Reads the kernels' status word (4 bytes, once per optimizer step, before the
        update is applied). The fused gradient reduce-scatter and the peer-memory barriers
        carry on after a time-out with whatever bytes sit in the peers' buffers, so a
        non-zero status means the gradients of this step are corrupt: raise instead of
        stepping. Callers that run under a ``HealthMonitor`` (``parallel.health.guarded_step``)
        publish the exception to the other ranks."""
        dev = next(iter(self.model.parameters())).device
        if dev.type != "cuda":
            return
        code = _lib.read_status(dev)
        if code != 0:
            raise DeviceWaitTimeout(f"a device-side wait timed out during the step (status "
                                    f"{code}); the optimizer update was not applied")


class SFTStepper(TrainStepper):
    def __init__(self, model, optimizer, scheduler=None, max_grad_norm: float = 1.0):
        super().__init__(model, optimizer, scheduler, model_forward_with_loss, max_grad_norm)

    def step(self, input_ids, labels, micro_batch_size: Optional[int] = None):
        return super().step(input_ids, labels, micro_batch_size=micro_batch_size)


def smoke_train_step(device="cuda:0"):
    """One SFT step of a tiny LLaMA through the sharded wrapper, fused kernels and AdamW."""
    from .models.model import ModelArgs, Transformer
    from .utils.memory_efficient_adam import MemoryEfficientAdamW
    torch.manual_seed(0)
    cfg = ModelArgs(block_size=256, vocab_size=512, n_layer=2, n_head=4, dim=512,
                    intermediate_size=1024)
    with torch.device(device):
        model = Transformer(cfg, freeze_tok_embeddings=True, freeze_output=True, freeze_norm=True)
    for _, t in list(model.named_parameters()) + list(model.named_buffers()):
        if t.dim() == 2:
            t.data.normal_(0.0, 0.02)
    model = model.to(torch.bfloat16)
    for p in model.parameters():
        p.data = p.data.float()
    sdp = ShardedDataParallel(model, process_group=None)
    sdp.train()
    opt = MemoryEfficientAdamW(list(sdp.optimizer_parameters()), lr=1e-4, optim_dtype=torch.bfloat16,
                               optim_device=torch.device(device))
    stepper = SFTStepper(sdp, opt)
    ids = torch.randint(0, cfg.vocab_size, (2, 128), device=device)
    loss, gn = stepper.step(ids, ids.clone())
    torch.cuda.synchronize()
    return float(loss), float(gn)


# ----------------------------------------------------------------------------- reward models

def pointwise_reward_loss(model, input_ids: torch.Tensor, labels: torch.Tensor,
                          weights: torch.Tensor) -> torch.Tensor:
    """Weighted binary cross-entropy of the per-token reward against per-token labels
    (train_rm_pointwise.py:78-112 of the reference): sum(w * bce) / (sum(w) + 1e-6)."""
    rewards = model(input_ids)
    loss = F.binary_cross_entropy_with_logits(rewards.float().view(-1), labels.float().view(-1),
                                              reduction="none")
    w = weights.float().view(-1)
    return (loss * w).sum() / (w.sum() + 1e-6)


def reward_modeling_metrics(logits: torch.Tensor, labels: torch.Tensor) -> dict:
    """accuracy / positive rates of ``logits >= 0`` against 0/1 labels
    (train_rm_pairwise.py:131-147 of the reference)."""
    pred = (logits >= 0.0).long()
    labels = labels.long()
    return dict(accuracy=pred.eq(labels).float().mean(),
                label_positive_rate=(labels == 1).float().mean(),
                positive_rate=(pred == 1).float().mean(),
                true_positive_rate=(pred * labels).float().sum() / labels.sum(),
                false_positive_rate=(pred * (1 - labels)).float().sum() / (1 - labels).sum())


def pairwise_reward_loss(model, input_ids: torch.Tensor, choice: torch.Tensor):
    """``input_ids`` [B, 2, T] (0-padded on the right), ``choice`` [B, 1]: BCE of
    ``reward(candidate 0) - reward(candidate 1)`` at the last non-pad token against ``choice``
    (train_rm_pairwise.py:80-128 of the reference). Returns (loss, metrics)."""
    B, C, T = input_ids.shape
    assert C == 2 and choice.shape == (B, 1)
    flat = input_ids.reshape(B * C, T)
    eos_pos = flat.ne(0).long().sum(dim=-1) - 1
    rewards = model(flat, eos_pos=eos_pos).view(B, C)
    logits = (rewards[:, 0] - rewards[:, 1]).float()
    loss = F.binary_cross_entropy_with_logits(logits.view(-1), choice.float().view(-1))
    return loss, reward_modeling_metrics(logits.detach().view(-1), choice.view(-1))


# ----------------------------------------------------------------------------- DPO

def sequence_logprobs(model, input_ids: torch.Tensor, labels: torch.Tensor):
    """Sum over the non-ignored positions of log p(labels[:, t+1] | input_ids[:, :t+1]) and the
    number of such positions, per sequence. Works for a sharded (trainable) policy and for a
    plain frozen ``Transformer``; on CUDA neither materialises the logits."""
    B, S = input_ids.shape
    tgt = torch.full_like(labels, IGNORE_INDEX)
    tgt[:, :-1] = labels[:, 1:]
    backbone = getattr(model, "backbone", model)
    if isinstance(model, ShardedDataParallel):
        hidden = model.hidden_states(input_ids)
    else:
        model.setup_caches(max_batch_size=B, max_seq_length=S, kv_cache=False)
        hidden = model(input_ids, torch.arange(S, device=input_ids.device), fully_causal=True,
                       return_hidden=True)
    w = backbone.output.weight
    vp = backbone.vocab_parallel and backbone.tp_size > 1
    kw = {}
    if vp:
        kw = dict(vocab_start=groups.get_model_parallel_rank() * w.shape[0],
                  group=groups.get_model_parallel_group(), world=backbone.tp_size)
    lp, _ = loss_ops.linear_logprobs(hidden.reshape(B * S, -1).to(w.dtype), w, tgt.reshape(-1),
                                     IGNORE_INDEX, **kw)
    count = (tgt != IGNORE_INDEX).float().sum(dim=-1)
    return lp.view(B, S).sum(dim=-1), count


def dpo_loss(model, ref_model, input_ids_w, labels_w, input_ids_l, labels_l, win_rate_w,
             win_rate_l, beta: float = 0.1, label_smoothing: float = 0.0, variant: str = "dpo"):
    """DPO and its variants (train_rl_dpo.py:77-196 of the reference): ``dpo`` (with optional
    conservative label smoothing), ``ipo``, ``rpo``; ``average`` in the variant name divides the
    sequence log-probs by their token counts. Returns (loss, metrics)."""
    with torch.no_grad():
        ref_w, n_w = sequence_logprobs(ref_model, input_ids_w, labels_w)
        ref_l, n_l = sequence_logprobs(ref_model, input_ids_l, labels_l)
    lp_w, _ = sequence_logprobs(model, input_ids_w, labels_w)
    lp_l, _ = sequence_logprobs(model, input_ids_l, labels_l)
    if "average" in variant:
        ref_w, ref_l = ref_w / (n_w + 1e-8), ref_l / (n_l + 1e-8)
        lp_w, lp_l = lp_w / (n_w + 1e-8), lp_l / (n_l + 1e-8)
    logits_1, logits_2 = lp_w - ref_w, lp_l - ref_l
    logits = logits_1 - logits_2
    win_rate_w, win_rate_l = win_rate_w.view(lp_w.shape).float(), win_rate_l.view(lp_l.shape).float()
    if "ipo" in variant:
        loss = (logits - 1.0 / (2 * beta)).pow(2).mean()
    elif "rpo" in variant:
        loss = ((logits_1 - (1.0 / beta) * (win_rate_w - 0.5)).pow(2).mean()
                + (logits_2 - (1.0 / beta) * (win_rate_l - 0.5)).pow(2).mean()) / 2.0
    elif label_smoothing == 0.0:
        loss = -F.logsigmoid(beta * logits).mean()
    else:
        loss = (-F.logsigmoid(beta * logits).mean() * (1 - label_smoothing)
                - F.logsigmoid(-beta * logits).mean() * label_smoothing)
    metrics = {"accuracy": (logits > 0.0).float().mean().detach(),
               "accuracy_policy": (lp_w > lp_l).float().mean().detach(),
               "accuracy_reference": (ref_w > ref_l).float().mean().detach()}
    return loss, metrics
