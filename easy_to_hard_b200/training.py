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


def prepare_batch(input_ids: torch.Tensor, labels: torch.Tensor, pad_id: int, unk_id: int,
                  use_tp: bool, sync_group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mask padded labels and make the batch identical on every rank of a tensor-parallel
    group by concatenating the ranks' batches (train_sft.py:425-449 of the reference)."""
    labels = labels.masked_fill(labels == pad_id, IGNORE_INDEX)
    if pad_id < 0:
        input_ids = input_ids.masked_fill(input_ids == pad_id, unk_id)
    if use_tp and groups.get_model_parallel_world_size() > 1:
        n = groups.get_model_parallel_world_size()
        group = sync_group if sync_group is not None else groups.get_model_parallel_group()
        ids = torch.empty((input_ids.shape[0] * n, input_ids.shape[1]), dtype=input_ids.dtype,
                          device=input_ids.device)
        lab = torch.empty_like(ids, dtype=labels.dtype)
        dist.all_gather_into_tensor(ids, input_ids.contiguous(), group=group)
        dist.all_gather_into_tensor(lab, labels.contiguous(), group=group)
        return ids, lab
    return input_ids, labels


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


class SFTStepper:
    """zero_grad -> micro-batch forward/backward -> clip -> optimizer -> scheduler."""

    def __init__(self, model, optimizer, scheduler=None, max_grad_norm: float = 1.0):
        self.model, self.optimizer, self.scheduler = model, optimizer, scheduler
        self.max_grad_norm = max_grad_norm
        self.sharded = isinstance(model, ShardedDataParallel)
        dev = next(iter(model.parameters())).device
        self.clipper = GradClipper(dev) if (dev.type == "cuda" and self.sharded
                                            and hasattr(optimizer, "clip_coef")) else None

    def step(self, input_ids: torch.Tensor, labels: torch.Tensor,
             micro_batch_size: Optional[int] = None):
        """Returns (loss of the last micro batch, gradient norm before clipping); both stay on
        the device."""
        model = self.model
        model.zero_grad()
        n = input_ids.shape[0]
        mb = micro_batch_size or n
        scale = 1.0 / (-(-n // mb))
        loss = None
        for a in range(0, n, mb):
            loss = model_forward_with_loss(model, input_ids[a:a + mb], labels[a:a + mb])
            (loss * scale).backward()
        if self.sharded:
            model.finish_backward()
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
        return loss.detach(), grad_norm


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
