"""Sharded data parallelism (ZeRO-3 style) for the LLaMA block stack, replacing the reference's
PyTorch-FSDP1 wrapping (training_utils/trainer_utils.py:70-99, ppo_trainer.py:1357-1392).

Layout. Every transformer block (plus one "root" unit for any other trainable tensor, e.g. a
reward head) owns one flat parameter: the trainable tensors of the block concatenated, padded
to a multiple of the data-parallel world size and split evenly. Each rank keeps

* ``shard``      fp32 (``param_dtype``) master copy of its slice -- what the optimizer updates,
* ``shard_lp``   the same slice in ``compute_dtype`` (bf16) -- what is all-gathered; refreshed by
                 the fused Adam kernel in the same pass that updates the master copy,
* ``shard.grad`` fp32 accumulator of the reduce-scattered gradient.

Step. ``forward`` walks the blocks; for block i the flat bf16 parameter is all-gathered into one
of two rotating buffers (the gather of block i+1 is issued on a side stream while block i
computes), the block runs with activation checkpointing semantics (only its input is saved),
and in the backward pass the parameter is gathered again, the block is recomputed and
back-propagated, its weight gradients land in one flat bf16 buffer that is reduce-scattered
(averaged over the group) into ``shard.grad``.

On CUDA the block itself is ``models.fused_block`` (explicit kernel sequence); on CPU (gloo
plumbing tests) it is the ``TransformerBlock`` module under ``torch.autograd``.

The wrapper also produces the data-parallel-unsharded views that checkpoints need
(``full_state_dict`` / ``full_optim_state_dict`` keyed by parameter name, and their loaders),
so checkpoint files stay in the reference's format.
"""
from __future__ import annotations

import math
from typing import Dict, Iterator, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as Fn
from . import collectives as coll
from . import groups

BLOCK_PARAM_ORDER = ("attention.wqkv", "attention.wo", "feed_forward.w1", "feed_forward.w3",
                     "feed_forward.w2")


def _group_size(group) -> Tuple[int, int]:
    if group is None or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


class ShardUnit:
    """One flat parameter: a list of (fqn, nn.Parameter) sharded over the data-parallel group."""

    def __init__(self, named_params: List[Tuple[str, nn.Parameter]], group, param_dtype,
                 compute_dtype, reduce_dtype):
        self.group = group
        self.world, self.rank = _group_size(group)
        self.names = [n for n, _ in named_params]
        self.params = [p for _, p in named_params]
        self.shapes = [tuple(p.shape) for p in self.params]
        self.numels = [p.numel() for p in self.params]
        self.offsets = [0]
        for n in self.numels:
            self.offsets.append(self.offsets[-1] + n)
        self.total = self.offsets[-1]
        self.shard_size = -(-self.total // self.world)
        # keep shards 16-byte aligned in bf16 for the gather / TMA consumers
        self.shard_size = -(-self.shard_size // 8) * 8
        self.padded = self.shard_size * self.world
        self.compute_dtype, self.reduce_dtype = compute_dtype, reduce_dtype
        dev = self.params[0].device
        flat = torch.zeros(self.padded, dtype=param_dtype, device=dev)
        for p, o, n in zip(self.params, self.offsets, self.numels):
            flat[o:o + n] = p.data.reshape(-1).to(param_dtype)
        lo = self.rank * self.shard_size
        self.shard = nn.Parameter(flat[lo:lo + self.shard_size].clone())
        self.shard_lp = self.shard.data.to(compute_dtype)
        if compute_dtype != param_dtype:
            # the fused AdamW kernel refreshes the low-precision copy while it updates the master
            self.shard._lp_copy = self.shard_lp
        del flat
        for p in self.params:             # the full tensors only exist while gathered
            p.data = torch.empty(0, dtype=compute_dtype, device=dev)
        self.gathered_in: Optional[torch.Tensor] = None
        self.lp_symm = None        # (SymmetricBuffer, byte offset) once shard_lp lives in one
        self.lp_peers = None       # index of each rank of this group inside that buffer's group

    def move_lp_to(self, sbuf, offset: int, peers=None) -> None:
        """Re-home the low-precision shard into symmetric memory (peers read it directly).
        ``peers``: for a buffer shared by a larger group than this unit's, the position of each
        rank of the unit's group inside that larger group."""
        self.lp_peers = list(peers) if peers is not None else None
        view = sbuf.view(offset, (self.shard_size,), self.compute_dtype)
        view.copy_(self.shard_lp)
        self.shard_lp = view
        if hasattr(self.shard, "_lp_copy"):
            self.shard._lp_copy = view
        self.lp_symm = (sbuf, offset)

    # -------------------------------------------------------------- parameters
    def gather_into(self, buf: torch.Tensor) -> None:
        """All-gather the bf16 shards into ``buf`` and point the parameters at views of it."""
        full = buf[: self.padded]
        if self.world > 1 and self.lp_symm is not None:
            # pull every rank's bf16 shard straight out of its symmetric memory (NVLink loads in
            # our own kernel); the shards only change at optimizer steps, which are fenced by
            # barriers on both sides (ShardedDataParallel.finish_backward / after_optimizer_step)
            import ctypes as C
            from ..ops import _lib
            sbuf, off = self.lp_symm
            arr = (C.c_void_p * 8)()
            for r in range(self.world):
                arr[r] = sbuf.peer_ptr(self.lp_peers[r] if self.lp_peers else r, off)
            rc = _lib.lib().e2h_p2p_all_gather(arr, self.world, full.data_ptr(),
                                               self.shard_size * 2, None, None, None, 0,
                                               _lib.status_word(full.device).data_ptr(),
                                               _lib.stream())
            _lib.check(rc, "p2p_all_gather")
        elif self.world > 1:
            dist.all_gather_into_tensor(full, self.shard_lp, group=self.group)
        else:
            full.copy_(self.shard_lp)
        for p, o, n, shp in zip(self.params, self.offsets, self.numels, self.shapes):
            p.data = full[o:o + n].view(shp)
        self.gathered_in = buf

    def release(self) -> None:
        for p in self.params:
            p.data = torch.empty(0, dtype=self.compute_dtype, device=p.device)
        self.gathered_in = None

    def grad_views(self, gradbuf: torch.Tensor) -> Dict[str, torch.Tensor]:
        full = gradbuf[: self.padded]
        return {n: full[o:o + k].view(shp)
                for n, o, k, shp in zip(self.names, self.offsets, self.numels, self.shapes)}

    def reduce_grads(self, gradbuf: torch.Tensor) -> None:
        """Average the flat gradient over the group and add this rank's slice to shard.grad."""
        full = gradbuf[: self.padded]
        if self.padded > self.total:
            full[self.total:].zero_()
        if self.world > 1:
            red = full.to(self.reduce_dtype) if full.dtype != self.reduce_dtype else full
            out = torch.empty(self.shard_size, dtype=red.dtype, device=red.device)
            if red.device.type == "cpu":
                dist.all_reduce(red, group=self.group)
                out.copy_(red[self.rank * self.shard_size:(self.rank + 1) * self.shard_size])
            else:
                dist.reduce_scatter_tensor(out, red, group=self.group)
            out = out.to(self.shard.dtype).div_(self.world)
        else:
            out = full[: self.shard_size].to(self.shard.dtype)
        if self.shard.grad is None:
            self.shard.grad = out.clone() if out.data_ptr() == full.data_ptr() else out
        else:
            self.shard.grad.add_(out)

    def reduce_grads_p2p(self, rs, slot: int, fresh: Optional[bool] = None) -> None:
        """Same result as ``reduce_grads`` through the fused kernel of ``ops/csrc/comm.cu``: the
        flat bf16 gradient already sits in slot ``slot`` of the symmetric buffers ``rs``; raise
        the flags, then pull this rank's slice from every rank, average in fp32 and write (or
        add to) ``shard.grad`` in one pass. ``fresh`` says that ``shard.grad`` was just created
        by the caller (on its own stream) and is to be written, not added to."""
        if self.padded > self.total:
            rs.grad_buffer(slot)[self.total:self.padded].zero_()
        rs.signal(slot)
        if fresh is None:
            fresh = self.shard.grad is None
            if fresh:
                self.shard.grad = torch.empty_like(self.shard.data)
        rs.reduce(slot, self.rank * self.shard_size, self.shard_size, self.shard.grad,
                  1.0 / self.world, accumulate=not fresh)

    def refresh_low_precision(self) -> None:
        """After an update of the master shard that did not write the low-precision copy."""
        self.shard_lp.copy_(self.shard.data)

    # -------------------------------------------------------------- full (unsharded) views
    def full_flat(self, src_shard: torch.Tensor) -> torch.Tensor:
        """Gather any per-rank shard-shaped tensor (master weights, Adam moments) to full size."""
        if self.world == 1:
            return src_shard.detach().clone()
        out = torch.empty(self.padded, dtype=src_shard.dtype, device=src_shard.device)
        dist.all_gather_into_tensor(out, src_shard.detach().contiguous(), group=self.group)
        return out

    def split_full(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {n: flat[o:o + k].view(shp).clone()
                for n, o, k, shp in zip(self.names, self.offsets, self.numels, self.shapes)}

    def load_named(self, state: Dict[str, torch.Tensor], into: torch.Tensor) -> List[str]:
        """Write this rank's slice of the named full tensors into a shard-shaped tensor."""
        lo, hi = self.rank * self.shard_size, (self.rank + 1) * self.shard_size
        missing = []
        for n, o, k in zip(self.names, self.offsets, self.numels):
            if n not in state:
                missing.append(n)
                continue
            a, b = max(o, lo), min(o + k, hi)
            if a < b:
                src = state[n].reshape(-1)[a - o:b - o]
                into.data[a - lo:b - lo] = src.to(device=into.device, dtype=into.dtype)
        return missing


class _BlockFn(torch.autograd.Function):
    """Checkpointed, parameter-gathering execution of one block."""

    @staticmethod
    def forward(ctx, x, sdp, idx, B, S):
        ctx.sdp, ctx.idx, ctx.BS = sdp, idx, (B, S)
        # position tables of this forward call (several calls may precede one backward)
        ctx.tables = (sdp._input_pos, sdp._freqs_pos, sdp._freqs, sdp._pos)
        ctx.save_for_backward(x)
        with torch.no_grad():
            # the budget is zero for forwards that need no backward (set in hidden_states)
            out, ctx.acts = sdp._run_block(idx, x, B, S, keep=True)
        return out

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        sdp = ctx.sdp
        sdp._input_pos, sdp._freqs_pos, sdp._freqs, sdp._pos = ctx.tables
        acts, ctx.acts = ctx.acts, None
        dx = ctx.sdp._backward_block(ctx.idx, x, dy.contiguous(), *ctx.BS, saved=acts)
        return dx, None, None, None, None


class ShardedDataParallel(nn.Module):
    _instances: List = []          # weak references, for sharing the activation budget

    def __init__(self, model: nn.Module, process_group=None, param_dtype=torch.float32,
                 compute_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16,
                 fused: Optional[bool] = None, keep_params: bool = False):
        """``keep_params``: the gathered low-precision parameters of every block stay resident
        between optimizer steps (gradients and optimizer state remain sharded): one all-gather
        per block and step instead of one per use. This is the reference's ``SHARD_GRAD_OP``
        choice for ``--slow_cross_node_comm`` (trainers/ppo_trainer.py:1384-1388)."""
        super().__init__()
        self.keep_params = keep_params
        import weakref
        ShardedDataParallel._instances.append(weakref.ref(self))
        self.module = model
        backbone = getattr(model, "backbone_model", model)
        self.backbone = backbone
        self.group = process_group
        self.world, self.rank = _group_size(process_group)
        dev = backbone.output.weight.device
        self.fused = (dev.type == "cuda") if fused is None else fused
        self.compute_dtype = compute_dtype if self.fused else param_dtype
        self.param_dtype = param_dtype
        if self.fused:
            # frozen tensors (embedding, norms, LM head, RoPE table) are only ever read by the
            # bf16 kernels
            for t in list(model.buffers()) + [p for p in model.parameters()
                                              if not p.requires_grad]:
                if t.is_floating_point() and t.dtype != compute_dtype:
                    t.data = t.data.to(compute_dtype)
        prefix = "backbone_model." if backbone is not model else ""
        self.units: List[ShardUnit] = []
        seen = set()
        for i, blk in enumerate(backbone.layers):
            named = []
            for rel in BLOCK_PARAM_ORDER:
                mod_name, _ = rel.split(".")
                p = getattr(getattr(blk, mod_name), rel.split(".")[1]).weight
                if isinstance(p, nn.Parameter) and p.requires_grad:
                    named.append((f"{prefix}layers.{i}.{rel}.weight", p))
                    seen.add(id(p))
            assert named, "every block must have trainable tensors"
            self.units.append(ShardUnit(named, process_group, param_dtype, self.compute_dtype,
                                        reduce_dtype if self.fused else param_dtype))
        rest = [(n, p) for n, p in model.named_parameters()
                if p.requires_grad and id(p) not in seen]
        self.root: Optional[ShardUnit] = None
        if rest:
            self.root = ShardUnit(rest, process_group, param_dtype, self.compute_dtype,
                                  reduce_dtype if self.fused else param_dtype)
        self._shards = nn.ParameterList([u.shard for u in self._all_units()])
        biggest = max(u.padded for u in self._all_units())
        if keep_params:      # one resident buffer per block
            self._param_bufs = [torch.empty(u.padded, dtype=self.compute_dtype, device=dev)
                                for u in self.units]
        else:                # two rotating buffers: the block in use and the prefetched one
            self._param_bufs = [torch.empty(biggest, dtype=self.compute_dtype, device=dev)
                                for _ in range(2)]
        self._resident = [False] * len(self.units)
        self.gathers = 0     # block all-gathers issued (what keep_params saves)
        self._grad_buf = torch.empty(biggest, dtype=self.compute_dtype, device=dev)
        # fused pull-based gradient reduce-scatter over peer memory (falls back to NCCL)
        self._rs = None
        self._lp_bar = None
        if (self.fused and self.world > 1 and param_dtype == torch.float32
                and self.compute_dtype == torch.bfloat16):
            from ..models.fused_block import p2p_reduce_enabled
            if p2p_reduce_enabled(process_group):
                from .symm import GradReduceScatter, P2PChannel, SymmetricBuffer
                self._rs = GradReduceScatter(biggest, process_group)
                # parameter all-gather as a pull over peer memory: every unit's bf16 shard lives
                # in one symmetric allocation
                sizes = [(u.shard_size * 2 + 255) // 256 * 256 for u in self._all_units()]
                self._lp_buf = SymmetricBuffer(sum(sizes), process_group)
                off = 0
                for u, nb in zip(self._all_units(), sizes):
                    u.move_lp_to(self._lp_buf, off)
                    off += nb
                self._lp_bar = P2PChannel(256, process_group)
                self._lp_bar.barrier()      # every rank's shards are in place
        self._root_buf = (torch.empty(self.root.padded, dtype=self.compute_dtype, device=dev)
                          if self.root else None)
        self._comm_stream = torch.cuda.Stream() if dev.type == "cuda" else None
        # the gradient reduce-scatter of block i runs on its own stream, under the backward
        # GEMMs of block i-1 (E2H_RS_OVERLAP=0 keeps it on the compute stream)
        import os
        self._rs_stream = (torch.cuda.Stream() if (dev.type == "cuda" and self._rs is not None
                           and os.environ.get("E2H_RS_OVERLAP", "1") != "0") else None)
        self._rs_events: Dict[int, "torch.cuda.Event"] = {}
        self._pending: Dict[int, "torch.cuda.Event"] = {}
        self._keep_budget = 0          # bytes of block intermediates kept per forward (0: recompute)
        self._keep_left = 0
        self._keep_planned = False
        self.micro_step = 0
        if self.root is not None:
            self.root.gather_into(self._root_buf)   # small: stays gathered

    # ------------------------------------------------------------------ plumbing
    def expose_shards(self, group=None) -> bool:
        """Make every unit's bf16 shard readable by all ranks of ``group`` (default: the world),
        not only by this wrapper's data-parallel group: the shards move into one symmetric
        allocation over ``group``. Needed by ``parallel.relayout.RolloutRelayout``, whose
        destination ranks pull from shards of other tensor-parallel columns. Collective over
        ``group``; returns False (nothing changed) where peer memory cannot reach all of it."""
        from .symm import SymmetricBuffer, peer_memory_usable
        dev = self.backbone.output.weight.device
        if dev.type != "cuda" or not dist.is_initialized() or not peer_memory_usable(group):
            return False
        if self.compute_dtype != torch.bfloat16:
            return False
        sizes = [(u.shard_size * 2 + 255) // 256 * 256 for u in self._all_units()]
        buf = SymmetricBuffer(sum(sizes), group)
        big = dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)
        mine = (dist.get_process_group_ranks(self.group) if self.group is not None
                else [dist.get_rank()])
        peers = [big.index(r) for r in mine]
        off = 0
        for u, nb in zip(self._all_units(), sizes):
            u.move_lp_to(buf, off, peers)
            off += nb
        self._lp_buf = buf
        if self._lp_bar is None and self.world > 1:
            from .symm import P2PChannel
            self._lp_bar = P2PChannel(256, self.group)
        torch.cuda.synchronize()
        dist.barrier(group)
        return True

    def _all_units(self) -> List[ShardUnit]:
        return self.units + ([self.root] if self.root is not None else [])

    def optimizer_parameters(self) -> Iterator[nn.Parameter]:
        return iter(u.shard for u in self._all_units())

    def grad_shards(self) -> Iterator[torch.Tensor]:
        return (u.shard.grad for u in self._all_units() if u.shard.grad is not None)

    def trainable_param_names(self) -> List[str]:
        return [n for u in self._all_units() for n in u.names]

    def _prefetch(self, idx: int) -> None:
        if not (0 <= idx < len(self.units)) or idx in self._pending:
            return
        if self.keep_params and self._resident[idx]:
            self._pending[idx] = None       # still gathered from an earlier use of this step
            return
        unit = self.units[idx]
        buf = self._param_bufs[idx if self.keep_params else idx % 2]
        self._resident[idx] = self.keep_params
        self.gathers += 1
        if self._comm_stream is None:
            unit.gather_into(buf)
            self._pending[idx] = None
            return
        self._comm_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._comm_stream):
            unit.gather_into(buf)
            ev = torch.cuda.Event()
            ev.record(self._comm_stream)
        self._pending[idx] = ev

    def _acquire(self, idx: int, nxt: int) -> ShardUnit:
        self._prefetch(idx)
        ev = self._pending.pop(idx)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        self._prefetch(nxt)        # overlaps with the compute of block idx
        return self.units[idx]

    def _block_weights(self, blk, unit: ShardUnit) -> Dict[str, torch.Tensor]:
        a, f = blk.attention, blk.feed_forward
        cd = self.compute_dtype
        return dict(wqkv=a.wqkv.weight.data, wo=a.wo.weight.data, w1=f.w1.weight.data,
                    w3=f.w3.weight.data, w2=f.w2.weight.data,
                    attention_norm=blk.attention_norm.weight.to(cd),
                    ffn_norm=blk.ffn_norm.weight.to(cd))

    def _shape(self, blk, B, S):
        from ..models.fused_block import BlockShape
        a = blk.attention
        return BlockShape(B, S, a.n_head, a.n_local_heads, a.head_dim, self.backbone.config.norm_eps,
                          tp=getattr(a, "tp_size", 1),
                          sequence_parallel=getattr(a, "sequence_parallel", False))

    def _run_block(self, idx: int, x: torch.Tensor, B: int, S: int, keep: bool = False):
        """One block forward. With ``keep`` (a training forward) the block's intermediates are
        kept for the backward while the activation budget lasts, instead of being recomputed:
        returns ``(out, saved or None)``."""
        unit = self._acquire(idx, idx + 1)
        blk = self.backbone.layers[idx]
        saved = None
        if self.fused:
            from ..models import fused_block as fb
            want = keep and self._keep_left > 0
            try:
                out, saved = fb.block_forward(x, self._block_weights(blk, unit), self._freqs,
                                              self._pos, self._shape(blk, B, S), keep=want)
            except torch.cuda.OutOfMemoryError:
                if not want or self.world > 1 or getattr(blk.attention, "tp_size", 1) > 1:
                    raise      # with peers, a one-sided retry would re-issue collectives
                # the budget was too optimistic: back to recomputation from here on
                self._keep_budget = self._keep_left = 0
                torch.cuda.empty_cache()
                out, saved = fb.block_forward(x, self._block_weights(blk, unit), self._freqs,
                                              self._pos, self._shape(blk, B, S), keep=False)
            if saved is not None:
                saved = {k: v for k, v in saved.items() if k not in ("act", "q", "k", "v")}
                nbytes = sum(t.numel() * t.element_size() for t in saved.values())
                if nbytes <= self._keep_left:
                    self._keep_left -= nbytes
                else:                      # does not fit: this block is recomputed instead
                    saved, self._keep_left = None, 0
        else:
            out = blk(x, self._input_pos, self._freqs_pos, None, True)
        if not self.keep_params:
            unit.release()
        return out, saved

    def _backward_block(self, idx: int, x: torch.Tensor, dy: torch.Tensor, B: int, S: int,
                        saved=None):
        unit = self._acquire(idx, idx - 1)
        blk = self.backbone.layers[idx]
        if self.fused:
            from ..models import fused_block as fb
            slot = self._rs.slot() if self._rs is not None else -1
            ev = self._rs_events.pop(slot, None)
            if ev is not None:      # the slot's previous reduce must have read it out
                torch.cuda.current_stream().wait_event(ev)
            gradbuf = self._rs.grad_buffer(slot) if self._rs is not None else self._grad_buf
            views = unit.grad_views(gradbuf)
            grads = {n.split(".")[-2]: v for n, v in views.items()}
            if saved is not None:          # q, k, v are views of the kept qkv
                shp = self._shape(blk, B, S)
                H, Hkv, D = shp.n_head, shp.n_kv, shp.head_dim
                qkv = saved["qkv"]
                saved["q"] = qkv[:, : H * D].view(B, S, H, D)
                saved["k"] = qkv[:, H * D: (H + Hkv) * D].view(B, S, Hkv, D)
                saved["v"] = qkv[:, (H + Hkv) * D:].view(B, S, Hkv, D)
            dx = fb.block_backward(dy, x, self._block_weights(blk, unit), grads, self._freqs,
                                   self._pos, self._shape(blk, B, S), saved=saved)
        else:
            for p in unit.params:
                p.grad = None
                p.requires_grad_(True)
            with torch.enable_grad():
                xin = x.detach().requires_grad_(True)
                out = blk(xin, self._input_pos, self._freqs_pos, None, True)
                torch.autograd.backward(out, dy)
            dx = xin.grad
            for (n, v), p in zip(unit.grad_views(self._grad_buf).items(), unit.params):
                v.copy_(p.grad if p.grad is not None else torch.zeros_like(v))
                p.grad = None
        if not self.keep_params:
            unit.release()
        if self.fused and self._rs is not None:
            if self._rs_stream is None:
                unit.reduce_grads_p2p(self._rs, slot)
            else:
                fresh = unit.shard.grad is None
                if fresh:           # created on the compute stream, which uses it later
                    unit.shard.grad = torch.empty_like(unit.shard.data)
                self._rs_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self._rs_stream):
                    unit.reduce_grads_p2p(self._rs, slot, fresh=fresh)
                    done = torch.cuda.Event()
                    done.record(self._rs_stream)
                self._rs_events[slot] = done
        else:
            unit.reduce_grads(self._grad_buf)
        return dx

    # ------------------------------------------------------------------ forward
    def hidden_states(self, idx: torch.Tensor) -> torch.Tensor:
        """Token ids [B, S] -> final-norm hidden states [B, S, dim] (differentiable w.r.t. the
        sharded block parameters)."""
        bb = self.backbone
        B, S = idx.shape
        dev = idx.device
        if bb.freqs_cis is None or bb.max_seq_length < S or bb.max_batch_size < B:
            bb.setup_caches(B, S, kv_cache=False)
        self._input_pos = torch.arange(S, device=dev)
        self._freqs_pos = bb.freqs_cis[:S]
        self._freqs = bb.freqs_cis
        self._pos = torch.arange(S, device=dev, dtype=torch.int32).repeat(B)
        self._pending.clear()
        self._keep_left = self._keep_budget if (torch.is_grad_enabled() and self.fused) else 0
        x = bb.embed(idx)
        sp = bb.sequence_parallel and bb.tp_size > 1 and self.training
        if sp:                       # rows of the batch are split over the tensor-parallel ranks
            x = coll.scatter_to_sequence_parallel(x)
        if self.fused:
            x = x.to(self.compute_dtype).reshape(-1, x.shape[-1])
        # the block function needs an input that is part of the graph to get a backward call
        x = x.detach().requires_grad_(True) if torch.is_grad_enabled() else x
        for i in range(len(bb.layers)):
            x = _BlockFn.apply(x, self, i, B, S)
        x = _rmsnorm_autograd(x, bb.norm.weight, bb.config.norm_eps)
        if sp:
            x = coll.gather_from_sequence_parallel(x, tensor_parallel_output_grad=False)
        return x.view(B, S, -1)

    def forward(self, idx: torch.Tensor, *args, **kwargs):
        """Same call convention as the wrapped model (logits for a ``Transformer``, rewards for
        a ``RewardModel``)."""
        hidden = self.hidden_states(idx)
        if self.backbone is not self.module:      # reward / value model
            rewards = self.module.token_rewards(hidden.to(self.backbone.output.weight.dtype))
            eos_pos = kwargs.get("eos_pos", args[0] if args else None)
            if eos_pos is not None:
                rewards = torch.gather(rewards, 1, eos_pos.unsqueeze(-1).long()).squeeze(-1)
            return rewards
        head = self.backbone.output
        if getattr(head, "tp_row_parallel", False):      # value head sharded over its input dim
            from ..models.tp import reward_head_forward
            return reward_head_forward(head, hidden.to(head.weight.dtype))
        return torch.nn.functional.linear(hidden, head.weight.to(hidden.dtype))

    def token_logprobs(self, idx: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                       temperature: float = 1.0):
        """(log p(labels[t]) per token [B, S], entropy [B, S]) without materialising logits."""
        from ..ops import loss
        hidden = self.hidden_states(idx)
        B, S, dim = hidden.shape
        w = self.backbone.output.weight
        lp, ent = loss.linear_logprobs(hidden.reshape(B * S, dim).to(w.dtype), w,
                                       labels.reshape(-1), ignore_index, temperature)
        return lp.view(B, S), ent.view(B, S)

    def logprobs_and_entropy(self, inputs: torch.Tensor, shifts, labels: torch.Tensor, tlen: int,
                             temperature: float, pad: int):
        """Log-probs and entropies of the last ``tlen`` positions of right-pad-rotated sequences
        (the hook ``models.rl_model.AutoregressivePolicy.forward`` looks for): hidden states are
        rotated back, positions ``[-tlen-1, -1)`` scored against ``labels`` through the fused
        LM-head loss. Differentiable w.r.t. the sharded parameters."""
        return lm_logprobs_and_entropy(self.backbone, self.hidden_states(inputs), shifts, labels,
                                       tlen, temperature, pad)

    def zero_grad(self, set_to_none: bool = True) -> None:
        for u in self._all_units():
            u.shard.grad = None

    def finish_backward(self) -> None:
        """Reduce the root unit's gradients (tensors outside the block stack). With parameter
        shards in peer-readable memory this is also the point where every rank has finished
        reading them for this step: a barrier before the optimizer may overwrite them."""
        for ev in self._rs_events.values():     # gradient reduces still running on their stream
            torch.cuda.current_stream().wait_event(ev)
        self._rs_events.clear()
        if self._lp_bar is not None:
            self._lp_bar.barrier()
        if self.root is None:
            return
        views = self.root.grad_views(self._grad_buf)
        for (n, v), p in zip(views.items(), self.root.params):
            v.copy_(p.grad if p.grad is not None else torch.zeros_like(v))
            p.grad = None
        self.root.reduce_grads(self._grad_buf)

    def plan_activation_budget(self, margin_bytes: int = 14 << 30) -> int:
        """How many bytes of block intermediates a training forward may keep for its backward
        instead of recomputing them (the reference always recomputes,
        models/model.py:233-243; with 180 GB per GPU the 7B model's 0.6 GB per block and
        micro-batch fit beside weights, gradients and optimizer state). Measured between steps,
        when only the static state is resident: free device memory plus what the caching
        allocator holds unused, minus ``margin_bytes`` for the transient buffers of a step.
        ``E2H_KEEP_ACTIVATIONS=0`` keeps the always-recompute behaviour, a number sets the
        budget in GiB."""
        import os
        env = os.environ.get("E2H_KEEP_ACTIVATIONS", "auto")
        dev = self.backbone.output.weight.device
        if not self.fused or dev.type != "cuda" or env == "0":
            self._keep_budget = 0
        elif env not in ("auto", "1", ""):
            self._keep_budget = int(float(env) * (1 << 30))
        else:
            free, _ = torch.cuda.mem_get_info(dev)
            cached = torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
            # several wrapped models in one process (PPO: policy and value) share what is left
            live = max(1, sum(1 for m in ShardedDataParallel._instances
                              if m() is not None and m().fused))
            self._keep_budget = max(0, int(free + cached - margin_bytes)) // live
        if dist.is_available() and dist.is_initialized() and dev.type == "cuda":
            # the same decision on every rank: a block that one tensor-parallel rank recomputes
            # (issuing its collectives again) must be recomputed by all of them
            t = torch.tensor([self._keep_budget], dtype=torch.int64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            self._keep_budget = int(t.item())
        return self._keep_budget

    def after_optimizer_step(self, lp_written: bool = False) -> None:
        """``lp_written``: the optimizer kernel already refreshed the low-precision shards."""
        if not self._keep_planned:
            # first optimizer step done: every piece of static state (moments, master weights,
            # gradient shards) now exists, so the memory left over can be measured
            self._keep_planned = True
            self.plan_activation_budget()
        if not lp_written:
            for u in self._all_units():
                u.refresh_low_precision()
        self._resident = [False] * len(self.units)     # resident copies are stale now
        self._lp_fence()
        if self.root is not None:
            self.root.gather_into(self._root_buf)

    def _lp_fence(self) -> None:
        """Every rank has written its low-precision shards before any rank pulls them."""
        if self._lp_bar is not None:
            self._lp_bar.barrier()

    # ------------------------------------------------------------------ checkpoints
    def full_state_dict(self, rank0_only: bool = True) -> Optional[Dict[str, torch.Tensor]]:
        out = {}
        for u in self._all_units():
            flat = u.full_flat(u.shard.data)
            if not rank0_only or self.rank == 0:
                out.update({k: v.cpu() for k, v in u.split_full(flat).items()})
        if rank0_only and self.rank != 0:
            return None
        for n, b in self.module.named_buffers():
            out.setdefault(n, b.detach().cpu())
        return out

    def load_full_state_dict(self, state: Dict[str, torch.Tensor], strict: bool = False):
        missing = []
        for u in self._all_units():
            missing += u.load_named(state, u.shard)
            u.refresh_low_precision()
        bufs = dict(self.module.named_buffers())
        for k, v in state.items():
            if k in bufs and bufs[k].shape == v.shape:
                bufs[k].data.copy_(v)
        self._resident = [False] * len(self.units)
        self._lp_fence()
        if self.root is not None:
            self.root.gather_into(self._root_buf)
        if strict and missing:
            raise KeyError(f"missing parameters: {missing}")
        return missing

    def full_optim_state_dict(self, optimizer, rank0_only: bool = True):
        """Optimizer state keyed by parameter name, data-parallel-unsharded:
        {"state": {fqn: {"step", "exp_avg", "exp_avg_sq"}}, "param_groups": [...]}"""
        state = {}
        for u in self._all_units():
            st = optimizer.state.get(u.shard, {})
            if not st:
                continue
            dev = u.shard.device
            m = u.split_full(u.full_flat(st["exp_avg"].to(dev)))
            v = u.split_full(u.full_flat(st["exp_avg_sq"].to(dev)))
            if not rank0_only or self.rank == 0:
                for n in u.names:
                    state[n] = {"step": int(st["step"]), "exp_avg": m[n].cpu(),
                                "exp_avg_sq": v[n].cpu()}
        if rank0_only and self.rank != 0:
            return None
        groups_ = [{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups]
        for g in groups_:
            g["params"] = list(state.keys())
        return {"state": state, "param_groups": groups_}

    def load_full_optim_state_dict(self, osd, optimizer) -> None:
        """Every rank reads the full state (from its own copy of the checkpoint file) and keeps
        its slice."""
        if osd is None:
            return
        for u in self._all_units():
            if not all(n in osd["state"] for n in u.names):
                continue
            st = optimizer.state[u.shard]
            ref = optimizer._new_state(u.shard) if hasattr(optimizer, "_new_state") else {
                "step": 0, "exp_avg": torch.zeros_like(u.shard),
                "exp_avg_sq": torch.zeros_like(u.shard)}
            for key in ("exp_avg", "exp_avg_sq"):
                tmp = torch.zeros_like(u.shard.data)
                u.load_named({n: osd["state"][n][key] for n in u.names}, tmp)
                ref[key].copy_(tmp.to(ref[key].dtype))
            ref["step"] = int(osd["state"][u.names[0]]["step"])
            st.update(ref)
        for g, saved in zip(optimizer.param_groups, osd.get("param_groups", [])):
            for k, v in saved.items():
                if k != "params":
                    g[k] = v


def lm_logprobs_and_entropy(backbone, hidden: torch.Tensor, shifts, labels: torch.Tensor,
                            tlen: int, temperature: float, pad: int):
    """hidden [B, L, dim] of right-pad-rotated sequences -> (logprobs, entropies) [B, tlen] of
    ``labels`` (0 where ``labels == pad``) at original positions ``[-tlen-1, -1)``."""
    from ..models.rl_model import restore_from_right_pad_sequences
    from ..ops import loss
    hidden = restore_from_right_pad_sequences(hidden, shifts)[:, -tlen - 1: -1]
    B = hidden.shape[0]
    from ..models.fused_block import dense_weight
    w = dense_weight(backbone.output)
    if w.dtype == torch.int8:            # CPU int8 module: dequantise in the activation dtype
        w = w.to(hidden.dtype) * backbone.output.scales.to(hidden.dtype)[:, None]
    kw = {}
    if backbone.vocab_parallel and backbone.tp_size > 1:
        kw = dict(vocab_start=groups.get_model_parallel_rank() * w.shape[0],
                  group=groups.get_model_parallel_group(), world=backbone.tp_size)
    lp, ent = loss.linear_logprobs(hidden.reshape(B * tlen, -1).to(w.dtype).contiguous(), w,
                                   labels.reshape(-1), pad, temperature, **kw)
    return lp.view(B, tlen), ent.view(B, tlen)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        ctx.save_for_backward(x, weight)
        ctx.eps = eps
        return Fn.rmsnorm(x, weight, eps)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        return Fn.rmsnorm_bwd(x, dy.contiguous(), weight, ctx.eps), None, None


def _rmsnorm_autograd(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _RMSNormFn.apply(x.contiguous(), weight.to(x.dtype), eps)
    from ..ops import reference
    return reference.rmsnorm(x, weight, eps)
