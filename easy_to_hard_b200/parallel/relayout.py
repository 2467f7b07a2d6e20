"""Weight re-layout from the training layout to the rollout layout of PPO.

Training shards a policy as TP_t tensor-parallel ranks x DP data-parallel shards (flat bf16
shards per block, ``parallel.fsdp``); generation wants it tensor parallel over more GPUs
(``--rollout_tensor_parallel_size`` TP_r, a multiple of TP_t, e.g. TP 2 x DP 4 for training and
TP 8 for rollouts). The reference keeps one TP degree and rebuilds an unsharded copy of the
policy from an FSDP full-state-dict gather before every rollout
(trainers/ppo_trainer.py:260-311 there). Here every rollout rank pulls exactly the rows /
columns it owns out of the peers' shards over NVLink (``ops/csrc/relayout.cu``): no rank ever
holds more than its rollout shard, and each byte crosses the link once.

Geometry. Global rank = dp * TP_t + tp. Rollout rank j (of TP_r) owns slice j of every split
dimension; that slice lies inside training shard i = j // (TP_r / TP_t), at sub-index
q = j % (TP_r / TP_t). Training shard i of a block is a flat buffer cut into DP pieces, piece d
sitting on global rank d * TP_t + i. Column-parallel tensors (wqkv per q/k/v segment, w1, w3)
take a row range of the training shard, row-parallel ones (wo, w2) a column range.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist


def _blocks_of(name: str, src_shape: Tuple[int, int], ratio: int, q: int, seg_rows: List[int]):
    """[(dst_row0, row0, col0, rows, cols)] of the training-shard tensor ``name`` that rollout
    sub-index ``q`` of ``ratio`` owns. ``seg_rows``: the q/k/v row counts of a training wqkv."""
    rows_t, cols_t = src_shape
    if ".wqkv." in name:
        out, start, dst0 = [], 0, 0
        for seg in seg_rows:
            assert seg % ratio == 0
            n = seg // ratio
            out.append((dst0, start + q * n, 0, n, cols_t))
            start += seg
            dst0 += n
        return out
    if ".w1." in name or ".w3." in name or name.endswith("output.weight"):
        assert rows_t % ratio == 0
        n = rows_t // ratio
        return [(0, q * n, 0, n, cols_t)]
    if ".wo." in name or ".w2." in name:
        assert cols_t % ratio == 0
        n = cols_t // ratio
        return [(0, 0, q * n, rows_t, n)]
    raise ValueError(f"no re-layout rule for {name}")


class RolloutRelayout:
    """Refreshes ``dst_model`` (TP_r-sharded rollout copy, bf16) from ``sdp``'s shards.

    ``sdp``: ``ShardedDataParallel`` over the training data-parallel group, whose bf16 shards
    have been made visible to ``world_group`` (``sdp.expose_shards``) on CUDA."""

    def __init__(self, sdp, dst_model, train_tp: int, rollout_tp: int, world_group=None):
        assert rollout_tp % train_tp == 0, "rollout TP must be a multiple of the training TP"
        self.sdp, self.dst = sdp, dst_model
        self.tp_t, self.tp_r, self.ratio = train_tp, rollout_tp, rollout_tp // train_tp
        self.world_group = world_group
        self.world = dist.get_world_size(world_group) if dist.is_initialized() else 1
        self.grank = dist.get_rank(world_group) if dist.is_initialized() else 0
        self.dp = self.world // train_tp
        assert self.world % rollout_tp == 0
        j = self.grank % rollout_tp
        self.src_tp, self.q = j // self.ratio, j % self.ratio
        att = dst_model.layers[0].attention
        D = att.head_dim
        self.seg_rows = [att.n_head * D * self.ratio, att.n_local_heads * D * self.ratio,
                         att.n_local_heads * D * self.ratio]
        self.dst_params: Dict[str, torch.Tensor] = dict(dst_model.named_parameters())
        self.dst_params.update(dict(dst_model.named_buffers()))
        self.plan = []          # (unit, dst tensor, flat0, pitch, dst_row0, row0, col0, rows, cols)
        for unit in sdp._all_units():
            for name, off, shp in zip(unit.names, unit.offsets, unit.shapes):
                key = name[len("backbone_model."):] if name.startswith("backbone_model.") else name
                if key not in self.dst_params:
                    continue
                dst = self.dst_params[key]
                for (d0, r0, c0, rows, cols) in _blocks_of(name, shp, self.ratio, self.q,
                                                           self.seg_rows):
                    assert dst.shape[1] == cols and d0 + rows <= dst.shape[0], (name, dst.shape)
                    self.plan.append((unit, dst, off, shp[1], d0, r0, c0, rows, cols))
        self.bytes_per_sync = sum(p[7] * p[8] * 2 for p in self.plan)

    # ------------------------------------------------------------------ execution
    def _shard_ptrs(self, unit):
        sbuf, _ = unit.lp_symm
        arr = (C.c_void_p * 8)()
        for d in range(self.dp):
            arr[d] = sbuf.ptrs[d * self.tp_t + self.src_tp]
        return arr

    @torch.no_grad()
    def run(self) -> None:
        """Collective over the world group (a barrier on each side keeps the pulls between the
        optimizer steps that rewrite the shards)."""
        if dist.is_initialized():
            dist.barrier(self.world_group)
        cuda = next(iter(self.dst_params.values())).is_cuda
        if cuda and all(u.lp_symm is not None for u in self.sdp._all_units()):
            self._run_pull()
        else:
            self._run_gather()
        if dist.is_initialized():
            dist.barrier(self.world_group)

    def _run_pull(self) -> None:
        from ..ops import _lib
        lib, stream = _lib.lib(), _lib.stream()
        for unit, dst, flat0, pitch, d0, r0, c0, rows, cols in self.plan:
            assert dst.dtype == torch.bfloat16 and dst.is_contiguous()
            rc = lib.e2h_relayout_pull(self._shard_ptrs(unit), self.dp, unit.lp_symm[1],
                                       unit.shard_size, flat0, pitch, r0, c0, rows, cols,
                                       dst[d0:d0 + rows].data_ptr(), stream)
            _lib.check(rc, "relayout_pull")

    def _run_gather(self) -> None:
        """Portable form (CPU / gloo, or peers without mapped memory): all-gather each block's
        shards over the world group, then slice."""
        done = {}
        for unit, dst, flat0, pitch, d0, r0, c0, rows, cols in self.plan:
            flat = done.get(id(unit))
            if flat is None:
                shard = unit.shard_lp.detach().contiguous()
                if self.world > 1:
                    every = torch.empty(self.world * unit.shard_size, dtype=shard.dtype,
                                        device=shard.device)
                    dist.all_gather_into_tensor(every, shard, group=self.world_group)
                    every = every.view(self.dp, self.tp_t, unit.shard_size)
                    flat = every[:, self.src_tp].reshape(-1)
                else:
                    flat = shard
                done = {id(unit): flat}          # keep one block's gather alive at a time
            block = flat.as_strided((rows, cols), (pitch, 1), flat0 + r0 * pitch + c0)
            dst[d0:d0 + rows].copy_(block.to(dst.dtype))
