"""Batched inference engine: prefill + CUDA-graph decode over the sm_100a kernels.

This is the B200 counterpart of the reference's ``torch.compile(mode="reduce-overhead")`` decode
(inference_generate.py:346-354, rl_model.py:54-62): instead of tracing the module tree, the engine
reads the weights of a (possibly tensor-parallel-sharded) ``Transformer`` and runs one decode step
as an explicit sequence of fused kernels, captured once in a CUDA graph and replayed per token:

    embedding + RMSNorm                                   (1 kernel, first layer only)
    per layer:
        QKV GEMM + RoPE + KV-cache scatter                (tcgen05, epilogue-fused)
        decode attention over the live cache range        (streams K/V once)
        wo GEMM + residual add                            (cluster split-K)
        RMSNorm
        w1/w3 GEMM + SwiGLU                               (dual accumulator)
        w2 GEMM + residual add                            (cluster split-K)
        RMSNorm (next layer's / final)
    LM-head GEMM (fp32 logits) ; fused top-k sampler      (advances the position on device)

Position, current tokens, EOS flags and the output sequence all live on the device, so the loop
needs no per-token host synchronisation (the reference syncs every token through
``eos_flag.all()``, rl_model.py:441).

With tensor parallelism the ``reduce`` strategy says how the partial sums of the row-parallel
GEMMs (wo, w2) meet:

``"fused"`` (default for TP > 1)
    the GEMM writes its bf16 partial into symmetric memory and its last CTA raises a flag on
    every peer; one kernel (``ops/csrc/tp_reduce.cu``) then sums the rows this rank owns over
    NVLink (plain peer loads, or ``multimem.ld_reduce`` through the NVSwitch where the group
    has a multicast mapping), adds the residual, normalises and writes the rows into every
    rank's activation buffer. No NCCL call sits in the decode graph.
``"nccl"``
    fp32 partial, ``dist.all_reduce``, then the local residual + norm kernel (the baseline).

A vocabulary-parallel model (``Transformer(vocab_parallel=True)`` under TP, the reference's
``--vocab_parallel`` flag: sharded embedding table and LM head, models/tp.py:85-119 and
models/rl_model.py:366-379 of the reference) runs on the fused strategy only: the embedding is a
masked lookup whose partial rows go through the same reduce kernel, and the ranks' logit shards
are gathered over peer memory before the (replicated, same-seed) sampler.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib, functional as Fn, gemm
from ..parallel import groups


class DecodeEngine:
    def __init__(self, model, max_batch_size: int, max_seq_length: int,
                 reduce: str = "auto", use_graph: bool = True, use_pdl: bool = True):
        cfg = model.config
        self.model = model
        self.cfg = cfg
        self.tp = getattr(model, "tp_size", 1)
        self.dev = model.output.weight.device
        assert self.dev.type == "cuda", "DecodeEngine needs a CUDA device"
        self.use_graph = use_graph
        self.use_pdl = use_pdl
        self.B = max_batch_size
        self.S = (max_seq_length + 7) // 8 * 8
        blk0 = model.layers[0].attention
        self.n_head, self.n_kv, self.D = blk0.n_head, blk0.n_local_heads, blk0.head_dim
        self.dim = model.tok_embeddings.weight.shape[1]
        w2 = model.layers[0].feed_forward.w2          # packed int4 weights are not [out, in]
        self.ffn = getattr(w2, "origin_in_features", None) or getattr(w2, "in_features", None) \
            or w2.weight.shape[1]
        self.vocab_parallel = bool(getattr(model, "vocab_parallel", False)) and self.tp > 1
        self.vocab_local = model.output.weight.shape[0]
        self.vocab = self.vocab_local * (self.tp if self.vocab_parallel else 1)
        # a model sharded over another group than the job's tensor-parallel one names it
        self.group = getattr(model, "tp_group", None)
        if self.group is None and self.tp > 1:
            self.group = groups.get_model_parallel_group()
        self.tp_rank = getattr(model, "tp_rank", None)
        if self.tp_rank is None:
            self.tp_rank = groups.get_model_parallel_rank() if self.tp > 1 else 0
        self.eps = cfg.norm_eps
        if reduce in ("auto", "p2p"):
            reduce = "local"
            if self.tp > 1:     # peer memory reaches every rank of a one-host group only
                from ..parallel.symm import peer_memory_usable
                reduce = "fused" if peer_memory_usable(self.group) else "nccl"
        if self.tp == 1:
            reduce = "local"
        # "fused_oneshot" / "fused_twophase" pin the form of the fused reduce (measurements);
        # plain "fused" picks by size (see parallel.symm.TPReduceSync)
        self.reduce_form = {"fused_oneshot": True, "fused_twophase": False}.get(reduce)
        if reduce.startswith("fused_"):
            reduce = "fused"
        if reduce not in ("local", "nccl", "fused"):
            raise ValueError(f"unknown reduce strategy {reduce!r}")
        if self.vocab_parallel and reduce != "fused":
            raise ValueError("a vocabulary-parallel model needs reduce='fused': its token ids "
                             "index a sharded embedding table and its logits are sharded")
        emb_rows = model.tok_embeddings.weight.shape[0]
        if not self.vocab_parallel and self.tp > 1 and emb_rows != cfg.vocab_size \
                and emb_rows * self.tp == cfg.vocab_size:
            raise ValueError("the embedding table is vocabulary-sharded but model.vocab_parallel "
                             "is off: global token ids would index past its end")
        self.reduce = reduce
        dev, bf = self.dev, torch.bfloat16
        B, S = self.B, self.S
        self.freqs = _freqs(S, self.D, cfg.rope_base, dev)
        self.kcache = [torch.zeros(B, self.n_kv, S, self.D, dtype=bf, device=dev)
                       for _ in model.layers]
        self.vcache = [torch.zeros(B, self.n_kv, S, self.D, dtype=bf, device=dev)
                       for _ in model.layers]
        # decode-step buffers
        self.h = torch.empty(B, self.dim, dtype=bf, device=dev)
        self.n_points = 2 * len(model.layers) + 2      # embedding, wo / w2 per layer, logits
        self.sync = self.sync_prefill = None
        if self.reduce == "fused":
            from ..parallel.symm import TPReduceSync
            self.sync = TPReduceSync(
                B, self.dim, self.n_points, self.group,
                extra_bytes=B * self.vocab_local * 4 if self.vocab_parallel else 0,
                oneshot=self.reduce_form)
            # the switch-side sum must give every rank the same bits, or their samplers drift
            # apart: checked once, plain peer loads otherwise
            self.sync.check_multimem_consistency(self.group)
        if self.sync is not None and not self.sync.oneshot:
            self.xn = self.sync.xn
        else:
            self.xn = torch.empty(B, self.dim, dtype=bf, device=dev)
        self.q = torch.empty(B, self.n_head * self.D, dtype=bf, device=dev)
        self.att = torch.empty(B, self.n_head * self.D, dtype=bf, device=dev)
        self.act = torch.empty(B, self.ffn, dtype=bf, device=dev)
        self.logits = torch.empty(B, self.vocab, dtype=torch.float32, device=dev)
        self.partial = (torch.empty(1, B, self.dim, dtype=torch.float32, device=dev)
                        if self.reduce == "nccl" else None)
        self.logits_shard = (self.sync.extra((B, self.vocab_local), torch.float32)
                             if self.vocab_parallel else None)
        self.seed_dev = torch.zeros(1, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.next_tok = torch.zeros(B, dtype=torch.int32, device=dev)
        self.left_pad = torch.zeros(B, dtype=torch.int32, device=dev)
        self.seq = torch.zeros(B, S, dtype=torch.int32, device=dev)
        self.eos_flag = torch.zeros(B, dtype=torch.int32, device=dev)
        self.n_unfinished = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        self._graphs = {}
        self.launches_per_step = 0
        self.W = [self._layer_weights(blk) for blk in model.layers]

    # ------------------------------------------------------------------ weights
    @staticmethod
    def _dense(linear):
        """(bf16 [out, in] weight, per-output-feature fp32 scale or None) as the GEMM kernels
        read them. bf16 modules hand out their own tensor (in-place updates of the model, e.g.
        the PPO rollout sync, are seen by captured graphs). Weight-only int8 stays int8 (the
        decode GEMM expands it to bf16 inside the SM) with its scales applied in the GEMM
        epilogue, exactly where the reference multiplies (models/quantize.py:397-398).
        Group-wise int4 (tinygemm packing in the checkpoint) is re-packed once into the
        row-major nibble layout of ``ops.gemm.Int4Weight`` and streams as int4; group sizes the
        kernel does not take (below 64) are dequantised once instead."""
        w = linear.weight
        if w.dtype == torch.int8 and hasattr(linear, "scales"):
            # stays int8 in memory: ops.gemm streams it through the converting kernel
            return w.contiguous(), linear.scales.float().contiguous()
        if w.dtype == torch.int32 and hasattr(linear, "scales_and_zeros"):
            from . import quantize as qz
            q = qz.unpack_int4_tinygemm(w, linear.inner_k_tiles)
            k = getattr(linear, "origin_in_features", q.shape[1])
            g = linear.groupsize
            if k % 128 == 0 and k % g == 0 and g >= 64 and (g & (g - 1)) == 0:
                # input columns added by the checkpoint's padding multiply zeros: dropped
                return gemm.Int4Weight.from_int(q[:, :k].contiguous(),
                                                linear.scales_and_zeros[: k // g], g), None
            full = qz.group_dequantize_tensor(q, linear.scales_and_zeros, 4, g)
            return full[:, :k].to(torch.bfloat16).contiguous(), None
        assert w.dtype == torch.bfloat16, f"unsupported weight dtype {w.dtype}"
        return w, None


    def _layer_weights(self, blk):
        a, f = blk.attention, blk.feed_forward
        out = {n: self._dense(m) for n, m in (("wqkv", a.wqkv), ("wo", a.wo), ("w1", f.w1),
                                              ("w3", f.w3), ("w2", f.w2))}
        s1, s3 = out["w1"][1], out["w3"][1]
        out["s13"] = None if s1 is None else torch.cat([s1, s3]).contiguous()
        return out

    # ------------------------------------------------------------------ layer pieces
    def _row_parallel(self, x, ws, h, next_norm_w, h_out, x_out, point: int = 0, sync=None):
        """h_out = h + x @ w^T (summed over TP ranks); x_out = rmsnorm(h_out) * next_norm_w.
        ``ws`` = (weight, per-feature scale or None). On the fused strategy ``x_out`` is the
        activation buffer of ``sync`` and only the token rows this rank owns are kept in
        ``h_out`` (the residual stream of a row lives on its owner)."""
        w, sc = ws
        T = x.shape[0]
        if self.reduce == "local":
            gemm.linear_residual(x, w, h, out=h_out, scale=sc)
            Fn.fused_residual_rmsnorm(h_out, next_norm_w, self.eps, x_out=x_out)
        elif self.reduce == "nccl":
            part = self.partial[:, :T] if T <= self.B else \
                torch.empty(1, T, self.dim, dtype=torch.float32, device=self.dev)
            gemm.linear(x, w, out=part[0], scale=sc)
            dist.all_reduce(part, group=self.group)
            Fn.fused_residual_rmsnorm(h, next_norm_w, self.eps, partials=part, h_out=h_out,
                                      x_out=x_out)
        else:
            gemm.linear(x, w, out=sync.partial_out(point, T), signal=sync.flag_a_signal(point),
                        ticket=sync.gemm_ticket[point:point + 1], scale=sc)
            sync.reduce_norm(point, h, h_out, next_norm_w, self.eps, T, xn_out=x_out)
        self._count(2)

    def _embed_norm(self, tok, h, xn, sync):
        """h = embedding(tok); xn = rmsnorm(h) * first attention norm."""
        m = self.model
        w0 = m.layers[0].attention_norm.weight
        if self.vocab_parallel:
            sync.embed_partial(0, tok, m.tok_embeddings.weight, self.tp_rank * self.vocab_local)
            sync.reduce_norm(0, None, h, w0, self.eps, tok.numel(), xn_out=xn)
            self._count(2)
        else:
            Fn.fused_residual_rmsnorm(None, w0, self.eps, tokens=tok, emb=m.tok_embeddings.weight,
                                      h_out=h, x_out=xn)
            self._count(1)

    def _head_sample(self, x, B, temperature, top_k, eos_id):
        """LM head on ``x`` [B, dim] and the fused sampler (advances the position)."""
        m = self.model
        logits = self.logits[:B]
        if self.vocab_parallel:
            pt = self.n_points - 1
            gemm.linear(x, m.output.weight, out=self.logits_shard[:B],
                        signal=self.sync.flag_a_signal(pt),
                        ticket=self.sync.gemm_ticket[pt:pt + 1])
            self.sync.gather_logits(pt, B, self.vocab_local, logits)
            self._count(1)
        else:
            gemm.linear(x, m.output.weight, out=logits)
        Fn.sample(logits, temperature=temperature, top_k=top_k, seed=0, seed_dev=self.seed_dev,
                  pos=self.pos, next_tok=self.next_tok[:B], seq=self.seq[:B], eos_id=eos_id,
                  eos_flag=self.eos_flag[:B], n_unfinished=self.n_unfinished, ticket=self.ticket,
                  advance_pos=True)
        self._count(2)

    def _count(self, n):
        self.launches_per_step += n

    def _layers(self, T: int, sq: int, h, xn, q, att, act, prefill_B: int = 0, sync=None):
        m = self.model
        for li, blk in enumerate(m.layers):
            W = self.W[li]
            gemm.linear_qkv_rope(xn, W["wqkv"][0], q, freqs=self.freqs, pos_base=self.pos,
                                 sq=sq, n_head=self.n_head, n_kv=self.n_kv, head_dim=self.D,
                                 kcache=self.kcache[li], vcache=self.vcache[li],
                                 scale=W["wqkv"][1])
            if sq == 1:
                Fn.attn_decode(q, self.kcache[li], self.vcache[li], self.pos, self.left_pad,
                               self.n_head, out=att)
            else:
                self._prefill_attention(li, q, att, prefill_B, sq)
            self._count(2)
            self._row_parallel(att, W["wo"], h, blk.ffn_norm.weight, h, xn, 1 + 2 * li, sync)
            gemm.linear_swiglu(xn, W["w1"][0], W["w3"][0], out=act, scale=W["s13"])
            self._count(1)
            nxt = (m.layers[li + 1].attention_norm.weight if li + 1 < len(m.layers)
                   else m.norm.weight)
            self._row_parallel(act, W["w2"], h, nxt, h, xn, 2 + 2 * li, sync)

    def _prefill_attention(self, li, q, att, B, S):
        from ..ops import attention as attn_ops
        attn_ops.prefill_attention(q.view(B, S, self.n_head, self.D), self.kcache[li],
                                   self.vcache[li], self.left_pad[:B], att.view(B, S, -1))

    # ------------------------------------------------------------------ decode
    def _decode_step(self, B, temperature, top_k, eos_id):
        h, xn, q, att, act = (t[:B] for t in (self.h, self.xn, self.q, self.att, self.act))
        self._embed_norm(self.next_tok[:B], h, xn, self.sync)
        self._layers(B, 1, h, xn, q, att, act, sync=self.sync)
        self._head_sample(xn, B, temperature, top_k, eos_id)

    def _graph_for(self, key):
        if key in self._graphs:
            return self._graphs[key]
        B, temperature, top_k, eos_id = key
        # warm up on a side stream (module loading, attribute setting), then capture
        saved = [t.clone() for t in (self.pos, self.next_tok, self.seq, self.eos_flag,
                                     self.n_unfinished)]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._decode_step(*key)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        self.launches_per_step = 0
        # programmatic dependent launch: each kernel's prologue overlaps its predecessor's tail
        old_pdl = _lib.lib().e2h_set_pdl(1 if self.use_pdl else 0)
        try:
            with torch.cuda.graph(g):
                self._decode_step(*key)
        finally:
            _lib.lib().e2h_set_pdl(old_pdl)
        for t, v in zip((self.pos, self.next_tok, self.seq, self.eos_flag, self.n_unfinished),
                        saved):
            t.copy_(v)
        self._graphs[key] = (g, self.launches_per_step)
        return self._graphs[key]

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor, left_pad_mask_pos: Optional[torch.Tensor],
                temperature: float, top_k: Optional[int], seed: int, eos_id: int):
        """prompt [B, T] (left padded). Fills the caches for positions 0..T-1 and samples the
        first new token into ``seq[:, T]``."""
        m = self.model
        B, T = prompt.shape
        assert B <= self.B and T < self.S
        dev, bf = self.dev, torch.bfloat16
        tok = prompt.to(device=dev, dtype=torch.int32).contiguous()
        self.seq[:B].zero_()
        self.seq[:B, :T] = tok
        self.eos_flag.zero_()
        self.n_unfinished.fill_(B)
        self.ticket.zero_()
        if left_pad_mask_pos is None:
            self.left_pad.zero_()
        else:
            self.left_pad[:B] = left_pad_mask_pos.to(device=dev, dtype=torch.int32)
        self.pos.zero_()
        self.seed_dev.fill_(int(seed) & (2 ** 63 - 1))
        n = B * T
        sync = None
        if self.reduce == "fused":
            sync = self._prefill_sync(n)
            xn = (torch.empty(n, self.dim, dtype=bf, device=dev) if sync.oneshot
                  else sync.xn[:n])
        else:
            xn = torch.empty(n, self.dim, dtype=bf, device=dev)
        h = torch.empty(n, self.dim, dtype=bf, device=dev)
        q = torch.empty(n, self.n_head * self.D, dtype=bf, device=dev)
        att = torch.empty(n, self.n_head * self.D, dtype=bf, device=dev)
        act = torch.empty(n, self.ffn, dtype=bf, device=dev)
        self.launches_per_step = 0
        self._embed_norm(tok.view(-1), h, xn, sync)
        self._layers(n, T, h, xn, q, att, act, prefill_B=B, sync=sync)
        last = xn.view(B, T, self.dim)[:, -1].contiguous()
        self.pos.fill_(T - 1)
        self._head_sample(last, B, temperature, top_k, eos_id)
        self.prefill_launches = self.launches_per_step + 3

    def _prefill_sync(self, n_tokens: int):
        """Symmetric buffers of the prompt pass, grown on demand (a collective: every rank
        prefills the same shape). They are separate from the decode buffers, whose addresses
        sit inside captured graphs."""
        sp = self.sync_prefill
        if sp is None or sp.T < n_tokens:
            from ..parallel.symm import TPReduceSync
            self.sync_prefill = sp = None
            torch.cuda.empty_cache()
            cap = 1 << max(10, (n_tokens - 1).bit_length())
            sp = TPReduceSync(cap, self.dim, self.n_points, self.group)
            self.sync_prefill = sp
        return sp

    # ------------------------------------------------------------------ generate
    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, left_pad_mask_pos: Optional[torch.Tensor],
                 max_new_tokens: int, temperature: float = 1.0, top_k: Optional[int] = None,
                 eos_id: Optional[int] = None, seed: int = 0, check_eos_every: int = 32):
        """Returns (seq [B, T+max_new_tokens] int32 on device, number of decode steps run).

        With an ``eos_id`` the loop stops once every row has produced it; the host looks at the
        device-side counter only every ``check_eos_every`` steps."""
        B, T = prompt.shape
        eos = -1 if eos_id is None else int(eos_id)
        self.prefill(prompt, left_pad_mask_pos, temperature, top_k, seed, eos)
        steps = 0
        key = (B, float(temperature), int(top_k) if top_k else 0, eos)
        n_dec = min(max_new_tokens - 1, self.S - T - 1)
        if self.use_graph:
            g, _ = self._graph_for(key)
        for i in range(n_dec):
            if self.use_graph:
                g.replay()
            else:
                self._decode_step(*key)
            steps += 1
            if eos >= 0 and (i + 1) % check_eos_every == 0 and self.n_unfinished.item() <= 0:
                break
        if self.reduce == "fused":
            self.check_status()
        return self.seq[:B, : T + max_new_tokens], steps

    def check_status(self) -> None:
        """Raises when a kernel of this device recorded a time-out (a tensor-parallel peer that
        never signalled): the tokens of that generation are not to be trusted."""
        code = _lib.read_status(self.dev)
        if code != 0:
            raise RuntimeError(f"decode engine: a device-side wait timed out (status {code}); "
                               "a tensor-parallel peer did not reach the same step")

    def decode_launches(self, key=None) -> int:
        if key is None and self._graphs:
            return next(iter(self._graphs.values()))[1]
        return self._graphs[key][1] if key in self._graphs else 0

    def weight_bytes(self) -> int:
        return sum(p.numel() * p.element_size()
                   for p in list(self.model.parameters()) + list(self.model.buffers()))


def _freqs(S, D, base, dev):
    from ..ops import reference
    return reference.precompute_freqs_cis(S, D, base, dtype=torch.bfloat16, device=dev)


def get_engine(model, batch_size: int, seq_length: int, **kw) -> DecodeEngine:
    """Engine cached on the model; rebuilt when a larger batch / sequence is requested."""
    eng = getattr(model, "_decode_engine", None)
    if eng is None or eng.B < batch_size or eng.S < seq_length:
        if eng is not None:
            del model._decode_engine
            torch.cuda.empty_cache()
        eng = DecodeEngine(model, batch_size, seq_length, **kw)
        model._decode_engine = eng
    return eng
