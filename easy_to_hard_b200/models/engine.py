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

With tensor parallelism the row-parallel GEMMs (wo, w2) write fp32 partial sums and the following
norm kernel adds the partials of all ranks; how the partials travel is the ``reduce`` strategy:
``"nccl"`` (all-reduce between the two kernels, the baseline) or ``"p2p"`` (the GEMM epilogue
pushes its partial tile straight into every peer's buffer over NVLink and raises a flag that the
norm kernel waits on, see ``parallel.symm``).
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
        self.vocab = model.output.weight.shape[0]
        self.eps = cfg.norm_eps
        if reduce == "auto":
            reduce = "local" if self.tp == 1 else "nccl"
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
        self.xn = torch.empty(B, self.dim, dtype=bf, device=dev)
        self.q = torch.empty(B, self.n_head * self.D, dtype=bf, device=dev)
        self.att = torch.empty(B, self.n_head * self.D, dtype=bf, device=dev)
        self.act = torch.empty(B, self.ffn, dtype=bf, device=dev)
        self.logits = torch.empty(B, self.vocab, dtype=torch.float32, device=dev)
        self.partial = (torch.empty(1, B, self.dim, dtype=torch.float32, device=dev)
                        if self.reduce == "nccl" else None)
        self.rp = None
        if self.reduce == "p2p":
            from ..parallel.symm import RowParallelReduce
            self.rp = RowParallelReduce(B, self.dim, groups.get_model_parallel_group())
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
    def _row_parallel(self, x, ws, h, next_norm_w, h_out, x_out):
        """h_out = h + x @ w^T (summed over TP ranks); x_out = rmsnorm(h_out) * next_norm_w.
        ``ws`` = (weight, per-feature scale or None)."""
        w, sc = ws
        if self.reduce == "local":
            gemm.linear_residual(x, w, h, out=h_out, scale=sc)
            Fn.fused_residual_rmsnorm(h_out, next_norm_w, self.eps, x_out=x_out)
            self._count(2)
        elif self.reduce == "nccl":
            part = self.partial[:, : x.shape[0]] if x.shape[0] <= self.B else \
                torch.empty(1, x.shape[0], self.dim, dtype=torch.float32, device=self.dev)
            gemm.linear(x, w, out=part[0], scale=sc)
            dist.all_reduce(part, group=groups.get_model_parallel_group())
            Fn.fused_residual_rmsnorm(h, next_norm_w, self.eps, partials=part, h_out=h_out,
                                      x_out=x_out)
            self._count(2)
        elif self.reduce == "p2p":
            T = x.shape[0]
            if T > self.rp.T:  # prefill-sized inputs take the NCCL route
                part = torch.empty(1, T, self.dim, dtype=torch.float32, device=self.dev)
                gemm.linear(x, w, out=part[0], scale=sc)
                dist.all_reduce(part, group=groups.get_model_parallel_group())
                Fn.fused_residual_rmsnorm(h, next_norm_w, self.eps, partials=part, h_out=h_out,
                                          x_out=x_out)
            else:
                rp = self.rp
                s = rp.slot()
                gemm.linear(x, w, out=rp.partial_out(s, T), signal=rp.signal_ptrs(s),
                            ticket=rp.gemm_ticket[s:s + 1], scale=sc)
                Fn.fused_residual_rmsnorm(h, next_norm_w, self.eps, partials=rp.partial_ptrs(s),
                                          h_out=h_out, x_out=x_out, flags=rp.flags(s),
                                          use_count=rp.use_count[s:s + 1],
                                          ticket=rp.norm_ticket[s:s + 1], T=T, dim=self.dim)
            self._count(2)
        else:
            raise ValueError(self.reduce)

    def _count(self, n):
        self.launches_per_step += n

    def _layers(self, T: int, sq: int, h, xn, q, att, act, prefill_B: int = 0):
        m = self.model
        for li, blk in enumerate(m.layers):
            W = self.W[li]
            gemm.linear_qkv_rope(xn, W["wqkv"][0], q, freqs=self.freqs, pos_base=self.pos,
                                 sq=sq, n_head=self.n_head, n_kv=self.n_kv, head_dim=self.D,
                                 kcache=self.kcache[li], vcache=self.vcache[li],
                                 scale=W["wqkv"][1])
            if sq == 1:
                Fn.attn_decode(q, self.kcache[li], self.vcache[li], self.pos, self.left_pad,
                               self.n_head, out=att, n_split=1 if T * self.n_kv >= 256 else 0)
            else:
                self._prefill_attention(li, q, att, prefill_B, sq)
            self._count(2)
            self._row_parallel(att, W["wo"], h, blk.ffn_norm.weight, h, xn)
            gemm.linear_swiglu(xn, W["w1"][0], W["w3"][0], out=act, scale=W["s13"])
            self._count(1)
            nxt = (m.layers[li + 1].attention_norm.weight if li + 1 < len(m.layers)
                   else m.norm.weight)
            self._row_parallel(act, W["w2"], h, nxt, h, xn)

    def _prefill_attention(self, li, q, att, B, S):
        from ..ops import attention as attn_ops
        attn_ops.prefill_attention(q.view(B, S, self.n_head, self.D), self.kcache[li],
                                   self.vcache[li], self.left_pad[:B], att.view(B, S, -1))

    # ------------------------------------------------------------------ decode
    def _decode_step(self, B, temperature, top_k, seed, eos_id):
        m = self.model
        h, xn, q, att, act = (t[:B] for t in (self.h, self.xn, self.q, self.att, self.act))
        Fn.fused_residual_rmsnorm(None, m.layers[0].attention_norm.weight, self.eps,
                                  tokens=self.next_tok[:B], emb=m.tok_embeddings.weight,
                                  h_out=h, x_out=xn)
        self._count(1)
        self._layers(B, 1, h, xn, q, att, act)
        logits = self.logits[:B]
        gemm.linear(xn, m.output.weight, out=logits)
        Fn.sample(logits, temperature=temperature, top_k=top_k, seed=seed, pos=self.pos,
                  next_tok=self.next_tok[:B], seq=self.seq[:B], eos_id=eos_id,
                  eos_flag=self.eos_flag[:B], n_unfinished=self.n_unfinished, ticket=self.ticket,
                  advance_pos=True)
        self._count(2)

    def _graph_for(self, key):
        if key in self._graphs:
            return self._graphs[key]
        B, temperature, top_k, seed, eos_id = key
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
        n = B * T
        h = torch.empty(n, self.dim, dtype=bf, device=dev)
        xn = torch.empty(n, self.dim, dtype=bf, device=dev)
        q = torch.empty(n, self.n_head * self.D, dtype=bf, device=dev)
        att = torch.empty(n, self.n_head * self.D, dtype=bf, device=dev)
        act = torch.empty(n, self.ffn, dtype=bf, device=dev)
        self.launches_per_step = 0
        Fn.fused_residual_rmsnorm(None, m.layers[0].attention_norm.weight, self.eps,
                                  tokens=tok.view(-1), emb=m.tok_embeddings.weight, h_out=h,
                                  x_out=xn)
        self._layers(n, T, h, xn, q, att, act, prefill_B=B)
        last = xn.view(B, T, self.dim)[:, -1].contiguous()
        logits = self.logits[:B]
        gemm.linear(last, m.output.weight, out=logits)
        self.pos.fill_(T - 1)
        Fn.sample(logits, temperature=temperature, top_k=top_k, seed=seed, pos=self.pos,
                  next_tok=self.next_tok[:B], seq=self.seq[:B], eos_id=eos_id,
                  eos_flag=self.eos_flag[:B], n_unfinished=self.n_unfinished, ticket=self.ticket,
                  advance_pos=True)
        self.prefill_launches = self.launches_per_step + 3

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
        key = (B, float(temperature), int(top_k) if top_k else 0, int(seed), eos)
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
        return self.seq[:B, : T + max_new_tokens], steps

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
