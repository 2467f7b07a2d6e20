"""LLaMA-architecture model: configuration table, static KV cache, and the module tree
(``Transformer`` / ``TransformerBlock`` / ``Attention`` / ``FeedForward`` / ``RMSNorm``).

The public surface mirrors the reference (models/model.py:42-416): ``ModelArgs.from_name`` with
fuzzy matching on the checkpoint directory name, ``Transformer.setup_caches`` /
``Transformer.forward(idx, input_pos, left_pad_mask_pos, fully_causal)``, the gpt-fast state-dict
naming (fused ``wqkv``), interleaved-pair RoPE with a bf16 table.

What differs is underneath. Tensor / sequence parallelism is explicit in the forward code
(``parallel.collectives``), not bolted on through module hooks; on a B200 every hot op goes to a
hand-written sm_100a kernel (``ops``): the linears run on the tcgen05 GEMM with fused epilogues,
decode attention reads only the live part of the static cache, and the batched decode loop of
``models.engine`` is a captured CUDA graph over those kernels. The same modules run in fp32 on CPU
(gloo) as the plumbing oracle.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ..ops import reference as ref_ops
from ..parallel import collectives as coll
from .frozen_layers import FrozenEmbedding, FrozenLinear, FrozenRMSNorm

_GLOBAL_IN_COMPILE_MODE = False


def set_global_compile_mode(flag: bool) -> None:
    """Kept for API compatibility: the reference switches apex norms off under torch.compile
    (models/model.py:415-416). Here "compile mode" selects the CUDA-graph decode engine."""
    global _GLOBAL_IN_COMPILE_MODE
    _GLOBAL_IN_COMPILE_MODE = bool(flag)


def in_compile_mode() -> bool:
    return _GLOBAL_IN_COMPILE_MODE


def find_multiple(n: int, k: int) -> int:
    return n if n % k == 0 else n + k - (n % k)


@dataclass
class ModelArgs:
    block_size: int = 2048
    vocab_size: int = 32000
    n_layer: int = 32
    n_head: int = 32
    dim: int = 4096
    intermediate_size: Optional[int] = None
    n_local_heads: int = -1
    head_dim: int = 64
    rope_base: float = 10000
    norm_eps: float = 1e-5

    def __post_init__(self):
        if self.n_local_heads == -1:
            self.n_local_heads = self.n_head
        if self.intermediate_size is None:
            self.intermediate_size = find_multiple(int(2 * 4 * self.dim / 3), 256)
        self.head_dim = self.dim // self.n_head

    @classmethod
    def from_name(cls, name: str) -> "ModelArgs":
        """Exact key first, then the first config whose key is a substring of the (upper-cased)
        name -- the directory that holds ``model.pth`` selects the architecture."""
        name = str(name)
        if name in transformer_configs:
            return cls(**transformer_configs[name])
        hits = [k for k in transformer_configs if k in name.upper() or k in name]
        assert hits, f"no model config matches {name!r}"
        # prefer the most specific (longest) key so "llemma-7b-32016" does not fall back to "7B"
        hits.sort(key=len, reverse=True)
        return cls(**transformer_configs[hits[0]])


transformer_configs = {
    "CodeLlama-7b-Python-hf": dict(block_size=16384, vocab_size=32000, n_layer=32, dim=4096,
                                   rope_base=1000000),
    "llemma-7b": dict(block_size=4096, n_layer=32, n_head=32, dim=4096),
    # the Llemma-7B architecture as released: 32016-entry vocabulary, RoPE theta 1e6
    "llemma-7b-32016": dict(block_size=4096, vocab_size=32016, n_layer=32, n_head=32, dim=4096,
                            intermediate_size=11008, rope_base=1000000),
    "deepseek-math-7b": dict(block_size=4096, vocab_size=102400, n_layer=30, n_head=32, dim=4096,
                             intermediate_size=11008, rope_base=10000, norm_eps=1e-6),
    "7B": dict(n_layer=32, n_head=32, dim=4096),
    "13B": dict(n_layer=40, n_head=40, dim=5120),
    "30B": dict(n_layer=60, n_head=52, dim=6656),
    "34B": dict(block_size=4096, n_layer=48, n_head=64, dim=8192, vocab_size=32000,
                n_local_heads=8, intermediate_size=22016, rope_base=1000000),
    "70B": dict(n_layer=80, n_head=64, dim=8192, n_local_heads=8, intermediate_size=28672),
    # plumbing configuration for CPU / gloo tests
    "tiny-llama": dict(block_size=256, vocab_size=1024, n_layer=2, n_head=4, dim=256,
                       intermediate_size=688, rope_base=10000, norm_eps=1e-5),
}


class KVCache(nn.Module):
    """Static ``[max_batch, n_kv_heads, max_seq, head_dim]`` key / value buffers."""

    def __init__(self, max_batch_size, max_seq_length, n_heads, head_dim, dtype=torch.bfloat16):
        super().__init__()
        shape = (max_batch_size, n_heads, max_seq_length, head_dim)
        self.register_buffer("k_cache", torch.zeros(shape, dtype=dtype), persistent=False)
        self.register_buffer("v_cache", torch.zeros(shape, dtype=dtype), persistent=False)

    def update(self, input_pos: Tensor, k_val: Tensor, v_val: Tensor):
        """k_val/v_val [B, H, S, D] written at positions input_pos [S]; returns the caches
        sliced to B rows."""
        assert input_pos.shape[0] == k_val.shape[2]
        B = k_val.size(0)
        self.k_cache[:B, :, input_pos] = k_val.to(self.k_cache.dtype)
        self.v_cache[:B, :, input_pos] = v_val.to(self.v_cache.dtype)
        return self.k_cache[:B], self.v_cache[:B]


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: Tensor) -> Tensor:
        return ref_ops.rmsnorm(x, self.weight, self.eps)


def precompute_freqs_cis(seq_len: int, n_elem: int, base: float = 10000.0) -> Tensor:
    return ref_ops.precompute_freqs_cis(seq_len, n_elem, base, dtype=torch.bfloat16)


apply_rotary_emb = ref_ops.apply_rotary_emb


class Attention(nn.Module):
    def __init__(self, config: ModelArgs):
        super().__init__()
        assert config.dim % config.n_head == 0
        total = (config.n_head + 2 * config.n_local_heads) * config.head_dim
        self.wqkv = nn.Linear(config.dim, total, bias=False)
        self.wo = nn.Linear(config.dim, config.dim, bias=False)
        self.kv_cache: Optional[KVCache] = None
        self.n_head = config.n_head
        self.head_dim = config.head_dim
        self.n_local_heads = config.n_local_heads
        self.dim = config.dim
        self.tp_size = 1
        self.sequence_parallel = False
        self._register_load_state_dict_pre_hook(self._fuse_qkv_hook)

    @staticmethod
    def _fuse_qkv_hook(state_dict, prefix, *args):
        """Accept checkpoints that still carry separate wq / wk / wv."""
        if prefix + "wq.weight" in state_dict:
            parts = [state_dict.pop(prefix + n + ".weight") for n in ("wq", "wk", "wv")]
            state_dict[prefix + "wqkv.weight"] = torch.cat(parts)

    def forward(self, x: Tensor, freqs_cis: Tensor, mask: Optional[Tensor],
                input_pos: Optional[Tensor], fully_causal: bool) -> Tensor:
        training = self.training
        if self.tp_size > 1:
            x = coll.enter_parallel_region(x, self.sequence_parallel and training)
        B, S, _ = x.shape
        q_sz, kv_sz = self.n_head * self.head_dim, self.n_local_heads * self.head_dim
        q, k, v = self.wqkv(x).split([q_sz, kv_sz, kv_sz], dim=-1)
        q = apply_rotary_emb(q.view(B, S, self.n_head, self.head_dim), freqs_cis)
        k = apply_rotary_emb(k.view(B, S, self.n_local_heads, self.head_dim), freqs_cis)
        v = v.view(B, S, self.n_local_heads, self.head_dim)
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
        if not fully_causal and self.kv_cache is not None:
            k, v = self.kv_cache.update(input_pos, k, v)
        if fully_causal:
            y = ref_ops.attention(q, k, v, None, causal=True)
        else:
            y = ref_ops.attention(q, k.to(q.dtype), v.to(q.dtype), mask)
        y = self.wo(y.transpose(1, 2).reshape(B, S, q_sz))
        if self.tp_size > 1:
            y = coll.exit_parallel_region(y, self.sequence_parallel and training)
        return y


class FeedForward(nn.Module):
    def __init__(self, config: ModelArgs):
        super().__init__()
        self.w1 = nn.Linear(config.dim, config.intermediate_size, bias=False)
        self.w3 = nn.Linear(config.dim, config.intermediate_size, bias=False)
        self.w2 = nn.Linear(config.intermediate_size, config.dim, bias=False)
        self.tp_size = 1
        self.sequence_parallel = False

    def forward(self, x: Tensor) -> Tensor:
        training = self.training
        if self.tp_size > 1:
            x = coll.enter_parallel_region(x, self.sequence_parallel and training)
        y = self.w2(F.silu(self.w1(x)) * self.w3(x))
        if self.tp_size > 1:
            y = coll.exit_parallel_region(y, self.sequence_parallel and training)
        return y


class TransformerBlock(nn.Module):
    def __init__(self, config: ModelArgs, freeze_norm: bool = False):
        super().__init__()
        self.attention = Attention(config)
        self.feed_forward = FeedForward(config)
        norm_cls = FrozenRMSNorm if freeze_norm else RMSNorm
        self.ffn_norm = norm_cls(config.dim, config.norm_eps)
        self.attention_norm = norm_cls(config.dim, config.norm_eps)

    def forward(self, x, input_pos, freqs_cis, mask, fully_causal: bool = False):
        h = x + self.attention(self.attention_norm(x), freqs_cis, mask, input_pos, fully_causal)
        return h + self.feed_forward(self.ffn_norm(h))


class Transformer(nn.Module):
    def __init__(self, config: ModelArgs, freeze_tok_embeddings: bool = False,
                 freeze_output: bool = False, freeze_norm: bool = False,
                 vocab_parallel: bool = False):
        super().__init__()
        self.config = config
        self.tok_embeddings = (FrozenEmbedding(config.vocab_size, config.dim)
                               if freeze_tok_embeddings
                               else nn.Embedding(config.vocab_size, config.dim))
        self.layers = nn.ModuleList(TransformerBlock(config, freeze_norm)
                                    for _ in range(config.n_layer))
        self.norm = (FrozenRMSNorm if freeze_norm else RMSNorm)(config.dim, config.norm_eps)
        self.output = (FrozenLinear(config.dim, config.vocab_size) if freeze_output
                       else nn.Linear(config.dim, config.vocab_size, bias=False))
        self.freqs_cis: Optional[Tensor] = None
        self.causal_mask: Optional[Tensor] = None
        self.max_batch_size = -1
        self.max_seq_length = -1
        self.kv_cache_enabled = False
        # Unlike the reference, which forces this flag to False (models/model.py:170) and so never
        # reaches its vocab-parallel code, the flag is honoured: apply_tp shards the LM head and
        # the losses / sampler take their vocab-parallel form.
        self.vocab_parallel = bool(vocab_parallel)
        self.tp_size = 1
        self.sequence_parallel = False
        self.activation_checkpointing = True

    @classmethod
    def from_name(cls, name: str, **kwargs) -> "Transformer":
        return cls(ModelArgs.from_name(name), **kwargs)

    # ------------------------------------------------------------------------------------
    def setup_caches(self, max_batch_size: int, max_seq_length: int, kv_cache: bool = True):
        """Allocate RoPE table, causal mask and (optionally) per-layer static KV caches. Like the
        reference (models/model.py:172-210) an existing, large-enough allocation is kept; unlike
        it, a larger request re-allocates instead of raising."""
        max_seq_length = find_multiple(max_seq_length, 8)
        have_kv = self.kv_cache_enabled or not kv_cache
        if (self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size
                and have_kv):
            return
        self.max_seq_length, self.max_batch_size = max_seq_length, max_batch_size
        dev = self.output.weight.device if hasattr(self.output, "weight") else None
        dtype = self.output.weight.dtype
        if kv_cache:
            self.kv_cache_enabled = True
            for blk in self.layers:
                att = blk.attention
                att.kv_cache = KVCache(max_batch_size, max_seq_length, att.n_local_heads,
                                       att.head_dim, dtype=dtype).to(dev)
        head_dim = self.config.dim // self.config.n_head
        self.freqs_cis = precompute_freqs_cis(max_seq_length, head_dim,
                                              self.config.rope_base).to(dev)
        self.causal_mask = torch.tril(torch.ones(max_seq_length, max_seq_length,
                                                 dtype=torch.bool, device=dev))

    def build_mask(self, input_pos: Tensor, left_pad_mask_pos: Optional[Tensor]) -> Tensor:
        """mask[b,0,i,j] = (j <= pos_i and j >= left_pad_b) or j == pos_i
        (models/model.py:221-228 of the reference)."""
        mask = self.causal_mask[None, None, input_pos]
        if left_pad_mask_pos is not None:
            j = torch.arange(self.max_seq_length, device=input_pos.device)
            pad_ok = j[None, None, None, :] >= left_pad_mask_pos[:, None, None, None]
            diag = j[None, None, None, :] == input_pos[None, None, :, None]
            mask = (mask & pad_ok) | diag
        return mask

    def logprobs_and_entropy(self, inputs: Tensor, shifts, labels: Tensor, tlen: int,
                             temperature: float, pad: int):
        """Scoring hook of ``rl_model.AutoregressivePolicy.forward`` for an unsharded model:
        hidden states of the right-pad-rotated ``inputs`` (fused kernels on CUDA under
        ``no_grad``), then the LM head + log-softmax of the last ``tlen`` positions without
        materialising the logits."""
        from ..parallel.fsdp import lm_logprobs_and_entropy
        B, L = inputs.shape
        if self.freqs_cis is None or self.max_seq_length < L or self.max_batch_size < B:
            self.setup_caches(B, L, kv_cache=self.kv_cache_enabled)
        hidden = self(inputs, torch.arange(L, device=inputs.device), fully_causal=True,
                      return_hidden=True)
        return lm_logprobs_and_entropy(self, hidden, shifts, labels, tlen, temperature, pad)

    def embed(self, idx: Tensor) -> Tensor:
        if self.vocab_parallel and self.tp_size > 1:
            return coll.vocab_parallel_embedding(idx, self.tok_embeddings.weight)
        return self.tok_embeddings(idx)

    def forward(self, idx: Tensor, input_pos: Optional[Tensor] = None,
                left_pad_mask_pos: Optional[Tensor] = None, fully_causal: bool = False,
                return_hidden: bool = False) -> Tensor:
        assert self.freqs_cis is not None, "call setup_caches first"
        if fully_causal and idx.is_cuda and not torch.is_grad_enabled():
            # scoring / log-prob passes: the whole stack on the fused sm_100a kernels
            from . import fused_block
            if fused_block.can_fuse(self, idx):
                x = fused_block.transformer_hidden(self, idx)
                return x if return_hidden else self.head(x)
        if input_pos is None:
            input_pos = torch.arange(idx.shape[1], device=idx.device)
        mask = None if fully_causal else self.build_mask(input_pos, left_pad_mask_pos)
        x = self.embed(idx)
        sp = self.sequence_parallel and self.training and self.tp_size > 1
        if sp:
            x = coll.scatter_to_sequence_parallel(x)
        freqs_cis = self.freqs_cis[input_pos]
        for blk in self.layers:
            if self.training and self.activation_checkpointing and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(blk, x, input_pos, freqs_cis, mask,
                                                      fully_causal, use_reentrant=False)
            else:
                x = blk(x, input_pos, freqs_cis, mask, fully_causal)
        x = self.norm(x)
        if sp:
            x = coll.gather_from_sequence_parallel(x, tensor_parallel_output_grad=False)
        if return_hidden:
            return x
        return self.head(x)

    def head(self, x: Tensor) -> Tensor:
        """The output projection: LM head, or a reward / value head that may be sharded over its
        input dimension (``models.tp.apply_reward_head_tp``)."""
        out = self.output
        if getattr(out, "tp_row_parallel", False):
            from .tp import reward_head_forward
            return reward_head_forward(out, x.to(out.weight.dtype))
        w = getattr(out, "weight", None)
        if isinstance(w, Tensor) and w.is_floating_point() and x.dtype != w.dtype:
            x = x.to(w.dtype)
        return out(x)
