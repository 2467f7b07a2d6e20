"""Policy / value wrappers for RL and the generic (module-path) sampling loop.

API of the reference's ``models/rl_model.py``: ``AutoregressivePolicy.{forward,respond}``,
``AutoregressiveValue``, ``prefill`` / ``decode_one_token`` / ``decode_n_tokens`` / ``sample``,
``compute_logprobs`` and the left/right padding helpers.

Scoring forward (rl_model.py:117-160 of the reference): queries are left-padded and responses
right-padded; the concatenation is rotated so that padding sits at the tail ("right-pad roll"),
run through the fully-causal model, rotated back, and the last ``target_max_len`` positions give
fp32 log-probs and entropies. Generation (rl_model.py:162-230): on CUDA it runs on the
``DecodeEngine`` (CUDA-graph decode, on-device EOS tracking); on CPU the same semantics run
through the module forward, one token at a time.
"""
from __future__ import annotations

import abc
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from ..ops import reference as ref_ops
from . import tp as tp_mod
from .model import Transformer


# ----------------------------------------------------------------------------- padding helpers

def _first_true(mask: Tensor) -> Tensor:
    """Index of the first True per row (0 for an all-False row)."""
    return torch.argmax(mask.to(torch.int32), dim=1)


def _rotate_rows(x: Tensor, shifts: Tensor) -> Tensor:
    """out[b, i] = x[b, (i + shifts[b]) mod T] for x [B, T, ...]."""
    T = x.size(1)
    idx = (torch.arange(T, device=x.device)[None, :] + shifts[:, None]) % T
    idx = idx.view(idx.shape + (1,) * (x.dim() - 2)).expand_as(x)
    return torch.gather(x, 1, idx)


def prepare_right_pad_sequences(input_ids: Tensor, attention_mask: Optional[Tensor] = None,
                                pad_token_id: int = 0) -> Tuple[Tensor, Tensor]:
    """Rotate every row left by its number of leading pads, so pads end up at the tail."""
    if attention_mask is None:
        attention_mask = input_ids != pad_token_id
    shifts = _first_true(attention_mask)
    return _rotate_rows(input_ids, shifts), shifts


def restore_from_right_pad_sequences(inputs: Tensor, shifts: Optional[Tensor]) -> Tensor:
    if shifts is None:
        return inputs
    return _rotate_rows(inputs, -shifts)


def prepare_left_pad_mask_pos(input_ids: Tensor, attention_mask: Optional[Tensor] = None,
                              pad_token_id: int = 0) -> Tensor:
    if attention_mask is None:
        attention_mask = input_ids != pad_token_id
    return _first_true(attention_mask)


# ----------------------------------------------------------------------------- sampling

def multinomial_sample_one_no_sync(probs: Tensor) -> Tensor:
    return ref_ops.sample_from_probs(probs)


logits_to_probs = ref_ops.logits_to_probs


def sample(logits: Tensor, vocab_parallel: bool, temperature: float = 1.0,
           top_k: Optional[int] = None) -> Tuple[Tensor, Tensor]:
    """Sample from the last position of ``logits`` [B, S, V(/tp)]."""
    last = logits[:, -1].float()
    if vocab_parallel and tp_mod.get_model_parallel_world_size() > 1:
        from ..parallel import collectives as coll
        last = coll._gather_last_dim(last)
    return ref_ops.sample(last, temperature, top_k)


def prefill(model: Transformer, x: Tensor, input_pos: Tensor, left_pad_mask_pos: Tensor,
            **sampling_kwargs) -> Tensor:
    logits = model(x, input_pos, left_pad_mask_pos)
    return sample(logits, model.vocab_parallel, **sampling_kwargs)[0]


def decode_one_token(model: Transformer, x: Tensor, input_pos: Tensor, left_pad_mask_pos: Tensor,
                     **sampling_kwargs) -> Tuple[Tensor, Tensor]:
    assert input_pos.shape[-1] == 1
    logits = model(x, input_pos, left_pad_mask_pos)
    return sample(logits, model.vocab_parallel, **sampling_kwargs)


def decode_n_tokens(model: Transformer, cur_token: Tensor, input_pos: Tensor,
                    left_pad_mask_pos: Tensor, num_new_tokens: int, eos_id: Optional[int] = None,
                    **sampling_kwargs):
    """Module-path decode loop (CPU oracle / fallback). Returns (tokens, probs, last index)."""
    eos_flag = torch.zeros_like(cur_token, dtype=torch.bool) if eos_id is not None else None
    new_tokens, new_probs = [], []
    i = -1
    for i in range(num_new_tokens):
        nxt, prob = decode_one_token(model, cur_token, input_pos, left_pad_mask_pos,
                                     **sampling_kwargs)
        input_pos = input_pos + 1
        new_tokens.append(nxt.clone().view(-1, 1))
        new_probs.append(prob)
        cur_token = nxt.view(-1, 1).to(cur_token.dtype)
        if eos_flag is not None:
            eos_flag |= cur_token == eos_id
            if bool(eos_flag.all()):
                break
    return new_tokens, new_probs, i


def compute_logprobs(logits: Tensor, labels: Tensor, ignore_index: int) -> Tensor:
    """Per-token log-probs of ``labels``; 0 where ``labels == ignore_index``."""
    return -F.cross_entropy(logits.permute(0, 2, 1), labels, reduction="none",
                            ignore_index=ignore_index)


@torch.no_grad()
def generate_tokens(model: Transformer, queries: Tensor, left_pad_mask_pos: Optional[Tensor],
                    max_new_tokens: int, temperature: float, top_k: Optional[int],
                    eos_id: Optional[int], seed: int = 0) -> Tensor:
    """Returns [B, T + max_new_tokens]; positions after an early stop stay 0."""
    B, T = queries.shape
    if queries.is_cuda:
        from .engine import get_engine
        eng = get_engine(model, B, T + max_new_tokens)
        seq, _ = eng.generate(queries, left_pad_mask_pos, max_new_tokens, temperature, top_k,
                              eos_id, seed=seed)
        return seq.to(queries.dtype)
    model.setup_caches(max_batch_size=B, max_seq_length=T + max_new_tokens)
    seq = torch.zeros(B, T + max_new_tokens, dtype=queries.dtype, device=queries.device)
    seq[:, :T] = queries
    kw = dict(temperature=temperature, top_k=top_k)
    nxt = prefill(model, queries, torch.arange(T, device=queries.device), left_pad_mask_pos, **kw)
    seq[:, T] = nxt.view(B)
    toks, _, _ = decode_n_tokens(model, nxt.view(B, 1).to(queries.dtype),
                                 torch.tensor([T], device=queries.device), left_pad_mask_pos,
                                 max_new_tokens - 1, eos_id, **kw)
    if toks:
        gen = torch.cat(toks, dim=-1).view(B, -1)
        seq[:, T + 1: T + 1 + gen.size(1)] = gen
    return seq


# ----------------------------------------------------------------------------- wrappers

class Policy(nn.Module, abc.ABC):
    def __init__(self, args, base_model: Transformer, base_tokenizer):
        super().__init__()
        self.args = args
        self.base_model = base_model
        self.base_tokenizer = base_tokenizer

    @abc.abstractmethod
    def forward(self, queries, query_attn_masks, responses=None, temperature=None, mode=None):
        raise NotImplementedError

    def respond(self, queries, query_attn_masks, temperature=None, num_return_sequences=1):
        assert not self.training, "Policy must be in eval mode for generation."
        return self._post_respond(
            self._respond(queries, query_attn_masks, temperature, num_return_sequences))

    @abc.abstractmethod
    def _respond(self, queries, query_attn_masks, temperature=None, num_return_sequences=1):
        raise NotImplementedError

    def _post_respond(self, respond_outputs):
        return respond_outputs


def _unwrap(m):
    return getattr(m, "module", m)


class AutoregressivePolicy(Policy):
    def forward(self, queries: Tensor, query_attn_masks: Tensor,
                responses: Optional[Tensor] = None, temperature: Optional[float] = None,
                mode: Optional[str] = None) -> Dict[str, Tensor]:
        if mode == "respond":
            return self.respond(queries, query_attn_masks, temperature)
        assert responses is not None
        temperature = self.args.temperature if temperature is None else temperature
        pad = self.base_tokenizer.pad_id
        tlen = self.args.target_max_len
        input_ids = torch.cat([queries, responses], dim=1)
        attn = input_ids.ne(pad)
        attn[:, : queries.size(1)] = query_attn_masks
        inputs, shifts = prepare_right_pad_sequences(input_ids, attn, pad)
        pos = torch.arange(input_ids.size(1), device=input_ids.device)
        base = _unwrap(self.base_model)
        labels = input_ids[:, -tlen:]
        fused = getattr(self.base_model, "logprobs_and_entropy", None)
        if fused is not None:
            # fused LM-head + log-softmax path: never materialises [B, T, V] logits
            logprobs, entropies = fused(inputs, shifts, labels, tlen, temperature, pad)
        else:
            logits = self.base_model(inputs, pos, fully_causal=True).float()
            logits = restore_from_right_pad_sequences(logits, shifts)
            logits = logits[:, -tlen - 1: -1] / temperature
            if base.vocab_parallel and tp_mod.get_model_parallel_world_size() > 1:
                logprobs = tp_mod.compute_vocab_parallel_logprobs(logits, labels, pad)
                from ..parallel import collectives as coll
                full = coll.gather_last_dim(logits)
            else:
                logprobs = compute_logprobs(logits, labels, ignore_index=pad)
                full = logits
            logp_all = full.log_softmax(dim=-1)
            entropies = -(logp_all.exp() * logp_all).sum(dim=-1)
        keep = labels.ne(pad).to(entropies.dtype)
        return dict(logprobs=logprobs, entropies=entropies, reg_entropies=entropies * keep,
                    reg_entropies_weight=keep)

    def _respond(self, queries: Tensor, query_attn_masks: Tensor,
                 temperature: Optional[float] = None, num_return_sequences=1):
        del num_return_sequences
        base = _unwrap(self.base_model)
        T = queries.size(1)
        tlen = self.args.target_max_len
        assert T + tlen <= base.config.block_size
        temperature = self.args.temperature if temperature is None else temperature
        shifts = prepare_left_pad_mask_pos(queries, query_attn_masks, self.base_tokenizer.pad_id)
        seq = generate_tokens(base, queries, shifts, tlen, temperature,
                              getattr(self.args, "rollout_top_k", 50),
                              self.base_tokenizer.eos_id,
                              seed=int(torch.randint(0, 2 ** 31 - 1, (1,)).item()))
        return dict(responses=seq[:, T:])


class Value(nn.Module, abc.ABC):
    def __init__(self, args, base_model, base_tokenizer):
        super().__init__()
        self.args = args
        self.base_model = base_model
        self.base_tokenizer = base_tokenizer
        self.initialized = False

    @abc.abstractmethod
    def forward(self, queries, query_attn_masks, responses):
        raise NotImplementedError


class AutoregressiveValue(Value):
    def forward(self, queries: Tensor, query_attn_masks: Tensor, responses: Tensor):
        assert self.initialized, "Value model must be initialized before forward pass."
        pad = self.base_tokenizer.pad_id
        sequences = torch.cat([queries, responses], dim=1)
        attn = sequences.ne(pad)
        attn[:, : queries.size(1)] = query_attn_masks
        inputs, shifts = prepare_right_pad_sequences(sequences, attn, pad)
        pos = torch.arange(sequences.size(1), device=queries.device)
        values = self.base_model(inputs, pos, fully_causal=True)
        if values.dim() == 3:
            values = values.mean(dim=-1)
        values = restore_from_right_pad_sequences(values, shifts)
        values = values[:, queries.size(1) - 1: -1]
        assert values.size(1) == responses.size(1)
        return dict(values=values)


def make_policy_with_base_model(args, base_model, base_tokenizer) -> AutoregressivePolicy:
    return AutoregressivePolicy(args, base_model, base_tokenizer)


def make_value_with_base_model(args, base_model, base_tokenizer) -> AutoregressiveValue:
    v = AutoregressiveValue(args, base_model, base_tokenizer)
    v.initialized = True
    return v
