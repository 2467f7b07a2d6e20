"""Single-sequence generation with optional speculative decoding and an interactive prompt loop
(same flags as the reference's ``interactive.py``).

    python interactive.py --checkpoint_path ckpts/llemma-7b-32016/model.pth \
        --prompt "Hello, my name is" --num_samples 3 --max_new_tokens 200 --top_k 200 \
        --temperature 0.8 [--draft_checkpoint_path ckpts/small/model.pth --speculate_k 5] \
        [--interactive] [--profile trace]

Plain decoding of a CUDA model runs on the ``DecodeEngine`` (CUDA-graph decode step, batch 1).
Speculative decoding follows interactive.py:87-160 of the reference: the draft model proposes
``speculate_k`` tokens one by one, the target model scores them in a single ``k+1``-token
forward against its KV cache, each draft token is accepted with probability min(1, q/p), and the
first rejection is replaced by a sample from the normalised positive part of ``q - p``; when all
are accepted one extra token is sampled from the target's last distribution. ``accept_counts``
report how many tokens each round produced.
"""
from __future__ import annotations

import argparse
import itertools
import sys
import time
from pathlib import Path
from typing import List, Optional, Tuple

import torch

from easy_to_hard_b200.models.model import Transformer
from easy_to_hard_b200.models.tokenizer_utils import AcceleraTokenizer
from easy_to_hard_b200.models.tp import initialize_model_parallel, maybe_init_dist
from easy_to_hard_b200.utils.checkpoint_utils import (get_latest_checkpoint_path,
                                                      load_inference_checkpoint)
from inference_generate import _load_model

B_INST, E_INST = "[INST]", "[/INST]"


def multinomial_sample_one_no_sync(probs: torch.Tensor) -> torch.Tensor:
    """argmax(p / Exp(1)) is a draw from p; needs no host synchronisation."""
    q = torch.empty_like(probs).exponential_(1)
    return torch.argmax(probs / q, dim=-1, keepdim=True).to(dtype=torch.int)


def logits_to_probs(logits: torch.Tensor, temperature: float = 1.0,
                    top_k: Optional[int] = None) -> torch.Tensor:
    logits = logits.float() / max(temperature, 1e-5)
    if top_k is not None:
        v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
        logits = torch.where(logits < v[..., -1:], -float("inf"), logits)
    return torch.softmax(logits, dim=-1)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None):
    probs = logits_to_probs(logits[0, -1], temperature, top_k)
    return multinomial_sample_one_no_sync(probs), probs


def model_forward(model: Transformer, x: torch.Tensor, input_pos: torch.Tensor) -> torch.Tensor:
    return model(x, input_pos)


def prefill(model, x, input_pos, **sampling_kwargs) -> torch.Tensor:
    return sample(model_forward(model, x, input_pos), **sampling_kwargs)[0]


def decode_one_token(model, x, input_pos, **sampling_kwargs):
    assert input_pos.shape[-1] == 1
    return sample(model_forward(model, x, input_pos), **sampling_kwargs)


def decode_n_tokens(model, cur_token, input_pos, num_new_tokens: int, callback=lambda _: _,
                    **sampling_kwargs) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
    new_tokens, new_probs = [], []
    for _ in range(num_new_tokens):
        next_token, next_prob = decode_one_token(model, cur_token, input_pos, **sampling_kwargs)
        input_pos = input_pos + 1
        new_tokens.append(next_token.clone())
        callback(new_tokens[-1])
        new_probs.append(next_prob.clone())
        cur_token = next_token.view(1, -1)
    return new_tokens, new_probs


def speculative_decode(model, draft_model, cur_token: torch.Tensor, input_pos: int,
                       speculate_k: int, **sampling_kwargs) -> torch.Tensor:
    device = cur_token.device
    pos0 = torch.tensor([input_pos], dtype=torch.int64, device=device)
    draft_tokens, draft_probs = decode_n_tokens(draft_model, cur_token.view(1, -1), pos0.clone(),
                                                speculate_k, **sampling_kwargs)
    draft_tokens = torch.cat(draft_tokens)
    target_logits = model_forward(
        model, torch.cat([cur_token.view(1), draft_tokens]).view(1, -1),
        torch.arange(input_pos, input_pos + speculate_k + 1, device=device))
    target_probs = logits_to_probs(target_logits[0], **sampling_kwargs)
    draft_probs = torch.stack(draft_probs)
    idx = torch.arange(speculate_k, device=device)
    p = draft_probs[idx, draft_tokens.long()]          # draft probability of its own proposal
    q = target_probs[idx, draft_tokens.long()]         # target probability of the same token
    accept = torch.minimum(torch.ones((), device=device), q / p)
    rejected = (torch.rand_like(accept) > accept).nonzero()
    if rejected.shape[0] == 0:                          # all accepted: one bonus token
        last = multinomial_sample_one_no_sync(target_probs[-1])
        model_forward(draft_model, draft_tokens[-1].view(1, -1), pos0 + speculate_k)
        return torch.cat([draft_tokens, last])
    n_ok = rejected[0].item()
    new = torch.clamp(target_probs[n_ok] - draft_probs[n_ok], min=0.0)
    new = new / new.sum()
    return torch.cat([draft_tokens[:n_ok], multinomial_sample_one_no_sync(new)])


@torch.no_grad()
def generate(model: Transformer, prompt: torch.Tensor, max_new_tokens: int, *, interactive: bool,
             draft_model: Optional[Transformer], speculate_k: int = 8, callback=lambda x: x,
             **sampling_kwargs):
    """prompt [T] -> (sequence [T + max_new_tokens], {"accept_counts": [...]})"""
    speculative = draft_model is not None
    T = prompt.size(0)
    T_new = T + max_new_tokens
    max_seq = 350 if interactive else min(T_new, model.config.block_size)
    max_seq = max(max_seq, T + 1)
    if speculative:
        max_seq += speculate_k + 1
    device, dtype = prompt.device, prompt.dtype
    accept_counts = [0] * (speculate_k + 1)
    if not speculative and prompt.is_cuda and not interactive:
        from easy_to_hard_b200.models.engine import get_engine
        eng = get_engine(model, 1, T_new)
        seq, _ = eng.generate(prompt.view(1, -1).int(), None, max_new_tokens,
                              sampling_kwargs.get("temperature", 1.0),
                              sampling_kwargs.get("top_k"), None,
                              seed=int(torch.randint(0, 2 ** 31 - 1, (1,)).item()))
        return seq[0].to(dtype), {"accept_counts": accept_counts}
    model.setup_caches(max_batch_size=1, max_seq_length=max_seq)
    if speculative and draft_model is not model:
        draft_model.setup_caches(max_batch_size=1, max_seq_length=max_seq)
    seq = torch.empty(T_new, dtype=dtype, device=device)
    seq[:T] = prompt
    input_pos = torch.arange(0, T, device=device)
    next_token = prefill(model, prompt.view(1, -1), input_pos, **sampling_kwargs)
    if speculative:
        prefill(draft_model, prompt.view(1, -1), input_pos, **sampling_kwargs)
    seq[T] = next_token
    if speculative:
        pos = T
        while pos < T_new - 1:
            nxt = speculative_decode(model, draft_model, next_token.view(()), pos, speculate_k,
                                     **sampling_kwargs)
            accept_counts[len(nxt) - 1] += 1
            n = min(T_new - pos - 1, len(nxt))
            seq[pos + 1: pos + n + 1] = nxt[:n]
            for t in nxt[:n]:
                callback(t)
            pos += n
            next_token = nxt[-1]
    else:
        toks, _ = decode_n_tokens(model, next_token.view(1, -1),
                                  torch.tensor([T], device=device, dtype=torch.int64),
                                  max_new_tokens - 1, callback=callback, **sampling_kwargs)
        if toks:
            seq[T + 1:] = torch.cat(toks)
    return seq, {"accept_counts": accept_counts}


def encode_tokens(tokenizer, string: str, bos: bool = True, device="cuda") -> torch.Tensor:
    return torch.tensor(tokenizer.encode(string, bos=bos, eos=False), dtype=torch.int,
                        device=device)


def main(prompt: str = "Hello, my name is", interactive: bool = False, num_samples: int = 5,
         max_new_tokens: int = 100, top_k: int = 200, temperature: float = 0.8,
         checkpoint_path: Path = Path("checkpoints/meta-Transformer/Transformer-2-7b-chat-hf/model.pth"),
         compile: bool = True, compile_prefill: bool = False, profile: Optional[Path] = None,
         draft_checkpoint_path: Optional[Path] = None,
         finetune_checkpoint_path: Optional[Path] = None, speculate_k: int = 5) -> dict:
    del compile, compile_prefill   # accepted for compatibility; no tracing compiler is used
    checkpoint_path = Path(checkpoint_path)
    assert checkpoint_path.is_file(), checkpoint_path
    tokenizer_path = checkpoint_path.parent / "tokenizer.model"
    assert tokenizer_path.is_file(), tokenizer_path
    rank = maybe_init_dist()
    use_tp = rank is not None
    if use_tp:
        initialize_model_parallel(torch.distributed.get_world_size())
    say = print if rank in (None, 0) else (lambda *a, **k: None)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    precision = torch.bfloat16 if device == "cuda" else torch.float32
    speculative = draft_checkpoint_path is not None
    is_chat = "chat" in str(checkpoint_path)

    say("Loading model ...")
    t0 = time.time()
    model = _load_model(checkpoint_path, device, precision, use_tp)
    if finetune_checkpoint_path is not None:
        path, _, _ = get_latest_checkpoint_path(finetune_checkpoint_path)
        say("Loading finetune model ...")
        if path is not None:
            load_inference_checkpoint(path, model)
    draft_model = (_load_model(Path(draft_checkpoint_path), device, precision, use_tp)
                   if speculative else None)
    say(f"Time to load model: {time.time() - t0:.02f} seconds")

    tokenizer = AcceleraTokenizer(tokenizer_path)
    encoded = encode_tokens(tokenizer, prompt, bos=True, device=device)
    torch.manual_seed(1234)
    model_size = sum(p.numel() * p.element_size()
                     for p in itertools.chain(model.parameters(), model.buffers()))
    metrics = {"tokens_per_sec": [], "accept_counts": []}
    for i in range(num_samples):
        if interactive:
            prompt = input("What is your prompt? ")
            if is_chat:
                prompt = f"{B_INST} {prompt.strip()} {E_INST}"
            encoded = encode_tokens(tokenizer, prompt, bos=True, device=device)
        buffer: List[str] = []
        period_id = tokenizer.encode(".", bos=False, eos=False)[-1]
        done = False

        def callback(x):
            nonlocal done
            if not interactive or done:
                return
            buffer.append(tokenizer.decode([period_id] + x.view(-1).tolist())[1:])
            if x.item() == tokenizer.eos_id:
                done = True
            if len(buffer) == 4 or done:
                print("".join(buffer), end="", flush=True)
                buffer.clear()
        prof = None
        if profile is not None and i == num_samples - 1 and (not use_tp or rank == 0):
            prof = torch.profiler.profile()
            prof.__enter__()
        if device == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        y, stats = generate(model, encoded, max_new_tokens, draft_model=draft_model,
                            speculate_k=speculate_k, interactive=interactive, callback=callback,
                            temperature=temperature, top_k=top_k)
        if device == "cuda":
            torch.cuda.synchronize()
        t = time.perf_counter() - t0
        metrics["accept_counts"].append(stats["accept_counts"])
        if prof is not None:
            prof.__exit__(None, None, None)
            prof.export_chrome_trace(f"{profile}_rank_{rank}.json" if use_tp else f"{profile}.json")
        if interactive:
            print()
        else:
            say(tokenizer.decode(y.tolist()))
        n_gen = y.size(0) - encoded.size(0)
        tps = n_gen / t
        metrics["tokens_per_sec"].append(tps)
        say(f"Time for inference {i + 1}: {t:.02f} sec total, {tps:.02f} tokens/sec")
        say(f"Bandwidth achieved: {model_size * tps / 1e9:.02f} GB/s")
    say("==========")
    if speculative:
        counts = [sum(c) for c in zip(*metrics["accept_counts"])]
        total = max(1, sum(counts))
        say(f"Acceptance probs: {[c / total for c in counts]}")
        say(f"Mean Accepted: {sum((k + 1) * c for k, c in enumerate(counts)) / total}")
    mean_tps = sum(metrics["tokens_per_sec"]) / max(1, len(metrics["tokens_per_sec"]))
    say(f"Average tokens/sec: {mean_tps:.2f}")
    if device == "cuda":
        say(f"Memory used: {torch.cuda.max_memory_reserved() / 1e9:.02f} GB")
    return metrics


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Generate from a prompt, optionally speculatively.")
    ap.add_argument("--prompt", type=str, default="Hello, my name is")
    ap.add_argument("--interactive", action="store_true")
    ap.add_argument("--num_samples", type=int, default=5)
    ap.add_argument("--max_new_tokens", type=int, default=200)
    ap.add_argument("--top_k", type=int, default=200)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--checkpoint_path", type=Path,
                    default=Path("checkpoints/meta-Transformer/Transformer-2-7b-chat-hf/model.pth"))
    ap.add_argument("--compile", action="store_true")
    ap.add_argument("--compile_prefill", action="store_true")
    ap.add_argument("--profile", type=Path, default=None)
    ap.add_argument("--speculate_k", type=int, default=5)
    ap.add_argument("--draft_checkpoint_path", type=Path, default=None)
    ap.add_argument("--finetune_checkpoint_path", type=Path, default=None)
    a = ap.parse_args()
    main(a.prompt, a.interactive, a.num_samples, a.max_new_tokens, a.top_k, a.temperature,
         a.checkpoint_path, a.compile, a.compile_prefill, a.profile, a.draft_checkpoint_path,
         a.finetune_checkpoint_path, a.speculate_k)
