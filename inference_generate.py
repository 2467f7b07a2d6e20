"""Batched generation entry point (same flags and file formats as the reference's
``inference_generate.py``).

    torchrun --nproc_per_node 8 inference_generate.py --prompt_file p.json --output_file o.jsonl \
        --checkpoint_path ckpts/llemma-7b-32016/model.pth --batch_size 64 --max_new_tokens 512 \
        --temperature 0.7 --top_k 50 --tensor_parallel_size 8 --compile

Reads a JSON list with ``prompt`` (or ``input``) fields, sorts prompts by token length, draws
``num_samples`` samples per prompt in left-padded batches that are dealt round-robin to the
data-parallel ranks, and appends ``{idx, sample_idx, prompt, output}`` lines to the output file
under an exclusive ``flock`` (tensor-parallel rank 0 of each group writes). ``--resume_generation``
skips the (idx, sample) pairs already present in the output file.

On CUDA, ``generate`` runs on the ``DecodeEngine`` (CUDA-graph decode over the sm_100a kernels,
static KV cache sized to prompt + new tokens instead of the whole ``block_size``); ``--compile``
is accepted for compatibility and selects the same engine.
"""
from __future__ import annotations

import argparse
import fcntl
import gc
import itertools
import json
import os
import time
from copy import deepcopy
from pathlib import Path
from typing import Optional, Tuple

import torch

from easy_to_hard_b200.models.model import Transformer, set_global_compile_mode
from easy_to_hard_b200.models.rl_model import generate_tokens
from easy_to_hard_b200.models.tokenizer_utils import AcceleraTokenizer, batch_encode_tokens
from easy_to_hard_b200.models.tp import (apply_tp, get_data_parallel_rank,
                                         get_data_parallel_world_size, get_model_parallel_rank,
                                         initialize_model_parallel, maybe_init_dist)


@torch.no_grad()
def generate(model: Transformer, prompt: torch.Tensor, left_pad_mask_pos: Optional[torch.Tensor],
             max_new_tokens: int, eos_id: Optional[int] = None, max_seq_len: Optional[int] = None,
             temperature: float = 1.0, top_k: Optional[int] = None,
             seed: int = 0) -> Tuple[torch.Tensor, int]:
    """Continue ``prompt`` [B, T] (left padded, ``left_pad_mask_pos`` = pad count per row) by
    ``max_new_tokens`` sampled tokens. Returns (sequences [B, T + max_new_tokens], number of
    decode steps after the prefill)."""
    del max_seq_len  # the cache is sized to what this call needs
    B, T = prompt.shape
    if prompt.is_cuda:
        from easy_to_hard_b200.models.engine import get_engine
        eng = get_engine(model, B, T + max_new_tokens)
        seq, steps = eng.generate(prompt, left_pad_mask_pos, max_new_tokens, temperature, top_k,
                                  eos_id, seed=seed)
        return seq, steps
    seq = generate_tokens(model, prompt, left_pad_mask_pos, max_new_tokens, temperature, top_k,
                          eos_id, seed=seed)
    return seq, max_new_tokens - 1


def _load_model(checkpoint_path: Path, device, precision, use_tp: bool) -> Transformer:
    """Meta-device build, quantised layouts picked from the file name (``int8`` /
    ``int4.g{G}``), mmap load, tensor-parallel sharding, move to the device."""
    with torch.device("meta"):
        model = Transformer.from_name(checkpoint_path.parent.name, freeze_tok_embeddings=True,
                                      freeze_output=True, freeze_norm=True)
    name = checkpoint_path.name
    if "int8" in name:
        from easy_to_hard_b200.models.quantize import WeightOnlyInt8QuantHandler
        model = WeightOnlyInt8QuantHandler(model).convert_for_runtime()
    if "int4" in name:
        from easy_to_hard_b200.models.quantize import WeightOnlyInt4QuantHandler
        group = name.split(".")[-2]
        assert group.startswith("g"), f"cannot parse the group size from {name}"
        model = WeightOnlyInt4QuantHandler(model, int(group[1:])).convert_for_runtime()
    state = torch.load(str(checkpoint_path), mmap=True, weights_only=True)
    if "int8" in name or "int4" in name:
        from easy_to_hard_b200.models.quantize import dequantize_head_in_state_dict
        g = int(name.split(".")[-2][1:]) if "int4" in name else 128
        state = dequantize_head_in_state_dict(dict(state), g)
    model.load_state_dict(state, assign=True)
    if use_tp:
        apply_tp(model)
    quantised = "int8" in name or "int4" in name
    model = model.to(device=device) if quantised else model.to(device=device, dtype=precision)
    return model.eval()


def post_process(tokens, tokenizer) -> str:
    """Cut at the first EOS and drop everything up to the last pad (left padding)."""
    tokens = list(tokens)
    if tokenizer.eos_id in tokens:
        tokens = tokens[: tokens.index(tokenizer.eos_id)]
    if tokenizer.pad_id in tokens:
        last = len(tokens) - 1 - tokens[::-1].index(tokenizer.pad_id)
        tokens = tokens[last + 1:]
    return tokenizer.decode(tokens)


def read_prompts(prompt_file: Path, tokenizer, num_samples: int):
    with open(prompt_file) as fh:
        raw = json.load(fh)
    assert "idx" not in raw[0], "Prompts already have idx field"
    key = "prompt" if "prompt" in raw[0] else "input" if "input" in raw[0] else None
    if key is None:
        raise ValueError("Prompts must have either prompt or input field")
    items = [{"idx": i, "prompt": r[key]} for i, r in enumerate(raw)]
    texts = [it["prompt"] for it in items]
    lens = tokenizer.batch_encode(texts, bos=[False] * len(texts), eos=[False] * len(texts))
    for it, ids in zip(items, lens):
        it["prompt_len"] = len(ids)
    items.sort(key=lambda it: it["prompt_len"])  # similar lengths share a batch: less padding
    out = []
    for it in items:
        for s in range(num_samples):
            c = deepcopy(it)
            c["sample_idx"] = s
            out.append(c)
    return out


def drop_finished(prompts, output_file: Path):
    """Remove as many samples of each idx as the output file already holds."""
    done = {}
    if os.path.isfile(output_file):
        with open(output_file) as fh:
            for line in fh:
                if line.strip():
                    i = json.loads(line)["idx"]
                    done[i] = done.get(i, 0) + 1
    keep = []
    for p in prompts:
        if done.get(p["idx"], 0) > 0:
            done[p["idx"]] -= 1
        else:
            keep.append(p)
    return keep


def main(seed: int, prompt_file: Path, output_file: Path, batch_size: int = 4,
         num_samples: int = 5, max_new_tokens: int = 100, top_k: int = 200,
         temperature: float = 0.8,
         checkpoint_path: Path = Path("checkpoints/llemma-7b/model.pth"), compile: bool = True,
         default_compile: bool = False, finetune_checkpoint_path: Optional[Path] = None,
         finetune_checkpoint_prefix: Optional[str] = None, resume_generation: bool = False,
         tensor_parallel_size: Optional[int] = None,
         on_the_fly_8bit_quantization: bool = False) -> None:
    assert checkpoint_path.is_file(), checkpoint_path
    assert not (compile and default_compile), "Cannot compile with both modes"
    set_global_compile_mode(compile or default_compile)
    tok_path = checkpoint_path.parent / "tokenizer.model"
    if not tok_path.is_file():
        tok_path = checkpoint_path.parent
    rank = maybe_init_dist()
    use_tp = rank is not None
    log = print if (rank in (None, 0)) else (lambda *a, **k: None)
    initialize_model_parallel(
        (tensor_parallel_size or torch.distributed.get_world_size()) if use_tp else 1)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    precision = torch.bfloat16 if device == "cuda" else torch.float32

    t0 = time.time()
    model = _load_model(checkpoint_path, device, precision, use_tp)
    if finetune_checkpoint_path is not None:
        from easy_to_hard_b200.utils.checkpoint_utils import (get_latest_checkpoint_path,
                                                              load_inference_checkpoint)
        path, _, _ = get_latest_checkpoint_path(finetune_checkpoint_path,
                                                prefix=finetune_checkpoint_prefix)
        if path is not None:
            log(f"Loading finetune model from {path} ...")
            load_inference_checkpoint(path, model)
        model = model.to(device=device).eval()
    if on_the_fly_8bit_quantization:
        from easy_to_hard_b200.models.quantize import WeightOnlyInt8QuantHandler
        model = WeightOnlyInt8QuantHandler(model).convert_for_runtime_on_the_fly()
        model = model.to(device=device).eval()
    if device == "cuda":
        torch.cuda.synchronize()
    log(f"Time to load model: {time.time() - t0:.02f} seconds")

    tokenizer = AcceleraTokenizer(tok_path, model_vocab_size=model.config.vocab_size)
    torch.manual_seed(seed)
    model_size = sum(p.numel() * p.element_size()
                     for p in itertools.chain(model.parameters(), model.buffers()))
    prompts = read_prompts(prompt_file, tokenizer, num_samples)
    if rank in (None, 0):
        output_file.parent.mkdir(exist_ok=True, parents=True)
    if use_tp:
        torch.distributed.barrier()
    if resume_generation:
        prompts = drop_finished(prompts, output_file)
    if not prompts:
        log("Nothing left to generate.")
        return
    while len(prompts) % batch_size:
        prompts.insert(0, prompts[0])
    dp_rank, dp_size = get_data_parallel_rank(), get_data_parallel_world_size()
    tp_rank = get_model_parallel_rank()
    writer = open(output_file, "a") if tp_rank == 0 else None
    gc.collect()

    for b, start in enumerate(range(0, len(prompts), batch_size), start=1):
        if b % dp_size != dp_rank:
            continue
        batch = prompts[start: start + batch_size]
        ids, left_pad = batch_encode_tokens(tokenizer, [p["prompt"] for p in batch], bos=True,
                                            device=device)
        T = ids.size(1)
        new = min(max_new_tokens, model.config.block_size - T - 1)
        if device == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        y, n_dec = generate(model, ids, left_pad, new, temperature=temperature, top_k=top_k,
                            eos_id=tokenizer.eos_id, seed=seed + b)
        rows = y.tolist()  # device -> host: also the synchronisation point of the timing
        dt = time.perf_counter() - t0
        toks = (n_dec + 1) * y.size(0)
        log(post_process(rows[0], tokenizer))
        log(f"Prompt length: {T}")
        log(f"Time for inference {start + batch_size} / {len(prompts)}: {dt:.02f} sec total, "
            f"{toks / dt:.02f} tokens/sec")
        log(f"Bandwidth achieved: {model_size * toks / dt / 1e9:.02f} GB/s")
        if writer is not None:
            fcntl.flock(writer, fcntl.LOCK_EX)
            try:
                for p, row in zip(batch, rows):
                    writer.write(json.dumps({"idx": p["idx"], "sample_idx": p["sample_idx"],
                                             "prompt": p["prompt"],
                                             "output": post_process(row[T:], tokenizer)}) + "\n")
                writer.flush()
            finally:
                fcntl.flock(writer, fcntl.LOCK_UN)
    if writer is not None:
        writer.close()


def _cli() -> argparse.Namespace:
    ap = argparse.ArgumentParser(description="Batched generation with a static KV cache.")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--prompt_file", type=Path, required=True)
    ap.add_argument("--output_file", type=Path, required=True)
    ap.add_argument("--batch_size", type=int, default=4)
    ap.add_argument("--num_samples", type=int, default=1)
    ap.add_argument("--max_new_tokens", type=int, default=200)
    ap.add_argument("--top_k", type=int, default=200)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--checkpoint_path", type=Path,
                    default=Path("checkpoints/llemma-7b/model.pth"))
    ap.add_argument("--compile", action="store_true")
    ap.add_argument("--default_compile", action="store_true")
    ap.add_argument("--finetune_checkpoint_path", type=Path, default=None)
    ap.add_argument("--finetune_checkpoint_prefix", type=str, default=None)
    ap.add_argument("--resume_generation", action="store_true")
    ap.add_argument("--tensor_parallel_size", type=int, default=None)
    ap.add_argument("--on_the_fly_8bit_quantization", action="store_true")
    return ap.parse_args()


if __name__ == "__main__":
    a = _cli()
    main(a.seed, a.prompt_file, a.output_file, a.batch_size, a.num_samples, a.max_new_tokens,
         a.top_k, a.temperature, a.checkpoint_path, a.compile, a.default_compile,
         a.finetune_checkpoint_path, a.finetune_checkpoint_prefix, a.resume_generation,
         a.tensor_parallel_size, a.on_the_fly_8bit_quantization)
