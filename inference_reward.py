"""Process-reward scoring entry point (same flags and file formats as the reference's
``inference_reward.py``), plus the best-of-N aggregation the reference leaves to external
scripts.

    torchrun --nproc_per_node 8 inference_reward.py --prompt_file samples.jsonl \
        --output_file scored.jsonl --checkpoint_path ckpts/llemma-7b-32016/model.pth \
        --finetune_checkpoint_path ckpts/prm --batch_size 64 --tensor_parallel_size 2 \
        --aggregate min --best_of_n_file best.jsonl

Input: JSON lines ``{idx, sample_idx, prompt, output}`` (what ``inference_generate.py`` writes).
Samples are sorted by token length, padded on the right, dealt round-robin to the
data-parallel ranks and scored in one fully-causal pass (fused sm_100a kernels on CUDA). The
reward of a reasoning step is the model's score at the first token of the blank line that ends
the step (inference_reward.py:379-453 of the reference). Output lines are appended under an
exclusive ``flock`` by tensor-parallel rank 0: ``{idx, sample_idx, prompt, output, reward:
[step scores]}``; with ``--aggregate`` an ``aggregate_reward`` field (min / prod / last / mean of
the step scores after a sigmoid) is added, and ``--best_of_n_file`` receives the best sample of
every ``idx``.
"""
from __future__ import annotations

import argparse
import fcntl
import gc
import itertools
import json
import math
import os
import time
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from easy_to_hard_b200.models.reward_model import RewardModel, apply_reward_modeling_head
from easy_to_hard_b200.models.tokenizer_utils import AcceleraTokenizer, batch_encode_tokens
from easy_to_hard_b200.models.tp import (apply_reward_head_tp, apply_tp, get_data_parallel_rank,
                                         get_data_parallel_world_size, get_model_parallel_rank,
                                         initialize_model_parallel, maybe_init_dist)
from easy_to_hard_b200.utils.checkpoint_utils import (get_latest_checkpoint_path,
                                                      load_inference_checkpoint)

BROKEN_ANSWER_SCORE = -5.0


@torch.no_grad()
def model_score(model: RewardModel, prompt: torch.Tensor,
                max_seq_len: Optional[int] = None) -> torch.Tensor:
    """Per-token rewards [B, T] of right-padded sequences."""
    B, T = prompt.shape
    model.backbone_model.setup_caches(max_batch_size=B, max_seq_length=max_seq_len or T,
                                      kv_cache=False)
    return model(prompt)


def _load_reward_model(checkpoint_path: Path, device, precision, use_tp: bool) -> RewardModel:
    for tag in ("int8", "int4"):
        if tag in str(checkpoint_path):
            raise NotImplementedError(f"{tag} quantization cannot be used for reward model!")
    with torch.device("meta"):
        model = RewardModel.from_name(checkpoint_path.parent.name)
    sd = torch.load(str(checkpoint_path), mmap=True, weights_only=True)
    model.backbone_model.load_state_dict(sd, assign=True)
    if use_tp:
        apply_tp(model.backbone_model)
    apply_reward_modeling_head(model.backbone_model)
    if use_tp:
        apply_reward_head_tp(model.backbone_model)
    return model.to(device=device, dtype=precision).eval()


def find_step_boundaries(ids: Sequence[int], newline_id: int) -> List[int]:
    """Indices i with ids[i] == ids[i+1] == newline_id, scanned left to right without overlap
    (a run of three newline tokens is one boundary)."""
    out, i, n = [], 0, len(ids)
    while i + 1 < n:
        if ids[i] == newline_id and ids[i + 1] == newline_id:
            out.append(i)
            i += 2
        else:
            i += 1
    return out


def post_process_newline_scores(encoded_full_seq: Sequence[int], scores: Sequence[float],
                                prompt: str, output: str, process_reward_with_answer: bool,
                                newline_id: int = 13, eos_id: int = 2, pad_id: int = 0
                                ) -> Tuple[List[float], str]:
    """Step scores of one sample and a human-readable rendering.

    The text is ``prompt`` (ending in a blank line) + ``output``; ``output`` is a sequence of
    steps separated by blank lines, optionally followed by ``# Answer`` / blank line / the
    answer. A step's score is read at the first newline token of the blank line closing it.
    Steps are those before ``# Answer``; the last of them is skipped, and the answer scored at
    its last token instead (``BROKEN_ANSWER_SCORE`` if the sequence does not end in EOS), when
    ``process_reward_with_answer`` is set. Steps cut off by truncation are dropped."""
    ids = [t for t in encoded_full_seq if t != pad_id]
    assert prompt.endswith("\n\n")
    n_prompt = prompt.count("\n\n")
    n_out = output.split("# Answer")[0].count("\n\n")
    bounds = find_step_boundaries(ids, newline_id)
    assert n_prompt + n_out <= len(bounds), (n_prompt, n_out, len(bounds))
    segments = output.split("\n\n")
    step_scores: List[float] = []
    pretty = [prompt.strip()]
    for k in range(min(n_out, len(segments))):
        pos = bounds[n_prompt + k]                 # first newline token of the k-th output gap
        last_step = k == n_out - 1
        if pos + 1 < len(scores) and not (last_step and process_reward_with_answer):
            step_scores.append(float(scores[pos]))
            near = ",".join(f"{scores[q]}" for q in (pos - 1, pos, pos + 1) if 0 <= q < len(scores))
            pretty.append(f"{segments[k]} ({near})")
        else:
            pretty.append(segments[k])
    for k in range(n_out, len(segments)):
        is_answer = k == n_out + 1
        if is_answer and process_reward_with_answer:
            if ids and ids[-1] == eos_id and len(ids) >= 2:
                step_scores.append(float(scores[len(ids) - 2]))
                pretty.append(f"{segments[k]} ({scores[len(ids) - 2]})")
            else:
                step_scores.append(BROKEN_ANSWER_SCORE)
                pretty.append(f"{segments[k]} (Broken)")
        else:
            pretty.append(segments[k])
    return step_scores, "\n\n".join(pretty)


def aggregate_step_scores(step_scores: Sequence[float], how: str) -> float:
    """One number per sample from its step scores (logits): sigmoid first, then ``min`` /
    ``prod`` / ``mean`` over the steps or the ``last`` step. An empty list scores 0."""
    if not step_scores:
        return 0.0
    probs = [1.0 / (1.0 + math.exp(-s)) for s in step_scores]
    if how == "min":
        return min(probs)
    if how == "prod":
        return math.prod(probs)
    if how == "mean":
        return sum(probs) / len(probs)
    if how == "last":
        return probs[-1]
    raise ValueError(f"unknown aggregation {how!r}")


def select_best_of_n(records: Sequence[Dict], key: str = "aggregate_reward") -> List[Dict]:
    """The highest-scoring sample of every ``idx`` (ties: lowest ``sample_idx``)."""
    best: Dict = {}
    for r in records:
        cur = best.get(r["idx"])
        if cur is None or (r[key], -r["sample_idx"]) > (cur[key], -cur["sample_idx"]):
            best[r["idx"]] = r
    return [best[k] for k in sorted(best)]


def main(prompt_file: Path, output_file: Path, batch_size: int = 4,
         checkpoint_path: Path = Path("checkpoints/meta-Transformer/Transformer-2-7b-chat-hf/model.pth"),
         compile: bool = True, finetune_checkpoint_path: Optional[Path] = None,
         resume_generation: bool = False, tensor_parallel_size: Optional[int] = None,
         on_the_fly_8bit_quantization: bool = False, process_reward_with_answer: bool = False,
         aggregate: Optional[str] = None, best_of_n_file: Optional[Path] = None) -> None:
    del compile  # accepted for compatibility: the fused kernels are always used on CUDA
    checkpoint_path = Path(checkpoint_path)
    assert checkpoint_path.is_file(), checkpoint_path
    tokenizer_path = checkpoint_path.parent / "tokenizer.model"
    assert tokenizer_path.is_file(), tokenizer_path

    rank = maybe_init_dist()
    use_tp = rank is not None
    if use_tp:
        initialize_model_parallel(tensor_parallel_size or torch.distributed.get_world_size())
    say = print if (rank in (None, 0)) else (lambda *a, **k: None)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    precision = torch.bfloat16 if device == "cuda" else torch.float32

    say("Loading model ...")
    t0 = time.time()
    model = _load_reward_model(checkpoint_path, device, precision, use_tp)
    if finetune_checkpoint_path is not None:
        path, _, _ = get_latest_checkpoint_path(finetune_checkpoint_path)
        say("Loading finetune model ...")
        if path is not None:
            load_inference_checkpoint(path, model)
        model = model.eval()
    if on_the_fly_8bit_quantization:
        say("Quantizing model ...")
        from easy_to_hard_b200.models.quantize import WeightOnlyInt8QuantHandler
        model = WeightOnlyInt8QuantHandler(model).convert_for_runtime_on_the_fly()
        model = model.to(device=device).eval()
    if device == "cuda":
        torch.cuda.synchronize()
    say(f"Time to load model: {time.time() - t0:.02f} seconds")

    tokenizer = AcceleraTokenizer(tokenizer_path)
    torch.manual_seed(1234)
    model_size = sum(p.numel() * p.element_size()
                     for p in itertools.chain(model.parameters(), model.buffers()))
    newline_ids = tokenizer.encode("\n\n", bos=False, eos=False)
    newline_id = newline_ids[-1] if newline_ids else 13

    with open(prompt_file, "r") as f:
        prompts = [json.loads(line) for line in f if line.strip()]
    assert prompts and "idx" in prompts[0] and "sample_idx" in prompts[0]
    say("Tokenizing prompts ...")
    full = [p["prompt"] + p["output"] for p in prompts]
    for p, toks in zip(prompts, tokenizer.batch_encode(full, bos=[False] * len(full),
                                                       eos=[False] * len(full))):
        p["full_seq"] = p["prompt"] + p["output"]
        p["full_seq_len"] = len(toks)
    prompts.sort(key=lambda x: x["full_seq_len"])

    if rank in (None, 0):
        Path(output_file).parent.mkdir(exist_ok=True, parents=True)
    if use_tp:
        torch.distributed.barrier()
    seen = set()
    if resume_generation and os.path.isfile(output_file):
        with open(output_file, "r") as f:
            for line in f:
                s = json.loads(line)
                seen.add((s["idx"], s["sample_idx"]))
    todo = []
    for p in prompts:                                 # also drops duplicated (idx, sample) pairs
        key = (p["idx"], p["sample_idx"])
        if key not in seen:
            todo.append(p)
            seen.add(key)
    prompts = todo
    if not prompts:
        say("Nothing left to score.")
    while prompts and len(prompts) % batch_size != 0:
        prompts.insert(0, prompts[0])

    dp_rank, tp_rank, dp_size = (get_data_parallel_rank(), get_model_parallel_rank(),
                                 get_data_parallel_world_size())
    writer = open(output_file, "a") if tp_rank == 0 else None
    gc.collect()
    max_seq_len = (prompts[-1]["full_seq_len"] + 2) if prompts else 0
    say("Max sequence length:", max_seq_len)
    vocab = model.backbone_model.config.vocab_size
    batch_idx = 0
    for start in range(0, len(prompts), batch_size):
        batch_idx += 1
        if batch_idx % dp_size != dp_rank:
            continue
        batch = prompts[start:start + batch_size]
        encoded = batch_encode_tokens(tokenizer, [b["full_seq"] for b in batch], bos=True,
                                      eos=True, device=device, padding_side="right")
        encoded[encoded >= vocab] = vocab - 1
        t0 = time.perf_counter()
        y = model_score(model, encoded, max_seq_len=max_seq_len)
        assert y.shape == encoded.shape
        inputs, outputs = encoded.tolist(), y.float().tolist()
        t = time.perf_counter() - t0
        results = [post_process_newline_scores(inputs[i], outputs[i], batch[i]["prompt"],
                                               batch[i]["output"], process_reward_with_answer,
                                               newline_id=newline_id, eos_id=tokenizer.eos_id,
                                               pad_id=(tokenizer.unk_id if tokenizer.pad_id < 0
                                                       else tokenizer.pad_id))
                   for i in range(len(batch))]
        toks_s = encoded.numel() / max(t, 1e-9)
        say(results[0][1] + "\n")
        say(f"Prompt length: {encoded.size(1)}")
        say(f"Time for inference {start + batch_size} / {len(prompts)}: {t:.02f} sec total, "
            f"{toks_s:.02f} tokens/sec")
        say(f"Bandwidth achieved: {model_size * toks_s / 1e9:.02f} GB/s")
        if writer is not None:
            fcntl.flock(writer, fcntl.LOCK_EX)
            try:
                for b, (step_scores, _) in zip(batch, results):
                    rec = {"idx": b["idx"], "sample_idx": b["sample_idx"], "prompt": b["prompt"],
                           "output": b["output"], "reward": step_scores}
                    if aggregate:
                        rec["aggregate_reward"] = aggregate_step_scores(step_scores, aggregate)
                    writer.write(json.dumps(rec) + "\n")
                writer.flush()
            finally:
                fcntl.flock(writer, fcntl.LOCK_UN)
    if writer is not None:
        writer.close()
    if use_tp:
        torch.distributed.barrier()
    if best_of_n_file is not None and aggregate and rank in (None, 0):
        with open(output_file, "r") as f:
            records = {(r["idx"], r["sample_idx"]): r for r in map(json.loads, f)}
        with open(best_of_n_file, "w") as f:
            for r in select_best_of_n(list(records.values())):
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Score samples with a process reward model.")
    ap.add_argument("--prompt_file", type=Path, required=True,
                    help="JSON lines with idx, sample_idx, prompt, output.")
    ap.add_argument("--output_file", type=Path, required=True)
    ap.add_argument("--batch_size", type=int, default=4)
    ap.add_argument("--checkpoint_path", type=Path,
                    default=Path("checkpoints/meta-Transformer/Transformer-2-7b-chat-hf/model.pth"))
    ap.add_argument("--compile", action="store_true")
    ap.add_argument("--finetune_checkpoint_path", type=Path, default=None)
    ap.add_argument("--resume_generation", action="store_true")
    ap.add_argument("--tensor_parallel_size", type=int, default=None)
    ap.add_argument("--on_the_fly_8bit_quantization", action="store_true")
    ap.add_argument("--process_reward_with_answer", action="store_true")
    ap.add_argument("--aggregate", choices=["min", "prod", "mean", "last"], default=None,
                    help="also write one aggregate score per sample")
    ap.add_argument("--best_of_n_file", type=Path, default=None,
                    help="with --aggregate: write the best sample of every idx here")
    a = ap.parse_args()
    main(a.prompt_file, a.output_file, a.batch_size, a.checkpoint_path, a.compile,
         a.finetune_checkpoint_path, a.resume_generation, a.tensor_parallel_size,
         a.on_the_fly_8bit_quantization, a.process_reward_with_answer, a.aggregate,
         a.best_of_n_file)
