"""Hugging Face LLaMA checkpoint -> ``model.pth`` in the gpt-fast layout that every entry point
loads (scripts/convert_hf_checkpoint.py of the reference).

    python scripts/convert_hf_checkpoint.py --checkpoint_dir checkpoints/EleutherAI/llemma_7b \
        --target_precision bf16

Key mapping: ``model.embed_tokens`` -> ``tok_embeddings``, ``self_attn.{q,k,v}_proj`` -> one
fused ``attention.wqkv`` (rows [q; k; v]), ``o_proj`` -> ``wo``, ``mlp.{gate,up,down}_proj`` ->
``feed_forward.{w1,w3,w2}``, the two layer norms, ``model.norm``, ``lm_head`` -> ``output``.
HF stores q/k rows with the two rotary halves of a head one after the other; the models here
rotate interleaved pairs, so q and k rows are permuted per head ([half, pair] -> [pair, half]).
Vocabularies padded to 32016 rows are cut back to 32000, as the reference does.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from pathlib import Path
from typing import Dict, Optional

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from easy_to_hard_b200.models.model import ModelArgs  # noqa: E402

WEIGHT_MAP = {
    "model.embed_tokens.weight": "tok_embeddings.weight",
    "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.wq.weight",
    "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.wk.weight",
    "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.wv.weight",
    "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
    "model.layers.{}.self_attn.rotary_emb.inv_freq": None,
    "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
    "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
    "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
    "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
    "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
    "model.norm.weight": "norm.weight",
    "lm_head.weight": "output.weight",
}
_DTYPES = {"fp32": None, "fp16": torch.float16, "bf16": torch.bfloat16}


def permute_rotary(w: torch.Tensor, n_head: int, head_dim: int) -> torch.Tensor:
    """[n_head * head_dim, dim] rows from HF order (first half | second half per head) to
    interleaved pairs."""
    dim = w.shape[1]
    return (w.view(n_head, 2, head_dim // 2, dim).transpose(1, 2)
            .reshape(head_dim * n_head, dim))


def unpermute_rotary(w: torch.Tensor, n_head: int, head_dim: int) -> torch.Tensor:
    """Inverse of ``permute_rotary``."""
    dim = w.shape[1]
    return (w.view(n_head, head_dim // 2, 2, dim).transpose(1, 2)
            .reshape(head_dim * n_head, dim))


def hf_to_gptfast(hf_state: Dict[str, torch.Tensor], config: ModelArgs,
                  trim_vocab_to: Optional[int] = 32000) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for key, value in hf_state.items():
        if "layers" in key:
            layer = re.search(r"\d+", key).group(0)
            new_key = WEIGHT_MAP[re.sub(r"(\d+)", "{}", key, count=1)]
            if new_key is None:
                continue
            new_key = new_key.format(layer)
        else:
            new_key = WEIGHT_MAP[key]
            if trim_vocab_to is not None and value.dim() == 2 and value.size(0) == 32016:
                value = value[:trim_vocab_to]
        out[new_key] = value
    for key in [k for k in out if k.endswith("attention.wq.weight")]:
        kk, kv = key.replace("wq", "wk"), key.replace("wq", "wv")
        q = permute_rotary(out.pop(key), config.n_head, config.head_dim)
        k = permute_rotary(out.pop(kk), config.n_local_heads, config.head_dim)
        out[key.replace("wq", "wqkv")] = torch.cat([q, k, out.pop(kv)])
    return out


def _load_shards(checkpoint_dir: Path) -> Dict[str, torch.Tensor]:
    merged: Dict[str, torch.Tensor] = {}
    index = checkpoint_dir / "pytorch_model.bin.index.json"
    st_index = checkpoint_dir / "model.safetensors.index.json"
    if index.is_file():
        files = sorted({checkpoint_dir / f for f in json.load(open(index))["weight_map"].values()})
        for f in files:
            merged.update(torch.load(str(f), map_location="cpu", mmap=True, weights_only=True))
    elif st_index.is_file() or (checkpoint_dir / "model.safetensors").is_file():
        from safetensors.torch import load_file
        files = (sorted({checkpoint_dir / f
                         for f in json.load(open(st_index))["weight_map"].values()})
                 if st_index.is_file() else [checkpoint_dir / "model.safetensors"])
        for f in files:
            merged.update(load_file(str(f)))
    elif (checkpoint_dir / "pytorch_model.bin").is_file():
        merged.update(torch.load(str(checkpoint_dir / "pytorch_model.bin"), map_location="cpu",
                                 mmap=True, weights_only=True))
    else:
        raise FileNotFoundError(f"no HF weight files under {checkpoint_dir}")
    return merged


@torch.inference_mode()
def convert_hf_checkpoint(*, checkpoint_dir: Path, model_name: Optional[str] = None,
                          target_precision: str = "fp32") -> Path:
    checkpoint_dir = Path(checkpoint_dir)
    config = ModelArgs.from_name(model_name or checkpoint_dir.name)
    print(f"Model config {config.__dict__}")
    if target_precision not in _DTYPES:
        raise ValueError(f"Unsupported target_precision {target_precision}")
    state = _load_shards(checkpoint_dir)
    dtype = _DTYPES[target_precision]
    if dtype is not None:
        state = {k: v.to(dtype) for k, v in state.items()}
    out = hf_to_gptfast(state, config)
    target = checkpoint_dir / "model.pth"
    print(f"Saving checkpoint to {target}")
    torch.save(out, target)
    return target


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Convert HuggingFace checkpoint.")
    ap.add_argument("--checkpoint_dir", type=Path,
                    default=Path("checkpoints/meta-llama/llama-2-7b-chat-hf"))
    ap.add_argument("--model_name", type=str, default=None)
    ap.add_argument("--target_precision", type=str, default="fp32")
    a = ap.parse_args()
    convert_hf_checkpoint(checkpoint_dir=a.checkpoint_dir, model_name=a.model_name,
                          target_precision=a.target_precision)
