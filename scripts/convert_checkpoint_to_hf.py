"""Tensor-parallel training checkpoint -> Hugging Face LLaMA weights
(scripts/convert_checkpoint_to_hf.py of the reference).

    python scripts/convert_checkpoint_to_hf.py --tp_ckpt_name ckpts/sft \
        --pretrain_name EleutherAI/llemma_7b --tokenizer_name EleutherAI/llemma_7b \
        --save_name_hf exported/llemma_7b_sft

Reads ``<tp_ckpt_name>/last_checkpoint`` (a file name with a ``_rank_*`` wildcard), merges the
per-rank files back to the unsharded layout (``utils.checkpoint_utils.merge_tp_checkpoint``),
splits the fused ``wqkv`` into q / k / v, undoes the interleaved-pair row permutation of q and
k, and writes the tensors over the pretrained HF model's state dict. Tensors that were not
trained (embeddings, norms, possibly the LM head) keep their pretrained values.
"""
from __future__ import annotations

import argparse
import glob
import os
import re
import sys
from typing import Dict, Optional, Tuple

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from easy_to_hard_b200.utils.checkpoint_utils import merge_tp_checkpoint  # noqa: E402
from scripts.convert_hf_checkpoint import unpermute_rotary  # noqa: E402

_HEADS_BY_DIM = {4096: (32, 32), 5120: (40, 40), 6656: (52, 52), 8192: (64, 8)}
_NAMES = {"attention.wo": "self_attn.o_proj", "feed_forward.w1": "mlp.gate_proj",
          "feed_forward.w3": "mlp.up_proj", "feed_forward.w2": "mlp.down_proj",
          "attention_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm"}


def gptfast_to_hf(state: Dict[str, torch.Tensor], heads: Optional[Tuple[int, int]] = None
                  ) -> Dict[str, torch.Tensor]:
    """Unsharded gpt-fast tensors -> HF parameter names and row order."""
    out: Dict[str, torch.Tensor] = {}
    for key, w in state.items():
        m = re.search(r"layers\.(\d+)\.(.+)\.weight$", key)
        if m is None:
            top = {"output.weight": "lm_head.weight", "norm.weight": "model.norm.weight",
                   "tok_embeddings.weight": "model.embed_tokens.weight"}
            if key not in top:
                raise ValueError(f"Invalid key: {key}")
            out[top[key]] = w
            continue
        layer, name = m.group(1), m.group(2)
        if name == "attention.wqkv":
            n_head, n_kv = heads or _HEADS_BY_DIM[w.shape[1]]
            head_dim = w.shape[0] // (n_head + 2 * n_kv)
            q, k, v = w.split([n_head * head_dim, n_kv * head_dim, n_kv * head_dim], dim=0)
            base = f"model.layers.{layer}.self_attn."
            out[base + "q_proj.weight"] = unpermute_rotary(q, n_head, head_dim)
            out[base + "k_proj.weight"] = unpermute_rotary(k, n_kv, head_dim)
            out[base + "v_proj.weight"] = v
        else:
            out[f"model.layers.{layer}.{_NAMES[name]}.weight"] = w
    return out


def load_and_merge_models(tp_ckpt_name: str, pretrain_name: str, tokenizer_name: str,
                          save_name_hf: Optional[str], push_to_hf_hub_name: Optional[str] = None):
    assert save_name_hf or push_to_hf_hub_name, "Please provide a name to save the HF model"
    with open(os.path.join(tp_ckpt_name, "last_checkpoint")) as f:
        pattern = os.path.join(tp_ckpt_name, f.readline().strip().split("/")[-1])
    files = sorted(glob.glob(pattern))
    print("Loading checkpoint files:", files)
    shards = [torch.load(f, mmap=True, weights_only=False)["model"] for f in files]
    from transformers import AutoConfig, AutoModelForCausalLM, AutoTokenizer
    model = AutoModelForCausalLM.from_pretrained(pretrain_name, torch_dtype=torch.bfloat16)
    hf_state = model.cpu().state_dict()
    cfg = model.config
    heads = (cfg.num_attention_heads, getattr(cfg, "num_key_value_heads",
                                              cfg.num_attention_heads))
    merged = merge_tp_checkpoint(shards, heads=heads) if len(shards) > 1 else shards[0]
    converted = gptfast_to_hf({k: v.cpu() for k, v in merged.items()}, heads)
    for name, w in converted.items():
        ref = hf_state[name]
        if name == "lm_head.weight" and w.shape[0] < ref.shape[0]:   # vocabulary padded in HF
            full = ref.clone()
            full[: w.shape[0]] = w.to(ref.dtype)
            w = full
        hf_state[name] = w.to(ref.dtype)
    print("Unreplaced keys:", sorted(set(hf_state) - set(converted)))
    model.load_state_dict(hf_state, strict=False)
    if save_name_hf is not None:
        model.save_pretrained(save_name_hf)
        AutoTokenizer.from_pretrained(tokenizer_name).save_pretrained(save_name_hf)
        AutoConfig.from_pretrained(pretrain_name).save_pretrained(save_name_hf)
    else:
        model.push_to_hub(push_to_hf_hub_name, private=True, safe_serialization=False)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Export a TP checkpoint to the HF format.")
    ap.add_argument("--tp_ckpt_name", type=str, required=True)
    ap.add_argument("--tokenizer_name", type=str, required=True)
    ap.add_argument("--pretrain_name", type=str, required=True)
    ap.add_argument("--save_name_hf", type=str, default=None)
    ap.add_argument("--push_to_hf_hub_name", type=str, default=None)
    a = ap.parse_args()
    load_and_merge_models(a.tp_ckpt_name, a.pretrain_name, a.tokenizer_name, a.save_name_hf,
                          a.push_to_hf_hub_name)
