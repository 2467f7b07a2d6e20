"""Decode-step time of ONE tensor-parallel rank's kernels, measured on one GPU.

    python bench/decode_shape_bench.py --tp 8 [--batch 64] [--ctx 512] [--steps 64]

Builds the Llemma-7B architecture with random weights, keeps rank 0's shard of a TP = ``--tp``
split (``models.tp.shard_linear`` with an explicit world and rank, no process group) and replays
the decode engine's CUDA graph with the reduce strategy "local": every kernel of the decode step
runs with the per-rank shapes, nothing crosses NVLink, and the row-parallel GEMMs simply leave
their partial sums in place (the tokens are meaningless, the timing is not). The figure is what
the kernels alone cost per token step when the work per rank shrinks, i.e. the part of the
strong-scaling loss that no collective can be blamed for.

Prints one JSON line: microseconds per decode step and per layer, launches per step, and the
bytes the step must stream (weights + live KV range) against the measured copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=512, help="cached positions when timing starts")
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--hbm_gbs", type=float, default=6453.1)
    a = ap.parse_args()
    from easy_to_hard_b200.models.model import ModelArgs, Transformer
    from easy_to_hard_b200.models import tp as tpm
    from easy_to_hard_b200.models.engine import DecodeEngine
    from easy_to_hard_b200.ops import _lib

    torch.cuda.set_device(0)
    cfg = ModelArgs.from_name("llemma-7b-32016")
    cfg.n_layer = a.layers
    with torch.device("cuda"):
        model = Transformer(cfg, freeze_tok_embeddings=True, freeze_output=True,
                            freeze_norm=True).to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(1234)
    for _, t in list(model.named_parameters()) + list(model.named_buffers()):
        if t.dim() == 2:
            t.data.normal_(0.0, 0.02, generator=g)
    n = a.tp
    if n > 1:
        for blk in model.layers:
            att, ffn = blk.attention, blk.feed_forward
            kv = att.n_local_heads * att.head_dim
            tpm.shard_linear(att.wqkv, "colwise", [att.n_head * att.head_dim, kv, kv],
                             world=n, rank=0)
            tpm.shard_linear(att.wo, "rowwise", world=n, rank=0)
            att.n_head //= n
            att.n_local_heads //= n
            att.dim //= n
            for name, style in (("w1", "colwise"), ("w3", "colwise"), ("w2", "rowwise")):
                tpm.shard_linear(getattr(ffn, name), style, world=n, rank=0)
        torch.cuda.empty_cache()
    model.eval()
    B = a.batch
    eng = DecodeEngine(model, B, a.ctx + a.steps * 3 + 16, reduce="local", use_pdl=bool(a.pdl))
    prompt = torch.randint(0, cfg.vocab_size, (B, a.ctx), device="cuda", dtype=torch.int32)
    eng.prefill(prompt, None, 0.7, 50, 0, -1)
    key = (B, 0.7, 50, -1)
    graph, launches = eng._graph_for(key)
    for _ in range(a.steps):          # warm-up, also moves the context forward
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.steps
    ctx_mid = a.ctx + a.steps + a.steps // 2
    w_bytes = sum(t.numel() * t.element_size() for blk in model.layers
                  for t in blk.parameters()) + model.output.weight.numel() * 2
    kv_bytes = 2 * a.layers * B * eng.n_kv * ctx_mid * eng.D * 2
    floor_us = (w_bytes + kv_bytes) / (a.hbm_gbs * 1e9) * 1e6
    print(json.dumps({
        "tp_shapes": n, "batch": B, "context": ctx_mid, "layers": a.layers,
        "us_per_step": round(us, 1), "us_per_layer": round(us / a.layers, 2),
        "launches_per_step": launches, "weight_mb": round(w_bytes / 1e6, 1),
        "kv_mb": round(kv_bytes / 1e6, 1), "hbm_floor_us": round(floor_us, 1),
        "fraction_of_measured_copy_bw": round(floor_us / us, 3),
        "status": _lib.read_status()}), flush=True)
    eng._graphs.clear()


if __name__ == "__main__":
    main()
