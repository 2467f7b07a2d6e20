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
    ap.add_argument("--gemm_phases", default="", help="run the GEMMs of the step through the "
                    "phase-stamp build (python -m easy_to_hard_b200.ops.build --phase-clock) and "
                    "write, per GEMM launch of one replayed step, the phase times (median over "
                    "its CTAs) on one clock; diagnosis only, the printed step time is then that "
                    "of the stamping build")
    ap.add_argument("--timeline", default="", help="write the kernels of one replayed step "
                    "(name, start, duration from the profiler's activity records) to this file; "
                    "for reading the gaps between kernels, never for a reported time")
    a = ap.parse_args()
    from easy_to_hard_b200.models.model import ModelArgs, Transformer
    from easy_to_hard_b200.models import tp as tpm
    from easy_to_hard_b200.models.engine import DecodeEngine
    from easy_to_hard_b200.ops import _lib

    torch.cuda.set_device(0)
    stamp_log = use_phase_build() if a.gemm_phases else None
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
    if stamp_log is not None:
        stamp_log["on"] = True
    graph, launches = eng._graph_for(key)
    if stamp_log is not None:
        stamp_log["on"] = False
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
    if a.timeline:
        write_timeline(graph, a.timeline)
    if stamp_log is not None:
        write_gemm_phases(graph, stamp_log, a.gemm_phases)
    eng._graphs.clear()


PHASES = ["entry", "set-up done", "producer past wait", "loads issued", "first stage landed",
          "MMAs issued", "accumulator ready", "exchange done", "values staged", "tile written",
          "tmem freed"]
STAMP_SLOTS = 256 * 16          # int64 words per launch: 16 per CTA


def use_phase_build():
    """Route e2h_gemm_umma through the stamping build; while ``log["on"]`` every launch gets its
    own region of the stamp buffer (the launches recorded into the decode graph)."""
    import ctypes as C
    from easy_to_hard_b200.ops import _lib, build
    from easy_to_hard_b200.ops._lib import GemmParams
    import os
    path = os.environ.get("E2H_PHASE_LIB")      # another stamping build, for A/B comparisons
    if not path:
        path = build.OUT_DIR / "libe2h_b200_phase.so"
        if not path.exists():
            path = build.build_phase_clock()
    phase = C.CDLL(str(path))
    phase.e2h_gemm_umma.argtypes = [C.POINTER(GemmParams), C.c_void_p]
    phase.e2h_gemm_umma.restype = C.c_int
    log = {"on": False, "launches": [],
           "stamps": torch.zeros(512 * STAMP_SLOTS, dtype=torch.int64, device="cuda")}
    real = _lib.lib()

    class WithStamps:
        def __getattr__(self, name):
            return getattr(real, name)

        def e2h_gemm_umma(self, pref, stream):
            p = pref._obj
            if log["on"] and len(log["launches"]) < 512:
                p.phase_clock = log["stamps"].data_ptr() + len(log["launches"]) * STAMP_SLOTS * 8
                log["launches"].append((p.F, p.K, p.splitk, p.dual))
            return phase.e2h_gemm_umma(C.byref(p), stream)

    shim = WithStamps()
    _lib.lib = lambda: shim
    return log


def write_gemm_phases(graph, log, path):
    log["stamps"].zero_()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    t = log["stamps"].view(-1, STAMP_SLOTS // 16, 16).cpu()
    base = None
    with open(path, "w") as f:
        f.write("# us since the first GEMM CTA of the step started; median over the CTAs of the "
                "launch (entry: min / median / max)\n")
        f.write("# F K splitk dual CTAs | " + " | ".join(PHASES) + "\n")
        for i, (F, K, sk, dual) in enumerate(log["launches"]):
            rows = t[i]
            rows = rows[rows[:, 0] > 0]
            if not len(rows):
                continue
            if base is None:
                base = int(rows[:, 0].min())
            cells = []
            for k in range(len(PHASES)):
                col = rows[:, k]
                col = (col[col > 0] - base).float() / 1e3
                if not len(col):
                    cells.append("-")
                elif k == 0:
                    cells.append(f"{float(col.min()):.1f}/{float(col.median()):.1f}/"
                                 f"{float(col.max()):.1f}")
                else:
                    cells.append(f"{float(col.median()):.1f}")
            last = (rows[:, 1:].max() - base).item() / 1e3
            f.write(f"{F} {K} {sk} {dual} {len(rows)} | " + " | ".join(cells)
                    + f" | end {last:.1f}\n")


def write_timeline(graph, path):
    """Kernel start / duration records of the second of two replays, and their summary: time
    covered by at least one kernel, idle time between kernels, overlap."""
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        graph.replay()
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
    ev = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                 if e.device_type == torch.autograd.DeviceType.CUDA and "memcpy" not in e.name.lower()
                 and "memset" not in e.name.lower()), key=lambda x: x[0])
    ev = ev[len(ev) // 2:]
    t0 = ev[0][0]
    covered, idle, end = 0.0, 0.0, ev[0][0]
    per = {}
    for s_, e_, name in ev:
        if s_ > end:
            idle += s_ - end
            covered += e_ - s_
        else:
            covered += max(0.0, e_ - end)
        end = max(end, e_)
        short = name.split("(")[0].split("<")[0].split("::")[-1]
        d = per.setdefault(short, [0, 0.0])
        d[0] += 1
        d[1] += e_ - s_
    with open(path, "w") as f:
        f.write(json.dumps({"kernels": len(ev), "span_us": round(end - t0, 1),
                            "covered_us": round(covered, 1), "idle_us": round(idle, 1),
                            "by_kernel": {k: [v[0], round(v[1], 1)] for k, v in per.items()}})
                + "\n")
        for s_, e_, name in ev:
            f.write(f"{s_ - t0:10.2f} {e_ - s_:8.2f} {name[:90]}\n")


if __name__ == "__main__":
    main()
