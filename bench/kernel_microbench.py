"""Event-timed micro-benchmarks of the sm_100a kernels on the shapes of the 7B model.

    python bench/kernel_microbench.py --case all
    python bench/kernel_microbench.py --case gemm_wgrad --tokens 6144 --iters 20

Each case prints one JSON line: duration (CUDA events on the launching stream, after warm-up,
L2 flushed between iterations by writing a 256 MB buffer), algorithmic FLOPs or bytes per
launch, the achieved rate and its fraction of the measured peaks (``MEASURED_PEAKS.json`` at
the repository root when present: cuBLAS bf16 burst TFLOP/s and copy GB/s).
The same command line is what the ``profiles/`` summaries were captured with under ``ncu``.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import sys

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, _ROOT)

from easy_to_hard_b200.ops import flash, functional as Fn, gemm, reference  # noqa: E402

DIM, FFN, HEADS, HEAD_DIM, VOCAB = 4096, 11008, 32, 128, 32016


def _peaks():
    try:
        with open(os.path.join(_ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 1590.0, 6650.0, "fallback"


def _time(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(iters):
        flush.zero_()                       # evict the 126 MB L2
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _bf(*shape):
    return (torch.randn(*shape, device="cuda") * 0.02).bfloat16()


def cases(T: int, B: int, S: int, ctx: int):
    """name -> (callable, flops, bytes). ``T`` tokens for the large GEMMs, ``B`` sequences of
    ``S`` tokens for attention, ``B`` decode rows against ``ctx`` cached positions."""
    x, xf = _bf(T, DIM), _bf(T, FFN)
    wqkv, wo, w1, w3, w2 = _bf(3 * DIM, DIM), _bf(DIM, DIM), _bf(FFN, DIM), _bf(FFN, DIM), \
        _bf(DIM, FFN)
    dy = _bf(T, DIM)
    gw2 = torch.empty(DIM, FFN, device="cuda", dtype=torch.bfloat16)
    out = {}
    out["gemm_fwd_wqkv"] = (lambda: gemm.linear(x, wqkv), 2.0 * T * DIM * 3 * DIM, 0)
    out["gemm_fwd_w13_dual"] = (lambda: gemm.linear_dual(x, w1, w3), 4.0 * T * DIM * FFN, 0)
    out["gemm_fwd_w2_residual"] = (lambda: gemm.linear_residual(xf, w2, x), 2.0 * T * DIM * FFN, 0)
    out["gemm_dgrad_w2"] = (lambda: gemm.linear_dgrad(dy, w2), 2.0 * T * DIM * FFN, 0)
    out["gemm_wgrad_w2"] = (lambda: gemm.linear_wgrad(dy, xf, out=gw2), 2.0 * T * DIM * FFN, 0)
    q, k, v = (_bf(B, S, HEADS, HEAD_DIM) for _ in range(3))
    o, lse = flash.flash_fwd(q, k, v, None, return_lse=True)
    do = torch.randn_like(o)
    att = 4.0 * B * HEADS * S * S * HEAD_DIM / 2          # causal: half of the score matrix
    out["flash_fwd"] = (lambda: flash.flash_fwd(q, k, v, None, return_lse=True), att, 0)
    out["flash_bwd"] = (lambda: flash.flash_bwd(q, k, v, o, do, lse), 2.5 * att, 0)
    # the bar on the same box: PyTorch's scaled_dot_product_attention with the flash backend,
    # which is what the reference model calls (models/model.py:338-342 of the reference)
    from torch.nn.attention import SDPBackend, sdpa_kernel
    qs, ks, vs = (t.transpose(1, 2).detach().clone().requires_grad_(True) for t in (q, k, v))
    dos = do.transpose(1, 2).contiguous()

    def sdpa_fwd():
        with sdpa_kernel(SDPBackend.FLASH_ATTENTION):
            return torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True)

    def sdpa_fwd_bwd():
        sdpa_fwd().backward(dos)
        qs.grad = ks.grad = vs.grad = None

    out["sdpa_flash_fwd"] = (lambda: sdpa_fwd(), att, 0)
    out["sdpa_flash_fwd_bwd"] = (sdpa_fwd_bwd, 3.5 * att, 0)
    # decode: 64 rows
    xd = _bf(64, DIM)
    hd = _bf(64, DIM)
    out["decode_gemm_wqkv"] = (lambda: gemm.linear(xd, wqkv), 0, 3 * DIM * DIM * 2)
    out["decode_gemm_w13_swiglu"] = (lambda: gemm.linear_swiglu(xd, w1, w3), 0, 2 * FFN * DIM * 2)
    xa = _bf(64, FFN)
    out["decode_gemm_w2_residual"] = (lambda: gemm.linear_residual(xa, w2, hd), 0, FFN * DIM * 2)
    w8 = torch.randint(-128, 128, (3 * DIM, DIM), device="cuda", dtype=torch.int8)
    s8 = torch.rand(3 * DIM, device="cuda") * 0.01
    w8b = torch.randint(-128, 128, (DIM, FFN // 64 * 64), device="cuda", dtype=torch.int8)
    s8b = torch.rand(DIM, device="cuda") * 0.01
    xa8 = _bf(64, FFN // 64 * 64)
    out["decode_gemm_w8_wqkv"] = (lambda: gemm.linear(xd, w8, scale=s8), 0, 3 * DIM * DIM)
    out["decode_gemm_w8_w2_residual"] = (lambda: gemm.linear_residual(xa8, w8b, hd, scale=s8b),
                                         0, (FFN // 64 * 64) * DIM)
    codes = torch.randint(0, 16, (3 * DIM, DIM), device="cuda", dtype=torch.int32)
    sz = (torch.rand(DIM // 128, 3 * DIM, 2, device="cuda") * 0.01).bfloat16()
    w4 = gemm.Int4Weight.from_int(codes, sz, 128)
    out["decode_gemm_w4_wqkv"] = (lambda: gemm.linear(xd, w4), 0, 3 * DIM * DIM // 2)
    kc, vc = _bf(64, HEADS, ctx, HEAD_DIM), _bf(64, HEADS, ctx, HEAD_DIM)
    qd = _bf(64, HEADS * HEAD_DIM)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    lp = torch.zeros(64, dtype=torch.int32, device="cuda")
    out["attn_decode"] = (lambda: Fn.attn_decode(qd, kc, vc, pos, lp, HEADS),
                          0, 2 * 64 * HEADS * ctx * HEAD_DIM * 2)
    nw = torch.ones(DIM, device="cuda", dtype=torch.bfloat16)
    out["rmsnorm"] = (lambda: Fn.rmsnorm(x, nw, 1e-5), 0, 2 * T * DIM * 2)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--tokens", type=int, default=6144)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=768)
    ap.add_argument("--ctx", type=int, default=768)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    torch.manual_seed(0)
    tf_peak, gb_peak, src = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    table = cases(a.tokens, a.batch, a.seq, a.ctx)
    names = list(table) if a.case == "all" else [a.case]
    for name in names:
        fn, flops, nbytes = table[name]
        ms = _time(fn, a.iters, flush)
        rec = {"case": name, "ms": round(ms, 4)}
        if flops:
            tf = flops / (ms * 1e-3) / 1e12
            rec.update(tflops=round(tf, 1), frac_of_peak=round(tf / tf_peak, 3),
                       peak=f"{tf_peak} TFLOP/s ({src})")
        if nbytes:
            gbs = nbytes / (ms * 1e-3) / 1e9
            rec.update(gbs=round(gbs, 1), frac_of_peak=round(gbs / gb_peak, 3),
                       peak=f"{gb_peak} GB/s ({src})")
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
