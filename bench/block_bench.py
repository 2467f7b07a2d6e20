"""Event-timed breakdown of one transformer block at the SFT micro-batch shape of the 7B model.

    python bench/block_bench.py [--batch 8] [--seq 768]

Prints the forward, the backward from kept intermediates and the backward that recomputes the
block, then every kernel of the block on its own (CUDA events, five back-to-back launches after
two warm-ups; weights and activations stay hot in L2 where they fit, so the figures are the ones
the training step sees, not cold-cache ones).
"""
import argparse

import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from easy_to_hard_b200.ops import flash, functional as Fn, gemm, reference  # noqa: E402
from easy_to_hard_b200.models import fused_block as fb  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=768)
    a = ap.parse_args()
    B, S, H, D, dim, ffn = a.batch, a.seq, 32, 128, 4096, 11008
    T = B * S
    dev = 'cuda'
    torch.manual_seed(0)
    w = dict(wqkv=torch.randn(3*dim, dim, device=dev).bfloat16()*0.02, wo=torch.randn(dim, dim, device=dev).bfloat16()*0.02,
             w1=torch.randn(ffn, dim, device=dev).bfloat16()*0.02, w3=torch.randn(ffn, dim, device=dev).bfloat16()*0.02,
             w2=torch.randn(dim, ffn, device=dev).bfloat16()*0.02,
             attention_norm=torch.ones(dim, device=dev).bfloat16(), ffn_norm=torch.ones(dim, device=dev).bfloat16())
    freqs = reference.precompute_freqs_cis(S, D, 1e6, dtype=torch.bfloat16).to(dev)
    pos = torch.arange(S, device=dev, dtype=torch.int32).repeat(B)
    x = torch.randn(T, dim, device=dev).bfloat16()
    dy = torch.randn(T, dim, device=dev).bfloat16()
    shape = fb.BlockShape(B, S, H, H, D, 1e-5)
    grads = {k: torch.empty_like(v) for k, v in w.items() if k.startswith('w')}
    def t(fn, n=5):
        for _ in range(2): fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n): fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n
    print("block fwd  ms", t(lambda: fb.block_forward(x, w, freqs, pos, shape)))
    print("block bwd (recompute) ms", t(lambda: fb.block_backward(dy, x, w, grads, freqs, pos, shape)))
    _, a = fb.block_forward(x, w, freqs, pos, shape, keep=True)
    sv = {k: v for k, v in a.items() if k != "act"}
    print("block bwd (kept) ms", t(lambda: fb.block_backward(dy, x, w, grads, freqs, pos, shape, saved=sv)))
    xn = a['xn1f']
    print("rmsnorm", t(lambda: Fn.rmsnorm(x, w['attention_norm'], 1e-5)))
    print("wqkv", t(lambda: gemm.linear(xn, w['wqkv'])))
    qkv = a['qkv']
    print("rope", t(lambda: Fn.rope(qkv, freqs, pos, 2*H, D, out=qkv)))
    print("flash fwd", t(lambda: flash.flash_fwd(a['q'], a['k'], a['v'], None, return_lse=True)))
    o2 = a['o'].view(T, H*D)
    print("wo+res", t(lambda: gemm.linear_residual(o2, w['wo'], x)))
    print("w13 dual", t(lambda: gemm.linear_dual(a['xn2f'], w['w1'], w['w3'])))
    print("swiglu", t(lambda: Fn.swiglu(a['g'], a['u'])))
    print("w2+res", t(lambda: gemm.linear_residual(a['act'], w['w2'], a['h'])))
    print("dgrad w2", t(lambda: gemm.linear_dgrad(dy, w['w2'])))
    print("wgrad w2", t(lambda: gemm.linear_wgrad(dy, a['act'], out=grads['w2'])))
    dact = torch.randn_like(a['act'])
    print("swiglu bwd", t(lambda: Fn.swiglu_bwd(a['g'], a['u'], dact)))
    dg = torch.randn_like(a['g'])
    print("dgrad w1", t(lambda: gemm.linear_dgrad(dg, w['w1'])))
    print("wgrad w1", t(lambda: gemm.linear_wgrad(dg, a['xn2f'], out=grads['w1'])))
    print("rmsnorm bwd", t(lambda: Fn.rmsnorm_bwd(a['h'], dy, w['ffn_norm'], 1e-5, dres=dy)))
    print("dgrad wo", t(lambda: gemm.linear_dgrad(dy, w['wo'])))
    print("wgrad wo", t(lambda: gemm.linear_wgrad(dy, o2, out=grads['wo'])))
    do = torch.randn_like(a['o'])
    dqkv = torch.empty_like(qkv)
    print("flash bwd", t(lambda: flash.flash_bwd(a['q'], a['k'], a['v'], a['o'], do, a['lse'],
          dq=dqkv[:, :H*D].view(B,S,H,D), dk=dqkv[:, H*D:2*H*D].view(B,S,H,D), dv=dqkv[:, 2*H*D:].view(B,S,H,D))))
    print("dgrad wqkv", t(lambda: gemm.linear_dgrad(dqkv, w['wqkv'])))
    print("wgrad wqkv", t(lambda: gemm.linear_wgrad(dqkv, xn, out=grads['wqkv'])))


if __name__ == "__main__":
    main()
