"""Where the time of a skinny (decode) GEMM goes, from time stamps inside the kernel.

    python -m easy_to_hard_b200.ops.build --phase-clock      # builds libe2h_b200_phase.so
    python bench/gemm_phase_bench.py [--cold 1]

Runs the 7B decode shapes (64 tokens) at the per-rank sizes of TP 1 and TP 8 through the build of
``gemm_umma.cu`` that stamps the nanosecond global timer at the phases of its pipeline (set-up,
first stage landed, last MMA issued, accumulator ready, split-K exchange, values staged in shared
memory, tile written), and prints, per phase, the minimum / median / maximum over the CTAs in
microseconds since the first CTA started. ``--cold 1`` flushes L2 before the measured launch.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from easy_to_hard_b200.ops import _lib, build, gemm  # noqa: E402
from easy_to_hard_b200.ops._lib import GemmParams  # noqa: E402

PHASES = ["entry", "set-up done", "producer past wait", "loads issued", "first stage landed",
          "MMAs issued", "accumulator ready", "exchange done", "values staged", "tile written",
          "tmem freed"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cold", type=int, default=0)
    a = ap.parse_args()
    path = build.OUT_DIR / "libe2h_b200_phase.so"
    if not path.exists():
        path = build.build_phase_clock()
    torch.cuda.set_device(0)
    phase = C.CDLL(str(path))
    phase.e2h_gemm_umma.argtypes = [C.POINTER(GemmParams), C.c_void_p]
    phase.e2h_gemm_umma.restype = C.c_int
    stamps = torch.zeros(4096 * 16, dtype=torch.int64, device="cuda")
    real = _lib.lib()

    class WithStamps:
        def __getattr__(self, name):
            return getattr(real, name)

        def e2h_gemm_umma(self, pref, stream):
            p = pref._obj
            p.phase_clock = stamps.data_ptr()
            return phase.e2h_gemm_umma(C.byref(p), stream)

    _lib.lib = lambda: WithStamps()
    flush = torch.empty(64 << 20, dtype=torch.float32, device="cuda")

    def mk(*s):
        return (torch.randn(*s, device="cuda") * 0.02).to(torch.bfloat16)

    def run(tag, F, K, dual=False, residual=False):
        x, w = mk(64, K), mk(F, K)
        w3 = mk(F, K) if dual else None
        res = mk(64, F) if residual else None
        out = torch.empty(64, F, dtype=torch.bfloat16, device="cuda")

        def call():
            if dual:
                gemm.linear_swiglu(x, w, w3, out=out)
            elif residual:
                gemm.linear_residual(x, w, res, out=out)
            else:
                gemm.linear(x, w, out=out)
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        if a.cold:
            flush.fill_(1.0)
        stamps.zero_()
        torch.cuda.synchronize()
        call()
        torch.cuda.synchronize()
        t = stamps.view(-1, 16).cpu()
        t = t[t[:, 0] > 0]
        base = int(t[:, 0].min())
        print(f"== {tag}: F={F} K={K} {'dual ' if dual else ''}{'residual ' if residual else ''}"
              f"CTAs={len(t)} {'cold' if a.cold else 'warm'} L2")
        for k, name in enumerate(PHASES):
            col = t[:, k]
            col = (col[col > 0] - base).float() / 1e3
            if len(col):
                print(f"   {name:20s} min {float(col.min()):7.2f}  med {float(col.median()):7.2f}"
                      f"  max {float(col.max()):7.2f}")

    run("wqkv TP1", 12288, 4096)
    run("w1/w3 SwiGLU TP1", 11008, 4096, dual=True)
    run("w2 + residual TP1", 4096, 11008, residual=True)
    run("wo + residual TP1", 4096, 4096, residual=True)
    run("wqkv TP8", 1536, 4096)
    run("wo TP8", 4096, 512)


if __name__ == "__main__":
    main()
