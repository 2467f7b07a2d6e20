"""Cost of the tensor-parallel reduce of the decode step, per strategy, on N GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench/tp_reduce_bench.py [--batch 64] [--iters 32] [--reps 30]

One iteration is the communication-bound part of a 7B decode layer at TP = N:

    act [B, ffn/N]  --w2 (row-parallel GEMM)-->  partial  --reduce + residual + RMSNorm-->  xn
    xn  [B, 4096]   --w1 (column-parallel GEMM)-->  act

``iters`` iterations are captured in one CUDA graph with programmatic dependent launch (as the
decode engine does) and replayed ``reps`` times between CUDA events; the figure is the time
per iteration, max over ranks. Strategies:

    local          no cross-rank traffic at all (GEMM + residual + norm): the floor
    nccl           fp32 partial, dist.all_reduce, norm kernel (the baseline)
    oneshot        tp_reduce.cu, every rank pulls all partials (plain peer loads)
    oneshot_mc     the same with one multimem.ld_reduce per 16 bytes (the switch adds)
    twophase       tp_reduce.cu, reduce-scatter + all-gather by rows (plain peer loads/stores)
    twophase_mc    the same through the NVSwitch (multimem.ld_reduce / multimem.st), if mapped

Prints one JSON line per strategy with the NVLink bytes a rank moves per reduce and the time
the reduce adds over ``local``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--iters", type=int, default=32)
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=11008)
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from easy_to_hard_b200.ops import _lib, functional as Fn, gemm
    from easy_to_hard_b200.parallel import groups
    from easy_to_hard_b200.parallel.symm import TPReduceSync

    groups.initialize_model_parallel(world)
    dev, bf = torch.device("cuda", local), torch.bfloat16
    B, dim, ffn = a.batch, a.dim, a.ffn // world // 64 * 64
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    n_w = 8                                   # distinct weight sets so that they stream from HBM
    w2 = [torch.randn(dim, ffn, device=dev, generator=g).mul_(0.02).to(bf) for _ in range(n_w)]
    w1 = [torch.randn(ffn, dim, device=dev, generator=g).mul_(0.02).to(bf) for _ in range(n_w)]
    nw = torch.ones(dim, device=dev, dtype=bf)
    act = torch.randn(B, ffn, device=dev, generator=g).to(bf)
    h = torch.zeros(B, dim, device=dev, dtype=bf)
    xn_local = torch.zeros(B, dim, device=dev, dtype=bf)
    part32 = torch.zeros(1, B, dim, device=dev, dtype=torch.float32)
    n_points = 2 * a.iters
    tp_group = groups.get_model_parallel_group() if world > 1 else None

    def make(strategy):
        sync = None
        if strategy in ("oneshot", "oneshot_mc", "twophase", "twophase_mc"):
            sync = TPReduceSync(B, dim, n_points + 1, tp_group,
                                oneshot=strategy.startswith("oneshot"),
                                multicast=strategy.endswith("_mc"))
            if strategy.endswith("_mc") and not sync.multicast:
                return None, None
            if strategy == "oneshot_mc" and not sync.check_multimem_consistency(tp_group, 64):
                if rank == 0:
                    print(json.dumps({"strategy": strategy, "ranks_got_different_bits": True}),
                          flush=True)
                return None, None
        xn = sync.xn[:B] if (sync is not None and not sync.oneshot) else xn_local

        def body():
            for i in range(a.iters):
                k = i % n_w
                if strategy == "local":
                    gemm.linear_residual(act, w2[k], h, out=h)
                    Fn.fused_residual_rmsnorm(h, nw, 1e-5, x_out=xn)
                elif strategy == "nccl":
                    gemm.linear(act, w2[k], out=part32[0])
                    dist.all_reduce(part32, group=tp_group)
                    Fn.fused_residual_rmsnorm(h, nw, 1e-5, partials=part32, h_out=h, x_out=xn)
                else:
                    gemm.linear(act, w2[k], out=sync.partial_out(i, B),
                                signal=sync.flag_a_signal(i),
                                ticket=sync.gemm_ticket[i:i + 1])
                    sync.reduce_norm(i, h, h, nw, 1e-5, B, xn_out=xn)
                gemm.linear(xn, w1[k], out=act)
        return body, sync

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    results = {}
    for strategy in ("local", "nccl", "oneshot", "oneshot_mc", "twophase", "twophase_mc"):
        if world == 1 and strategy != "local":
            continue
        body, sync = make(strategy)
        if body is None:
            if rank == 0:
                print(json.dumps({"strategy": strategy, "unavailable": "no multicast mapping"}),
                      flush=True)
            continue
        h.zero_()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            body()
        torch.cuda.current_stream().wait_stream(s)
        barrier()
        graph = torch.cuda.CUDAGraph()
        old = _lib.lib().e2h_set_pdl(1)
        try:
            with torch.cuda.graph(graph):
                body()
        finally:
            _lib.lib().e2h_set_pdl(old)
        for _ in range(3):
            graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.reps):
            graph.replay()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item()) * 1e3 / (a.reps * a.iters)
        status = _lib.read_status()
        results[strategy] = us
        part = B * dim * 2
        nvlink = {"local": 0, "nccl": None, "oneshot": (world - 1) * part, "oneshot_mc": part,
                  "twophase": 2 * (world - 1) * part // world,
                  "twophase_mc": 2 * part // world}[strategy]
        if rank == 0:
            print(json.dumps({
                "strategy": strategy, "n_gpus": world, "batch": B, "us_per_iteration": round(us, 2),
                "reduce_adds_us": round(us - results["local"], 2),
                "nvlink_bytes_per_rank_per_reduce": nvlink,
                "algorithmic_bytes": 2 * (world - 1) * part // world,
                "link_floor_us": (None if not nvlink else round(nvlink / 770e9 * 1e6, 2)),
                "status": status}), flush=True)
        del graph
        barrier()
    barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
