"""Headline benchmark: batched decode tokens/s of the Llemma-7B architecture.

    python bench.py [--gpus N --steps K --warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (fixed): LLaMA-2-7B architecture with the Llemma vocabulary (32 layers, dim 4096, 32
heads, ffn 11008, vocab 32016, RoPE theta 1e6), random normal(0, 0.02) bf16 weights, batch 64,
256-token random prompts, 512 new tokens, temperature 0.7, top-k 50, static KV cache, tensor
parallel over the N GPUs. One "step" is one whole batched generation (prefill + 511 decode
steps); ``value`` = 64 * 512 * K / time, the reference's own metric
(inference_generate.py:484-492: decoded tokens x batch / time, prefill included), device-timed
with CUDA events between barriers, max over ranks.

``e2e`` is the same metric through the public API (``inference_generate.generate``) with the
prompt copied from pinned host memory and the generated tokens copied back to pinned host memory
inside the timed region of every step.

``--impl reference`` runs the unmodified reference from ``baseline/_ref`` (its ``Transformer``,
``apply_tp`` and ``generate`` with its ``torch.compile``'d decode step) on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, PROMPT, NEW = 64, 256, 512
TEMPERATURE, TOP_K = 0.7, 50
MODEL = "llemma-7b-32016"


def decode_config(world: int, quant: str = "none") -> dict:
    """The workload description both arms print (identical keys and values for one N)."""
    return {"model": "Llemma-7B architecture (32 layers, dim 4096, 32 heads, ffn 11008, "
                     "vocab 32016, rope 1e6)",
            "global_batch": BATCH, "seq_len": PROMPT + NEW, "prompt_len": PROMPT,
            "new_tokens": NEW, "temperature": TEMPERATURE, "top_k": TOP_K,
            "weights": "bf16" if quant == "none" else quant,
            "parallelism": f"tp{world}",
            "step": "one batched generation: prefill + 511 decode steps",
            "l2": "inputs larger than L2 (weights 13.5 GB + KV cache stream per step)"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "sft", "prm"],
                    help="decode: batched generation (headline); sft: full-parameter SFT step")
    ap.add_argument("--quant", default="none", choices=["none", "int8", "int4"],
                    help="decode: weight-only quantisation of the linears (int4: groups of 128)")
    ap.add_argument("--micro", type=int, default=16, help="sft: sequences per micro batch")
    ap.add_argument("--tp", type=int, default=1, help="sft: tensor-parallel size (rest is FSDP)")
    ap.add_argument("--reduce", default="auto", help="TP reduce strategy of the engine: auto | "
                    "fused | fused_oneshot | fused_twophase | nccl")
    ap.add_argument("--vocab_parallel", type=int, default=1, help="decode, N > 1: shard the "
                    "embedding table and the LM head over the ranks (the reference's "
                    "--vocab_parallel flag, which its own model ignores)")
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch in the "
                    "decode graph (1) or plain stream order (0)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(n):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def max_over_ranks(x: float) -> float:
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync():
    import torch
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


def timed(fn, steps):
    """K calls of fn between barriers, CUDA events on the launching stream; ms, max over ranks."""
    import torch
    barrier_sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    barrier_sync()
    return max_over_ranks(e0.elapsed_time(e1))


def run_ours(a):
    import torch
    rank, local, world = dist_setup(a.gpus)
    from easy_to_hard_b200.models.model import ModelArgs, Transformer
    from easy_to_hard_b200.models import tp
    from easy_to_hard_b200.models.engine import get_engine
    from easy_to_hard_b200.ops import _lib
    import inference_generate as api

    tp.initialize_model_parallel(world)
    cfg = ModelArgs.from_name(MODEL)

    def build(reduce, vocab_parallel):
        """Model (random init, sharded over the N ranks) and its decode engine."""
        c = ModelArgs.from_name(MODEL)
        torch.manual_seed(0)
        with torch.device("cuda"):
            model = Transformer(c, freeze_tok_embeddings=True, freeze_output=True,
                                freeze_norm=True,
                                vocab_parallel=vocab_parallel).to(torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(1234)
        for name, t in list(model.named_parameters()) + list(model.named_buffers()):
            if t.dim() == 2:
                t.data.normal_(0.0, 0.02, generator=g)
        if world > 1:
            tp.apply_tp(model)
            torch.cuda.empty_cache()
        if a.quant == "int8":
            from easy_to_hard_b200.models.quantize import WeightOnlyInt8QuantHandler
            model = WeightOnlyInt8QuantHandler(model).convert_for_runtime_on_the_fly()
        elif a.quant == "int4":
            from easy_to_hard_b200.models.quantize import WeightOnlyInt4QuantHandler
            h = WeightOnlyInt4QuantHandler(model, groupsize=128, inner_k_tiles=8)
            sd = h.create_quantized_state_dict()
            model = h.convert_for_runtime()
            model.load_state_dict(sd, strict=False)
            del sd
        if a.quant != "none":
            model = model.cuda()
            torch.cuda.empty_cache()
        model.eval()
        return model, get_engine(model, BATCH, PROMPT + NEW, reduce=reduce, use_pdl=bool(a.pdl))

    def all_ok(flag: bool) -> bool:
        if world == 1:
            return flag
        import torch.distributed as dist
        t = torch.tensor([int(flag)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def ranks_agree(model, probe):
        """Every rank must produce the same tokens (same seed, bit-identical activations) and
        no device-side wait may have run out. Every rank reaches every collective here whatever
        happened on it, so a failure on one rank is seen by all."""
        digest, err = -1, None
        try:
            seq, _ = api.generate(model, probe, None, 24, temperature=TEMPERATURE, top_k=TOP_K,
                                  seed=123)
            torch.cuda.synchronize()
            if _lib.read_status() == 0:
                digest = int((seq.long() * torch.arange(1, seq.shape[1] + 1,
                                                        device="cuda")).sum())
        except Exception as e:  # noqa: BLE001
            err = e
        ok = digest >= 0
        if world > 1:
            import torch.distributed as dist
            mine = torch.tensor([digest], dtype=torch.int64, device="cuda")
            every = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(every, mine)
            ok = ok and all(int(e) == int(every[0]) for e in every)
        return all_ok(ok), err

    def bring_up(reduce, vocab_parallel):
        """(model, engine, None) when the strategy works on every rank, else (None, None, why)."""
        model = eng = err = None
        try:
            model, eng = build(reduce, vocab_parallel)
        except Exception as e:  # noqa: BLE001
            err = e
        if not all_ok(err is None):
            return None, None, f"build: {type(err).__name__}: {str(err)[:160]}" if err \
                else "build failed on a peer"
        ok, err = ranks_agree(model, probe)
        if not ok:
            return None, None, (f"{type(err).__name__}: {str(err)[:160]}" if err else
                                "ranks disagree or a device-side wait timed out")
        return model, eng, None

    vocab_parallel = bool(a.vocab_parallel) and world > 1 and a.reduce != "nccl" \
        and cfg.vocab_size % world == 0
    probe = torch.randint(0, cfg.vocab_size, (BATCH, PROMPT), dtype=torch.int32,
                          generator=torch.Generator().manual_seed(99)).cuda()
    fallback = None
    model, eng, why = bring_up(a.reduce, vocab_parallel)
    if model is None:
        if world == 1 or a.reduce == "nccl":
            raise RuntimeError(why)
        # a peer-memory path that does not come up on this box: the library baseline between
        # our kernels instead, and the bench line says so
        fallback = why
        torch.cuda.empty_cache()
        _lib.read_status()
        model, eng, why = bring_up("nccl", False)
        if model is None:
            raise RuntimeError(f"the NCCL strategy failed as well: {why}")

    gen = torch.Generator().manual_seed(7)
    host_prompts = [torch.randint(0, cfg.vocab_size, (BATCH, PROMPT), generator=gen,
                                  dtype=torch.int32).pin_memory()
                    for _ in range(a.steps + a.warmup)]
    dev_prompts = [p.cuda() for p in host_prompts]
    host_out = torch.empty(BATCH, PROMPT + NEW, dtype=torch.int32).pin_memory()

    def step_device(i):
        api.generate(model, dev_prompts[i % len(dev_prompts)], None, NEW,
                     temperature=TEMPERATURE, top_k=TOP_K, seed=i)

    def step_e2e(i):
        p = host_prompts[i % len(host_prompts)].to("cuda", non_blocking=True)
        seq, _ = api.generate(model, p, None, NEW, temperature=TEMPERATURE, top_k=TOP_K, seed=i)
        host_out.copy_(seq, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(a.warmup):
        step_device(i)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(lambda i: step_device(a.warmup + i), a.steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(lambda i: step_e2e(a.warmup + i), a.steps)
    status = _lib.read_status()
    agree = ranks_agree(model, probe)[0] if world > 1 else True
    toks = BATCH * NEW * a.steps
    key = next(iter(eng._graphs)) if eng._graphs else None
    launches = (eng.prefill_launches + (NEW - 1) * eng.decode_launches(key)) * a.steps
    if rank == 0:
        out = {
            "metric": "batched_decode_tokens_per_s", "value": toks / (ms / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16" if a.quant == "none" else f"bf16 activations, {a.quant} weights",
            "data": "synthetic (random token ids, random-init weights)",
            "impl": "ours",
            "config": decode_config(world, a.quant),
            "impl_notes": {"tp_reduce": eng.reduce,
                           "tp_reduce_form": (None if eng.sync is None else
                                              "one-shot pull" + (" (multimem.ld_reduce)"
                                                                 if eng.sync.multicast else "")
                                              if eng.sync.oneshot else
                                              "two-phase" + (" (multimem)" if eng.sync.multicast
                                                             else "")),
                           "vocab_parallel": eng.vocab_parallel, "ranks_agree": agree,
                           "fell_back_to_nccl_because": fallback,
                           "kv_cache": "sized to prompt + new tokens, only the live range is read"},
            "clocks": clocks,
            "e2e": {"value": toks / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": BATCH * PROMPT * 4,
                    "d2h_bytes_per_step": BATCH * (PROMPT + NEW) * 4},
            "gpu_launches": launches, "kernel_status": status,
        }
        print(json.dumps(out), flush=True)
    eng._graphs.clear()


def finish():
    """Ends the process. The result line is out and every rank has synchronised. CUDA graphs are
    dropped first (they may hold collective kernels), then the interpreter's exit callbacks run
    (so that anything registered with ``atexit``, e.g. a hook that records which shared libraries
    this process mapped, still sees a live process), then the process leaves without running the
    static destructors of the communication libraries: tearing a communicator down at
    interpreter exit has blocked on this stack before. A watchdog bounds the whole sequence."""
    import atexit

    def _bail():
        time.sleep(90)
        os._exit(0)

    threading.Thread(target=_bail, daemon=True).start()
    try:
        import torch
        import torch.distributed as dist
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()
            torch.cuda.synchronize()
    except Exception:  # noqa: BLE001
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    try:
        atexit._run_exitfuncs()
    except Exception:  # noqa: BLE001
        pass
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


SFT_SEQ, SFT_GLOBAL_BATCH = 768, 64


def sft_config(world: int, tp: int) -> dict:
    """The SFT workload description both arms print."""
    return {"model": "Llemma-7B architecture (32 layers, dim 4096, 32 heads, ffn 11008, "
                     "vocab 32016, rope 1e6)",
            "global_batch": SFT_GLOBAL_BATCH, "seq_len": SFT_SEQ,
            "parallelism": f"tp{tp}xfsdp{world // tp}",
            "sequence_parallel": tp > 1,
            "optimizer": "AdamW lr 2e-5 betas 0.9/0.95, fp32 master weights, fp32 moments, "
                         "bf16 compute, gradient clipping at 1.0",
            "loss": "cross-entropy on response tokens (prompt 64..384 masked)",
            "step": "one optimizer step over the global batch",
            "l2": "inputs larger than L2 (13 GB of bf16 weights per pass)"}


def sft_batches(n, vocab, per_rank, rank):
    """Random token ids; per sequence a prompt of 64..384 tokens whose labels are ignored
    (cross-entropy on the response tokens only). Pinned host tensors."""
    import torch
    gen = torch.Generator().manual_seed(100 + rank)
    out = []
    for _ in range(n):
        ids = torch.randint(0, vocab, (per_rank, SFT_SEQ), generator=gen, dtype=torch.int64)
        plen = torch.randint(64, 385, (per_rank, 1), generator=gen)
        labels = ids.clone()
        labels[torch.arange(SFT_SEQ)[None, :] < plen] = -100
        out.append((ids.pin_memory(), labels.pin_memory()))
    return out


def run_ours_sft(a):
    """Full-parameter SFT step of the 7B architecture: fp32 master weights, bf16 compute, AdamW
    with fp32 moments (lr 2e-5, betas 0.9/0.95), global batch 64 x 768 tokens, TP=a.tp
    (sequence parallel) x sharded data parallel over the rest. value = trained tokens/s of the
    whole job."""
    import torch
    rank, local, world = dist_setup(a.gpus)
    from easy_to_hard_b200.models.model import ModelArgs, Transformer
    from easy_to_hard_b200.models import tp
    from easy_to_hard_b200.parallel import groups
    from easy_to_hard_b200.parallel.fsdp import ShardedDataParallel
    from easy_to_hard_b200.training import SFTStepper, prepare_batch
    from easy_to_hard_b200.utils.memory_efficient_adam import MemoryEfficientAdamW
    from easy_to_hard_b200.ops import _lib

    tp.initialize_model_parallel(a.tp)
    dp = world // a.tp
    cfg = ModelArgs.from_name(MODEL)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = Transformer(cfg, freeze_tok_embeddings=True, freeze_output=True,
                            freeze_norm=True).to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(1234)
    for name, t in list(model.named_parameters()) + list(model.named_buffers()):
        if t.dim() == 2:
            t.data.normal_(0.0, 0.02, generator=g)
    if a.tp > 1:
        tp.apply_tp(model, requires_grad=True, sequence_parallel=True)
    model.requires_grad_(True)
    sdp = ShardedDataParallel(model, process_group=groups.get_data_parallel_group(),
                              param_dtype=torch.float32, compute_dtype=torch.bfloat16,
                              reduce_dtype=torch.bfloat16)
    sdp.train()
    torch.cuda.empty_cache()
    opt = MemoryEfficientAdamW(list(sdp.optimizer_parameters()), lr=2e-5, betas=(0.9, 0.95),
                               weight_decay=0.0, optim_dtype=torch.float32,
                               optim_device=torch.device("cuda"))
    stepper = SFTStepper(sdp, opt)
    per_rank = SFT_GLOBAL_BATCH // world            # rows each rank loads; a TP group pools them
    host = sft_batches(a.steps + a.warmup, cfg.vocab_size, per_rank, rank)
    dev = [(i.cuda(), l.cuda()) for i, l in host]
    host_loss = torch.zeros(1, dtype=torch.float32).pin_memory()
    micro = max(1, min(a.micro, per_rank * a.tp))     # sequences per forward/backward pass

    def step_device(i):
        ids, labels = prepare_batch(*dev[i % len(dev)], -1, 0, a.tp > 1)
        stepper.step(ids, labels, micro)

    def step_e2e(i):
        ids, labels = host[i % len(host)]
        ids = ids.to("cuda", non_blocking=True)
        labels = labels.to("cuda", non_blocking=True)
        ids, labels = prepare_batch(ids, labels, -1, 0, a.tp > 1)
        loss, _ = stepper.step(ids, labels, micro)
        host_loss.copy_(loss.float().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(a.warmup):
        step_device(i)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(lambda i: step_device(a.warmup + i), a.steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(lambda i: step_e2e(a.warmup + i), a.steps)
    status = _lib.read_status()
    toks = SFT_GLOBAL_BATCH * SFT_SEQ * a.steps
    n_micro = -(-(per_rank * a.tp) // micro)
    # per block and micro batch: forward 9 kernels, backward 17 (+ 9 where the block is
    # recomputed; blocks whose intermediates fit the activation budget are not); plus CE chunks
    kept = int(getattr(sdp, "_keep_budget", 0) > 0)
    launches = (cfg.n_layer * (9 + 17 + (0 if kept else 9)) * n_micro + cfg.n_layer * 2 + 40) \
        * a.steps
    if rank == 0:
        flops = 6 * 6.74e9 * SFT_GLOBAL_BATCH * SFT_SEQ     # model FLOPs, recomputation not counted
        out = {
            "metric": "sft_train_tokens_per_s", "value": toks / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random token ids, random-init weights)", "impl": "ours",
            "config": sft_config(world, a.tp),
            "impl_notes": {"micro_batch": micro,
                           "activations": ("block intermediates kept within %.0f GiB, rest "
                                           "recomputed" % (getattr(sdp, "_keep_budget", 0) / 2 ** 30)),
                           "model_tflops_per_gpu": flops / (ms / a.steps / 1e3) / 1e12 / world,
                           "peak_memory_gib": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)},
            "clocks": clocks,
            "e2e": {"value": toks / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * per_rank * SFT_SEQ * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "kernel_status": status,
        }
        print(json.dumps(out), flush=True)


PRM_SEQ, PRM_PER_DEVICE = 1024, 16


def run_ours_prm(a):
    """Process-reward-model training step of the 7B architecture (the reference's recipe,
    examples/README.md:59-79 of the reference: TP 1, sharded data parallel over all ranks, 16
    sequences of 1024 tokens per device): backbone + two-row reward head, weighted per-token
    binary cross-entropy, fp32 master weights and moments, bf16 compute. value = trained
    tokens/s of the whole job (weak scaling: the global batch grows with N)."""
    import torch
    rank, local, world = dist_setup(a.gpus)
    from easy_to_hard_b200.models.model import ModelArgs
    from easy_to_hard_b200.models import tp
    from easy_to_hard_b200.models.reward_model import (RewardArgs, RewardModel,
                                                      apply_reward_modeling_head)
    from easy_to_hard_b200.parallel import groups
    from easy_to_hard_b200.parallel.fsdp import ShardedDataParallel
    from easy_to_hard_b200.training import TrainStepper, pointwise_reward_loss
    from easy_to_hard_b200.utils.memory_efficient_adam import MemoryEfficientAdamW
    from easy_to_hard_b200.ops import _lib

    tp.initialize_model_parallel(1)
    cfg = ModelArgs.from_name(MODEL)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = RewardModel(RewardArgs(backbone_args=cfg), freeze_tok_embeddings=True,
                            freeze_output=True, freeze_norm=True).to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(1234)
    for name, t in list(model.named_parameters()) + list(model.named_buffers()):
        if t.dim() == 2:
            t.data.normal_(0.0, 0.02, generator=g)
    apply_reward_modeling_head(model.backbone_model, requires_grad=True, init_sceheme="random")
    model.requires_grad_(True)
    sdp = ShardedDataParallel(model, process_group=groups.get_data_parallel_group(),
                              param_dtype=torch.float32, compute_dtype=torch.bfloat16,
                              reduce_dtype=torch.bfloat16)
    sdp.train()
    torch.cuda.empty_cache()
    opt = MemoryEfficientAdamW(list(sdp.optimizer_parameters()), lr=2e-5, betas=(0.9, 0.95),
                               weight_decay=0.0, optim_dtype=torch.float32,
                               optim_device=torch.device("cuda"))
    stepper = TrainStepper(sdp, opt, None, pointwise_reward_loss, 1.0)
    gen = torch.Generator().manual_seed(200 + rank)
    host = []
    for _ in range(a.steps + a.warmup):
        ids = torch.randint(0, cfg.vocab_size, (PRM_PER_DEVICE, PRM_SEQ), generator=gen)
        labels = torch.randint(0, 2, (PRM_PER_DEVICE, PRM_SEQ), generator=gen).float()
        # step boundaries (one position in ~24) carry the weight, as the step-level labels do
        weights = (torch.rand(PRM_PER_DEVICE, PRM_SEQ, generator=gen) < 1 / 24).float()
        host.append(tuple(t.pin_memory() for t in (ids, labels, weights)))
    dev = [tuple(t.cuda() for t in b) for b in host]
    host_loss = torch.zeros(1, dtype=torch.float32).pin_memory()
    micro = max(1, min(a.micro, PRM_PER_DEVICE))

    def step_device(i):
        stepper.step(*dev[i % len(dev)], micro_batch_size=micro)

    def step_e2e(i):
        batch = tuple(t.to("cuda", non_blocking=True) for t in host[i % len(host)])
        loss, _ = stepper.step(*batch, micro_batch_size=micro)
        host_loss.copy_(loss.float().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(a.warmup):
        step_device(i)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(lambda i: step_device(a.warmup + i), a.steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = timed(lambda i: step_e2e(a.warmup + i), a.steps)
    status = _lib.read_status()
    toks = PRM_PER_DEVICE * world * PRM_SEQ * a.steps
    n_micro = -(-PRM_PER_DEVICE // micro)
    kept = int(getattr(sdp, "_keep_budget", 0) > 0)
    launches = (cfg.n_layer * (9 + 17 + (0 if kept else 9)) * n_micro + cfg.n_layer * 2 + 40) \
        * a.steps
    if rank == 0:
        flops = 6 * 6.6e9 * PRM_PER_DEVICE * world * PRM_SEQ
        out = {
            "metric": "prm_train_tokens_per_s", "value": toks / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random token ids, labels and step weights, random-init weights)",
            "impl": "ours",
            "config": {"model": "Llemma-7B architecture + 2-row reward head",
                       "global_batch": PRM_PER_DEVICE * world, "seq_len": PRM_SEQ,
                       "parallelism": f"tp1xfsdp{world}",
                       "optimizer": "AdamW lr 2e-5 betas 0.9/0.95, fp32 master weights, fp32 "
                                    "moments, bf16 compute, gradient clipping at 1.0",
                       "loss": "weighted per-token binary cross-entropy",
                       "l2": "inputs larger than L2 (13 GB of bf16 weights per pass)"},
            "impl_notes": {"micro_batch": micro,
                           "model_tflops_per_gpu": flops / (ms / a.steps / 1e3) / 1e12 / world,
                           "peak_memory_gib": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)},
            "clocks": clocks,
            "e2e": {"value": toks / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": PRM_PER_DEVICE * PRM_SEQ * 16, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "kernel_status": status,
        }
        print(json.dumps(out), flush=True)


def run_reference(a):
    """The unmodified reference on the same workload: its own generate() for decode, its own
    training step (FSDP1, its AdamW, its tensor-parallel hooks) for SFT."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")

    def unavailable(why):
        if int(os.environ.get("RANK", 0)) == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)

    if not os.path.isdir(os.path.join(ref_dir, "models")):
        return unavailable("reference is not installed under baseline/_ref "
                           "(the reference ships neither setup.py nor pyproject.toml: install it from a copy "
                           "with a minimal setup.py, --no-deps)")
    try:
        from baseline import reference_runner, reference_sft_runner
    except Exception as e:  # noqa: BLE001
        return unavailable(f"reference runner import failed: {type(e).__name__}: {e}")
    if a.workload == "prm":
        return unavailable("no reference arm is wired for the reward-model training workload")
    try:
        if a.workload == "sft":
            reference_sft_runner.run(a, dict(seq=SFT_SEQ, global_batch=SFT_GLOBAL_BATCH,
                                             sequence_parallel=True, config=sft_config),
                                     ClockSampler)
        else:
            reference_runner.run(a, dict(batch=BATCH, prompt=PROMPT, new=NEW,
                                         temperature=TEMPERATURE, top_k=TOP_K, quant=a.quant,
                                         config=decode_config), ClockSampler)
    except Exception as e:  # noqa: BLE001
        unavailable(f"reference failed: {type(e).__name__}: {str(e)[:300]}")


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "sft":
        run_ours_sft(args)
    elif args.workload == "prm":
        run_ours_prm(args)
    else:
        run_ours(args)
    finish()
