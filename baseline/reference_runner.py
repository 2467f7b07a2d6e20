"""Runs the UNMODIFIED reference (installed under ``baseline/_ref``) on the headline workload.

Nothing of this framework is imported here: the model is the reference's ``Transformer``, sharded
by its ``apply_tp``, and tokens come from its ``generate`` with its decode step wrapped in
``torch.compile(mode="reduce-overhead", fullgraph=True)`` exactly as its ``main`` does
(inference_generate.py:346-354 of the reference). The static KV cache is therefore sized to the
model's ``block_size`` and read in full every step -- that is the reference's stock behaviour.
"""
from __future__ import annotations

import json
import os
import sys


def run(a, wl, ClockSampler):
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "_ref"))
    import torch
    import torch.distributed as dist
    from models.model import ModelArgs, Transformer
    from models.tp import apply_tp, initialize_model_parallel, maybe_init_dist
    import inference_generate as ref

    B, T, NEW = wl["batch"], wl["prompt"], wl["new"]
    rank = maybe_init_dist()
    use_tp = rank is not None
    if use_tp:
        initialize_model_parallel(dist.get_world_size())
    world = dist.get_world_size() if use_tp else 1
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)

    def build(block_size):
        cfg = ModelArgs(block_size=block_size, vocab_size=32016, n_layer=32, n_head=32, dim=4096,
                        intermediate_size=11008, rope_base=1000000)
        with torch.device("cuda"):
            m = Transformer(cfg, freeze_tok_embeddings=True, freeze_output=True, freeze_norm=True,
                            vocab_parallel=True).to(torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(1234)
        for t in list(m.parameters()) + list(m.buffers()):
            if t.dim() == 2:
                t.data.normal_(0.0, 0.02, generator=g)
        if use_tp:
            apply_tp(m)
        m = m.to(device="cuda", dtype=torch.bfloat16).eval()
        quant = wl.get("quant", "none")
        if quant == "int8":
            # the reference's own on-the-fly path (inference_generate.py:319-326 there)
            from models.quantize import WeightOnlyInt8QuantHandler
            m = WeightOnlyInt8QuantHandler(m).convert_for_runtime_on_the_fly()
            m = m.to(device="cuda").eval()
        elif quant == "int4":
            # its offline path, run in memory: quantised state dict, runtime modules, load
            from models.quantize import WeightOnlyInt4QuantHandler
            h = WeightOnlyInt4QuantHandler(m, 128)
            sd = h.create_quantized_state_dict()
            m = h.convert_for_runtime()
            m.load_state_dict(sd, assign=True)
            m = m.to(device="cuda").eval()
        return m

    eager_decode = ref.decode_one_token
    gen = torch.Generator().manual_seed(7)
    host_prompts = [torch.randint(0, 32016, (B, T), generator=gen, dtype=torch.int32).pin_memory()
                    for _ in range(a.steps + a.warmup)]

    def one(model, i, e2e=False):
        p = host_prompts[i % len(host_prompts)].to("cuda", non_blocking=True)
        y, n = ref.generate(model, p, None, NEW, temperature=wl["temperature"],
                            top_k=wl["top_k"], eos_id=2)
        if e2e:
            return y.tolist()
        return None

    # The reference's stock decode modes, fastest first: --compile (reduce-overhead, CUDA
    # graphs), the same with PyTorch's legacy CUDA-graph runner (a PyTorch setting, the
    # reference is untouched), --default_compile, and plain eager. The first one that survives
    # the warm-up on this PyTorch version is the one that is timed.
    import torch._inductor.config as ind_cfg
    modes = [("compile: reduce-overhead", "reduce-overhead", True),
             ("compile: reduce-overhead, cudagraph_trees=False", "reduce-overhead", False),
             ("default_compile", "default", True),
             ("eager (no compile)", None, True)]
    notes = []
    model = None
    for block_size in (4096, 2048):
        for label, mode, trees in modes:
            try:
                import gc
                gc.collect()
                torch.cuda.empty_cache()
                torch._dynamo.reset()
                ind_cfg.triton.cudagraph_trees = trees
                ref.decode_one_token = (eager_decode if mode is None else
                                        torch.compile(eager_decode, mode=mode, fullgraph=True))
                if model is None:
                    model = build(block_size)
                    ref.remove_all_backward_hooks(model)
                for i in range(a.warmup):
                    one(model, i)
                torch.cuda.synchronize()
                notes.append(f"ran with {label}, block_size {block_size}")
                break
            except (NotImplementedError, ImportError, ModuleNotFoundError, AttributeError) as e:
                if model is None:      # the quantised model itself could not be built
                    raise RuntimeError(f"{type(e).__name__}: {str(e)[:200]}") from e
                notes.append(f"{label}: {type(e).__name__}: {str(e)[:120]}")
                continue
            except torch.cuda.OutOfMemoryError:
                notes.append(f"{label}, block_size {block_size}: out of memory")
                model = None
                break
            except Exception as e:  # noqa: BLE001
                notes.append(f"{label}: {type(e).__name__}: {str(e)[:120]}")
                continue
        else:
            model = None
        if model is not None and notes and notes[-1].startswith("ran with"):
            break
        model = None
    note = "; ".join(notes)
    if model is None:
        raise RuntimeError(note or "reference model could not be built")

    def sync():
        if use_tp:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.steps):
            fn(a.warmup + i)
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if use_tp:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local)
    if rank in (None, 0):
        sampler.start()
    ms = timed(lambda i: one(model, i))
    clocks = sampler.stop() if rank in (None, 0) else None
    ms_e2e = timed(lambda i: one(model, i, e2e=True))
    toks = B * NEW * a.steps
    if rank in (None, 0):
        print(json.dumps({
            "metric": "batched_decode_tokens_per_s", "value": toks / (ms / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16" if wl.get("quant", "none") == "none"
            else f"bf16 activations, {wl['quant']} weights",
            "data": "synthetic (random token ids, random-init weights)", "impl": "reference",
            "config": wl["config"](world, wl.get("quant", "none")),
            "impl_notes": {"kv_cache": f"sized to block_size {model.config.block_size} and read "
                           "in full every step (the reference's stock generate)",
                           "decode_mode": note},
            "clocks": clocks,
            "e2e": {"value": toks / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": B * T * 4, "d2h_bytes_per_step": B * (T + NEW) * 4},
        }), flush=True)
