"""Runs the UNMODIFIED reference (installed under ``baseline/_ref``) on the SFT workload.

Nothing of this framework is imported here. The step is the reference's own: its ``Transformer``
(frozen embeddings / norms / head, as ``load_model_from_from_ckpt`` builds it), ``apply_tp`` with
its sequence-parallel hooks, ``create_fsdp_model_for_finetune`` (FSDP1 over the data-parallel
group), ``create_optimizer`` (its ``MemoryEfficientAdamW``), and per iteration exactly what
``train_sft.main`` does (train_sft.py:341-375 of the reference): ``model.zero_grad``,
``prepare_batch`` (the tensor-parallel all-gather of the batch), autocast
``model_forward_with_loss`` per micro batch, backward, ``clip_grad_norm_(model, 1.0)``,
``optimizer.step``. Only the data loader is replaced by synthetic batches of the benchmark's
shape and the checkpoint file by random-init weights of the same architecture.

The reference's trainers need a process group (its ``maybe_init_dist`` returns None for a single
process and the training script then dereferences groups that do not exist), so the arm needs
N >= 2 ranks.
"""
from __future__ import annotations

import json
import os
import sys
from types import SimpleNamespace


def run(a, wl, ClockSampler):
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "_ref"))
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank0 = int(os.environ.get("RANK", 0)) == 0
    if world < 2:
        if rank0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "the reference's training scripts need a process group of at least "
                              "2 ranks (train_sft.py dereferences the data-parallel group)"}),
                  flush=True)
        return
    # The reference targets PyTorch 2.2 and imports a private FSDP helper whose signature has
    # since grown two arguments (models/tp.py:22, :847 there call _get_grad_norm(params,
    # norm_type)). The helper is wrapped on the PyTorch side so that the old call still works;
    # the reference's files are untouched.
    import torch.distributed.fsdp.fully_sharded_data_parallel as _fsdp_mod
    import inspect
    if len(inspect.signature(_fsdp_mod._get_grad_norm).parameters) == 4:
        _orig_norm = _fsdp_mod._get_grad_norm

        def _get_grad_norm_compat(params, norm_type, zero=None, device=None):
            params = list(params)
            if device is None:
                device = (params[0].device if params
                          else torch.device("cuda", torch.cuda.current_device()))
            if zero is None:
                zero = torch.tensor(0.0, device=device)
            return _orig_norm(params, norm_type, zero, device)

        _fsdp_mod._get_grad_norm = _get_grad_norm_compat
    from models.model import ModelArgs, Transformer
    from models.tp import (apply_tp, clip_grad_norm_, get_data_parallel_world_size,
                           get_model_parallel_group, initialize_model_parallel, maybe_init_dist)
    import train_sft as ref
    from training_utils.trainer_utils import create_fsdp_model_for_finetune, create_optimizer

    rank = maybe_init_dist()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    tp = a.tp
    initialize_model_parallel(tp)
    dp = world // tp
    seq, gb = wl["seq"], wl["global_batch"]
    args = SimpleNamespace(learning_rate=2e-5, adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-8,
                           weight_decay=0.0, optim_dtype=torch.float32,
                           compute_dtype=torch.bfloat16, param_dtype=torch.float32)
    cfg = ModelArgs(block_size=4096, vocab_size=32016, n_layer=32, n_head=32, dim=4096,
                    intermediate_size=11008, rope_base=1000000)
    # bf16 like a checkpoint, initialised and sharded on the device, then cast to the
    # parameter dtype as load_model_from_from_ckpt does
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = Transformer(cfg, freeze_tok_embeddings=True, freeze_output=True,
                            freeze_norm=True, vocab_parallel=False).to(torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(1234)
    for t in list(model.parameters()) + list(model.buffers()):
        if t.dim() == 2:
            t.data.normal_(0.0, 0.02, generator=g)
    apply_tp(model, requires_grad=True, sequence_parallel=bool(wl["sequence_parallel"]) and tp > 1)
    model.requires_grad_(True)
    model = model.to(device="cuda", dtype=args.param_dtype).train(True)
    use_fsdp = get_data_parallel_world_size() > 1
    if use_fsdp:
        model = create_fsdp_model_for_finetune(args, model)
    optimizer = create_optimizer(args, model=model, optimizer_cpu_offload=False,
                                 model_cpu_offload=False)
    tokenizer = SimpleNamespace(pad_id=-1, unk_id=0)
    per_rank = gb // world
    micro = max(1, min(a.micro, per_rank * tp))
    gen = torch.Generator().manual_seed(100 + dist.get_rank())
    host = []
    for _ in range(a.steps + a.warmup):
        ids = torch.randint(0, 32016, (per_rank, seq), generator=gen, dtype=torch.int64)
        plen = torch.randint(64, 385, (per_rank, 1), generator=gen)
        labels = ids.clone()
        labels[torch.arange(seq)[None, :] < plen] = -100
        host.append((ids.pin_memory(), labels.pin_memory()))
    host_loss = torch.zeros(1, dtype=torch.float32).pin_memory()

    def step(i, e2e=False):
        ids, labels = host[i % len(host)]
        model.zero_grad()
        ids = ids.to("cuda", non_blocking=True)
        labels = labels.to("cuda", non_blocking=True)
        ids, labels = ref.prepare_batch(ids, labels, tokenizer=tokenizer, use_tp=True,
                                        sync_group=get_model_parallel_group())
        n = ids.size(0)
        n_micro = -(-n // micro)
        for s in range(0, n, micro):
            with torch.cuda.amp.autocast(dtype=args.compute_dtype):
                loss = ref.model_forward_with_loss(model, ids[s:s + micro], labels[s:s + micro])
            (loss / n_micro).backward()
        clip_grad_norm_(model, 1.0)
        optimizer.step()
        if e2e:
            host_loss.copy_(loss.detach().float().reshape(1), non_blocking=True)
            torch.cuda.current_stream().synchronize()

    def sync():
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
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for i in range(a.warmup):
        step(i)
    sampler = ClockSampler(local)
    if rank0:
        sampler.start()
    ms = timed(lambda i: step(i))
    clocks = sampler.stop() if rank0 else None
    ms_e2e = timed(lambda i: step(i, e2e=True))
    toks = gb * seq * a.steps
    if rank0:
        print(json.dumps({
            "metric": "sft_train_tokens_per_s", "value": toks / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random token ids, random-init weights)", "impl": "reference",
            "config": wl["config"](world, tp),
            "impl_notes": {"micro_batch": micro, "fsdp": "PyTorch FSDP1 FULL_SHARD" if use_fsdp
                           else "none (data-parallel size 1)",
                           "activation_checkpointing": "every block (the reference's forward)",
                           "pytorch_compat": "private FSDP helper _get_grad_norm wrapped for the "
                                             "reference's PyTorch 2.2 call signature",
                           "peak_memory_gib": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)},
            "clocks": clocks,
            "e2e": {"value": toks / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * per_rank * seq * 8, "d2h_bytes_per_step": 4},
        }), flush=True)
