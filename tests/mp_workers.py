"""Worker bodies for the multi-process CPU (gloo) tests. Every worker writes its result with
``torch.save`` to ``<out>/rank<k>.pt``; the test process compares the files."""
from __future__ import annotations

import datetime
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, out, kwargs):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      LOCAL_RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    backend = kwargs.pop("backend", "gloo")
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        if world > 1:
            extra = {"device_id": torch.device("cuda", rank)} if backend == "nccl" else {}
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    timeout=datetime.timedelta(seconds=kwargs.pop("pg_timeout", 120)),
                                    **extra)
        res = fn(rank, world, **kwargs)
        torch.save(res, os.path.join(out, f"rank{rank}.pt"))
        if backend == "nccl" and world > 1:
            # communicators referenced by captured CUDA graphs can block in their destructor:
            # synchronise, then leave the child without tearing NCCL down
            torch.cuda.synchronize()
            dist.barrier()
            os._exit(0)
    except Exception:  # noqa: BLE001 -- the parent only sees files
        with open(os.path.join(out, f"rank{rank}.err"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run(fn, world: int, out: str, **kwargs):
    """Run ``fn(rank, world, **kwargs)`` on ``world`` gloo ranks; returns the per-rank results."""
    os.makedirs(out, exist_ok=True)
    port = free_port()
    if world == 1:
        saved = {k: os.environ.get(k) for k in ("MASTER_ADDR", "MASTER_PORT", "RANK", "LOCAL_RANK",
                                                "WORLD_SIZE")}
        try:
            _entry(0, 1, port, fn, out, dict(kwargs))
        finally:
            for k, v in saved.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
    else:
        mp.spawn(_entry, args=(world, port, fn, out, dict(kwargs)), nprocs=world, join=True)
    return [torch.load(os.path.join(out, f"rank{r}.pt"), weights_only=False)
            for r in range(world)]


# ------------------------------------------------------------------------------- model helpers

def tiny_model(seed=0, dtype=torch.float32, vocab_parallel=False, name="tiny-llama"):
    from easy_to_hard_b200.models.model import Transformer
    torch.manual_seed(seed)
    m = Transformer.from_name(name, freeze_tok_embeddings=True, freeze_output=True,
                              freeze_norm=True, vocab_parallel=vocab_parallel)
    g = torch.Generator().manual_seed(seed + 1)
    for _, t in list(m.named_parameters()) + list(m.named_buffers()):
        if t.dim() == 2:
            t.data.copy_(torch.randn(t.shape, generator=g) * 0.05)
    return m.to(dtype)


def sft_batch(vocab=1024, batch=4, seq=128, seed=3):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (batch, seq), generator=g)
    labels = ids.clone()
    labels[:, :64] = -100            # loss over positions 64..127 only
    return ids, labels


def _merged_state(sdp):
    """Full (data-parallel-unsharded) state dict; tensor-parallel shards stay as they are."""
    return sdp.full_state_dict(rank0_only=False)


def sft_step_and_generate(rank, world, tp=1, sequence_parallel=False, vocab_parallel=False,
                          steps=1, micro=None, gen=True, device="cpu", keep_params=False):
    """One (or more) SFT steps on the tiny model with TP=tp, DP=world/tp, then greedy decode."""
    from easy_to_hard_b200.models import tp as tpm
    from easy_to_hard_b200.parallel import groups
    from easy_to_hard_b200.parallel.fsdp import ShardedDataParallel
    from easy_to_hard_b200.training import SFTStepper
    from easy_to_hard_b200.utils.memory_efficient_adam import MemoryEfficientAdamW
    from easy_to_hard_b200.models.rl_model import generate_tokens
    from easy_to_hard_b200.utils.checkpoint_utils import merge_tp_checkpoint

    tpm.initialize_model_parallel(tp)
    device = torch.device(device if device == "cpu" else f"cuda:{rank}")
    model = tiny_model(vocab_parallel=vocab_parallel).to(device)
    heads = (model.config.n_head, model.config.n_local_heads)
    if tp > 1:
        tpm.apply_tp(model, requires_grad=True, sequence_parallel=sequence_parallel)
    for n, p in model.named_parameters():
        p.requires_grad_(True)
    sdp = ShardedDataParallel(model, process_group=groups.get_data_parallel_group(),
                              keep_params=keep_params)
    sdp.train()
    opt = MemoryEfficientAdamW(list(sdp.optimizer_parameters()), lr=1e-4, weight_decay=0.0,
                               optim_dtype=torch.float32, optim_device=device)
    stepper = SFTStepper(sdp, opt)
    ids, labels = (t.to(device) for t in sft_batch())
    dp, dp_rank = groups.get_data_parallel_world_size(), groups.get_data_parallel_rank()
    per = ids.shape[0] // dp                       # every data-parallel rank takes its rows
    my_ids, my_lab = ids[dp_rank * per:(dp_rank + 1) * per], labels[dp_rank * per:(dp_rank + 1) * per]
    losses, norms = [], []
    for _ in range(steps):
        loss, gn = stepper.step(my_ids, my_lab, micro)
        l = loss.detach().clone()
        if dp > 1:
            dist.all_reduce(l, group=groups.get_data_parallel_group())
            l /= dp
        losses.append(float(l))
        norms.append(float(gn))
    state = _merged_state(sdp)
    state = {k: v.cpu() for k, v in state.items() if "layers" in k and k.endswith("weight")
             and "norm" not in k}
    if tp > 1:   # gather the tensor-parallel shards and merge them to the TP=1 layout
        shards = [None] * tp
        dist.all_gather_object(shards, state, group=groups.get_model_parallel_group())
        state = merge_tp_checkpoint(shards, heads=heads)
    out = {"loss": losses, "grad_norm": norms, "state": state, "gathers": sdp.gathers}
    if gen:
        # decode with the updated weights through the plain module path
        for u in sdp.units:
            u.gather_into(torch.empty(u.padded, dtype=u.shard_lp.dtype, device=device))
        model.eval()
        g = torch.Generator().manual_seed(11)
        prompts = torch.randint(0, 1024, (4, 32), generator=g).to(device)
        with torch.no_grad():
            seq = generate_tokens(model, prompts, None, 16, temperature=0.0, top_k=None,
                                  eos_id=None)
        out["tokens"] = seq.cpu()
    return out


def checkpoint_roundtrip(rank, world, tp=1, save_dir=None):
    """Train 2 steps, save through checkpoint_utils, train 1 more; a fresh model resumes from the
    file and must reproduce the third step."""
    from types import SimpleNamespace
    from easy_to_hard_b200.models import tp as tpm
    from easy_to_hard_b200.parallel import groups
    from easy_to_hard_b200.parallel.fsdp import ShardedDataParallel
    from easy_to_hard_b200.training import SFTStepper
    from easy_to_hard_b200.utils import checkpoint_utils as cu
    from easy_to_hard_b200.utils.memory_efficient_adam import MemoryEfficientAdamW
    from easy_to_hard_b200.utils.trainer_utils import get_cosine_schedule_with_warmup

    tpm.initialize_model_parallel(tp)

    def build():
        model = tiny_model()
        if tp > 1:
            tpm.apply_tp(model, requires_grad=True)
        model.requires_grad_(True)
        names = [n for n, p in model.named_parameters() if p.requires_grad]
        sdp = ShardedDataParallel(model, process_group=groups.get_data_parallel_group())
        sdp.train()
        opt = MemoryEfficientAdamW(list(sdp.optimizer_parameters()), lr=1e-3,
                                   optim_dtype=torch.float32, optim_device=torch.device("cpu"))
        sch = get_cosine_schedule_with_warmup(opt, 1, 10)
        return sdp, opt, sch, names

    ids, labels = sft_batch(batch=2 * max(1, world // tp))
    dp, dp_rank = groups.get_data_parallel_world_size(), groups.get_data_parallel_rank()
    per = ids.shape[0] // dp
    my = slice(dp_rank * per, (dp_rank + 1) * per)
    sdp, opt, sch, names = build()
    st = SFTStepper(sdp, opt, sch)
    for _ in range(2):
        st.step(ids[my], labels[my])
    path = cu.get_checkpoint_path(save_dir, 0, 2, groups.get_model_parallel_rank(), "")
    cu.save_checkpoint(path, sdp, opt, sch, 0, 2, groups.get_model_parallel_rank(), False, None,
                       True, names, "", None, torch.float32)
    if dist.is_initialized():
        dist.barrier()
    l3, _ = st.step(ids[my], labels[my])

    sdp2, opt2, sch2, _ = build()
    found, epoch, step = cu.get_latest_checkpoint_path(save_dir)
    cu.load_checkpoint(found, sdp2, opt2, sch2, use_fsdp=True)
    st2 = SFTStepper(sdp2, opt2, sch2)
    l3b, _ = st2.step(ids[my], labels[my])
    a, b = sdp.full_state_dict(rank0_only=False), sdp2.full_state_dict(rank0_only=False)
    diff = max(float((a[k].float() - b[k].float()).abs().max()) for k in a if "layers" in k)
    return {"l3": float(l3), "l3_resumed": float(l3b), "step": step, "param_diff": diff,
            "lr": (sch.get_last_lr()[0], sch2.get_last_lr()[0])}


# ------------------------------------------------------------------------------- failure paths

def rank_raises(rank, world, bad_rank=1):
    """A rank fails on the host between steps; the others learn of it from the store before the
    next collective (no collective is left hanging)."""
    from easy_to_hard_b200.parallel.health import HealthMonitor
    mon = HealthMonitor(rank, world, heartbeat_s=0.05, dead_after_s=1.0)
    mon.start()
    status = "ok"
    try:
        for step in range(50):
            mon.check()                      # raises PeerFailure if someone reported an error
            if rank == bad_rank and step == 3:
                raise RuntimeError("injected host-side failure")
            t = torch.ones(4)
            dist.all_reduce(t)
            import time
            time.sleep(0.02)
    except RuntimeError as e:
        if "injected" in str(e):
            mon.report_failure(str(e))
            status = "failed"
        else:
            status = f"peer-failure:{e}"
    except Exception as e:  # noqa: BLE001
        status = f"peer-failure:{type(e).__name__}"
    finally:
        mon.stop()
    return status


def rank_never_joins(rank, world):
    """Rank 1 leaves before the collective; a short process-group timeout ends the others' wait
    with an error instead of a hang."""
    if rank == 1:
        return "left"
    try:
        t = torch.ones(2)
        dist.all_reduce(t)
        return "completed"
    except Exception as e:  # noqa: BLE001
        return f"error:{type(e).__name__}"


def p2p_channel_ops(rank, world, device="cuda"):
    """Stand-alone peer-memory collectives (parallel/symm.P2PChannel) against NCCL."""
    from easy_to_hard_b200.ops import _lib
    from easy_to_hard_b200.parallel.symm import P2PChannel
    torch.manual_seed(100 + rank)
    n = 1 << 16
    ch = P2PChannel(n * 2, wait_ms=20000)
    res = {}
    for rep in range(3):
        x = torch.randn(n, device="cuda").bfloat16()
        ref = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(ref, x)
        got = ch.all_gather(x)
        res[f"gather{rep}"] = bool(torch.equal(got, torch.stack(ref)))
        want = torch.stack(ref).float().sum(0)
        one = ch.all_reduce(x, "one_shot")
        two = ch.all_reduce(x, "two_shot")
        res[f"one{rep}"] = float((one.float() - want).abs().max() / want.abs().max())
        res[f"two{rep}"] = float((two.float() - want).abs().max() / want.abs().max())
        res[f"same{rep}"] = bool(torch.equal(one, two))
        rs = ch.reduce_scatter(x)
        res[f"rs{rep}"] = bool(torch.equal(rs, one.view(world, -1)[rank]))
        ch.barrier()
    torch.cuda.synchronize()
    res["status"] = _lib.read_status()
    return res


def decode_engine_tp(rank, world, vocab_parallel=False, reduce="fused", dim_name="tiny-llama",
                     new_tokens=24):
    """Batched generation on the CUDA decode engine with TP = world: greedy and sampled tokens,
    the device status word, and whether the multicast (NVLS) form of the reduce was used."""
    from easy_to_hard_b200.models import tp as tpm
    from easy_to_hard_b200.models.engine import DecodeEngine
    from easy_to_hard_b200.ops import _lib

    tpm.initialize_model_parallel(world)
    dev = torch.device(f"cuda:{rank}")
    model = tiny_model(dtype=torch.bfloat16, vocab_parallel=vocab_parallel, name=dim_name).to(dev)
    if world > 1:
        tpm.apply_tp(model)
    model.eval()
    eng = DecodeEngine(model, 8, 96, reduce=reduce)
    g = torch.Generator().manual_seed(21)
    prompts = torch.randint(0, 1024, (8, 32), generator=g).to(dev)
    left_pad = torch.tensor([0, 3, 0, 7, 1, 0, 0, 12], device=dev)
    out = {"reduce": eng.reduce, "multicast": bool(eng.sync.multicast) if eng.sync else False}
    seq, _ = eng.generate(prompts, left_pad, new_tokens, temperature=0.0, top_k=None)
    out["greedy"] = seq.cpu().clone()
    seq, _ = eng.generate(prompts, left_pad, new_tokens, temperature=0.8, top_k=20, seed=5)
    out["sampled5"] = seq.cpu().clone()
    n_graphs = len(eng._graphs)
    seq, _ = eng.generate(prompts, left_pad, new_tokens, temperature=0.8, top_k=20, seed=6)
    out["sampled6"] = seq.cpu().clone()
    out["graphs_reused"] = len(eng._graphs) == n_graphs
    torch.cuda.synchronize()
    out["status"] = _lib.read_status()
    eng._graphs.clear()
    return out


def generate_main(rank, world, checkpoint=None, prompt_file=None, output_file=None,
                  resume=False, tp=1, num_samples=2):
    """``inference_generate.main`` as one rank of a gloo job (data-parallel batches, shared
    output file under flock)."""
    from pathlib import Path
    import inference_generate
    inference_generate.main(seed=3, prompt_file=Path(prompt_file), output_file=Path(output_file),
                            batch_size=2, num_samples=num_samples, max_new_tokens=6, top_k=20,
                            temperature=0.8, checkpoint_path=Path(checkpoint), compile=False,
                            resume_generation=resume, tensor_parallel_size=tp)
    return {"rank": rank}


def rollout_relayout(rank, world, tp=1, rollout_tp=2, device="cpu", generate=True):
    """Training layout TP=tp x DP=world/tp -> rollout layout TP=rollout_tp: after one SFT step
    the rollout copy is refreshed from the training shards; returns the largest deviation from
    the directly re-sharded full weights, and greedy tokens generated at the rollout degree."""
    from easy_to_hard_b200.models import tp as tpm
    from easy_to_hard_b200.models.rl_model import generate_tokens
    from easy_to_hard_b200.parallel import groups
    from easy_to_hard_b200.parallel.fsdp import ShardedDataParallel
    from easy_to_hard_b200.parallel.relayout import RolloutRelayout
    from easy_to_hard_b200.training import SFTStepper
    from easy_to_hard_b200.utils.checkpoint_utils import merge_tp_checkpoint
    from easy_to_hard_b200.utils.memory_efficient_adam import MemoryEfficientAdamW

    tpm.initialize_model_parallel(tp)
    groups.initialize_rollout_parallel(rollout_tp)
    dev = torch.device(device if device == "cpu" else f"cuda:{rank}")
    cuda = dev.type == "cuda"
    dt = torch.bfloat16 if cuda else torch.float32
    model = tiny_model(dtype=dt).to(dev)
    heads = (model.config.n_head, model.config.n_local_heads)
    if tp > 1:
        tpm.apply_tp(model, requires_grad=True)
    model.requires_grad_(True)
    if cuda:
        for p in model.parameters():
            p.data = p.data.float()
    sdp = ShardedDataParallel(model, process_group=groups.get_data_parallel_group())
    sdp.train()
    opt = MemoryEfficientAdamW(list(sdp.optimizer_parameters()), lr=1e-2, weight_decay=0.0,
                               optim_dtype=torch.float32, optim_device=dev)
    ids, labels = (t.to(dev) for t in sft_batch())
    SFTStepper(sdp, opt).step(ids[:2], labels[:2])
    # the rollout copy starts from the initial weights and must pick up the trained ones
    g, ranks, size, rrank = groups.get_rollout_parallel()
    copy_ = tiny_model(dtype=dt).to(dev)
    tpm.apply_tp(copy_, world=size, rank=rrank, group=g)
    copy_ = copy_.to(torch.bfloat16 if cuda else torch.float32).eval()
    exposed = sdp.expose_shards(None) if cuda else False
    rl = RolloutRelayout(sdp, copy_, tp, rollout_tp)
    rl.run()
    # expectation: the full (TP- and DP-unsharded) trained weights, re-sharded at the rollout degree
    state = {k: v.cpu() for k, v in sdp.full_state_dict(rank0_only=False).items()
             if "layers" in k and k.endswith("weight") and "norm" not in k}
    if tp > 1:
        shards = [None] * tp
        dist.all_gather_object(shards, state, group=groups.get_model_parallel_group())
        state = merge_tp_checkpoint(shards, heads=heads)
    ref = tiny_model(dtype=torch.float32)
    ref.load_state_dict({k: v.float() for k, v in state.items()}, strict=False)
    tpm.apply_tp(ref, world=size, rank=rrank, group=g)
    got = dict(copy_.named_parameters())
    got.update(dict(copy_.named_buffers()))
    worst = 0.0
    for k, v in ref.state_dict().items():
        if "layers" in k and k.endswith("weight") and "norm" not in k:
            worst = max(worst, float((got[k].detach().float().cpu() - v.float()).abs().max()))
    out = {"max_diff": worst, "pulled": bool(exposed), "bytes": rl.bytes_per_sync}
    if generate:
        gq = torch.Generator().manual_seed(31)
        prompts = torch.randint(0, 1024, (4, 16), generator=gq).to(dev)
        with groups.model_parallel_as(g, ranks, size, rrank), torch.no_grad():
            seq = generate_tokens(copy_, prompts, None, 8, temperature=0.0, top_k=None,
                                  eos_id=None)
        out["tokens"] = seq.cpu()
        if cuda:
            from easy_to_hard_b200.ops import _lib
            torch.cuda.synchronize()
            out["status"] = _lib.read_status()
    return out


def ppo_main(rank, world, argv=None):
    """``train_rl_ppo.main`` as one rank of a gloo job; returns the per-step statistics."""
    import train_rl_ppo
    from easy_to_hard_b200.utils.arguments import Arguments
    from easy_to_hard_b200.utils.hf_argparser import HfArgumentParser
    args = HfArgumentParser((Arguments,)).parse_args_into_dataclasses(list(argv))[0]
    history = train_rl_ppo.main(args)
    return {"steps": len(history),
            "keys": sorted(history[0].keys()) if history else [],
            "policy_loss": [float(h["ppo/loss/policy"]) for h in history],
            "grad_norm": [float(h["ppo/loss/grad_norm_policy"]) for h in history]}
