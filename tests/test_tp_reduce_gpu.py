"""The decode engine's fused tensor-parallel reduce (ops/csrc/tp_reduce.cu) with the ranks of a
group emulated inside one process on one GPU: every "rank" has its own buffers, producers run
before consumers in stream order and the phase-B wait is issued as a separate launch after all
ranks' kernels, so no launch ever waits on a later one. Checked against plain fp32 PyTorch."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(hs, parts, w, eps, world):
    """Row t is owned by rank t*world//T... (owner = the rank whose [row0, row1) holds t)."""
    T, dim = parts[0].shape
    total = torch.stack([p.float() for p in parts]).sum(0).bfloat16().float()
    h = torch.empty(T, dim, dtype=torch.float32, device=parts[0].device)
    for r in range(world):
        r0, r1 = r * T // world, (r + 1) * T // world
        src = hs[r][r0:r1].float() if hs is not None else 0.0
        h[r0:r1] = (src + total[r0:r1]).bfloat16().float()
    rstd = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    xn = ((h * rstd).bfloat16().float() * w.float()).bfloat16()
    return h.bfloat16(), xn


def _signal(sync, point):
    from easy_to_hard_b200.ops import _lib
    arr = (C.c_void_p * 8)()
    for r, p in enumerate(sync.flag_a_remote(point)):
        arr[r] = p
    _lib.check(_lib.lib().e2h_signal_peers(arr, sync.world, _lib.stream()), "signal")


@pytest.mark.parametrize("world,T,dim", [(2, 64, 4096), (4, 64, 512), (8, 64, 4096), (8, 5, 256),
                                         (2, 300, 1024), (4, 7, 8192)])
@pytest.mark.parametrize("oneshot", [False, True], ids=["two_phase", "one_shot"])
def test_reduce_norm_matches_reference_and_replays(world, T, dim, oneshot):
    from easy_to_hard_b200.ops import _lib
    from easy_to_hard_b200.parallel.symm import TPReduceSync
    torch.manual_seed(world * 1000 + T)
    dev = "cuda"
    syncs = TPReduceSync.emulated(T, dim, 3, world, oneshot=oneshot)
    w = (torch.randn(dim, device=dev) * 0.5 + 1).bfloat16()
    _lib.read_status()
    for use in range(3):
        point = use % 2 + 1
        parts = [(torch.randn(T, dim, device=dev) * 0.3).bfloat16() for _ in range(world)]
        hs = [torch.randn(T, dim, device=dev).bfloat16() for _ in range(world)] if use != 1 else None
        if oneshot and hs is not None:       # every rank keeps the whole residual stream
            hs = [hs[0]] * world
        for r, s in enumerate(syncs):
            s.partial_out(point, T).copy_(parts[r])
            if not oneshot:
                s.xn.zero_()
            _signal(s, point)
        outs, xns = [], []
        for r, s in enumerate(syncs):
            h_out = torch.zeros(T, dim, dtype=torch.bfloat16, device=dev)
            xn = torch.zeros(T, dim, dtype=torch.bfloat16, device=dev) if oneshot else None
            s.reduce_norm(point, None if hs is None else hs[r], h_out, w, 1e-5, T, wait_b=False,
                          xn_out=xn)
            outs.append(h_out)
            xns.append(xn if oneshot else s.xn[:T])
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        h_ref, xn_ref = _ref(hs, parts, w, 1e-5, world)
        for r, s in enumerate(syncs):
            r0, r1 = (0, T) if oneshot else (r * T // world, (r + 1) * T // world)
            assert torch.equal(outs[r][r0:r1], h_ref[r0:r1]), (use, r)
            # every rank holds every row, bit-identical on all ranks
            torch.testing.assert_close(xns[r].float(), xn_ref.float(), atol=2e-2, rtol=2e-2)
            assert torch.equal(xns[r], xns[0])
            n_use = {0: 1, 1: 1, 2: 2}[use]       # uses of this point so far
            assert int(s.count[point]) == n_use
            assert s.flag_b(point)[:world].tolist() == [0 if oneshot else n_use] * world
            assert s.flag_a(point)[:world].tolist() == [n_use] * world
            assert s.buf.check_canary()


def test_wait_runs_out_sets_status_and_returns():
    """A flag that nothing raises: the kernel gives up after its limit, records 105, still
    terminates, and the context stays usable."""
    from easy_to_hard_b200.ops import _lib
    from easy_to_hard_b200.parallel.symm import TPReduceSync
    syncs = TPReduceSync.emulated(8, 256, 2, 2, wait_ms=20)
    w = torch.ones(256, dtype=torch.bfloat16, device="cuda")
    h = torch.zeros(8, 256, dtype=torch.bfloat16, device="cuda")
    _lib.read_status()
    _signal(syncs[0], 0)                      # rank 1 never signals
    syncs[0].reduce_norm(0, h, h, w, 1e-5, 8, wait_b=True)
    torch.cuda.synchronize()
    assert _lib.read_status() == 105
    one = TPReduceSync.emulated(8, 256, 2, 2, wait_ms=20, oneshot=True)
    _signal(one[0], 1)
    one[0].reduce_norm(1, h, h, w, 1e-5, 8, xn_out=torch.empty_like(h))
    torch.cuda.synchronize()
    assert _lib.read_status() == 105
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    # with the status word set, later waits return at once instead of stacking time-outs
    _lib.status_word().fill_(105)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(20):
        syncs[0].reduce_norm(1, h, h, w, 1e-5, 8, wait_b=True)
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 200.0
    assert _lib.read_status() == 105


@pytest.mark.parametrize("world", [2, 8])
def test_vocab_parallel_embedding_and_logit_gather(world):
    from easy_to_hard_b200.ops import _lib
    from easy_to_hard_b200.parallel.symm import TPReduceSync
    torch.manual_seed(5)
    dev, T, dim, V = "cuda", 16, 512, 1024 if world == 2 else 8 * 126
    vs = V // world
    table = torch.randn(V, dim, device=dev).bfloat16()
    tok = torch.randint(0, V, (T,), device=dev, dtype=torch.int32)
    syncs = TPReduceSync.emulated(T, dim, 2, world, extra_bytes=T * vs * 4)
    w = torch.ones(dim, dtype=torch.bfloat16, device=dev)
    _lib.read_status()
    for r, s in enumerate(syncs):
        s.embed_partial(0, tok, table[r * vs:(r + 1) * vs].contiguous(), r * vs)
    outs = []
    for r, s in enumerate(syncs):
        h = torch.zeros(T, dim, dtype=torch.bfloat16, device=dev)
        s.reduce_norm(0, None, h, w, 1e-5, T, wait_b=False)
        outs.append(h)
    torch.cuda.synchronize()
    ref = table[tok.long()]
    for r in range(world):
        r0, r1 = r * T // world, (r + 1) * T // world
        assert torch.equal(outs[r][r0:r1], ref[r0:r1])
    # logits: every rank's fp32 shard [T, vs] -> [T, V] on every rank
    logits = torch.randn(T, V, device=dev)
    for r, s in enumerate(syncs):
        s.extra((T, vs), torch.float32).copy_(logits[:, r * vs:(r + 1) * vs])
        _signal(s, 1)
    for r, s in enumerate(syncs):
        out = torch.zeros(T, V, device=dev)
        s.gather_logits(1, T, vs, out)
        torch.cuda.synchronize()
        assert torch.equal(out, logits)
    assert _lib.read_status() == 0


def test_out_of_range_token_id_is_reported_not_dereferenced():
    from easy_to_hard_b200.ops import _lib, functional as Fn
    dev = "cuda"
    table = torch.randn(32, 256, device=dev).bfloat16()
    tok = torch.tensor([3, 31, 32, 100000, -1], device=dev, dtype=torch.int32)
    w = torch.ones(256, dtype=torch.bfloat16, device=dev)
    _lib.read_status()
    out = Fn.embedding(tok, table)
    torch.cuda.synchronize()
    assert _lib.read_status() == 106
    assert torch.equal(out[:2], table[[3, 31]]) and float(out[2:].abs().max()) == 0.0
    h = torch.empty(5, 256, dtype=torch.bfloat16, device=dev)
    x = torch.empty_like(h)
    Fn.fused_residual_rmsnorm(None, w, 1e-5, tokens=tok, emb=table, h_out=h, x_out=x)
    torch.cuda.synchronize()
    assert _lib.read_status() == 106
    assert torch.equal(h[:2], table[[3, 31]]) and float(h[2:].abs().max()) == 0.0
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0


def _signal_ptrs(ptrs, world):
    from easy_to_hard_b200.ops import _lib
    arr = (C.c_void_p * 8)()
    for r, p in enumerate(ptrs):
        arr[r] = p
    _lib.check(_lib.lib().e2h_signal_peers(arr, world, _lib.stream()), "signal")


@pytest.mark.parametrize("world,T,dim", [(2, 512, 4096), (4, 96, 512), (8, 40, 1024), (2, 7, 256)])
def test_sequence_parallel_collectives_match_reference(world, T, dim):
    """Reduce-scatter, reduce-scatter + norm + all-gather, and (norm +) all-gather by token rows,
    each twice (the flags count uses), emulated ranks on one GPU."""
    from easy_to_hard_b200.ops import _lib
    from easy_to_hard_b200.parallel.symm import SequenceParallelSync
    torch.manual_seed(world + T)
    dev = "cuda"
    syncs = SequenceParallelSync.emulated(T, dim, world)
    w = (torch.randn(dim, device=dev) * 0.5 + 1).bfloat16()
    _lib.read_status()

    def own(t, r):
        r0, n = syncs[r].rows(T)
        return t[r0:r0 + n].contiguous()

    def rms(x):
        x = x.float()
        return ((x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)).bfloat16().float()
                * w.float()).bfloat16()

    for rep in range(2):
        parts = [(torch.randn(T, dim, device=dev) * 0.3).bfloat16() for _ in range(world)]
        res = torch.randn(T, dim, device=dev).bfloat16()
        total = torch.stack([p.float() for p in parts]).sum(0).bfloat16().float()
        # --- reduce-scatter (+ residual)
        slots = []
        for r, s in enumerate(syncs):
            slot, part = s.next_partial(T)
            part.copy_(parts[r])
            slots.append(slot)
            _signal_ptrs(s.signal_ptrs(2), world)
        outs = [s.reduce(2, slots[r], own(res, r), T) for r, s in enumerate(syncs)]
        none = [None] * world
        torch.cuda.synchronize()
        want = (res.float() + total).bfloat16()
        for r in range(world):
            assert torch.equal(outs[r], own(want, r)), ("reduce", rep, r)
        # --- reduce-scatter + norm + all-gather
        for r, s in enumerate(syncs):
            slot, part = s.next_partial(T)
            part.copy_(parts[r])
            slots[r] = slot
            s.xn.zero_()
            _signal_ptrs(s.signal_ptrs(1), world)
        hs = []
        for r, s in enumerate(syncs):
            h, _ = s.reduce_norm_gather(1, slots[r], own(res, r), w, 1e-5, T, wait_b=False)
            hs.append(h)
        torch.cuda.synchronize()
        for r, s in enumerate(syncs):
            assert torch.equal(hs[r], own(want, r))
            torch.testing.assert_close(s.xn[:T].float(), rms(want).float(), atol=2e-2, rtol=2e-2)
            assert torch.equal(s.xn[:T], syncs[0].xn[:T])
        # --- all-gather of rows, plain and normalised
        for weight in (None, w):
            pt = 3 if weight is None else 0
            for s in syncs:
                s.xn.zero_()
                _signal_ptrs(s.signal_ptrs(pt), world)
            for r, s in enumerate(syncs):
                s.gather(pt, own(res, r), T, weight, 1e-5, wait_b=False, barrier=False)
            torch.cuda.synchronize()
            for s in syncs:
                if weight is None:
                    assert torch.equal(s.xn[:T], res)
                else:
                    torch.testing.assert_close(s.xn[:T].float(), rms(res).float(),
                                               atol=2e-2, rtol=2e-2)
        assert _lib.read_status() == 0
        for s in syncs:
            assert s.buf.check_canary()
            assert s.count[:4].tolist() == [rep + 1] * 4
