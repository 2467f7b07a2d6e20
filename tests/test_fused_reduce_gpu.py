"""Fused row-parallel GEMM -> all-reduce -> residual + RMSNorm protocol, emulated on one GPU:
the "ranks" are buffers of one process and every producer runs before any consumer in stream
order, so no launch waits on a later one."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,T", [(2, 64), (4, 64), (8, 64), (2, 512), (4, 384)])
def test_row_parallel_reduce_emulated(world, T):
    from easy_to_hard_b200.ops import _lib, functional as Fn, gemm, reference
    from easy_to_hard_b200.parallel.symm import RowParallelReduce, SymmetricBuffer
    torch.manual_seed(0)
    dim, K = 1024, 512 * world   # T >= 256 takes the vectorised consumer kernel
    g = torch.Generator(device="cuda").manual_seed(1)
    x = (torch.randn(T, K, generator=g, device="cuda")).bfloat16()
    w = (torch.randn(dim, K, generator=g, device="cuda") / math.sqrt(K)).bfloat16()
    h = torch.randn(T, dim, generator=g, device="cuda").bfloat16()
    nw = torch.randn(dim, generator=g, device="cuda").bfloat16()
    proto = RowParallelReduce.__new__(RowParallelReduce)
    slot_bytes = T * dim * 4 + 256
    bufs = SymmetricBuffer.emulated(2 * slot_bytes, world)
    ranks = [RowParallelReduce(T, dim, buf=b) for b in bufs]
    ks = K // world
    for use in range(3):  # three uses: both slots and a reuse
        outs = []
        slots = [r.slot() for r in ranks]
        assert len(set(slots)) == 1
        s = slots[0]
        for r, rp in enumerate(ranks):   # producers
            gemm.linear(x[:, r * ks:(r + 1) * ks].contiguous(),
                        w[:, r * ks:(r + 1) * ks].contiguous(), out=rp.partial_out(s, T),
                        signal=rp.signal_ptrs(s), ticket=rp.gemm_ticket[s:s + 1])
        for r, rp in enumerate(ranks):   # consumers
            h_out, x_out = torch.empty_like(h), torch.empty_like(h)
            Fn.fused_residual_rmsnorm(h, nw, 1e-5, partials=rp.partial_ptrs(s), h_out=h_out,
                                      x_out=x_out, flags=rp.flags(s),
                                      use_count=rp.use_count[s:s + 1],
                                      ticket=rp.norm_ticket[s:s + 1], T=T, dim=dim)
            outs.append((h_out, x_out))
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        want_h = (h.float() + (x.float() @ w.float().T).bfloat16().float()).bfloat16()
        want_x = reference.rmsnorm(want_h, nw, 1e-5)
        for h_out, x_out in outs:
            assert torch.allclose(h_out.float(), want_h.float(), rtol=2e-2, atol=6e-2)
            assert torch.allclose(x_out.float(), want_x.float(), rtol=3e-2, atol=8e-2)
        for rp in ranks:
            assert int(rp.flags(s).min()) == int(rp.use_count[s]) == use // 2 + 1


def test_wait_times_out_with_error_status():
    """A flag that nobody sets: the bounded wait gives up, reports a status code, and the
    context stays usable."""
    from easy_to_hard_b200.ops import _lib, functional as Fn
    from easy_to_hard_b200.parallel.symm import RowParallelReduce, SymmetricBuffer
    T, dim = 4, 256
    bufs = SymmetricBuffer.emulated(2 * (T * dim * 4 + 256), 2)
    rp = RowParallelReduce(T, dim, buf=bufs[0])
    h = torch.zeros(T, dim, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(dim, dtype=torch.bfloat16, device="cuda")
    out = torch.empty_like(h)
    Fn.fused_residual_rmsnorm(h, w, 1e-5, partials=rp.partial_ptrs(0), h_out=out, x_out=out,
                              flags=rp.flags(0), use_count=rp.use_count[0:1],
                              ticket=rp.norm_ticket[0:1], T=T, dim=dim)
    torch.cuda.synchronize()
    assert _lib.read_status() == 105  # kStatusTimeoutFlag
    assert _lib.read_status() == 0    # cleared; the device still works
    assert torch.ones(2, device="cuda").sum().item() == 2


@pytest.mark.parametrize("world", [2, 4])
def test_gradient_reduce_scatter_emulated(world):
    """Fused reduce-scatter + cast + average + accumulate (ops/csrc/comm.cu), ranks emulated as
    buffers of one process: all producers signal before any consumer runs."""
    from easy_to_hard_b200.ops import _lib
    from easy_to_hard_b200.parallel.symm import GradReduceScatter, SymmetricBuffer
    torch.manual_seed(0)
    shard = 4096 + 8
    numel = shard * world
    proto = GradReduceScatter.__new__(GradReduceScatter)
    slot_bytes = (numel * 2 + 255) // 256 * 256 + 256
    bufs = SymmetricBuffer.emulated(2 * slot_bytes, world)
    ranks = [GradReduceScatter(numel, buf=b, wait_ms=1000) for b in bufs]
    outs = [torch.zeros(shard, device="cuda") for _ in range(world)]
    total = torch.zeros(numel, device="cuda")
    for use in range(4):                      # both slots, then both again (accumulating)
        slots = [r.slot() for r in ranks]
        s = slots[0]
        grads = [(torch.randn(numel, device="cuda") * 0.1).bfloat16() for _ in range(world)]
        for r, rs in enumerate(ranks):        # producers
            rs.grad_buffer(s).copy_(grads[r])
            rs.signal(s)
        for r, rs in enumerate(ranks):        # consumers
            rs.reduce(s, r * shard, shard, outs[r], 1.0 / world, accumulate=use > 0)
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        total += sum(g.float() for g in grads) / world
        for r in range(world):
            assert torch.allclose(outs[r], total[r * shard:(r + 1) * shard], atol=1e-5, rtol=1e-5)
        for rs in ranks:
            assert int(rs.flags(s).min()) == int(rs.use_count[s]) == use // 2 + 1
