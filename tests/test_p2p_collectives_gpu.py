"""Stand-alone peer-memory collectives (ops/csrc/comm.cu, parallel/symm.P2PChannel) on one GPU:
``world`` emulated ranks post first and consume afterwards, so no launch waits on a later one.
A wait whose flag nobody raises must time out into the status word and leave the context usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _channels(world, nbytes):
    from easy_to_hard_b200.parallel.symm import P2PChannel, SymmetricBuffer
    slot_bytes = (nbytes + 255) // 256 * 256 + 256
    bufs = SymmetricBuffer.emulated(2 * slot_bytes, world)
    return [P2PChannel(nbytes, buf=b, wait_ms=2000) for b in bufs]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_gather_and_one_shot_all_reduce(world):
    from easy_to_hard_b200.ops import _lib
    n = 4096 + 64
    ch = _channels(world, n * 2)
    xs = [torch.randn(n, device="cuda").bfloat16() for _ in range(world)]
    for rep in range(3):                                   # slots alternate and are reused
        slots = [c.post(x) for c, x in zip(ch, xs)]
        for c in ch:
            got = c.gather_posted(slots[c.rank], xs[0])
            assert torch.equal(got, torch.stack(xs))
        slots = [c.post(x) for c, x in zip(ch, xs)]
        want = torch.stack(xs).float().sum(0)
        outs = []
        for c in ch:
            out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
            c.reduce_posted(slots[c.rank], 0, n, out, 1.0)
            outs.append(out)
        assert all(torch.equal(o, outs[0]) for o in outs)  # same order of additions everywhere
        assert float((outs[0].float() - want).abs().max()) <= 0.02 * float(want.abs().max())
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert all(c.buf.check_canary() for c in ch)            # nothing wrote past a payload
    ch[0].buf._raw[-1] = 0                                  # and the check does see an overrun
    assert not ch[0].buf.check_canary()


def test_reduce_scatter_slices_and_two_shot():
    from easy_to_hard_b200.ops import _lib
    world, n = 4, 8192
    ch = _channels(world, n * 2)
    ch2 = _channels(world, n * 2 // world)
    xs = [torch.randn(n, device="cuda").bfloat16() for _ in range(world)]
    want = torch.stack(xs).float().sum(0)
    slots = [c.post(x) for c, x in zip(ch, xs)]
    parts = []
    for c in ch:
        out = torch.empty(n // world, dtype=torch.bfloat16, device="cuda")
        parts.append(c.reduce_posted(slots[c.rank], c.rank * (n // world), n // world, out, 0.5))
    got = torch.cat(parts).float()
    assert float((got - 0.5 * want).abs().max()) <= 0.02 * float(want.abs().max())
    # second shot: all-gather of the reduced slices
    slots2 = [c.post(p) for c, p in zip(ch2, parts)]
    for c in ch2:
        full = c.gather_posted(slots2[c.rank], parts[0]).view(-1)
        assert torch.equal(full, torch.cat(parts))
    torch.cuda.synchronize()
    assert _lib.read_status() == 0


def test_barrier_and_a_wait_that_runs_out():
    from easy_to_hard_b200.ops import _lib
    ch = _channels(2, 256)
    slots = [c.post(None) for c in ch]
    for c in ch:
        c.wait_posted(slots[c.rank])
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    assert [int(c.use_count[slots[c.rank]]) for c in ch] == [1, 1]
    # only rank 0 posts: rank 1's flag on rank 0 never rises -> bounded wait, status code, no hang
    ch[0].wait_ms = 20
    s0 = ch[0].post(None)
    ch[0].wait_posted(s0)
    torch.cuda.synchronize()
    assert _lib.read_status() != 0
    x = torch.ones(8, device="cuda")
    assert float((x + 1).sum()) == 16.0                    # the context still works


@pytest.mark.parametrize("dp,rows_src,pitch,row0,col0,rows,cols", [
    (1, 64, 256, 0, 0, 64, 256), (2, 96, 512, 32, 0, 32, 512), (4, 128, 1024, 0, 256, 128, 256),
    (8, 344, 256, 86, 0, 86, 256), (4, 256, 688 * 2, 0, 344, 256, 344 - 344 % 8)])
def test_relayout_pull_kernel_matches_slicing(dp, rows_src, pitch, row0, col0, rows, cols):
    """The weight re-layout kernel (training shards -> rollout shard) with the data-parallel
    shards of one flat parameter buffer as separate allocations of one GPU: the pulled block
    equals the slice of the unsharded matrix."""
    import ctypes as C
    from easy_to_hard_b200.ops import _lib
    torch.manual_seed(dp + rows)
    flat0 = 1024                                  # the tensor starts inside the flat buffer
    total = flat0 + rows_src * pitch + 512
    shard = -(-total // dp // 8) * 8
    flat = torch.randn(shard * dp, device="cuda").bfloat16()
    unit_off = 256                                # byte offset of the unit inside each buffer
    bufs = [torch.zeros(unit_off // 2 + shard, dtype=torch.bfloat16, device="cuda")
            for _ in range(dp)]
    for d in range(dp):
        bufs[d][unit_off // 2:] = flat[d * shard:(d + 1) * shard]
    arr = (C.c_void_p * 8)()
    for d in range(dp):
        arr[d] = bufs[d].data_ptr()
    dst = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
    rc = _lib.lib().e2h_relayout_pull(arr, dp, unit_off, shard, flat0, pitch, row0, col0, rows,
                                      cols, dst.data_ptr(), _lib.stream())
    assert rc == 0
    torch.cuda.synchronize()
    want = flat[flat0:flat0 + rows_src * pitch].view(rows_src, pitch)[row0:row0 + rows,
                                                                     col0:col0 + cols]
    assert torch.equal(dst, want)
    # a block that leaves the source, or sizes that are not multiples of 8, are refused
    assert _lib.lib().e2h_relayout_pull(arr, dp, unit_off, shard, flat0, pitch, row0, col0,
                                        rows, pitch + 8, dst.data_ptr(), _lib.stream()) == -1
    assert _lib.lib().e2h_relayout_pull(arr, dp, unit_off, shard, flat0 + 4, pitch, row0, col0,
                                        rows, cols, dst.data_ptr(), _lib.stream()) == -1
