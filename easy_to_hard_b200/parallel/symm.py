"""Symmetric (peer-mapped) buffers for the in-kernel tensor-parallel collectives.

A ``SymmetricBuffer`` is the same allocation on every rank of a group, mapped into every peer's
address space over NVLink, so a kernel on rank r can load from / store to rank j's copy directly
(``ptrs[j]``) -- the transport of the fused GEMM + all-reduce of the decode engine:

* every rank's row-parallel GEMM writes its fp32 partial into its *own* buffer and, when its grid
  is done, bumps a flag word in every peer's buffer (one ``red.release.sys`` per peer);
* the following residual+RMSNorm kernel waits (bounded) for all flags and sums the partials
  straight out of the peers' memory with system-scope loads.

Allocation and the pointer exchange ride on ``torch.distributed._symmetric_memory``; the
kernels only see raw addresses. ``SymmetricBuffer.emulated`` builds the same structure inside one
process (n "ranks" on one GPU) for single-GPU tests, where the producers run before the consumer
in stream order so that no launch ever waits on a later one.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def peer_wait_ms() -> int:
    """Limit of one cross-rank device wait of the training kernels. Ranks of a training job can
    drift apart by seconds (data loading, first-use initialisation), not by minutes: ten
    seconds by default, ``E2H_PEER_WAIT_MS`` overrides."""
    import os
    return int(os.environ.get("E2H_PEER_WAIT_MS", "10000"))


def peer_memory_usable(group=None) -> bool:
    """True when every rank of ``group`` sits on the same host, i.e. when peer-mapped
    (symmetric) memory can reach all of them; groups that span hosts keep the NCCL collectives.
    A collective call (one small object all-gather), cached per group."""
    if not dist.is_initialized():
        return False
    key = id(group) if group is not None else 0
    hit = _PEER_OK.get(key)
    if hit is not None:
        return hit
    import socket
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
        names = [None] * dist.get_world_size(group)
        dist.all_gather_object(names, socket.gethostname(), group=group)
        ok = len(set(names)) == 1
    except Exception:  # noqa: BLE001
        ok = False
    _PEER_OK[key] = ok
    return ok


_PEER_OK: dict = {}


class SymmetricBuffer:
    GUARD = 256        # bytes of canary after the payload
    CANARY = 0xA5

    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        assert dist.is_initialized(), "SymmetricBuffer needs an initialised process group"
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        nbytes = (nbytes + 255) // 256 * 256
        # one guard block after the payload: peers write into this allocation with raw
        # pointers, so an overrun would otherwise go unnoticed (see check_canary)
        self._raw = symm_mem.empty(nbytes + self.GUARD, dtype=torch.uint8, device=dev)
        self._raw.zero_()
        self._raw[nbytes:].fill_(self.CANARY)
        self.local = self._raw[:nbytes]
        self.handle = symm_mem.rendezvous(self._raw, group)
        # the handle's addresses are those of the allocation block; the tensor may sit at an
        # offset inside it
        shift = self._raw.data_ptr() - int(self.handle.buffer_ptrs[self.rank])
        assert 0 <= shift and shift % 16 == 0
        self.ptrs: List[int] = [int(p) + shift for p in self.handle.buffer_ptrs]
        self.multicast_ptr = 0
        import os
        if os.environ.get("E2H_MULTIMEM", "1") != "0":
            try:
                mc = int(self.handle.multicast_ptr)
                self.multicast_ptr = mc + shift if mc else 0
            except Exception:  # noqa: BLE001 -- no NVSwitch multicast on this system
                self.multicast_ptr = 0
        torch.cuda.synchronize()
        dist.barrier(group)

    @classmethod
    def emulated(cls, nbytes: int, world: int, device="cuda") -> List["SymmetricBuffer"]:
        """``world`` buffers in one process; buffer r plays rank r's copy."""
        nbytes = (nbytes + 255) // 256 * 256
        raws = [torch.zeros(nbytes + cls.GUARD, dtype=torch.uint8, device=device)
                for _ in range(world)]
        for t in raws:
            t[nbytes:].fill_(cls.CANARY)
        locals_ = [t[:nbytes] for t in raws]
        out = []
        for r in range(world):
            b = cls.__new__(cls)
            b.world, b.rank, b.local, b._raw = world, r, locals_[r], raws[r]
            b.handle, b.multicast_ptr = None, 0
            b.ptrs = [t.data_ptr() for t in locals_]
            out.append(b)
        return out

    def check_canary(self) -> bool:
        """True while nothing (this rank's kernels or a peer's stores) has written past the end
        of the payload. Synchronises the device; meant for tests and post-mortems."""
        guard = self._raw[self.local.numel():]
        return bool((guard == self.CANARY).all().item())

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        """Typed view of the local copy at a byte offset."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset: offset + nbytes].view(dtype).view(*shape)

    def peer_ptr(self, rank: int, offset: int) -> int:
        return self.ptrs[rank] + offset


class RowParallelReduce:
    """Buffers and counters of the fused "row-parallel GEMM -> all-reduce -> residual + norm".

    Layout of the symmetric buffer: two slots (alternating between consecutive uses, which is
    what makes reuse safe without an extra hand-shake), each ``[max_tokens, dim]`` fp32 partial
    + ``world`` int32 flag words."""

    def __init__(self, max_tokens: int, dim: int, group=None, buf: Optional[SymmetricBuffer] = None,
                 device="cuda", dtype: torch.dtype = torch.float32):
        """``dtype``: element type of the partial sums (fp32 for the decode path, bf16 for the
        large-token training path, whose GEMM stores through its TMA epilogue)."""
        self.T, self.dim, self.dtype = max_tokens, dim, dtype
        self.part_bytes = max_tokens * dim * torch.empty((), dtype=dtype).element_size()
        self.slot_bytes = self.part_bytes + 256
        if buf is None:
            buf = SymmetricBuffer(2 * self.slot_bytes, group)
        self.buf = buf
        self.world, self.rank = buf.world, buf.rank
        dev = buf.local.device
        self.use_count = torch.zeros(2, dtype=torch.int32, device=dev)
        self.norm_ticket = torch.zeros(2, dtype=torch.int32, device=dev)
        self.gemm_ticket = torch.zeros(2, dtype=torch.int32, device=dev)
        self.next_slot = 0

    def slot(self):
        s = self.next_slot
        self.next_slot ^= 1
        return s

    def partial_out(self, slot: int, T: int) -> torch.Tensor:
        """This rank's [T, dim] partial (the GEMM writes here)."""
        return self.buf.view(slot * self.slot_bytes, (self.T, self.dim), self.dtype)[:T]

    def signal_ptrs(self, slot: int) -> List[int]:
        """Address of *this rank's* flag word inside every rank's slot."""
        off = slot * self.slot_bytes + self.part_bytes + 4 * self.rank
        return [self.buf.peer_ptr(r, off) for r in range(self.world)]

    def flags(self, slot: int) -> torch.Tensor:
        return self.buf.view(slot * self.slot_bytes + self.part_bytes, (self.world,),
                             torch.int32)

    def partial_ptrs(self, slot: int) -> List[int]:
        return [self.buf.peer_ptr(r, slot * self.slot_bytes) for r in range(self.world)]


class GradReduceScatter:
    """Buffers and counters of the fused gradient reduce-scatter of sharded data parallelism
    (``ops/csrc/comm.cu``): two alternating slots, each a flat bf16 gradient buffer of ``numel``
    elements followed by ``world`` int32 flag words, in symmetric memory."""

    def __init__(self, numel: int, group=None, buf: Optional[SymmetricBuffer] = None,
                 wait_ms: Optional[int] = None):
        wait_ms = peer_wait_ms() if wait_ms is None else wait_ms
        self.numel = (numel + 7) // 8 * 8
        self.grad_bytes = self.numel * 2
        self.slot_bytes = (self.grad_bytes + 255) // 256 * 256 + 256
        if buf is None:
            buf = SymmetricBuffer(2 * self.slot_bytes, group)
        self.buf = buf
        self.world, self.rank = buf.world, buf.rank
        dev = buf.local.device
        self.use_count = torch.zeros(2, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(2, dtype=torch.int32, device=dev)
        self.wait_ms = wait_ms
        self.next_slot = 0

    def slot(self) -> int:
        s = self.next_slot
        self.next_slot ^= 1
        return s

    def _flag_off(self, slot: int) -> int:
        return slot * self.slot_bytes + (self.grad_bytes + 255) // 256 * 256

    def grad_buffer(self, slot: int) -> torch.Tensor:
        """This rank's flat bf16 gradient buffer of ``slot`` (the weight-gradient GEMMs write
        views of it)."""
        return self.buf.view(slot * self.slot_bytes, (self.numel,), torch.bfloat16)

    def flags(self, slot: int) -> torch.Tensor:
        return self.buf.view(self._flag_off(slot), (self.world,), torch.int32)

    def signal(self, slot: int) -> None:
        """Tell every rank that this rank's buffer of ``slot`` is complete (stream-ordered after
        the kernels that wrote it)."""
        import ctypes as C
        from ..ops import _lib
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.buf.peer_ptr(r, self._flag_off(slot) + 4 * self.rank)
        _lib.check(_lib.lib().e2h_signal_peers(arr, self.world, _lib.stream()), "signal_peers")

    def reduce(self, slot: int, offset: int, n: int, out: torch.Tensor, scale: float,
               accumulate: bool) -> None:
        """out[:n] (+)= scale * sum over ranks of their buffer[offset : offset + n] (fp32 out)."""
        import ctypes as C
        from ..ops import _lib
        assert out.dtype == torch.float32 and out.is_contiguous() and n % 8 == 0 and offset % 8 == 0
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.buf.peer_ptr(r, slot * self.slot_bytes + 2 * offset)
        rc = _lib.lib().e2h_reduce_scatter_accum(
            arr, self.world, out.data_ptr(), n, float(scale), int(accumulate),
            self.flags(slot).data_ptr(), self.use_count[slot:slot + 1].data_ptr(),
            self.ticket[slot:slot + 1].data_ptr(), int(self.wait_ms),
            _lib.status_word(out.device).data_ptr(), _lib.stream())
        _lib.check(rc, "reduce_scatter_accum")


class P2PChannel:
    """Stand-alone collectives over peer memory with the flag protocol of the fused kernels
    (``ops/csrc/comm.cu``): all-gather (pull), one-shot all-reduce, reduce-scatter, two-shot
    all-reduce (reduce-scatter + all-gather) and a barrier, each wait bounded by ``wait_ms``
    (a time-out lands in the device status word, ``ops._lib.read_status``).

    Every use is ``post`` (copy the payload into this rank's slot, then raise this rank's flag
    on every peer, stream-ordered) followed by one consuming kernel that waits for all flags and
    pulls from the peers. Two slots alternate; all ranks must issue the same sequence of uses.
    The split into ``post`` / ``*_posted`` lets a single process play several ranks on one GPU
    (all posts first, then the consumers), which is how the single-GPU tests run it."""

    def __init__(self, nbytes: int, group=None, buf: Optional[SymmetricBuffer] = None,
                 wait_ms: Optional[int] = None):
        wait_ms = peer_wait_ms() if wait_ms is None else wait_ms
        self.nbytes = (nbytes + 255) // 256 * 256
        self.slot_bytes = self.nbytes + 256
        if buf is None:
            buf = SymmetricBuffer(2 * self.slot_bytes, group)
        self.buf = buf
        self.world, self.rank = buf.world, buf.rank
        dev = buf.local.device
        self.use_count = torch.zeros(2, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(2, dtype=torch.int32, device=dev)
        self.wait_ms = wait_ms
        self.next_slot = 0
        self._second: Optional["P2PChannel"] = None
        self._group = group

    # ---- building blocks
    def _flag_off(self, slot: int) -> int:
        return slot * self.slot_bytes + self.nbytes

    def flags(self, slot: int) -> torch.Tensor:
        return self.buf.view(self._flag_off(slot), (self.world,), torch.int32)

    def payload(self, slot: int, shape, dtype) -> torch.Tensor:
        return self.buf.view(slot * self.slot_bytes, shape, dtype)

    def _ptr_array(self, slot: int, byte_offset: int = 0):
        import ctypes as C
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.buf.peer_ptr(r, slot * self.slot_bytes + byte_offset)
        return arr

    def _ctl(self, slot: int):
        from ..ops import _lib
        return (self.flags(slot).data_ptr(), self.use_count[slot:slot + 1].data_ptr(),
                self.ticket[slot:slot + 1].data_ptr(), int(self.wait_ms),
                _lib.status_word(self.buf.local.device).data_ptr(), _lib.stream())

    def post(self, x: Optional[torch.Tensor]) -> int:
        """Stage ``x`` (any dtype, contiguous) in the next slot and signal every rank."""
        import ctypes as C
        from ..ops import _lib
        slot = self.next_slot
        self.next_slot ^= 1
        if x is not None:
            nb = x.numel() * x.element_size()
            assert x.is_contiguous() and nb <= self.nbytes
            self.payload(slot, tuple(x.shape), x.dtype).copy_(x)
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.buf.peer_ptr(r, self._flag_off(slot) + 4 * self.rank)
        _lib.check(_lib.lib().e2h_signal_peers(arr, self.world, _lib.stream()), "signal_peers")
        return slot

    def gather_posted(self, slot: int, like: torch.Tensor) -> torch.Tensor:
        from ..ops import _lib
        nb = like.numel() * like.element_size()
        assert nb % 16 == 0, "payloads are moved as 16-byte vectors"
        out = torch.empty((self.world,) + tuple(like.shape), dtype=like.dtype, device=like.device)
        rc = _lib.lib().e2h_p2p_all_gather(self._ptr_array(slot), self.world, out.data_ptr(), nb,
                                           *self._ctl(slot))
        _lib.check(rc, "p2p_all_gather")
        return out

    def reduce_posted(self, slot: int, offset: int, n: int, out: torch.Tensor,
                      scale: float = 1.0) -> torch.Tensor:
        """out[:n] = bf16(scale * sum over ranks of their payload[offset : offset + n])."""
        from ..ops import _lib
        assert out.dtype == torch.bfloat16 and n % 8 == 0 and offset % 8 == 0
        rc = _lib.lib().e2h_p2p_reduce_bf16(self._ptr_array(slot, 2 * offset), self.world,
                                            out.data_ptr(), n, float(scale), *self._ctl(slot))
        _lib.check(rc, "p2p_reduce_bf16")
        return out

    def wait_posted(self, slot: int) -> None:
        from ..ops import _lib
        flags, use, _, wait_ms, status, stream = self._ctl(slot)
        _lib.check(_lib.lib().e2h_wait_flags(flags, self.world, use, 1, wait_ms, status, stream),
                   "wait_flags")

    def second(self) -> "P2PChannel":
        """Channel of the second phase of a two-shot all-reduce (the reduced slices)."""
        if self._second is None:
            self._second = P2PChannel(self.nbytes // self.world + 256, self._group,
                                      wait_ms=self.wait_ms)
        return self._second

    # ---- collectives (one rank per process)
    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """[world, *x.shape]: every rank's ``x`` (same shape and dtype on all ranks)."""
        return self.gather_posted(self.post(x), x)

    def reduce_scatter(self, x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """This rank's slice (numel / world elements) of the element-wise sum of bf16 ``x``."""
        n = x.numel() // self.world
        assert x.dtype == torch.bfloat16 and x.numel() % (8 * self.world) == 0
        slot = self.post(x.reshape(-1))
        out = torch.empty(n, dtype=torch.bfloat16, device=x.device)
        return self.reduce_posted(slot, self.rank * n, n, out, scale)

    def all_reduce(self, x: torch.Tensor, algo: str = "one_shot", scale: float = 1.0) -> torch.Tensor:
        """Element-wise sum of bf16 ``x`` over the ranks. ``one_shot``: every rank pulls and adds
        all payloads (latency-optimal, world x traffic); ``two_shot``: each rank reduces one
        slice, then the reduced slices are all-gathered (bandwidth-optimal)."""
        assert x.dtype == torch.bfloat16 and x.numel() % 8 == 0
        if algo == "one_shot" or self.world == 1:
            slot = self.post(x.reshape(-1))
            out = torch.empty_like(x)
            self.reduce_posted(slot, 0, x.numel(), out.view(-1), scale)
            return out
        assert algo == "two_shot" and x.numel() % (8 * self.world) == 0
        part = self.reduce_scatter(x, scale)
        return self.second().all_gather(part).view(x.shape)

    def barrier(self) -> None:
        self.wait_posted(self.post(None))


class TPReduceSync:
    """Buffers, flag words and use counters of the decode engine's fused tensor-parallel
    reductions (``ops/csrc/tp_reduce.cu``). The row-parallel GEMM of call site ``point`` writes
    its bf16 partial into ``partial_out(point)`` and raises flag A of that point on every rank;
    ``reduce_norm`` is the consumer. One symmetric allocation holds

        region 0 [T, dim] bf16 | region 1 [T, dim] bf16 | extra | flags A [points, 8] | flags B

    and the per-point use counters and tickets live in local memory. Two forms:

    ``oneshot`` (decode-sized inputs, latency-bound): both regions are partial slots, taken in
        turn by consecutive points; every rank pulls all partials with plain loads, sums them
        in rank order and writes its own local activations. One NVLink round trip per use.
    two-phase (large inputs, bandwidth-bound): region 0 is the partial, region 1 the
        activation buffer ``xn`` that the owners of the token rows write into on every rank
        (reduce-scatter + all-gather by rows). With an NVSwitch multicast mapping of the
        allocation the sum is one ``multimem.ld_reduce`` and the write-out one ``multimem.st``
        per 16 bytes.

    All ranks must issue the same sequence of uses. ``emulated`` builds the ``world`` ranks'
    objects inside one process for single-GPU tests."""

    def __init__(self, max_tokens: int, dim: int, n_points: int, group=None, extra_bytes: int = 0,
                 multicast: bool = True, wait_ms: int = 5000, oneshot: Optional[bool] = None,
                 buf: Optional[SymmetricBuffer] = None, world: Optional[int] = None):
        self.T, self.dim, self.n_points = max_tokens, dim, n_points
        self.part_bytes = (max_tokens * dim * 2 + 255) // 256 * 256
        self.extra_off = 2 * self.part_bytes
        self.extra_bytes = (extra_bytes + 255) // 256 * 256
        self.flag_a_off = self.extra_off + self.extra_bytes
        self.flag_b_off = self.flag_a_off + n_points * 32
        total = self.flag_b_off + n_points * 32
        if buf is None:
            buf = SymmetricBuffer(total, group)
        self.buf = buf
        self.world, self.rank = buf.world, buf.rank
        if oneshot is None:      # every rank pulls world x the partial: fine while that is small
            oneshot = self.world * self.part_bytes <= self.ONESHOT_MAX_BYTES
        self.oneshot = bool(oneshot)
        dev = buf.local.device
        self.count = torch.zeros(n_points, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(n_points, dtype=torch.int32, device=dev)
        self.gemm_ticket = torch.zeros(n_points, dtype=torch.int32, device=dev)
        self.multicast = bool(multicast and buf.multicast_ptr)
        self.wait_ms = wait_ms
        self._regions = [buf.view(0, (max_tokens, dim), torch.bfloat16),
                         buf.view(self.part_bytes, (max_tokens, dim), torch.bfloat16)]
        self.xn = None if self.oneshot else self._regions[1]

    ONESHOT_MAX_BYTES = 16 << 20

    @classmethod
    def emulated(cls, max_tokens: int, dim: int, n_points: int, world: int, extra_bytes: int = 0,
                 wait_ms: int = 50, oneshot: bool = False, device="cuda") -> List["TPReduceSync"]:
        part = (max_tokens * dim * 2 + 255) // 256 * 256
        total = 2 * part + (extra_bytes + 255) // 256 * 256 + 2 * n_points * 32
        bufs = SymmetricBuffer.emulated(total, world, device)
        return [cls(max_tokens, dim, n_points, extra_bytes=extra_bytes, multicast=False,
                    wait_ms=wait_ms, oneshot=oneshot, buf=b) for b in bufs]

    # ---- addresses
    def _ptrs(self, offset: int):
        import ctypes as C
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.buf.peer_ptr(r, offset)
        return arr

    def _region(self, point: int) -> int:
        return (point & 1) if self.oneshot else 0

    def partial_out(self, point: int, T: int) -> torch.Tensor:
        """Where this rank's producer of ``point`` writes its [T, dim] bf16 partial."""
        return self._regions[self._region(point)][:T]

    def flag_a_remote(self, point: int) -> List[int]:
        """Address of this rank's flag-A word of ``point`` in every rank's buffer (what a
        producer bumps when its partial is complete)."""
        off = self.flag_a_off + point * 32 + 4 * self.rank
        return [self.buf.peer_ptr(r, off) for r in range(self.world)]

    def flag_a_signal(self, point: int):
        """What a producer GEMM takes as ``signal=``: with a multicast mapping the one address
        through which a single ``multimem.red`` raises this rank's flag-A word on every rank
        (the per-rank adds of ``flag_a_remote`` cost a microsecond each at eight ranks),
        otherwise the list of per-rank addresses."""
        import os
        if self.buf.multicast_ptr and self.world > 1 and \
                os.environ.get("E2H_MULTIMEM_SIGNAL", "1") != "0":
            from ..ops.gemm import MulticastSignal
            return MulticastSignal(self.buf.multicast_ptr + self.flag_a_off + point * 32
                                   + 4 * self.rank)
        return self.flag_a_remote(point)

    def flag_a(self, point: int) -> torch.Tensor:
        return self.buf.view(self.flag_a_off + point * 32, (8,), torch.int32)

    def flag_b(self, point: int) -> torch.Tensor:
        return self.buf.view(self.flag_b_off + point * 32, (8,), torch.int32)

    def extra(self, shape, dtype) -> torch.Tensor:
        return self.buf.view(self.extra_off, shape, dtype)

    def extra_ptrs(self):
        return self._ptrs(self.extra_off)

    # ---- kernels
    def reduce_norm(self, point: int, h_in: Optional[torch.Tensor], h_out: torch.Tensor,
                    weight: torch.Tensor, eps: float, T: int, wait_b: bool = True,
                    xn_out: Optional[torch.Tensor] = None) -> None:
        """h_out = h_in + sum of all ranks' partials of ``point``; activations = rmsnorm(h_out)
        * weight. One-shot form: all rows, activations into the local ``xn_out``. Two-phase
        form: the rows this rank owns, written into every rank's ``xn``; returns once (on the
        stream) every rank's rows have arrived in the local ``xn`` unless ``wait_b`` is off
        (single-process emulation, where the other ranks' kernels only run later)."""
        import ctypes as C
        from ..ops import _lib
        assert T <= self.T and h_out.dtype == torch.bfloat16 and h_out.stride(0) == self.dim
        mc = 0
        parts = self._ptrs(self._region(point) * self.part_bytes)
        fb = None
        if self.oneshot:
            assert xn_out is not None and xn_out.stride(0) == self.dim
            xn = (C.c_void_p * 8)()
            xn[0] = xn_out.data_ptr()
            if self.multicast:      # one multimem.ld_reduce per 16 bytes instead of n peer loads
                mc = 1
                parts[0] = self.buf.multicast_ptr + self._region(point) * self.part_bytes
        else:
            xn = self._ptrs(self.part_bytes)
            fb = self._ptrs(self.flag_b_off + point * 32 + 4 * self.rank)
            if self.multicast:
                mc = 3
                parts[0] = self.buf.multicast_ptr
                xn[0] = self.buf.multicast_ptr + self.part_bytes
        rc = _lib.lib().e2h_tp_reduce_norm(
            _lib.ptr(h_in), h_out.data_ptr(), weight.data_ptr(), parts, xn, fb,
            self.flag_a(point).data_ptr(), self.flag_b(point).data_ptr(),
            self.count[point:point + 1].data_ptr(), self.ticket[point:point + 1].data_ptr(),
            self.world, self.rank, T, self.dim, float(eps), mc, int(wait_b), int(self.oneshot),
            int(self.wait_ms), _lib.status_word(h_out.device).data_ptr(), _lib.stream())
        _lib.check(rc, "tp_reduce_norm")

    def check_multimem_consistency(self, group=None, trials: int = 16) -> bool:
        """One-shot form with ``multimem.ld_reduce``: every rank asks the switch for the sum of
        the same addresses on its own, and the ranks only stay in lock step if they all get the
        same bits. This runs the reduce on random partials and compares the results of all ranks
        bit for bit; on any difference the multicast form is switched off for this object (the
        plain loads sum in rank order and are identical by construction). Collective; uses the
        last call site, whose counters advance by ``trials`` on every rank."""
        if not (self.oneshot and self.multicast and self.world > 1):
            return True
        dev = self.buf.local.device
        point = self.n_points - 1
        T = min(self.T, 64)
        g = torch.Generator(device=dev).manual_seed(1000 + self.rank)
        w = torch.ones(self.dim, dtype=torch.bfloat16, device=dev)
        h = torch.zeros(T, self.dim, dtype=torch.bfloat16, device=dev)
        xn = torch.empty(T, self.dim, dtype=torch.bfloat16, device=dev)
        same = True
        import ctypes as C
        from ..ops import _lib
        for _ in range(trials):
            part = self.partial_out(point, T)
            part.copy_((torch.randn(T, self.dim, device=dev, generator=g) * 3).to(torch.bfloat16))
            arr = (C.c_void_p * 8)()
            for r, p in enumerate(self.flag_a_remote(point)):
                arr[r] = p
            _lib.check(_lib.lib().e2h_signal_peers(arr, self.world, _lib.stream()), "signal")
            out = torch.empty(T, self.dim, dtype=torch.bfloat16, device=dev)
            self.reduce_norm(point, h, out, w, 1e-5, T, xn_out=xn)
            every = [torch.empty_like(out) for _ in range(self.world)]
            dist.all_gather(every, out, group=group)
            same = same and all(torch.equal(e, every[0]) for e in every)
            dist.barrier(group)      # nobody overwrites its partial while a peer still reads it
        flag = torch.tensor([int(same)], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        same = bool(flag.item())
        if not same:
            self.multicast = False
        return same

    def embed_partial(self, point: int, tokens: torch.Tensor, table: torch.Tensor, v0: int) -> None:
        """partial[t] = table[tokens[t] - v0] for ids this rank's vocabulary shard holds, zeros
        otherwise; raises flag A of ``point`` on every rank."""
        import ctypes as C
        from ..ops import _lib
        T = tokens.numel()
        assert T <= self.T and tokens.dtype == torch.int32 and table.shape[1] == self.dim
        fa = (C.c_void_p * 8)()
        sig = self.flag_a_signal(point)
        if isinstance(sig, list):
            n_sig = self.world
            for r, p in enumerate(sig):
                fa[r] = p
        else:                       # one multimem.red on the flag's multicast address
            n_sig = -1
            fa[0] = sig.address
        rc = _lib.lib().e2h_tp_embed_partial(
            tokens.data_ptr(), table.data_ptr(), int(v0), table.shape[0],
            self.partial_out(point, T).data_ptr(), T, self.dim, fa, n_sig,
            self.gemm_ticket[point:point + 1].data_ptr(), _lib.stream())
        _lib.check(rc, "tp_embed_partial")

    def gather_logits(self, point: int, B: int, vs: int, out: torch.Tensor) -> None:
        """out[b, r * vs:(r + 1) * vs] = rank r's fp32 shard [B, vs] (in ``extra``), for all r."""
        from ..ops import _lib
        assert out.dtype == torch.float32 and out.shape[1] >= self.world * vs
        rc = _lib.lib().e2h_tp_gather_logits(
            self.extra_ptrs(), self.world, B, vs, out.data_ptr(), out.stride(0),
            self.flag_a(point).data_ptr(), self.count[point:point + 1].data_ptr(),
            self.ticket[point:point + 1].data_ptr(), int(self.wait_ms),
            _lib.status_word(out.device).data_ptr(), _lib.stream())
        _lib.check(rc, "tp_gather_logits")


class SequenceParallelSync:
    """The sequence-parallel collectives of training as peer-memory kernels (``e2h_tp_rows`` in
    ``ops/csrc/tp_reduce.cu``) for activations of ``[T, dim]`` token rows, rank r owning rows
    ``[r*T/n, (r+1)*T/n)`` (the reference's ``_gather_along_first_dim`` /
    ``_reduce_scatter_along_first_dim``, models/tp.py:713-777, on its batch-major layout).

    One symmetric allocation holds two partial slots (the row-parallel GEMMs write them in turn
    and raise flag A of the call site on every rank), one gathered-activation buffer ``xn`` and
    the flag words of ``n_points`` call sites. A call site must always be used the same way
    (its flags count its uses); all ranks issue the same sequence of calls.

    * ``reduce(point, slot, residual)``: this rank's rows of the sum of all ranks' partials
      (+ residual): the reduce-scatter after a row-parallel GEMM.
    * ``reduce_norm_gather(point, slot, residual, weight)``: the same rows, plus their RMSNorm
      written into every rank's ``xn``: reduce-scatter, norm and the next all-gather in one pass.
    * ``gather(point, rows, weight=None)``: all-gather of this rank's rows (optionally of their
      RMSNorm) into every rank's ``xn``. Nothing before it on the peers orders them against this
      rank's earlier readers of ``xn``, so the kernel opens with a flag barrier.

    ``xn`` is overwritten by the next gathering call: copy what must live longer. With an
    NVSwitch multicast mapping the sum is ``multimem.ld_reduce`` and the write-out
    ``multimem.st``. ``emulated`` builds the ranks of one group inside a process (tests)."""

    def __init__(self, max_tokens: int, dim: int, n_points: int = 8, group=None,
                 multicast: bool = True, wait_ms: Optional[int] = None,
                 buf: Optional[SymmetricBuffer] = None):
        self.T, self.dim, self.n_points = max_tokens, dim, n_points
        self.part_bytes = (max_tokens * dim * 2 + 255) // 256 * 256
        self.xn_off = 2 * self.part_bytes
        self.flag_a_off = 3 * self.part_bytes
        self.flag_b_off = self.flag_a_off + n_points * 32
        total = self.flag_b_off + n_points * 32
        if buf is None:
            buf = SymmetricBuffer(total, group)
        self.buf = buf
        self.world, self.rank = buf.world, buf.rank
        dev = buf.local.device
        self.count = torch.zeros(n_points, dtype=torch.int32, device=dev)
        self.ticket = torch.zeros(n_points, dtype=torch.int32, device=dev)
        self.gemm_ticket = torch.zeros(n_points, dtype=torch.int32, device=dev)
        self.multicast = bool(multicast and buf.multicast_ptr)
        self.wait_ms = peer_wait_ms() if wait_ms is None else wait_ms
        self.xn = buf.view(self.xn_off, (max_tokens, dim), torch.bfloat16)
        self._slots = [buf.view(i * self.part_bytes, (max_tokens, dim), torch.bfloat16)
                       for i in range(2)]
        self._next_slot = 0

    @staticmethod
    def total_bytes(max_tokens: int, dim: int, n_points: int = 8) -> int:
        return 3 * ((max_tokens * dim * 2 + 255) // 256 * 256) + 2 * n_points * 32

    @classmethod
    def emulated(cls, max_tokens: int, dim: int, world: int, n_points: int = 8,
                 wait_ms: int = 50, device="cuda") -> List["SequenceParallelSync"]:
        bufs = SymmetricBuffer.emulated(cls.total_bytes(max_tokens, dim, n_points), world, device)
        return [cls(max_tokens, dim, n_points, multicast=False, wait_ms=wait_ms, buf=b)
                for b in bufs]

    def rows(self, T: int):
        """(first row, number of rows) this rank owns of a [T, dim] tensor."""
        r0 = self.rank * T // self.world
        return r0, (self.rank + 1) * T // self.world - r0

    def _ptrs(self, offset: int):
        import ctypes as C
        arr = (C.c_void_p * 8)()
        for r in range(self.world):
            arr[r] = self.buf.peer_ptr(r, offset)
        return arr

    def next_partial(self, T: int):
        """(slot index, [T, dim] view) of the partial buffer the next row-parallel GEMM writes."""
        s = self._next_slot
        self._next_slot ^= 1
        return s, self._slots[s][:T]

    def signal_ptrs(self, point: int) -> List[int]:
        off = self.flag_a_off + point * 32 + 4 * self.rank
        return [self.buf.peer_ptr(r, off) for r in range(self.world)]

    def _run(self, ops: int, point: int, slot: int, h_in, h_out, weight, eps: float, T: int,
             wait_b: bool = True) -> None:
        from ..ops import _lib
        assert T <= self.T and 0 <= point < self.n_points
        parts = self._ptrs(slot * self.part_bytes)
        xn = self._ptrs(self.xn_off)
        mc = 0
        if self.multicast:
            mc = 3
            parts[0] = self.buf.multicast_ptr + slot * self.part_bytes
            xn[0] = self.buf.multicast_ptr + self.xn_off
        fa = self._ptrs(self.flag_a_off + point * 32 + 4 * self.rank)
        fb = self._ptrs(self.flag_b_off + point * 32 + 4 * self.rank)
        dev = self.buf.local.device
        rc = _lib.lib().e2h_tp_rows(
            ops | 16, _lib.ptr(h_in), _lib.ptr(h_out), _lib.ptr(weight), parts, xn, fa, fb,
            self.buf.view(self.flag_a_off + point * 32, (8,), torch.int32).data_ptr(),
            self.buf.view(self.flag_b_off + point * 32, (8,), torch.int32).data_ptr(),
            self.count[point:point + 1].data_ptr(), self.ticket[point:point + 1].data_ptr(),
            self.world, self.rank, T, self.dim, float(eps), mc, int(wait_b), int(self.wait_ms),
            _lib.status_word(dev).data_ptr(), _lib.stream())
        _lib.check(rc, "tp_rows")

    def _own(self, t: Optional[torch.Tensor], T: int):
        if t is not None:
            want = (self.rows(T)[1], self.dim)
            assert t.dtype == torch.bfloat16 and t.is_contiguous() and tuple(t.shape) == want, \
                (tuple(t.shape), want)
        return t

    def reduce(self, point: int, slot: int, residual: Optional[torch.Tensor], T: int,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """[T/n, dim]: this rank's rows of (sum of the partials in ``slot``) + residual."""
        if out is None:
            out = torch.empty(self.rows(T)[1], self.dim, dtype=torch.bfloat16,
                              device=self.buf.local.device)
        self._run(1, point, slot, self._own(residual, T), self._own(out, T), None, 0.0, T)
        return out

    def reduce_norm_gather(self, point: int, slot: int, residual: Optional[torch.Tensor],
                           weight: torch.Tensor, eps: float, T: int, wait_b: bool = True):
        """(h [T/n, dim] = reduce(...), xn [T, dim] view = every rank's rmsnorm(h) * weight)."""
        h = torch.empty(self.rows(T)[1], self.dim, dtype=torch.bfloat16,
                        device=self.buf.local.device)
        self._run(1 | 2 | 4, point, slot, self._own(residual, T), h, weight, eps, T, wait_b)
        return h, self.xn[:T]

    def gather(self, point: int, rows: torch.Tensor, T: int,
               weight: Optional[torch.Tensor] = None, eps: float = 0.0,
               wait_b: bool = True, barrier: bool = True) -> torch.Tensor:
        """[T, dim] view of ``xn``: every rank's ``rows`` (their RMSNorm when ``weight`` is
        given). ``barrier=False`` leaves raising flag A of ``point`` to the caller (the
        single-process emulation raises all ranks' flags before the first kernel runs)."""
        ops = 4 | (8 if barrier else 0) | (2 if weight is not None else 0)
        self._run(ops, point, 0, self._own(rows, T), None, weight, eps, T, wait_b)
        return self.xn[:T]
