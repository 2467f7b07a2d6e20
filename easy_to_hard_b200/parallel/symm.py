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


class SymmetricBuffer:
    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        assert dist.is_initialized(), "SymmetricBuffer needs an initialised process group"
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        nbytes = (nbytes + 255) // 256 * 256
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, group)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr)
        except Exception:  # no NVLS multicast on this system
            self.multicast_ptr = 0
        torch.cuda.synchronize()
        dist.barrier(group)

    @classmethod
    def emulated(cls, nbytes: int, world: int, device="cuda") -> List["SymmetricBuffer"]:
        """``world`` buffers in one process; buffer r plays rank r's copy."""
        nbytes = (nbytes + 255) // 256 * 256
        locals_ = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        out = []
        for r in range(world):
            b = cls.__new__(cls)
            b.world, b.rank, b.local = world, r, locals_[r]
            b.handle, b.multicast_ptr = None, 0
            b.ptrs = [t.data_ptr() for t in locals_]
            out.append(b)
        return out

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
                 wait_ms: int = 120000):
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
