"""Python front-end of the tcgen05 flash-attention kernels (csrc/flash_attn.cu)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib


def _strides_bshd(t: torch.Tensor):
    """(batch, seq, head) element strides of a [B, S, H, D] view with contiguous D."""
    assert t.dim() == 4 and t.stride(3) == 1
    return t.stride(0), t.stride(1), t.stride(2)


def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              left_pad: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              return_lse: bool = False):
    """Causal attention. q [B, Sq, H, D], k / v [B, Sk, Hkv, D] (any strides with contiguous D,
    k and v sharing theirs), query i aligned to key i + Sk - Sq; keys before ``left_pad[b]`` are
    hidden (the diagonal always stays visible). Returns out [B, Sq, H, D] (+ lse [B, H, Sq])."""
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    assert k.stride() == v.stride() and q.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(B, Sq, H, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device) if return_lse else None
    qs, ks, os_ = _strides_bshd(q), _strides_bshd(k), _strides_bshd(out)
    rc = _lib.lib().e2h_flash_fwd(
        q.data_ptr(), qs[0], qs[1], qs[2], k.data_ptr(), v.data_ptr(), ks[0], ks[1], ks[2],
        out.data_ptr(), os_[0], os_[1], os_[2], _lib.ptr(lse), _lib.ptr(left_pad), B, H, Hkv, Sq,
        Sk, D, 1.0 / math.sqrt(D), _lib.status_word(q.device).data_ptr(), _lib.stream())
    _lib.check(rc, "flash_fwd")
    return (out, lse) if return_lse else out


def flash_fwd_cache(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                    left_pad: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """Prefill attention against the static cache: q [B, S, H, D]; caches
    [max_batch, Hkv, Smax, D], rows 0..S-1 live; out [B, S, H*D]."""
    B, S, H, D = q.shape
    k = kcache[:B, :, :S].transpose(1, 2)   # [B, S, Hkv, D] view
    v = vcache[:B, :, :S].transpose(1, 2)
    flash_fwd(q, k, v, left_pad, out=out.view(B, S, H, D))
    return out


def flash_bwd(q, k, v, o, d_o, lse, left_pad: Optional[torch.Tensor] = None, dq=None, dk=None,
              dv=None):
    """Gradients (dq, dk, dv) of ``flash_fwd``. The outputs share the strides of q / k / v, so
    they may be passed in as views of one fused ``dqkv`` buffer."""
    B, Sq, H, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    assert k.stride() == v.stride()
    d_o = d_o if d_o.stride(3) == 1 else d_o.contiguous()
    def like(t):
        return torch.empty_like(t) if t.is_contiguous() else torch.empty_strided(
            t.shape, t.stride(), dtype=t.dtype, device=t.device)
    dq = like(q) if dq is None else dq
    dk = like(k) if dk is None else dk
    dv = like(v) if dv is None else dv
    assert dq.stride() == q.stride() and dk.stride() == k.stride() == dv.stride()
    delta = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device)
    qs, ks, os_, ds = (_strides_bshd(t) for t in (q, k, o, d_o))
    rc = _lib.lib().e2h_flash_bwd(
        q.data_ptr(), qs[0], qs[1], qs[2], k.data_ptr(), v.data_ptr(), ks[0], ks[1], ks[2],
        o.data_ptr(), os_[0], os_[1], os_[2], d_o.data_ptr(), ds[0], ds[1], ds[2],
        lse.data_ptr(), delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
        _lib.ptr(left_pad), B, H, Hkv, Sq, Sk, D, 1.0 / math.sqrt(D),
        _lib.status_word(q.device).data_ptr(), _lib.stream())
    _lib.check(rc, "flash_bwd")
    return dq, dk, dv


class FlashAttnFunc(torch.autograd.Function):
    """Causal attention with the tcgen05 kernels in both directions."""

    @staticmethod
    def forward(ctx, q, k, v):
        q, k, v = (t if t.stride(3) == 1 else t.contiguous() for t in (q, k, v))
        if k.stride() != v.stride():
            k, v = k.contiguous(), v.contiguous()
        out, lse = flash_fwd(q, k, v, None, return_lse=True)
        ctx.save_for_backward(q, k, v, out, lse)
        return out

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, out, lse = ctx.saved_tensors
        return flash_bwd(q, k, v, out, d_o, lse)


def causal_attention(q, k, v):
    """q [B, S, H, D], k / v [B, S, Hkv, D] -> [B, S, H, D]; differentiable."""
    return FlashAttnFunc.apply(q, k, v)
