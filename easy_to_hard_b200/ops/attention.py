"""Attention front-ends: causal flash attention (training / scoring) and the left-pad-aware
prefill attention of batched generation."""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib, reference


def prefill_mask(S: int, left_pad: Optional[torch.Tensor], device) -> torch.Tensor:
    """mask[b, 1, i, j] = (j <= i and j >= left_pad[b]) or j == i  (True = attend)."""
    i = torch.arange(S, device=device)
    causal = i[None, :] <= i[:, None]
    if left_pad is None:
        return causal[None, None]
    ok = causal[None] & (i[None, None, :] >= left_pad[:, None, None].to(device))
    return (ok | torch.eye(S, dtype=torch.bool, device=device)[None])[:, None]


def prefill_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      left_pad: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """q [B, S, H, D] (already rotated) against cache rows 0..S-1; out [B, S, H*D]."""
    B, S, H, D = q.shape
    lib = _lib.lib() if q.is_cuda else None
    if lib is not None and hasattr(lib, "e2h_flash_fwd"):
        from . import flash
        return flash.flash_fwd_cache(q, kcache, vcache, left_pad, out)
    k = kcache[:B, :, :S]
    v = vcache[:B, :, :S]
    o = reference.attention(q.transpose(1, 2), k, v, prefill_mask(S, left_pad, q.device))
    out.copy_(o.transpose(1, 2).reshape(B, S, H * D))
    return out
