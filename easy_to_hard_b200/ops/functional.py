"""Front-ends of the non-GEMM kernels. CUDA tensors run the native sm_100a kernels; CPU
tensors run the PyTorch restatements in ``reference.py`` (the oracle of the tests)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib, reference


def _s():
    return _lib.stream()


def _part_array(parts):
    """ctypes array of up to 8 device pointers from tensors / raw addresses."""
    import ctypes as C
    arr = (C.c_void_p * 8)()
    for i, t in enumerate(parts):
        arr[i] = t if isinstance(t, int) else t.data_ptr()
    return arr


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not x.is_cuda:
        return reference.rmsnorm(x, weight, eps)
    dim = x.shape[-1]
    x2 = x.reshape(-1, dim)
    assert x2.is_contiguous() and x.dtype == torch.bfloat16
    if out is None:
        out = torch.empty_like(x2)
    rc = _lib.lib().e2h_rmsnorm_fwd(x2.data_ptr(), None, None, 0, _part_array([]), 0,
                                    weight.data_ptr(), None, out.data_ptr(), None, x2.shape[0],
                                    dim, eps, None, None, None,
                                    _lib.status_word(x.device).data_ptr(), _s())
    _lib.check(rc, "rmsnorm_fwd")
    return out.view(x.shape)


def fused_residual_rmsnorm(h: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                           *, partials=None, tokens: Optional[torch.Tensor] = None,
                           emb: Optional[torch.Tensor] = None,
                           h_out: Optional[torch.Tensor] = None,
                           x_out: Optional[torch.Tensor] = None,
                           flags: Optional[torch.Tensor] = None,
                           use_count: Optional[torch.Tensor] = None,
                           ticket: Optional[torch.Tensor] = None, T: Optional[int] = None,
                           dim: Optional[int] = None):
    """h' = (h | emb[tokens]) + sum_i partials[i];  x = rmsnorm(h') * weight.

    ``partials`` is an fp32 tensor [n, T, dim] or a list of n fp32 [T, dim] tensors / raw device
    addresses (a tensor-parallel peer's buffer, read over NVLink). With ``flags`` (int32 [n],
    local) the kernel first waits, bounded, until every rank has bumped its flag for this use
    (``use_count`` and ``ticket`` are the device-side counters of the protocol)."""
    ref = tokens if tokens is not None else (h if h is not None else x_out)
    T = T if T is not None else ref.shape[0]
    if dim is None:
        dim = (emb if tokens is not None else (h if h is not None else x_out)).shape[-1]
    if partials is None:
        parts = []
    elif torch.is_tensor(partials):
        parts = [partials[i] for i in range(partials.shape[0])]
    else:
        parts = list(partials)
    dev = ref.device
    rc = _lib.lib().e2h_rmsnorm_fwd(
        _lib.ptr(h) if tokens is None else None, _lib.ptr(tokens), _lib.ptr(emb),
        0 if emb is None else emb.shape[0], _part_array(parts), len(parts), _lib.ptr(weight), _lib.ptr(h_out), _lib.ptr(x_out), None,
        T, dim, eps, _lib.ptr(flags), _lib.ptr(use_count), _lib.ptr(ticket),
        _lib.status_word(dev).data_ptr(), _s())
    _lib.check(rc, "rmsnorm_fwd")
    return h_out, x_out


def reduce_residual_norm_bf16(h: torch.Tensor, weight: Optional[torch.Tensor], eps: float, *,
                              partials, h_out: torch.Tensor,
                              x_out: Optional[torch.Tensor] = None, flags=None, use_count=None,
                              ticket=None):
    """h_out = h + sum of bf16 [T, dim] partials given by raw device addresses (this rank's and
    its tensor-parallel peers' symmetric buffers); x_out = rmsnorm(h_out) * weight when asked.
    Large-token (T >= 1) form of ``fused_residual_rmsnorm`` with the same flag protocol."""
    T, dim = h.shape
    parts = list(partials)
    rc = _lib.lib().e2h_reduce_residual_norm_bf16(
        h.data_ptr(), _part_array(parts), len(parts), _lib.ptr(weight), h_out.data_ptr(),
        _lib.ptr(x_out), T, dim, eps, _lib.ptr(flags), _lib.ptr(use_count), _lib.ptr(ticket),
        _lib.status_word(h.device).data_ptr(), _s())
    _lib.check(rc, "reduce_residual_norm_bf16")
    return h_out, x_out


def rmsnorm_bwd(x, dy, weight, eps, dres=None):
    dim = x.shape[-1]
    x2, dy2 = x.reshape(-1, dim), dy.reshape(-1, dim)
    dx = torch.empty_like(x2)
    rc = _lib.lib().e2h_rmsnorm_bwd(x2.data_ptr(), dy2.data_ptr(), weight.data_ptr(),
                                    _lib.ptr(dres), dx.data_ptr(), x2.shape[0], dim, eps, _s())
    _lib.check(rc, "rmsnorm_bwd")
    return dx.view(x.shape)


def embedding(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not table.is_cuda:
        return torch.nn.functional.embedding(tokens.long(), table)
    tk = tokens.reshape(-1).to(torch.int32)
    out = torch.empty(tk.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    _lib.check(_lib.lib().e2h_embedding(tk.data_ptr(), table.data_ptr(), table.shape[0],
                                        out.data_ptr(), tk.numel(), table.shape[1],
                                        _lib.status_word(table.device).data_ptr(), _s()),
               "embedding")
    return out.view(*tokens.shape, table.shape[1])


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    if not g.is_cuda:
        return reference.swiglu(g, u)
    out = torch.empty_like(g)
    _lib.check(_lib.lib().e2h_swiglu_fwd(g.data_ptr(), u.data_ptr(), out.data_ptr(), g.numel(),
                                         _s()), "swiglu_fwd")
    return out


def swiglu_bwd(g, u, dact):
    dg, du = torch.empty_like(g), torch.empty_like(u)
    _lib.check(_lib.lib().e2h_swiglu_bwd(g.data_ptr(), u.data_ptr(), dact.data_ptr(),
                                         dg.data_ptr(), du.data_ptr(), g.numel(), _s()),
               "swiglu_bwd")
    return dg, du


def rope(x: torch.Tensor, freqs: torch.Tensor, pos: torch.Tensor, n_heads: int, head_dim: int,
         inverse: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, >= n_heads*head_dim] (row stride = x.stride(0)); rotates the first n_heads heads."""
    if out is None:
        out = torch.empty_like(x)
    assert out.stride(0) == x.stride(0)
    _lib.check(_lib.lib().e2h_rope(x.data_ptr(), out.data_ptr(), freqs.data_ptr(),
                                   pos.data_ptr(), x.shape[0], n_heads, head_dim, x.stride(0),
                                   int(inverse), _s()), "rope")
    return out


_ATTN_SCRATCH: dict = {}


def attn_decode_splits(B: int, n_kv: int, smax: Optional[int] = None) -> int:
    """How many CTAs may share one (sequence, kv head) in ``attn_decode``: the kernel deals the
    32-key chunks of all pairs out evenly, so a pair may be cut by run boundaries; 8 lets the
    runs be as short as an eighth of the longest context. ``E2H_ATTN_SPLITS=1`` gives every
    pair a CTA of its own (no scratch, no merge)."""
    import os
    forced = os.environ.get("E2H_ATTN_SPLITS")
    return max(1, min(8, int(forced))) if forced else 8


def attn_decode(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, pos: torch.Tensor,
                left_pad: Optional[torch.Tensor], n_head: int, out: Optional[torch.Tensor] = None,
                n_split: int = 0, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query token per sequence against the static cache, live range [left_pad[b], pos].

    q [B, n_head*D] bf16; caches [max_batch, n_kv, smax, D]; pos int32 device scalar.
    ``n_split`` (1..8, 0 = default) is the number of CTAs that may share one (sequence, kv head);
    their partial results go to ``scratch`` (a per-device buffer by default, so calls on one
    device must be ordered on one stream) and are merged by the last of them to finish."""
    B = q.shape[0]
    n_kv, smax, D = kcache.shape[1], kcache.shape[2], kcache.shape[3]
    if out is None:
        out = torch.empty_like(q)
    if n_split <= 0:
        n_split = attn_decode_splits(B, n_kv, smax)
    n_split = min(n_split, 8)
    tickets = None
    if n_split > 1:
        need = B * n_head * n_split * (D + 2)
        key = q.device.index
        buf = _ATTN_SCRATCH.get(key)
        if buf is None or buf[0].numel() < need or buf[1].numel() < B * n_kv:
            buf = (torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device),
                   torch.zeros(max(B * n_kv, 4096), dtype=torch.int32, device=q.device))
            _ATTN_SCRATCH[key] = buf
        tickets = buf[1]
        if scratch is None:
            scratch = buf[0]
        assert scratch.numel() >= need and scratch.dtype == torch.float32
    rc = _lib.lib().e2h_attn_decode(q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(),
                                    out.data_ptr(), _lib.ptr(scratch), pos.data_ptr(),
                                    _lib.ptr(left_pad), B, n_head, n_kv, D, smax,
                                    1.0 / math.sqrt(D), n_split, _lib.ptr(tickets),
                                    _lib.status_word(q.device).data_ptr(), _s())
    _lib.check(rc, "attn_decode")
    return out


def sample(logits: torch.Tensor, *, temperature: float, top_k: Optional[int], seed: int,
           pos: torch.Tensor, next_tok: torch.Tensor, advance_pos: bool = True,
           seq: Optional[torch.Tensor] = None, eos_id: int = -1,
           eos_flag: Optional[torch.Tensor] = None, n_unfinished: Optional[torch.Tensor] = None,
           ticket: Optional[torch.Tensor] = None, vocab: Optional[int] = None,
           seed_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Fused top-k / temperature / exponential-race sampler (fp32 logits [B, ld]). With
    ``seed_dev`` (int64 device scalar) the kernel reads the seed from device memory, so a
    captured graph does not bake it in."""
    B = logits.shape[0]
    vocab = vocab or logits.shape[1]
    rc = _lib.lib().e2h_sample(
        logits.data_ptr(), logits.stride(0), B, vocab, float(temperature),
        int(top_k) if top_k else 0, int(seed) & (2 ** 64 - 1), pos.data_ptr(), int(advance_pos),
        next_tok.data_ptr(), _lib.ptr(seq), 0 if seq is None else seq.stride(0),
        0 if seq is None else seq.shape[1], int(eos_id), _lib.ptr(eos_flag),
        _lib.ptr(n_unfinished), _lib.ptr(ticket), _lib.ptr(seed_dev), _s())
    _lib.check(rc, "sample")
    return next_tok


def reward_head(x: torch.Tensor, norm_weight: torch.Tensor, head_weight: torch.Tensor, eps: float,
                *, index: Optional[torch.Tensor] = None, k0: int = 0, finalize: bool = True,
                labels: Optional[torch.Tensor] = None, weights: Optional[torch.Tensor] = None):
    """Final RMSNorm + 2-row reward head + mean (+ weighted BCE-with-logits) in one kernel.

    ``x`` [rows, dim] bf16 is the residual stream BEFORE the final norm; ``head_weight`` [2, klen]
    holds columns ``[k0, k0 + klen)`` of the head (the whole head when unsharded). ``index``
    (int32 [n]) picks the rows to score. Returns ``(reward [n] fp32, dots [n, 2] fp32,
    loss_acc [2] fp32 or None)``: with ``finalize=False`` (a tensor-parallel slice) only ``dots``
    (fp32 partial sums) is meaningful and the caller reduces it over the ranks.
    Reference semantics: models/reward_model.py:80-88, train_rm_pointwise.py:101-110."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    dim = x.shape[1]
    head_weight = head_weight.to(torch.bfloat16)
    if head_weight.stride(1) != 1:
        head_weight = head_weight.contiguous()
    klen = head_weight.shape[1]
    n = int(index.numel()) if index is not None else x.shape[0]
    if index is not None:
        index = index.to(torch.int32).contiguous()
    reward = torch.empty(n, dtype=torch.float32, device=x.device)
    dots = torch.empty(n, 2, dtype=torch.float32, device=x.device)
    acc = None
    if labels is not None:
        acc = torch.zeros(2, dtype=torch.float32, device=x.device)
        labels = labels.to(torch.float32).contiguous()
        weights = weights.to(torch.float32).contiguous() if weights is not None else None
    nw = norm_weight.to(torch.bfloat16).contiguous()
    rc = _lib.lib().e2h_reward_head(
        x.data_ptr(), x.stride(0), nw.data_ptr(), head_weight.data_ptr(), head_weight.stride(0),
        dim, k0, klen, eps, _lib.ptr(index), n, x.shape[0], dots.data_ptr(), reward.data_ptr(),
        int(finalize), _lib.ptr(labels), _lib.ptr(weights), _lib.ptr(acc), _s())
    _lib.check(rc, "reward_head")
    return reward, dots, acc
