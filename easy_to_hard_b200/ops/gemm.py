"""Python front-end of the tcgen05 GEMM (csrc/gemm_umma.cu) and its fused epilogues.

Every function takes 2-D bf16 CUDA tensors whose last dimension is contiguous. The
"feature" operand (a weight ``[F, K]``) rides on the TMEM lanes and the "token" operand
(activations ``[T, K]``) on the TMEM columns, so ``linear(x, w)`` = ``x @ w.T`` is the
natural call for any token count.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _lib
from ._lib import (EPI_DUAL_STORE, EPI_RESIDUAL, EPI_ROPE_KV, EPI_ROWMAJOR_BF16,
                   EPI_ROWMAJOR_F32_ACC, EPI_STORE_BF16, EPI_STORE_F32, EPI_SWIGLU, GemmParams)

N_SM = 148


def _ld(t: torch.Tensor) -> int:
    assert t.dim() == 2 and t.stride(1) == 1, "operands must be 2-D with a contiguous last dim"
    return t.stride(0)


def _smem_bytes(bn: int, tf: int, dual: bool, splitk: int, stages: int, kps: int = 1) -> int:
    stage = kps * (tf * 128 * (2 if dual else 1) + bn * 128)
    xchg = (splitk - 1) * (bn // splitk) * tf * 4 * (2 if dual else 1) if splitk > 1 else 0
    return 2048 + stages * stage + xchg


def pick_tiles(F: int, T: int, K: int, dual: bool, splitk: Optional[int], bn: Optional[int],
               stages: int = 0, tf: Optional[int] = None, kps: int = 0):
    """Tile shape (features x tokens), cluster split-K factor, pipeline depth and k-blocks per
    pipeline stage.

    Skinny GEMMs (decode: at most one token tile) stream the weight once, so the aim is one CTA
    per SM on as many of the 148 SMs as possible: K is split across a cluster while the CTA count
    stays <= 148, and several 64-wide k-blocks share one pipeline stage because the per-stage
    barrier hand-shake (not the tensor work) bounds the k-loop at this size. Measured on B200:
    4 k-blocks per stage for a single accumulator, 2 for the dual (SwiGLU) one or when the tiles
    need more than one wave. Large GEMMs take the widest tile, one k-block per stage."""
    if bn is None:
        if T <= 64:
            bn = 64
        elif T <= 128 or dual:
            bn = 128
        else:
            bn = 256
    kb = -(-K // 64)
    t_tiles = -(-T // bn)
    skinny = bn <= 128 and t_tiles == 1
    if tf is None:
        tf = 128
    if tf == 64 and bn == 256:
        tf = 128
    tiles = -(-F // tf) * t_tiles
    if splitk is None:
        splitk = 1
        if skinny:
            while (splitk < 8 and tiles * splitk * 2 <= N_SM and kb // (splitk * 2) >= 4
                   and bn % (splitk * 2 * 8) == 0):
                splitk *= 2
    if kps <= 0:
        if not skinny or K % 64:
            kps = 1
        elif dual or tiles * splitk > N_SM:
            kps = 2
        else:
            kps = 4
    return bn, splitk, stages, tf, kps


class MulticastSignal:
    """``signal=`` for a GEMM whose completion flag lives in a symmetric allocation with an
    NVSwitch multicast mapping: the flag word's address in the multicast view. The last CTA
    bumps the word on every GPU with one ``multimem.red`` instead of one remote add per rank."""

    def __init__(self, address: int):
        self.address = int(address)


def pick_stream_tiles(F: int, K: int, bn: int, dual: bool):
    """Feature-tile height of a skinny K-major GEMM that runs without split-K, or None to keep
    128-row tiles. The kernel is a weight stream: with 128-row tiles a wide layer leaves SMs
    idle (11008 features = 86 tiles on 148 SMs), with lower tiles one wave covers nearly all of
    them (138 tiles of 80 rows). Measured on B200 at 64 tokens (cold L2): the dual w1/w3 GEMM
    74 -> 54 us; single-accumulator GEMMs, whose tiles already cover 96+ SMs, and anything that
    needs a split-K cluster (cluster placement, not the SM count, bounds its wave) do not gain,
    so they keep their tiles."""
    tiles128 = -(-F // 128)
    if tiles128 * 2 <= N_SM or tiles128 > N_SM or not dual:
        return None
    th = -(-F // N_SM)
    th = max(64, min(128, -(-th // 8) * 8))
    if -(-F // th) > N_SM:
        return None
    return th


def gemm(a: torch.Tensor, b: torch.Tensor, *, epi: int, out: Optional[torch.Tensor] = None,
         a2: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None,
         aux: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None,
         a_mn_major: bool = False, b_mn_major: bool = False, accumulate: bool = False,
         splitk: Optional[int] = None, bn: Optional[int] = None, stages: int = 0,
         rope: Optional[dict] = None, pdl: bool = False, tf: Optional[int] = None,
         tiled_shape: Optional[tuple] = None, kps: int = 0,
         signal=None, ticket: Optional[torch.Tensor] = None,
         persistent: Optional[bool] = None, pair: Optional[bool] = None,
         th: Optional[int] = None) -> None:
    """Raw launch. Shapes: a is [F, K] (or [K, F] when a_mn_major), b is [T, K] (or [K, T]).
    An int8 ``a`` (weight-only quantisation; ``scale`` holds the per-feature scales) streams as
    int8 through the converting kernel for up to 128 tokens and is expanded to a scratch bf16
    matrix first for larger token counts."""
    assert a.is_cuda and b.is_cuda and b.dtype == torch.bfloat16
    w4 = isinstance(a, Int4Weight)
    if w4:
        assert not a_mn_major and not b_mn_major and tiled_shape is None and scale is None
        assert a2 is None or isinstance(a2, Int4Weight)
        K4 = a.shape[1]
        if (b.shape[0] > 128 or K4 % 128 or a.groupsize < 64 or a.groupsize & (a.groupsize - 1)
                or (K4 // 2) % 16):
            a = _expand_int4(a, 0)            # many tokens: one dequantisation pass, then bf16
            a2 = _expand_int4(a2, 1) if a2 is not None else None
            w4 = False
    w8 = not w4 and a.dtype == torch.int8
    if w8:
        assert scale is not None and not a_mn_major and not b_mn_major and tiled_shape is None
        if a2 is not None:
            assert a2.dtype == torch.int8
        if b.shape[0] > 128 or a.shape[1] % 128 or _ld(a) % 16:
            a = _expand_int8(a, 0)
            a2 = _expand_int8(a2, 1) if a2 is not None else None
            w8 = False
    assert w8 or w4 or a.dtype == torch.bfloat16
    if w4:
        F, K = a.shape
    elif tiled_shape is not None:      # a is a TiledWeight payload: logical shape given
        F, K = tiled_shape
        assert tf is not None, "a tile-major weight fixes the feature-tile height"
    elif a_mn_major:
        K, F = a.shape
    else:
        F, K = a.shape
    if b_mn_major:
        Kb, T = b.shape
    else:
        T, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    dual = a2 is not None
    if (w8 or w4) and bn is None:
        bn = 64 if (T <= 64 or dual) else 128
    auto_tiles = (splitk is None and tf is None and kps <= 0 and th is None and not w8 and not w4
                  and not a_mn_major and not b_mn_major and tiled_shape is None
                  and K % 64 == 0 and STREAM_TILES)
    bn, splitk, stages, tf, kps = pick_tiles(F, T, K, dual, splitk, bn, stages, tf, kps)
    th = th or 0
    if auto_tiles and not th and bn <= 128 and T <= bn and splitk == 1:
        choice = pick_stream_tiles(F, K, bn, dual)
        if choice is not None:
            th, kps = choice, 4
    if (w8 or w4) and not th and splitk == 1 and STREAM_TILES:
        # the converting kernel is bound by bytes in flight per SM: a tile height that puts a
        # CTA on (nearly) every SM; rows per tile a multiple of 8 (int8) or 16 (int4)
        q = 16 if w4 else 8
        tiles128 = -(-F // 128)
        if tiles128 * 2 > N_SM and tiles128 <= N_SM:
            cand = max(64, min(128, -(-(-(-F // N_SM)) // q) * q))
            if -(-F // cand) <= N_SM:
                th = cand
    p = GemmParams()
    p.F, p.T, p.K = F, T, K
    p.splitk, p.epi, p.stages = splitk, epi, stages
    p.a_mn_major, p.b_mn_major = int(a_mn_major), int(b_mn_major)
    p.bn, p.dual, p.accumulate, p.pdl = bn, int(dual), int(accumulate), int(pdl)
    p.tf = tf
    p.th = th
    if isinstance(signal, MulticastSignal):
        assert ticket is not None
        p.n_signal = -1
        p.signal[0] = signal.address
        p.ticket = ticket.data_ptr()
    elif signal:
        assert ticket is not None and len(signal) <= 8
        p.n_signal = len(signal)
        for i, f in enumerate(signal):
            p.signal[i] = f if isinstance(f, int) else f.data_ptr()
        p.ticket = ticket.data_ptr()
    p.kps = kps
    p.a_tiled = int(tiled_shape is not None)
    if w4:
        p.lda, p.ldb = _ld(a.q), _ld(b)
        p.a, p.b = a.q.data_ptr(), b.data_ptr()
        p.qsz, p.groupsize = a.sz.data_ptr(), a.groupsize
        if dual:
            assert a2.shape == a.shape and a2.groupsize == a.groupsize
            p.a2, p.lda2, p.qsz2 = a2.q.data_ptr(), _ld(a2.q), a2.sz.data_ptr()
    else:
        p.lda, p.ldb = (64 if tiled_shape is not None else _ld(a)), _ld(b)
        p.a, p.b = a.data_ptr(), b.data_ptr()
        if dual:
            assert a2.shape == a.shape
            p.a2, p.lda2 = a2.data_ptr(), (64 if tiled_shape is not None else _ld(a2))
    if out is not None:
        p.out, p.ldo = out.data_ptr(), out.stride(0)
    if out2 is not None:
        p.out2, p.ldo2 = out2.data_ptr(), out2.stride(0)
    if aux is not None:
        p.aux = aux.data_ptr()
    if scale is not None:
        assert scale.dtype == torch.float32
        p.scale = scale.data_ptr()
    if rope is not None:
        p.freqs = rope["freqs"].data_ptr()
        p.pos_base = rope["pos_base"].data_ptr()
        p.sq = rope["sq"]
        p.n_head, p.n_kv, p.head_dim = rope["n_head"], rope["n_kv"], rope["head_dim"]
        p.smax = rope["smax"]
        p.kcache, p.vcache = rope["kcache"].data_ptr(), rope["vcache"].data_ptr()
    p.status = _lib.status_word(a.device).data_ptr()
    # more than one token tile: the persistent kernel (double-buffered accumulator, TMA-store
    # epilogue); skinny / split-K shapes: the latency-oriented one-tile-per-CTA kernel
    if w8:
        _lib.check(_lib.lib().e2h_gemm_w8(C.byref(p), _lib.stream()), "e2h_gemm_w8")
        return
    if w4:
        _lib.check(_lib.lib().e2h_gemm_w4(C.byref(p), _lib.stream()), "e2h_gemm_w4")
        return
    big = (persistent if persistent is not None else
           (T > bn and splitk == 1 and tf == 128 and tiled_shape is None
            and bn >= 128))
    if big:
        if (pair if pair is not None else PAIR_DEFAULT) and not dual and bn == 256:
            p.tf = 256      # CTA-pair (cta_group::2) tiles where the shape allows them
        _lib.check(_lib.lib().e2h_gemm_persistent(C.byref(p), _lib.stream()),
                   "e2h_gemm_persistent")
    else:
        _lib.check(_lib.lib().e2h_gemm_umma(C.byref(p), _lib.stream()), "e2h_gemm_umma")


class Int4Weight:
    """Group-wise int4 weight as the decode GEMM streams it: ``q`` uint8 ``[F, K / 2]`` where each
    32-bit word holds 8 consecutive k as ``sum_j q[2j] << 4j | q[2j+1] << (16 + 4j)`` (the pair
    (2j, 2j+1) then sits in bf16x2 position after one shift and mask), and ``sz`` bf16
    ``[K / g, F, 2]`` (scale, zero) exactly as the reference's checkpoints store it
    (models/quantize.py:60-70 of the reference). ``from_int`` builds it from integer codes
    ``[F, K]`` in 0..15 (``models.quantize.unpack_int4_tinygemm`` yields those)."""

    def __init__(self, q: torch.Tensor, sz: torch.Tensor, groupsize: int, shape):
        self.q, self.sz, self.groupsize, self.shape = q, sz, groupsize, tuple(shape)
        self.dtype, self.device, self.is_cuda = torch.uint8, q.device, q.is_cuda

    @classmethod
    def from_int(cls, codes: torch.Tensor, sz: torch.Tensor, groupsize: int) -> "Int4Weight":
        F, K = codes.shape
        assert K % 8 == 0
        c = codes.to(torch.int32).view(F, K // 8, 4, 2)
        sh = torch.arange(4, device=codes.device, dtype=torch.int32) * 4
        word = ((c[..., 0] << sh) | (c[..., 1] << (sh + 16))).sum(-1, dtype=torch.int64)
        word = word.to(torch.int32)                      # bit 31 may be set: wraps as intended
        q = word.view(torch.uint8).view(F, K // 2).contiguous()
        return cls(q, sz.to(torch.bfloat16).contiguous(), groupsize, (F, K))

    def codes(self) -> torch.Tensor:
        """Integer codes [F, K] (inverse of ``from_int``)."""
        F, K = self.shape
        w = self.q.view(torch.int32).view(F, K // 8, 1)
        sh = torch.arange(4, device=self.q.device, dtype=torch.int32) * 4
        lo, hi = (w >> sh) & 15, (w >> (sh + 16)) & 15
        return torch.stack([lo, hi], -1).view(F, K)

    def dequant(self) -> torch.Tensor:
        """bf16 [F, K]: ((q - 8) * scale + zero), each step rounded to bf16 as the reference does."""
        F, K = self.shape
        g = self.groupsize
        x = (self.codes() - 8).to(torch.bfloat16).view(F, K // g, g)
        s = self.sz[..., 0].t().unsqueeze(-1)            # [F, K/g, 1]
        z = self.sz[..., 1].t().unsqueeze(-1)
        return (x * s + z).view(F, K)


_INT8_SCRATCH: dict = {}
# large GEMMs on CTA pairs (cta_group::2, 256 x 256 tiles): E2H_GEMM_PAIR=0 keeps single-CTA tiles
PAIR_DEFAULT = os.environ.get("E2H_GEMM_PAIR", "1") != "0"
# skinny GEMMs: feature-tile height and split-K chosen so that the tiles fill one wave of the SMs
# (E2H_STREAM_TILES=0 keeps 128-row tiles)
STREAM_TILES = os.environ.get("E2H_STREAM_TILES", "1") != "0"


def _expand_int8(w: torch.Tensor, which: int) -> torch.Tensor:
    """bf16 image of an int8 weight in a per-device scratch buffer (two buffers, so that both
    matrices of a dual GEMM can be live). Used for token counts where re-converting the weights
    per token tile would cost more than one expansion pass."""
    key = (w.device.index, which)
    buf = _INT8_SCRATCH.get(key)
    if buf is None or buf.numel() < w.numel():
        buf = torch.empty(w.numel(), dtype=torch.bfloat16, device=w.device)
        _INT8_SCRATCH[key] = buf
    out = buf[: w.numel()].view(w.shape)
    out.copy_(w)
    return out


def _expand_int4(w: "Int4Weight", which: int) -> torch.Tensor:
    """bf16 image of an int4 weight in the per-device scratch buffers of ``_expand_int8``."""
    key = (w.device.index, which)
    n = w.shape[0] * w.shape[1]
    buf = _INT8_SCRATCH.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(n, dtype=torch.bfloat16, device=w.device)
        _INT8_SCRATCH[key] = buf
    out = buf[:n].view(w.shape)
    out.copy_(w.dequant())
    return out


def tile_weight(w: torch.Tensor, tf: int = 128) -> torch.Tensor:
    """[F, K] -> tile-major [ceil(F/tf) * ceil(K/64) * tf, 64] (zero padded): every (tf x 64)
    tile that one CTA streams per k-step is one contiguous block, so the weight stream is a
    sequence of full-page DRAM bursts instead of 128-byte pieces one row pitch apart."""
    F, K = w.shape
    Fp, Kp = -(-F // tf) * tf, -(-K // 64) * 64
    if (Fp, Kp) != (F, K):
        w = torch.nn.functional.pad(w, (0, Kp - K, 0, Fp - F))
    return (w.view(Fp // tf, tf, Kp // 64, 64).permute(0, 2, 1, 3).contiguous()
            .view(Fp // tf * (Kp // 64) * tf, 64))


def linear(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype=torch.bfloat16, scale=None, **kw) -> torch.Tensor:
    """x [T, K] @ w[F, K]^T -> [T, F]."""
    T, F = x.shape[0], w.shape[0]
    if out is None:
        out = torch.empty(T, F, dtype=out_dtype, device=x.device)
    epi = EPI_STORE_BF16 if out.dtype == torch.bfloat16 else EPI_STORE_F32
    gemm(w, x, epi=epi, out=out, scale=scale, **kw)
    return out


def linear_residual(x, w, residual, out=None, scale=None, **kw):
    """residual + x @ w^T (bf16)."""
    if out is None:
        out = torch.empty_like(residual)
    assert out.stride(0) == residual.stride(0)
    gemm(w, x, epi=EPI_RESIDUAL, out=out, aux=residual, scale=scale, **kw)
    return out


def linear_swiglu(x, w1, w3, out=None, **kw):
    """silu(x @ w1^T) * (x @ w3^T) with both products accumulated in one pass over x."""
    if out is None:
        out = torch.empty(x.shape[0], w1.shape[0], dtype=torch.bfloat16, device=x.device)
    gemm(w1, x, a2=w3, epi=EPI_SWIGLU, out=out, **kw)
    return out


def linear_dual(x, w1, w3, out1=None, out2=None, **kw):
    """(x @ w1^T, x @ w3^T) in one pass (training forward keeps both for the backward)."""
    T, F = x.shape[0], w1.shape[0]
    if out1 is None:
        out1 = torch.empty(T, F, dtype=torch.bfloat16, device=x.device)
    if out2 is None:
        out2 = torch.empty(T, F, dtype=torch.bfloat16, device=x.device)
    if T > 256 and not kw and w1.dtype == torch.bfloat16:
        # many tokens: two single-accumulator passes with 128 x 256 tiles. A dual tile has to be
        # 128 x 128 per matrix (tensor-memory budget), and the tensor core's operand fetch makes
        # that shape ~20% slower per FLOP than the wide one; re-reading x from L2 costs less.
        gemm(w1, x, epi=EPI_STORE_BF16, out=out1)
        gemm(w3, x, epi=EPI_STORE_BF16, out=out2)
        return out1, out2
    gemm(w1, x, a2=w3, epi=EPI_DUAL_STORE, out=out1, out2=out2, **kw)
    return out1, out2


def linear_qkv_rope(x, wqkv, q_out, *, freqs, pos_base, sq, n_head, n_kv, head_dim, kcache,
                    vcache, **kw):
    """Fused QKV projection + RoPE(q, k) + scatter of k, v into the static KV cache.

    q_out [T, n_head*head_dim]; caches [max_batch, n_kv, smax, head_dim]; token t belongs to
    sequence t // sq and sits at cache position pos_base + t % sq."""
    rope = dict(freqs=freqs, pos_base=pos_base, sq=sq, n_head=n_head, n_kv=n_kv,
                head_dim=head_dim, smax=kcache.shape[2], kcache=kcache, vcache=vcache)
    gemm(wqkv, x, epi=EPI_ROPE_KV, out=q_out, rope=rope, **kw)
    return q_out


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out=None, **kw) -> torch.Tensor:
    """dx [T, K] = dy [T, F] @ w [F, K] (w read as an MN-major operand, no transpose copy)."""
    T, K = dy.shape[0], w.shape[1]
    if out is None:
        out = torch.empty(T, K, dtype=torch.bfloat16, device=dy.device)
    gemm(w, dy, epi=EPI_STORE_BF16, out=out, a_mn_major=True, **kw)
    return out


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 accumulate: bool = False, **kw) -> torch.Tensor:
    """dw [F, K] (+)= dy[T, F]^T @ x[T, K]; fp32 (gradient accumulation buffer) or bf16 out."""
    F, K = dy.shape[1], x.shape[1]
    if out is None:
        out = torch.zeros(F, K, dtype=torch.float32, device=dy.device)
    epi = EPI_ROWMAJOR_F32_ACC if out.dtype == torch.float32 else EPI_ROWMAJOR_BF16
    gemm(dy, x, epi=epi, out=out, a_mn_major=True, b_mn_major=True, accumulate=accumulate, **kw)
    return out
