"""Weight-only int8 / int4 quantisation in the reference's checkpoint formats.

Formats (models/quantize.py:383-394, 502-545 of the reference):

* int8: ``*.weight`` int8 ``[N, K]`` + ``*.scales`` bf16 ``[N]``; symmetric per output channel,
  ``scale = max|w| / 127.5``, values clamped to [-128, 127]; ``y = (x @ W_int8^T) * scales``.
* int4: ``*.weight`` int32 in the tinygemm fragment layout ``[N/8, K/(ikt*16), 32, ikt/2]`` +
  ``*.scales_and_zeros`` bf16 ``[K/g, N, 2]``; asymmetric per group of ``g`` input features,
  ``scale = (max-min)/15``, ``zero = min + 8*scale``, ``w = (q - 8) * scale + zero``.

File names ``model_int8.pth`` / ``model_int4.g{G}.pth`` select the format at load time.

The packing into the tinygemm layout is restated here in plain PyTorch (``pack_int4_tinygemm`` /
``unpack_int4_tinygemm``) so that checkpoints can be produced and read on any device; the B200
decode path re-lays the weight out once at load time for its dequantising tcgen05 GEMM
(``ops.quant``), and the modules below are the device-agnostic definition of the numerics.
The reference's GPTQ handler depends on a ``models/GPTQ`` module that is not in its tree
(models/quantize.py:25-30) and is not reproduced.
"""
from __future__ import annotations

import time
from pathlib import Path
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .model import Transformer, find_multiple

# ------------------------------------------------------------------ int8 primitives


def dynamically_quantize_per_channel(x: torch.Tensor, quant_min: int, quant_max: int,
                                     target_dtype: torch.dtype):
    """Symmetric per-row quantisation. Returns (q, scales, zero_points)."""
    eps = torch.finfo(torch.float32).eps
    lo, hi = torch.aminmax(x, dim=1)
    absmax = torch.maximum(-torch.clamp(lo, max=0), torch.clamp(hi, min=0))
    scales = torch.clamp(absmax / (float(quant_max - quant_min) / 2), min=eps).to(x.dtype)
    q = torch.clamp(torch.round(x / scales.unsqueeze(-1)), quant_min, quant_max).to(target_dtype)
    return q, scales, torch.zeros_like(lo, dtype=torch.int64)


# ------------------------------------------------------------------ int4 primitives


def get_group_qparams(w: torch.Tensor, n_bit: int = 4, groupsize: int = 128):
    groupsize = min(groupsize, w.shape[-1])
    assert groupsize > 1 and w.dim() == 2 and w.shape[-1] % groupsize == 0
    g = w.reshape(-1, groupsize)
    hi, lo = g.amax(dim=1, keepdim=True), g.amin(dim=1, keepdim=True)
    scales = (hi - lo).clamp(min=1e-6) / (2 ** n_bit - 1)
    zeros = lo + scales * (2 ** (n_bit - 1))
    return (scales.to(torch.bfloat16).reshape(w.shape[0], -1),
            zeros.to(torch.bfloat16).reshape(w.shape[0], -1))


def pack_scales_and_zeros(scales: torch.Tensor, zeros: torch.Tensor) -> torch.Tensor:
    """[N, K/g] x2 -> [K/g, N, 2] bf16."""
    assert scales.shape == zeros.shape and scales.dtype == zeros.dtype == torch.bfloat16
    return torch.stack([scales, zeros], dim=-1).transpose(0, 1).contiguous()


def unpack_scales_and_zeros(scales_and_zeros: torch.Tensor):
    assert scales_and_zeros.dim() == 3 and scales_and_zeros.shape[2] == 2
    t = scales_and_zeros.transpose(0, 1)
    return t[..., 0].contiguous(), t[..., 1].contiguous()


def group_quantize_tensor_from_qparams(w, scales, zeros, n_bit: int = 4, groupsize: int = 128):
    if groupsize > w.shape[-1] and scales.shape[-1] == 1:
        groupsize = w.shape[-1]
    assert w.dim() == 2 and w.shape[-1] % groupsize == 0
    g = w.reshape(-1, groupsize)
    s, z = scales.reshape(-1, 1), zeros.reshape(-1, 1)
    lo = z - s * (2 ** (n_bit - 1))
    q = g.sub(lo).div(s).round().clamp_(0, 2 ** n_bit - 1).to(torch.int32)
    return q.reshape_as(w)


def group_quantize_tensor(w, n_bit: int = 4, groupsize: int = 128):
    scales, zeros = get_group_qparams(w, n_bit, groupsize)
    q = group_quantize_tensor_from_qparams(w, scales, zeros, n_bit, groupsize)
    return q, pack_scales_and_zeros(scales, zeros)


def group_dequantize_tensor_from_qparams(q, scales, zeros, n_bit: int = 4, groupsize: int = 128):
    if groupsize > q.shape[-1] and scales.shape[-1] == 1:
        groupsize = q.shape[-1]
    g = q.reshape(-1, groupsize)
    s, z = scales.reshape(-1, 1), zeros.reshape(-1, 1)
    return g.sub(2 ** (n_bit - 1)).mul(s).add(z).reshape_as(q)


def group_dequantize_tensor(q, scales_and_zeros, n_bit: int = 4, groupsize: int = 128):
    scales, zeros = unpack_scales_and_zeros(scales_and_zeros)
    return group_dequantize_tensor_from_qparams(q, scales, zeros, n_bit, groupsize)


def _tinygemm_index(inner_k_tiles: int):
    """For one (n-tile, k-outer-tile): the k offset and nibble shift of every packed value.

    Lane t of the warp owns row ``t // 4`` of the 8-row tile; each int32 packs two 16-wide
    k-tiles: nibble j (bits 4j..4j+3) holds k = tile(j) * 16 + (t % 4) * 2 + pair(j) where the
    nibble order is [k0, k0+8, k0+16, k0+24, k0+1, k0+9, k0+17, k0+25] relative to the int32's
    first k-tile (the m16n8k16 B-fragment order)."""
    t = torch.arange(32)
    koff = torch.tensor([0, 8, 16, 24, 1, 9, 17, 25])        # nibble j -> k offset
    k = (t % 4 * 2)[:, None, None] + koff[None, None, :]      # [32, 1, 8]
    pair = torch.arange(inner_k_tiles // 2) * 32              # each int32 spans 32 k
    k = k + pair[None, :, None]                               # [32, ikt/2, 8]
    row = (t // 4)[:, None, None].expand_as(k)
    return row, k


def pack_int4_tinygemm(q: torch.Tensor, inner_k_tiles: int = 8) -> torch.Tensor:
    """int32 ``[N, K]`` with values in [0, 15] -> int32 ``[N/8, K/(ikt*16), 32, ikt/2]``."""
    N, K = q.shape
    kt = inner_k_tiles * 16
    assert N % 8 == 0 and K % kt == 0
    row, k = _tinygemm_index(inner_k_tiles)
    row, k = row.to(q.device), k.to(q.device)
    tiles = q.reshape(N // 8, 8, K // kt, kt).permute(0, 2, 1, 3)      # [N/8, K/kt, 8, kt]
    vals = tiles[:, :, row, k].to(torch.int64) & 0xF                    # [.., 32, ikt/2, 8]
    shifts = (torch.arange(8, device=q.device) * 4).to(torch.int64)
    packed = (vals << shifts).sum(-1)
    packed = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed)
    return packed.to(torch.int32).contiguous()


def unpack_int4_tinygemm(packed: torch.Tensor, inner_k_tiles: Optional[int] = None):
    """Inverse of ``pack_int4_tinygemm``: -> int32 ``[N, K]``."""
    n8, ko, lanes, half = packed.shape
    assert lanes == 32
    ikt = inner_k_tiles or half * 2
    kt = ikt * 16
    row, k = _tinygemm_index(ikt)
    row, k = row.to(packed.device), k.to(packed.device)
    shifts = (torch.arange(8, device=packed.device) * 4).to(torch.int64)
    vals = ((packed.to(torch.int64) & 0xFFFFFFFF).unsqueeze(-1) >> shifts) & 0xF
    out = torch.zeros(n8, ko, 8, kt, dtype=torch.int32, device=packed.device)
    out[:, :, row, k] = vals.to(torch.int32)
    return out.permute(0, 2, 1, 3).reshape(n8 * 8, ko * kt)


def prepare_int4_weight_and_scales_and_zeros(weight_bf16, groupsize: int, inner_k_tiles: int):
    q, sz = group_quantize_tensor(weight_bf16, 4, groupsize)
    return pack_int4_tinygemm(q, inner_k_tiles), sz


def linear_forward_int4(x, weight_int4pack, scales_and_zeros, out_features: int, groupsize: int):
    """Dequantise-then-matmul definition of the int4 linear (device agnostic)."""
    q = unpack_int4_tinygemm(weight_int4pack)
    w = group_dequantize_tensor(q.float(), scales_and_zeros.float(), 4, groupsize)
    y = F.linear(x.reshape(-1, x.shape[-1]).to(torch.float32), w).to(x.dtype)
    return y.reshape(*x.shape[:-1], out_features)


def _check_linear_int4_k(k: int, groupsize: int = 1, inner_k_tiles: int = 1) -> bool:
    return k % groupsize == 0 and k % (inner_k_tiles * 16) == 0


# ------------------------------------------------------------------ modules


class WeightOnlyInt8Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None,
                 dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight", torch.empty(out_features, in_features, dtype=torch.int8,
                                                   device=device))
        self.register_buffer("scales", torch.ones(out_features, dtype=torch.bfloat16,
                                                  device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight.to(dtype=x.dtype)) * self.scales.to(x.dtype)


class WeightOnlyInt4Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None,
                 dtype=None, groupsize: int = 128, inner_k_tiles: int = 8, padding: bool = True):
        super().__init__()
        self.padding = padding
        if padding:
            self.origin_in_features = in_features
            in_features = find_multiple(in_features, 1024)
        self.in_features, self.out_features = in_features, out_features
        self.groupsize, self.inner_k_tiles = groupsize, inner_k_tiles
        assert out_features % 8 == 0 and in_features % (inner_k_tiles * 16) == 0
        self.register_buffer("weight", torch.empty(
            out_features // 8, in_features // (inner_k_tiles * 16), 32, inner_k_tiles // 2,
            dtype=torch.int32, device=device))
        self.register_buffer("scales_and_zeros", torch.empty(
            in_features // groupsize, out_features, 2, dtype=torch.bfloat16, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.padding:
            x = F.pad(x, pad=(0, self.in_features - self.origin_in_features))
        return linear_forward_int4(x, self.weight, self.scales_and_zeros, self.out_features,
                                   self.groupsize)


def _swap_linears(module: nn.Module, make, skip=("output",), prefix: str = "") -> None:
    for name, child in list(module.named_children()):
        fqn = f"{prefix}{name}"
        if isinstance(child, nn.Linear) and name not in skip:
            setattr(module, name, make(child, fqn))
        else:
            _swap_linears(child, make, skip, fqn + ".")


def _copy_tp_attrs(old: nn.Module, new: nn.Module) -> None:
    for a in ("tp_row_parallel",):
        if hasattr(old, a):
            setattr(new, a, getattr(old, a))


class WeightOnlyInt8QuantHandler:
    """Weight-only int8. The state dict covers every ``nn.Linear`` of the model, the LM head
    included when it is one, as the reference's files do (models/quantize.py:383-394 there);
    the runtime conversion swaps the block linears only, and a quantised head found in a file
    is expanded to bf16 at load time (``dequantize_head_in_state_dict``), because the head of an
    inference model is a frozen bf16 buffer."""

    def __init__(self, mod: nn.Module):
        self.mod = mod

    @torch.no_grad()
    def create_quantized_state_dict(self) -> Dict[str, torch.Tensor]:
        sd = self.mod.state_dict()
        for fqn, m in self.mod.named_modules():
            if isinstance(m, nn.Linear):
                q, scales, _ = dynamically_quantize_per_channel(m.weight.float(), -128, 127,
                                                                torch.int8)
                sd[f"{fqn}.weight"] = q
                sd[f"{fqn}.scales"] = scales.to(torch.bfloat16)
        return sd

    def convert_for_runtime(self) -> nn.Module:
        _swap_linears(self.mod, lambda lin, fqn: WeightOnlyInt8Linear(
            lin.in_features, lin.out_features, device=lin.weight.device))
        return self.mod

    @torch.no_grad()
    def convert_for_runtime_on_the_fly(self) -> nn.Module:
        """Quantise already-loaded (possibly TP-sharded) weights in place, e.g. the frozen
        reference policy / reward model of PPO (ppo_trainer.py:1343-1352 of the reference)."""
        def make(lin, fqn):
            new = WeightOnlyInt8Linear(lin.in_features, lin.out_features,
                                       device=lin.weight.device)
            q, scales, _ = dynamically_quantize_per_channel(lin.weight.float(), -128, 127,
                                                            torch.int8)
            new.weight.copy_(q)
            new.scales.copy_(scales.to(torch.bfloat16))
            _copy_tp_attrs(lin, new)
            return new
        _swap_linears(self.mod, make)
        return self.mod


class WeightOnlyInt4QuantHandler:
    def __init__(self, mod: nn.Module, groupsize: int = 128, inner_k_tiles: int = 8,
                 padding: bool = True):
        assert groupsize in (32, 64, 128, 256) and inner_k_tiles in (2, 4, 8)
        self.mod, self.groupsize, self.inner_k_tiles, self.padding = (mod, groupsize,
                                                                      inner_k_tiles, padding)

    @torch.no_grad()
    def create_quantized_state_dict(self) -> Dict[str, torch.Tensor]:
        sd = self.mod.state_dict()
        for fqn, m in self.mod.named_modules():
            if not isinstance(m, nn.Linear):
                continue
            assert m.out_features % 8 == 0, "int4 needs out_features divisible by 8"
            w = m.weight.data
            # input features are padded to a multiple of 1024 only when the plain layout does
            # not fit (models/quantize.py:513-535 of the reference): the 7B / 13B / 34B FFN
            # widths (11008, 13824, 22016) pass the check and are stored unpadded
            if not _check_linear_int4_k(m.in_features, self.groupsize, self.inner_k_tiles):
                if not self.padding:
                    continue
                w = F.pad(w, pad=(0, find_multiple(m.in_features, 1024) - m.in_features))
            packed, sz = prepare_int4_weight_and_scales_and_zeros(
                w.to(torch.bfloat16), self.groupsize, self.inner_k_tiles)
            sd[f"{fqn}.weight"] = packed
            sd[f"{fqn}.scales_and_zeros"] = sz
        return sd

    def convert_for_runtime(self) -> nn.Module:
        """Block linears become ``WeightOnlyInt4Linear``: unpadded where the input width fits
        the packed layout, padded otherwise (or left alone when padding is off), exactly the
        choice of the reference's ``replace_linear_int4`` (models/quantize.py:460-490)."""
        def make(lin, fqn):
            fits = _check_linear_int4_k(lin.in_features, self.groupsize, self.inner_k_tiles)
            if not fits and not self.padding:
                return lin
            return WeightOnlyInt4Linear(lin.in_features, lin.out_features,
                                        device=lin.weight.device, groupsize=self.groupsize,
                                        inner_k_tiles=self.inner_k_tiles, padding=not fits)
        _swap_linears(self.mod, make)
        return self.mod


def dequantize_head_in_state_dict(state: Dict[str, torch.Tensor], groupsize: int = 128,
                                  name: str = "output") -> Dict[str, torch.Tensor]:
    """Quantised checkpoints written from a model whose LM head is an ``nn.Linear`` carry the
    head as int8 (+ ``scales``) or packed int4 (+ ``scales_and_zeros``). Inference models keep
    the head as a frozen bf16 buffer, so it is expanded here, in place, before
    ``load_state_dict``; files without a quantised head pass through unchanged."""
    w = state.get(f"{name}.weight")
    if w is None:
        return state
    if f"{name}.scales" in state and w.dtype == torch.int8:
        sc = state.pop(f"{name}.scales").float()
        state[f"{name}.weight"] = (w.float() * sc.unsqueeze(-1)).to(torch.bfloat16)
    elif f"{name}.scales_and_zeros" in state and w.dtype == torch.int32:
        sz = state.pop(f"{name}.scales_and_zeros")
        q = unpack_int4_tinygemm(w, w.shape[-1] * 2)
        state[f"{name}.weight"] = group_dequantize_tensor(
            q, sz, 4, groupsize).to(torch.bfloat16)
    return state


def quantize(checkpoint_path: Path, mode: str = "int8", groupsize: int = 128,
             label: str = "") -> Path:
    """Read ``model.pth`` and write ``model{label}int8.pth`` / ``model{label}int4.g{G}.pth``
    next to it (the CLI's default label is ``_``)."""
    checkpoint_path = Path(checkpoint_path)
    assert checkpoint_path.is_file(), checkpoint_path
    t0 = time.time()
    with torch.device("meta"):
        model = Transformer.from_name(checkpoint_path.parent.name)
    sd = torch.load(str(checkpoint_path), mmap=True, weights_only=True)
    model.load_state_dict(sd, assign=True)
    model = model.to(dtype=torch.bfloat16, device="cpu")
    base = checkpoint_path.name
    if mode == "int8":
        out_sd = WeightOnlyInt8QuantHandler(model).create_quantized_state_dict()
        new_name = base.replace(".pth", f"{label}int8.pth")
    elif mode == "int4":
        out_sd = WeightOnlyInt4QuantHandler(model, groupsize).create_quantized_state_dict()
        new_name = base.replace(".pth", f"{label}int4.g{groupsize}.pth")
    else:
        raise ValueError(f"unknown quantisation mode {mode!r} (int8 | int4)")
    out = checkpoint_path.parent / new_name
    if out.exists():
        out.unlink()
    torch.save(out_sd, out)
    print(f"Quantization complete took {time.time() - t0:.02f} seconds -> {out}")
    return out


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="Quantize a model.")
    ap.add_argument("--checkpoint_path", type=Path,
                    default=Path("checkpoints/meta-llama/Llama-2-7b-chat-hf/model.pth"))
    ap.add_argument("--mode", "-q", type=str, default="int8", choices=["int8", "int4"])
    ap.add_argument("--groupsize", type=int, default=32)
    ap.add_argument("--label", type=str, default="_")
    a = ap.parse_args()
    quantize(a.checkpoint_path, a.mode, a.groupsize, a.label)
