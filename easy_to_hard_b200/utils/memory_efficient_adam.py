"""AdamW whose moments live in a chosen dtype on a chosen device (GPU or pinned host memory).

Same contract as the reference optimizer (training_utils/memory_efficient_adam.py:19-262):
``exp_avg`` / ``exp_avg_sq`` are kept in ``optim_dtype`` on ``optim_device``; with a CPU
``optim_device`` they are pinned and staged through the GPU around every update; decoupled weight
decay is applied to the parameter first; ``load_state_dict`` casts loaded state to the configured
dtype / device. On CUDA the whole update is one fused kernel per tensor (``ops/csrc/optim.cu``)
that can also apply a device-resident gradient-clip coefficient, so clipping needs no host sync.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch.optim import Optimizer

from ..ops import _lib, reference

_DT = {torch.float32: 0, torch.bfloat16: 1}


def fused_adamw_(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step,
                 clip_coef: Optional[torch.Tensor] = None,
                 bf16_copy: Optional[torch.Tensor] = None) -> None:
    """In-place AdamW on flat/contiguous CUDA tensors of dtype fp32 or bf16."""
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    ok = (p.is_cuda and p.is_contiguous() and g.is_contiguous() and m.is_cuda and
          all(t.dtype in _DT for t in (p, g, m)))
    if not ok:
        if clip_coef is not None:
            g = g * clip_coef.to(g.dtype)
        reference.adamw_step(p, g.to(p.dtype), m, v, lr, beta1, beta2, eps, weight_decay, step)
        if bf16_copy is not None:
            bf16_copy.copy_(p)
        return
    rc = _lib.lib().e2h_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(),
                              _DT[p.dtype], _DT[g.dtype], _DT[m.dtype], lr, beta1, beta2, eps,
                              weight_decay, bc1, bc2, _lib.ptr(clip_coef), _lib.ptr(bf16_copy),
                              _lib.stream())
    _lib.check(rc, "adamw")


class MemoryEfficientAdamW(Optimizer):
    def __init__(self, model_params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0,
                 adamw_mode=True, optim_dtype=torch.bfloat16,
                 optim_device=torch.device("cpu")):
        super().__init__(model_params, dict(lr=lr, betas=betas, eps=eps,
                                            weight_decay=weight_decay))
        self.adamw_mode = adamw_mode
        self.optim_dtype = optim_dtype
        self.optim_device = torch.device(optim_device)
        self.clip_coef: Optional[torch.Tensor] = None  # device scalar set by the trainer

    def _new_state(self, p):
        def z():
            t = torch.zeros_like(p, device=self.optim_device, dtype=self.optim_dtype)
            if self.optim_device.type == "cpu" and torch.cuda.is_available():
                t = t.pin_memory()
            return t
        return {"step": 0, "exp_avg": z(), "exp_avg_sq": z()}

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        offload = self.optim_device.type == "cpu"
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if len(st) == 0:
                    st.update(self._new_state(p))
                st["step"] += 1
                g = p.grad
                if group["weight_decay"] != 0 and not self.adamw_mode:
                    g = g.add(p, alpha=group["weight_decay"])
                wd = group["weight_decay"] if self.adamw_mode else 0.0
                m, v = st["exp_avg"], st["exp_avg_sq"]
                if offload and p.is_cuda:
                    m_dev = m.to(p.device, non_blocking=True)
                    v_dev = v.to(p.device, non_blocking=True)
                else:
                    m_dev, v_dev = m, v
                fused_adamw_(p.data, g.data, m_dev, v_dev, lr=group["lr"], beta1=beta1,
                             beta2=beta2, eps=group["eps"], weight_decay=wd, step=st["step"],
                             clip_coef=self.clip_coef,
                             bf16_copy=getattr(p, "_lp_copy", None))
                if m_dev is not m:
                    m.copy_(m_dev, non_blocking=True)
                    v.copy_(v_dev, non_blocking=True)
        return loss

    def load_state_dict(self, state_dict):
        """Standard load, then move / cast every moment to ``optim_dtype`` on ``optim_device``
        (pinned when on the host), whatever the checkpoint held."""
        super().load_state_dict(state_dict)
        for st in self.state.values():
            for k in ("exp_avg", "exp_avg_sq"):
                if k in st:
                    t = st[k].to(device=self.optim_device, dtype=self.optim_dtype)
                    if self.optim_device.type == "cpu" and torch.cuda.is_available():
                        t = t.pin_memory()
                    st[k] = t
            if "step" in st and torch.is_tensor(st["step"]):
                st["step"] = int(st["step"].item())
