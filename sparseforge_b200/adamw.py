"""Mask-aware AdamW on one fused kernel per tensor.

Mirror of the reference optimizer ``legacy/adamw.py:9-176``: same constructor, same
``step(closure=None, decay=None)``, same state keys (``step``, ``exp_avg``, ``exp_avg_sq``) with
the state kept in the parameter's dtype. For a ``SparseLinear`` weight the kernel also writes the
new masked weight ``W * M_eff`` the next forward pass consumes, so no separate masking pass runs.
Parameters must live on a CUDA device.
"""
from __future__ import annotations

import torch
from torch.optim.optimizer import Optimizer

from . import ops


class AdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False,
                 srste_decay=None, adaptive_l1_decay=0.0):
        if not 0.0 <= lr:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if not 0.0 <= eps:
            raise ValueError("Invalid epsilon value: {}".format(eps))
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError("Invalid beta parameter at index 0: {}".format(betas[0]))
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError("Invalid beta parameter at index 1: {}".format(betas[1]))
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad)
        self.decay = srste_decay if srste_decay is not None else 0.0
        self.adaptive_l1_decay = float(adaptive_l1_decay) if adaptive_l1_decay is not None else 0.0
        super().__init__(params, defaults)

    def __setstate__(self, state):
        super().__setstate__(state)
        for group in self.param_groups:
            group.setdefault("amsgrad", False)

    @torch.no_grad()
    def step(self, closure=None, decay=None):
        """legacy/adamw.py:65-176, one kernel launch per parameter tensor."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if decay is not None:
            self.decay = decay
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if not p.is_cuda:
                    raise RuntimeError("sparseforge_b200.AdamW: parameters must live on a CUDA device")
                grad = p.grad.data
                if grad.shape != p.data.shape:
                    if grad.numel() == p.data.numel() and p.data.numel() > 0:
                        grad = grad.view_as(p.data)
                    else:
                        # The reference applies the decoupled weight decay before it finds out that the
                        # gradient cannot be aligned (legacy/adamw.py:85-96); keep that order.
                        p.data.mul_(1 - group["lr"] * group["weight_decay"])
                        continue
                if grad.dtype != p.dtype:
                    grad = grad.to(p.dtype)
                mask = getattr(p, "mask", None)
                if mask is not None and mask.shape != p.data.shape:
                    mask = mask.view_as(p.data) if (mask.numel() == p.data.numel() and p.data.numel() > 0) else None
                if mask is not None and mask.dtype != torch.float32:
                    mask = mask.float()
                state = self.state[p]
                if len(state) == 0 or state["exp_avg"].shape != p.data.shape:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p.data)
                    state["exp_avg_sq"] = torch.zeros_like(p.data)
                    if group["amsgrad"]:
                        state["max_exp_avg_sq"] = torch.zeros_like(p.data)
                state["step"] += 1
                if p.data.numel() % 8 != 0 or p.dtype not in (torch.float32, torch.bfloat16):
                    self._small_tensor_step(p, grad, mask, state, group)
                    continue
                owner = getattr(p, "_sf_owner", None)
                layer = owner() if owner is not None else None
                wm, hx = (None, 1.0)
                ams = state.get("max_exp_avg_sq") if group["amsgrad"] else None
                fused = layer._optimizer_score_target() if (layer is not None and mask is not None and ams is None) \
                    else None
                if fused is not None:
                    # the mask update of this step follows: write the score of the new weight here
                    # and leave the masked weight to that update
                    metric, H = fused
                    ops.adamw_masked_score(p.data, grad.contiguous(), state["exp_avg"], state["exp_avg_sq"],
                                           mask=mask.data.contiguous(), lr=group["lr"], beta1=beta1, beta2=beta2,
                                           eps=group["eps"], weight_decay=group["weight_decay"], decay=float(self.decay),
                                           step=state["step"], adaptive_l1=self.adaptive_l1_decay, H=H,
                                           score=layer._score, norm=layer._norm, scratch=layer._scratch, metric=metric)
                    layer._optimizer_wrote_score()
                    continue
                if layer is not None:
                    layer._score_key = None
                if layer is not None and mask is not None and layer.mode == "sparse_forward" \
                        and layer.mask_type == "structured" and ams is None:
                    wm, hx = layer._adamw_emit_target()
                ops.adamw_masked(p.data, grad.contiguous(), state["exp_avg"], state["exp_avg_sq"],
                                 mask=None if mask is None else mask.data.contiguous(), lr=group["lr"], beta1=beta1,
                                 beta2=beta2, eps=group["eps"], weight_decay=group["weight_decay"],
                                 decay=float(self.decay), step=state["step"],
                                 adaptive_l1=self.adaptive_l1_decay if p.data.dim() >= 2 else 0.0, wm=wm, hx=hx,
                                 v_max=ams)
                if wm is not None:
                    layer._adamw_emitted()
                elif layer is not None:
                    layer.weight._sf_wm_stale = True  # the weight moved and no masked weight was written
        return loss

    def _small_tensor_step(self, p, grad, mask, state, group):
        """Tensors the vector kernel cannot take (size not a multiple of 8, other dtypes): the same
        update written with torch ops on the device (legacy/adamw.py:85-174)."""
        beta1, beta2 = group["betas"]
        p.data.mul_(1 - group["lr"] * group["weight_decay"])
        if mask is not None:
            grad = grad.add(p.data * (1 - mask), alpha=float(self.decay))
        m, v = state["exp_avg"], state["exp_avg_sq"]
        bc1 = 1 - beta1 ** state["step"]
        bc2 = 1 - beta2 ** state["step"]
        m.mul_(beta1).add_(grad, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
        if group["amsgrad"]:
            torch.max(state["max_exp_avg_sq"], v, out=state["max_exp_avg_sq"])
            v = state["max_exp_avg_sq"]
        denom = (v.sqrt() / (bc2 ** 0.5)).add_(group["eps"])
        p.data.addcdiv_(m, denom, value=-(group["lr"] / bc1))
        if self.adaptive_l1_decay > 0.0 and p.data.dim() >= 2 and mask is not None:
            p.data.add_(self.adaptive_l1_decay * torch.sign(p.data) / denom, alpha=-group["lr"])
