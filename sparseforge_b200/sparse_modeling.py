"""SparseLinear and its autograd functions on the B200 kernels.

Host-side mirror of the reference's ``legacy/sparse_modeling.py`` interface (same class and
method names, argument meaning and error behaviour) for the structured 2:4 path:

* ``SparseLinearConfig``  — legacy/sparse_modeling.py:136-239 (same fields and defaults)
* ``STE`` / ``SRSTE``      — :23-53
* ``FusedMaskedLinearSTE`` — :56-132 (``apply(x, weight, bias, mask, decay, scale_factor)``)
* ``SparseLinear``         — :242-1666

What differs by design: the masked weight ``W * M_eff`` is materialised once per change of
weight or mask (by the mask-update and AdamW kernels) instead of twice per step; the mask
update is one fused kernel that also emits 2:4 metadata, the flip count and the mask sums;
all three products run on tcgen05 kernels and stay differentiable to second order, which the
Hutchinson estimator needs. Tensors must live on a CUDA device; there is no CPU path.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from . import _lib, ops


@dataclass
class SparseLinearConfig:
    """Field-for-field the reference's dataclass (legacy/sparse_modeling.py:136-239)."""

    change_mask: bool = True
    mode: str = "sparse_forward"  # "sparse_forward" | "dense_forward"
    mask_type: str = "structured"  # "structured" | "unstructured" | "none"
    mask_metric: str = "hessian_obd"  # magnitude | movement | hessian_obd | hessian_ratio | hessian | wanda
    sparsity_ratio: float = 0.5
    N: int = 2
    M: int = 4
    beta: float = 0.99
    score_ema_beta: float = 0.99
    mask_update_period: int = 10
    mask_update_switch_step: int = 0
    mask_update_period_before: Optional[int] = None
    mask_update_period_after: Optional[int] = None
    mask_lr: float = 0.10
    mask_penalty_lr: float = None
    mask_penalty_mode: str = "mid"
    temp_init: float = 1.0
    temp_min: float = 0.05
    temp_decay: float = 0.97
    mask_binarize_decay: float = 0
    mask_hardening_start: int = 1000
    mask_hardening_duration: int = 10000
    sparsity_warmup_steps: int = 100
    tau_sample_size: int = 262144
    temperature: float = 1.0
    freeze_low: float = 0.0
    freeze_high: float = 1.0
    SLoRB: bool = False
    SLoRB_k: int = 64
    SLoRB_init_type: str = "mean"
    trainable_projection: bool = False
    structured_exact: bool = False
    hard_mask_type: str = "match"
    beta_structural_start: int = 0
    beta_structural_end: int = 0
    gradient_checkpointing: bool = False
    srste_decay: float = 0.0
    glu_joint_mask: bool = False
    weight_scaling: bool = False


# ----------------------------------------------------------------------------------------
# differentiable GEMM primitives (closed under differentiation, so any order works)
# ----------------------------------------------------------------------------------------
class _MatmulNT(torch.autograd.Function):
    """a[M,K] @ b[N,K]^T on the forward-product kernel."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return ops.gemm_fwd(a.contiguous(), b.contiguous())

    @staticmethod
    def backward(ctx, gy):
        a, b = ctx.saved_tensors
        ga = _MatmulNN.apply(gy, b) if ctx.needs_input_grad[0] else None
        gb = _MatmulTN.apply(gy, a) if ctx.needs_input_grad[1] else None
        return ga, gb


class _MatmulNN(torch.autograd.Function):
    """a[M,K] @ b[K,N] on the dgrad kernel."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return ops.gemm_dgrad(a.contiguous(), b.contiguous())

    @staticmethod
    def backward(ctx, gy):
        a, b = ctx.saved_tensors
        ga = _MatmulNT.apply(gy, b) if ctx.needs_input_grad[0] else None
        gb = _MatmulTN.apply(a, gy) if ctx.needs_input_grad[1] else None
        return ga, gb


class _MatmulTN(torch.autograd.Function):
    """a[K,M]^T @ b[K,N] on the wgrad kernel."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return ops.gemm_wgrad(a.contiguous(), b.contiguous())

    @staticmethod
    def backward(ctx, gy):
        a, b = ctx.saved_tensors
        ga = _MatmulNT.apply(b, gy) if ctx.needs_input_grad[0] else None
        gb = _MatmulNN.apply(a, gy) if ctx.needs_input_grad[1] else None
        return ga, gb


class _MaskedWeight(torch.autograd.Function):
    """weight * cast(M_eff) with its true gradient g * cast(M_eff) (no gradient to the mask).

    Stands for ``weight_cast * mask_for_grad`` in the reference's backward
    (legacy/sparse_modeling.py:113), which is built from differentiable ops there.
    """

    @staticmethod
    def forward(ctx, weight, mask, hx, finalized, wm_cached, proj=None):
        ctx.save_for_backward(mask)
        ctx.hx, ctx.finalized, ctx.proj = hx, finalized, proj
        if wm_cached is not None:
            return wm_cached.view_as(wm_cached)
        wm = torch.empty_like(weight)
        if proj is not None:
            proj(weight.detach().contiguous(), wm)
        else:
            ops.effective_weight(weight.detach().contiguous(), mask, wm, hx=hx, finalized=finalized)
        return wm

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        out = torch.empty_like(g)
        if ctx.proj is not None:
            ctx.proj(g.contiguous(), out)
        else:
            ops.effective_weight(g.contiguous(), mask, out, hx=ctx.hx, finalized=ctx.finalized)
        return out, None, None, None, None, None


class STE(torch.autograd.Function):
    """Forward weight * mask; backward passes the gradient to the dense weight
    (legacy/sparse_modeling.py:23-35)."""

    @staticmethod
    def forward(ctx, weight, mask):
        return weight * mask

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


class SRSTE(torch.autograd.Function):
    """STE plus decay * weight where mask < 0.5 (legacy/sparse_modeling.py:38-53)."""

    @staticmethod
    def forward(ctx, weight, mask, decay):
        ctx.save_for_backward(weight)
        ctx.mask, ctx.decay = mask, decay
        return weight * mask

    @staticmethod
    def backward(ctx, grad_output):
        (weight,) = ctx.saved_tensors
        return grad_output + ctx.decay * weight * (ctx.mask < 0.5).to(weight.dtype), None, None


def _as_f32_mask(mask: torch.Tensor) -> torch.Tensor:
    return mask if mask.dtype == torch.float32 else mask.float()


class FusedMaskedLinearSTE(torch.autograd.Function):
    """Masked linear with a straight-through weight gradient.

    ``apply(x, weight, bias, mask, decay, scale_factor=1.0)`` as in the reference
    (legacy/sparse_modeling.py:72-132): ``mask`` is the effective mask. Two extra trailing
    arguments are used by ``SparseLinear``: a cached masked weight and (hx, finalized), in which
    case ``mask`` is the soft mask and the effective mask is formed inside the kernels.
    The backward pass is made of differentiable functions, so ``create_graph=True`` works.
    """

    @staticmethod
    def forward(ctx, x, weight, bias, mask, decay, scale_factor=1.0, wm_cached=None, hx=1.0, finalized=True, proj=None,
                z=None, sw=None):
        if not x.is_cuda:
            raise RuntimeError("FusedMaskedLinearSTE: tensors must live on a CUDA device (there is no CPU path)")
        cd = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else weight.dtype
        mask32 = _as_f32_mask(mask.detach())
        if wm_cached is None:
            wm = torch.empty_like(weight)
            ops.effective_weight(weight.detach().contiguous(), mask32.contiguous(), wm, hx=hx, finalized=finalized)
        else:
            wm = wm_cached
        x2 = x.reshape(-1, x.shape[-1])
        b_cd = None if bias is None else bias.to(cd).contiguous()
        if z is None:
            y2 = ops.gemm_fwd(x2.to(cd).contiguous(), wm.to(cd), b_cd, alpha=float(scale_factor))
        else:
            # low-rank bypass z @ sw^T (legacy/sparse_modeling.py:790-794) added to the product: inside the
            # same launch where the kernel allows it (bf16, more than 128 rows, no output scale)
            z2, sw_cd = z.reshape(-1, z.shape[-1]).to(cd).contiguous(), sw.to(cd).contiguous()
            if cd == torch.bfloat16 and x2.shape[0] > 128 and float(scale_factor) == 1.0 and z2.shape[1] % 8 == 0:
                y2 = ops.gemm_fwd_lowrank(x2.to(cd).contiguous(), wm.to(cd), z2, sw_cd, b_cd)
            else:
                y2 = ops.gemm_fwd(x2.to(cd).contiguous(), wm.to(cd), b_cd, alpha=float(scale_factor))
                y2 = y2 + ops.gemm_fwd(z2, sw_cd)
        ctx.save_for_backward(x, weight, mask32, z, sw)
        ctx.has_bias = bias is not None
        ctx.decay = float(decay)
        ctx.hx, ctx.finalized = float(hx), bool(finalized)
        ctx.proj = proj  # writes src * cast(M_eff) for hard views other than 2:4 (a layer's bound method)
        ctx.wm = wm if wm.dtype == cd else None
        return y2.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_out):
        x, weight, mask32, z, sw = ctx.saved_tensors
        cd = grad_out.dtype
        gy = grad_out.reshape(-1, grad_out.shape[-1])
        x2 = x.reshape(-1, x.shape[-1]).to(cd)
        grad_x = grad_w = grad_b = grad_z = grad_sw = None
        if z is not None and ctx.needs_input_grad[10]:
            grad_z = _MatmulNN.apply(gy, sw.to(cd)).view_as(z).to(z.dtype)
        if z is not None and ctx.needs_input_grad[11]:
            grad_sw = _MatmulTN.apply(gy, z.reshape(-1, z.shape[-1]).to(cd)).to(sw.dtype)
        if ctx.needs_input_grad[0]:
            w = _MaskedWeight.apply(weight.to(cd), mask32, ctx.hx, ctx.finalized, ctx.wm, ctx.proj)
            grad_x = _MatmulNN.apply(gy, w).view_as(x)
        if ctx.needs_input_grad[1]:
            grad_w = _MatmulTN.apply(gy, x2)
            if ctx.decay != 0.0:
                eff_lt = (_effective_mask_tensor(mask32, ctx.hx, ctx.finalized) < 0.5).to(cd)
                grad_w = grad_w + ctx.decay * weight.to(cd) * eff_lt
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = gy.sum(dim=0) if torch.is_grad_enabled() else ops.bias_grad(gy.contiguous()).to(cd)
        return grad_x, grad_w, grad_b, None, None, None, None, None, None, None, grad_z, grad_sw


def _effective_mask_tensor(mask32, hx, finalized):
    """hx * mask + (1 - hx) * top2(mask) as a tensor (legacy/sparse_modeling.py:759-771)."""
    if finalized or hx >= 1.0 - 1e-6:
        return mask32
    hard, _ = ops.project_nm24(mask32)
    return (hx * mask32) + ((1.0 - hx) * hard)


# ----------------------------------------------------------------------------------------
# SparseLinear
# ----------------------------------------------------------------------------------------
_SUPPORTED_METRICS = ("magnitude", "movement", "hessian_obd", "hessian_ratio", "hessian", "wanda")


class SparseLinear(nn.Linear):
    """``nn.Linear`` with a continuous 2:4 mask driven by no-grad dynamics
    (legacy/sparse_modeling.py:242-1666).

    State-dict keys match the reference: ``weight bias mask grad_ema hessian_diag
    frozen_mask_flags scaler_row`` (1-element placeholders where unused). ``mask`` and
    ``hessian_diag`` are kept in float32 whatever the weight dtype.
    """

    def __init__(self, in_features, out_features, sparselinear_config=None, bias=True, **kwargs):
        super().__init__(in_features, out_features, bias=bias, **kwargs)
        assert sparselinear_config is not None
        cfg = sparselinear_config
        self.cfg = cfg
        self.mode = cfg.mode
        self.change_mask = cfg.change_mask
        self.mask_type = cfg.mask_type
        self.mask_metric = cfg.mask_metric
        self.sparsity_ratio = cfg.sparsity_ratio
        self.N, self.M = cfg.N, cfg.M
        dev = self.weight.device

        def frozen(shape, fill=0.0, dtype=torch.float32):
            return nn.Parameter(torch.full(shape, fill, device=dev, dtype=dtype), requires_grad=False)

        self.mask = frozen((out_features, in_features), 1.0)
        if cfg.change_mask and cfg.mask_metric == "movement":
            self.grad_ema = frozen((out_features, in_features), dtype=self.weight.dtype)
        else:
            self.grad_ema = frozen((1,), dtype=self.weight.dtype)
            self._grad_ema_placeholder = True
        if cfg.change_mask and (cfg.mask_metric in ("hessian_obd", "hessian_ratio", "hessian")
                                or getattr(cfg, "enable_hutchinson", False)):
            self.hessian_diag = frozen((out_features, in_features))
        else:
            self.hessian_diag = frozen((1,))
            self._hessian_diag_placeholder = True
        if cfg.change_mask and (cfg.freeze_low > 0.0 or cfg.freeze_high < 1.0):
            # fp32 like the mask: the update kernel reads and raises the flags in the same pass
            self.frozen_mask_flags = frozen((out_features, in_features), 0.0)
        else:
            self.frozen_mask_flags = frozen((1,), dtype=self.weight.dtype)
            self._frozen_mask_flags_placeholder = True
        if cfg.mask_metric == "wanda":
            self.scaler_row = frozen((in_features,), 0.0, dtype=self.weight.dtype)
        else:
            self.scaler_row = frozen((1,), dtype=self.weight.dtype)
            self._scaler_row_placeholder = True
        self.nsamples = 0

        self.weight.mask = self.mask
        self.weight.flipped_mask = 0
        self.weight.init_flipped_mask = 0
        self.weight.param_count = self.weight.numel()
        self.weight._sf_owner = weakref.ref(self)
        self.srste_decay = cfg.srste_decay
        self.mask_penalty_lr = float(cfg.mask_penalty_lr) if cfg.mask_penalty_lr is not None else float(cfg.mask_lr)
        self.hard_mask_type = str(getattr(cfg, "hard_mask_type", "match") or "match")
        self.hardening_x = 1.0
        self.SLoRB = cfg.SLoRB
        if self.SLoRB:
            # low-rank bypass out += (x x_proj^T) SLoRB_Weight^T; parameters registered here and filled
            # by init_SLoRB, as the reference does (legacy/sparse_modeling.py:388-408)
            self.SLoRB_k = cfg.SLoRB_k
            self.SLoRB_init_type = cfg.SLoRB_init_type
            self.trainable_projection = cfg.trainable_projection
            k = int(self.SLoRB_k)
            assert k > 0, f"SLoRB_k must be > 0 (got {k})"
            assert in_features % k == 0, f"in_features ({in_features}) must be divisible by SLoRB_k ({k})."
            self.x_proj = nn.Parameter(torch.zeros(in_features // k, in_features, device=dev, dtype=self.weight.dtype),
                                       requires_grad=bool(self.trainable_projection))
            self.SLoRB_Weight = nn.Parameter(torch.zeros(out_features, in_features // k, device=dev,
                                                         dtype=self.weight.dtype), requires_grad=True)
        # device-side caches (not part of the state dict)
        self._wm = None          # W * cast(M_eff) in the weight dtype
        self._wm_key = None      # what the cache was built from
        self._meta = None        # packed 2:4 metadata of top2(mask)
        self._score = None
        self._norm = None
        self._stats = None
        self._scratch = None
        self.last_mask_stats = None  # device float64[8] written by the last update_mask
        self._row_shard_group = None  # set by sharding.RowShardedLinear when this is one shard of a layer
        self._row_sharded = False
        # Score fusion with the optimizer: when the last update_mask call predicts that the next step
        # updates the mask too, this package's AdamW writes the score of the new weight in its own
        # pass (and leaves the masked weight to the mask update), and the Hutchinson accumulation
        # only updates H. _score_key records what that score was computed from.
        self.fuse_score_with_optimizer = True
        self._fuse_score_next = False
        self._score_key = None

    # -- helpers -------------------------------------------------------------------------
    def _apply(self, fn, recurse=True):
        """``.to(dtype)`` / ``.half()`` / ``.bfloat16()`` convert the weight; the soft mask and the
        Hessian diagonal stay float32 (the kernels read them as such), moved to the new device."""
        keep = {n: getattr(self, n).data for n in ("mask", "hessian_diag") if not self._is_placeholder(n)}
        out = super()._apply(fn, recurse) if recurse is not True else super()._apply(fn)
        for n, old in keep.items():
            prm = getattr(self, n)
            if prm.dtype != torch.float32:
                prm.data = old.to(device=prm.device, dtype=torch.float32)
        self.weight.mask = self.mask
        self.weight._sf_owner = weakref.ref(self)
        self._wm_key = None
        return out

    def _is_placeholder(self, name: str) -> bool:
        return getattr(self, f"_{name}_placeholder", False)

    def _resolved_hard_type(self) -> str:
        return self.mask_type if self.hard_mask_type == "match" else self.hard_mask_type

    def _block_size(self) -> int:
        """16 / 32 in the block-sparse soft-mask modes, else 0."""
        return {"block_sparse16": 16, "block_sparse32": 32}.get(self.hard_mask_type, 0)

    def _tile16_keep_k(self) -> int:
        """Entries kept per 16 x 16 tile in the 'block16' mode (legacy/sparse_modeling.py:553-555)."""
        return max(0, min(256, int(round((1.0 - float(self.sparsity_ratio)) * 256))))

    def _is_tile16(self) -> bool:
        return self._resolved_hard_type() == "block16"

    def _check_tile16(self):
        if self.out_features % 16 or self.in_features % 16:
            raise NotImplementedError("hard_mask_type='block16' is built for layer sizes that are multiples of 16")

    def _block_keep(self, block_values: torch.Tensor) -> torch.Tensor:
        """uint8 [ob, ib]: the round((1 - sparsity_ratio) * blocks) blocks with the largest value, ties
        to the lower flat index (legacy/sparse_modeling.py:621-637, 671-687)."""
        flat = block_values.flatten()
        total = flat.numel()
        keep_n = max(0, min(total, int(round((1.0 - float(self.sparsity_ratio)) * total))))
        keep = torch.zeros(total, dtype=torch.uint8, device=flat.device)
        if keep_n > 0:
            keep[torch.sort(flat, descending=True, stable=True).indices[:keep_n]] = 1
        return keep.view_as(block_values)

    def _buffers_ready(self):
        dev = self.weight.device
        if self._score is None or self._score.device != dev or self._score.shape != self.weight.shape:
            self._score = torch.empty(self.weight.shape, dtype=torch.float32, device=dev)
            self._norm = torch.zeros(2, dtype=torch.float32, device=dev)
            self._stats = torch.zeros(_lib.MSTAT_COUNT, dtype=torch.float64, device=dev)
            self._scratch = ops.hutch_score_scratch(dev)
            self._meta = torch.zeros((self.out_features, (self.in_features + 7) // 8), dtype=torch.uint8, device=dev)
            self._wm = torch.empty_like(self.weight.data)
            self._wm_key = None

    def _threshold_view(self) -> bool:
        """True when the hard view is ``mask > 0.5`` (hard_mask_type 'unstructured',
        legacy/sparse_modeling.py:526-527)."""
        return self._resolved_hard_type() == "unstructured"

    def _general_nm(self) -> bool:
        """True when the hard view is not top-2-of-4 (other N:M, or the 0.5 threshold): the general
        one-thread-per-group kernels then take the place of the 2:4 ones (no sparse tensor-core metadata, no
        fused optimizer output)."""
        return self._threshold_view() or (int(self.N), int(self.M)) != (2, 4)

    def _check_2to4(self):
        """Sizes and modes the N:M kernels (2:4 or general) accept."""
        n, m = int(self.N), int(self.M)
        if not self._general_nm():
            if self.in_features % 8 != 0:
                raise ValueError(f"in_features ({self.in_features}) must be a multiple of 8 for the 2:4 kernels")
            return
        if self._resolved_hard_type() not in ("structured", "unstructured"):
            raise NotImplementedError(
                f"N:M = {n}:{m} with hard_mask_type={self._resolved_hard_type()!r}: gate groups and hard view must agree "
                "(use hard_mask_type='structured' or 'match' with mask_type='structured')")
        if m not in (2, 4, 8, 16, 32) or not 1 <= n < m:
            raise NotImplementedError(f"N:M = {n}:{m}: M must be 2, 4, 8, 16 or 32 and 1 <= N < M")
        if self.in_features % m != 0:
            raise ValueError(f"in_features ({self.in_features}) must be divisible by M ({m}).")

    def _is_2to4_view(self) -> bool:
        """True when the layer's hard view is top-2-of-4 along the input dimension."""
        t = self._resolved_hard_type()
        return t == "nm_2_4" or (t == "structured" and not self._general_nm())

    def _check_strict_2to4(self, what: str):
        if not self._is_2to4_view():
            raise NotImplementedError(f"{what} needs a 2:4 hard view (the layer has N:M = {self.N}:{self.M}, "
                                      f"hard_mask_type={self._resolved_hard_type()!r})")

    @torch.no_grad()
    def initialize(self):
        """legacy/sparse_modeling.py:410-439."""
        self.mask.fill_(1.0)
        if not self._is_placeholder("frozen_mask_flags"):
            self.frozen_mask_flags.zero_()
        if not self._is_placeholder("grad_ema"):
            self.grad_ema.zero_()
        if not self._is_placeholder("hessian_diag"):
            self.hessian_diag.fill_(1.0 if self.mask_metric == "hessian_obd" else 0.0)
        self.sync_weight()
        self.invalidate_masked_weight()

    @torch.no_grad()
    def add_batch(self, inp, out=None):
        """WANDA calibration (legacy/sparse_modeling.py:884-898): folds the squared L2 norm of every
        input channel over this batch into ``scaler_row`` as a running mean over samples."""
        if self._is_placeholder("scaler_row"):
            return
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        batch = inp.shape[0]
        x2d = inp.reshape(-1, inp.shape[-1]).contiguous()
        keep = self.nsamples / (self.nsamples + batch + 1e-8)
        self.nsamples += batch
        ops.wanda_add_batch(x2d, self.scaler_row.data, keep, max(self.nsamples, 1))
        self._score_key = None  # the kernel wrote scaler_row behind autograd's version counter

    @torch.no_grad()
    def sync_weight(self):
        """legacy/sparse_modeling.py:441-458."""
        self.weight.mask = self.mask
        self.weight._sf_owner = weakref.ref(self)
        self.weight.flipped_mask = int(getattr(self.weight, "flipped_mask", 0))
        self.weight.init_flipped_mask = int(getattr(self.weight, "init_flipped_mask", 0))
        self.weight.param_count = int(getattr(self.weight, "param_count", self.weight.numel()))

    @torch.no_grad()
    def _blockify_tensor(self, tensor):
        """Block means broadcast back over each whole block (legacy/sparse_modeling.py:461-508)."""
        bs = self._block_size()
        if not bs or tensor.dim() != 2 or tensor.shape[0] < bs or tensor.shape[1] < bs:
            return tensor
        out = tensor.float().contiguous().clone()
        s, _ = ops.block_sums(out, bs, want_sq=False)
        keep = torch.ones(s.shape, dtype=torch.uint8, device=out.device)
        ops.block_mask_apply(out, bs, keep, value=(s / float(bs * bs)).contiguous())
        return out.to(tensor.dtype)

    # -- hard projection -----------------------------------------------------------------
    @torch.no_grad()
    def _hard_mask_from_soft(self, soft_mask: torch.Tensor) -> torch.Tensor:
        """legacy/sparse_modeling.py:510-735 for 'none', 'unstructured', 'structured', 'nm_2_4'."""
        mt = self._resolved_hard_type()
        if mt == "none":
            return torch.ones_like(soft_mask)
        if mt == "unstructured" or soft_mask.dim() != 2:
            return (soft_mask > 0.5).to(dtype=soft_mask.dtype)
        if mt == "nm_2_4":
            return ops.project_nm24(soft_mask)[0]
        if mt == "block16" and soft_mask.dim() == 2:
            # top entries of every 16 x 16 tile (:537-574)
            if soft_mask.shape[0] % 16 or soft_mask.shape[1] % 16:
                raise NotImplementedError("hard_mask_type='block16' is built for sizes that are multiples of 16")
            return ops.project_tile16(soft_mask.float().contiguous(), self._tile16_keep_k()).to(soft_mask.dtype)
        if mt in ("block_sparse16", "block_sparse32"):
            # whole blocks kept by the RMS of the soft mask over the block (:607-718)
            bs = 16 if mt == "block_sparse16" else 32
            hard = torch.ones_like(soft_mask, dtype=torch.float32)
            if soft_mask.shape[0] < bs or soft_mask.shape[1] < bs:
                return hard.to(soft_mask.dtype)
            _, sq = ops.block_sums(soft_mask.float().contiguous(), bs)
            keep = self._block_keep(torch.sqrt(sq / float(bs * bs)))
            ops.block_mask_apply(hard, bs, keep, value=keep.float().contiguous())
            return hard.to(soft_mask.dtype)
        if mt != "structured":
            raise ValueError(f"Invalid hard mask_type: {mt}")
        n, m = int(self.N), int(self.M)
        if soft_mask.shape[1] % m != 0:
            raise ValueError(f"in_features ({soft_mask.shape[1]}) must be divisible by M ({self.M}).")
        if (n, m) == (2, 4):
            return ops.project_nm24(soft_mask)[0]
        if m not in (2, 4, 8, 16, 32) or not 1 <= n < m:
            raise NotImplementedError(f"N:M = {n}:{m}: M must be 2, 4, 8, 16 or 32 and 1 <= N < M")
        if soft_mask.dtype not in (torch.float32, torch.bfloat16):
            return ops.project_nm(soft_mask.float(), n, m).to(soft_mask.dtype)
        return ops.project_nm(soft_mask, n, m)

    @torch.no_grad()
    def metadata(self) -> torch.Tensor:
        """Packed 2:4 metadata of top2(mask) ([out, in/8] uint8), as left by the last mask update
        or masked-weight refresh."""
        self._check_strict_2to4("metadata()")
        self.masked_weight()
        return self._meta

    # -- masked weight cache ---------------------------------------------------------------
    def invalidate_masked_weight(self):
        """Call after changing ``weight``, ``mask`` or ``hessian_diag`` through ``.data`` (edits that
        autograd's version counters do not see) outside ``update_mask`` / the AdamW of this package:
        drops the cached masked weight and the score the optimizer pass may have left."""
        self._wm_key = None
        self._score_key = None

    def _adamw_emit_target(self):
        """(wm buffer, hx) the AdamW kernel should write the new masked weight with."""
        self._check_2to4()
        if self._general_nm():
            return None, 1.0  # the optimizer kernel ranks groups of four; masked_weight() rebuilds the product
        self._buffers_ready()
        fin = bool(getattr(self, "_hardening_finalized", False))
        return self._wm, (1.0 if fin else float(self.hardening_x))

    def _adamw_emitted(self):
        self._wm_key = self._current_key()
        self.weight._sf_wm_stale = False
        self.weight._sf_managed = True

    def _current_key(self):
        fin = bool(getattr(self, "_hardening_finalized", False))
        return (self.weight.data_ptr(), self.weight._version, self.mask.data_ptr(), self.mask._version,
                float(self.hardening_x), fin, self.weight.dtype)

    @torch.no_grad()
    def masked_weight(self) -> torch.Tensor:
        """W * cast(M_eff). Rebuilt on every call unless this package's AdamW manages the weight (it
        and ``update_mask`` then rewrite the cache whenever they change weight or mask); under a
        managed weight, code that edits ``weight.data`` or ``mask.data`` itself must call
        ``invalidate_masked_weight()``."""
        if self._block_size():
            return self._masked_weight_block()
        if self._is_tile16():
            self._check_tile16()
            self._buffers_ready()
            fin = bool(getattr(self, "_hardening_finalized", False))
            ops.project_tile16(self.mask.data, self._tile16_keep_k(), want_hard=False, W=self.weight.data, wm=self._wm,
                               hx=1.0 if fin else float(self.hardening_x))
            return self._wm
        self._check_2to4()
        self._buffers_ready()
        key = self._current_key()
        managed = getattr(self.weight, "_sf_managed", False)  # set by this package's AdamW
        if (not managed) or self._wm_key != key or getattr(self.weight, "_sf_wm_stale", True):
            if self._general_nm():
                ops.effective_weight_nm(self.weight.data, self.mask.data, self._wm, int(self.N), int(self.M),
                                        hx=float(self.hardening_x), finalized=key[5], threshold_view=self._threshold_view())
            else:
                ops.effective_weight(self.weight.data, self.mask.data, self._wm, meta=self._meta,
                                     hx=float(self.hardening_x), finalized=key[5])
            self._wm_key = key
            self.weight._sf_wm_stale = False
        return self._wm

    @torch.no_grad()
    def _apply_effective_mask(self, src: torch.Tensor, dst: torch.Tensor) -> None:
        """dst <- src * cast(M_eff) with the layer's current mask, hardening and hard view; the
        backward of the masked weight (second-order products pass through it) for the hard views
        other than 2:4."""
        hx = float(self.hardening_x)
        fin = bool(getattr(self, "_hardening_finalized", False))
        bs = self._block_size()
        if bs:
            keep = torch.ones((self.out_features // bs, self.in_features // bs), dtype=torch.uint8, device=src.device)
            if not fin and hx < 1.0 - 1e-6:
                _, sq = ops.block_sums(self.mask.data, bs)
                keep = self._block_keep(torch.sqrt(sq / float(bs * bs)))
            ops.block_mask_apply(self.mask.data, bs, keep, W=src, wm=dst, hx=1.0 if fin else hx)
        elif self._is_tile16():
            ops.project_tile16(self.mask.data, self._tile16_keep_k(), want_hard=False, W=src, wm=dst,
                               hx=1.0 if fin else hx)
        elif self._general_nm():
            ops.effective_weight_nm(src, self.mask.data, dst, int(self.N), int(self.M), hx=hx, finalized=fin,
                                    threshold_view=self._threshold_view())
        else:
            ops.effective_weight(src, self.mask.data, dst, hx=hx, finalized=fin)

    @torch.no_grad()
    def _masked_weight_block(self) -> torch.Tensor:
        """W * cast(hx * mask + (1 - hx) * block-hard(mask)) in the block-sparse modes, rebuilt on every
        call (one pass for the block sums of the mask, one for the product)."""
        bs = self._block_size()
        self._buffers_ready()
        hx = float(self.hardening_x)
        fin = bool(getattr(self, "_hardening_finalized", False))
        keep = torch.ones((self.out_features // bs, self.in_features // bs), dtype=torch.uint8, device=self.weight.device)
        if not fin and hx < 1.0 - 1e-6:
            _, sq = ops.block_sums(self.mask.data, bs)
            keep = self._block_keep(torch.sqrt(sq / float(bs * bs)))
        ops.block_mask_apply(self.mask.data, bs, keep, W=self.weight.data, wm=self._wm, hx=1.0 if fin else hx)
        return self._wm

    # -- forward -----------------------------------------------------------------------------
    def _compute_weight_scale_factor(self) -> float:
        """legacy/sparse_modeling.py:799-827."""
        mt = self._resolved_hard_type()
        if mt == "none":
            return 1.0
        if mt == "structured":
            n, m = int(self.N), int(self.M)
            return 1.0 if (n <= 0 or m <= 0 or n >= m) else float(m) / float(n)
        if mt == "nm_2_4":
            return 2.0
        sr = float(self.sparsity_ratio)
        return 1.0 if (sr <= 0.0 or sr >= 1.0) else 1.0 / (1.0 - sr)

    # -- inference on the sparse tensor cores ---------------------------------------------------
    @torch.no_grad()
    def compress_for_inference(self):
        """Bakes weight * top2(mask) into the compressed 2:4 form the sparse tensor cores read
        (values [out, in/2] bf16 + metadata) and switches ``mode`` to ``"sparse24_forward"``.
        The reference's inference bake-in multiplies the hard mask into a dense weight and runs a
        dense GEMM (legacy/eval_wiki_ppl.py:548-651); this is the same function with half the
        weight bytes and half the tensor-core work. Forward only; the dense weight is kept."""
        self._check_strict_2to4("compress_for_inference (the sparse tensor cores' format)")
        self._check_2to4()
        if self.weight.dtype != torch.bfloat16:
            raise TypeError("compress_for_inference: the sparse tensor-core GEMM is bfloat16 only")
        if self.in_features % 16 != 0:
            raise ValueError(f"compress_for_inference: in_features ({self.in_features}) must be a multiple of 16")
        values, meta = ops.sparse24_compress(self.weight.data.contiguous(), self.mask.data.float().contiguous())
        self._sp_values = values
        self._sp_meta = meta
        self._sp_meta_tc = ops.sparse24_pack_meta(meta, self.out_features, self.in_features)
        self._sp_status = torch.zeros(4, dtype=torch.int32, device=self.weight.device)
        self.mode = "sparse24_forward"
        self._inference_optimized = True
        return self

    def _sparse24_forward(self, x):
        if torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad and self.training):
            raise RuntimeError("mode 'sparse24_forward' is inference only; call it under torch.no_grad() / eval()")
        if getattr(self, "_sp_values", None) is None:
            raise RuntimeError("mode 'sparse24_forward' without compressed buffers: call compress_for_inference()")
        x2d = x.reshape(-1, self.in_features)
        if x2d.dtype != torch.bfloat16:
            x2d = x2d.to(torch.bfloat16)
        y = ops.sparse24_gemm(x2d.contiguous(), self._sp_values, self._sp_meta_tc, bias=self.bias, status=self._sp_status)
        return y.view(*x.shape[:-1], self.out_features).to(x.dtype)

    def forward(self, x):
        """legacy/sparse_modeling.py:737-796."""
        if self.mode == "sparse24_forward":
            out = self._sparse24_forward(x)
            if self.SLoRB and hasattr(self, "x_proj"):
                # the low-rank bypass stays on at inference (legacy/eval_wiki_ppl.py:560-575, 623)
                out = out + self._slorb(x)
            return out
        if self.mode == "dense_forward" or self.mask_type == "none":
            ones = torch.ones_like(self.mask.data)
            return FusedMaskedLinearSTE.apply(x, self.weight, self.bias, ones, 0.0, 1.0, self.weight.detach(), 1.0, True)
        if self.mode != "sparse_forward":
            raise ValueError(f"Invalid mode: {self.mode}")
        if self._resolved_hard_type() not in ("structured", "nm_2_4", "unstructured", "block_sparse16", "block_sparse32",
                                              "block16"):
            raise NotImplementedError(f"hard mask type {self._resolved_hard_type()!r} is outside the kernel paths")
        hx = float(getattr(self, "hardening_x", 1.0))
        finalized = bool(getattr(self, "_hardening_finalized", False))
        scale = 1.0
        if getattr(self.cfg, "weight_scaling", False) and hx < 1.0 - 1e-6:
            scale = 1.0 + (1.0 - hx) * (self._compute_weight_scale_factor() - 1.0)
        wm = self.masked_weight()
        other_view = self._block_size() or self._is_tile16() or self._general_nm()
        proj = self._apply_effective_mask if other_view else None
        if self.SLoRB and hasattr(self, "x_proj"):
            # z = x x_proj^T as a product of its own (differentiable); z SLoRB_Weight^T rides in the main
            # product's K loop
            cd = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else self.weight.dtype
            x2 = x.reshape(-1, x.shape[-1]).to(cd)
            z = _MatmulNT.apply(x2, self.x_proj.to(cd))
            return FusedMaskedLinearSTE.apply(x, self.weight, self.bias, self.mask, 0.0, scale, wm, hx, finalized, proj,
                                              z, self.SLoRB_Weight)
        return FusedMaskedLinearSTE.apply(x, self.weight, self.bias, self.mask, 0.0, scale, wm, hx, finalized, proj)

    def _slorb(self, x):
        """(x x_proj^T) SLoRB_Weight^T, legacy/sparse_modeling.py:790-794, as two products on the
        tensor-core kernels (differentiable with respect to x, the projection and the weight)."""
        x2 = x.reshape(-1, x.shape[-1])
        z = _MatmulNT.apply(x2, self.x_proj.to(x2.dtype))
        y = _MatmulNT.apply(z, self.SLoRB_Weight.to(x2.dtype))
        return y.view(*x.shape[:-1], self.out_features)

    @torch.no_grad()
    def init_SLoRB(self):
        """legacy/sparse_modeling.py:830-872: x_proj sums blocks of k input features (or is drawn
        xavier-uniform); SLoRB_Weight starts from the mean / sum over each block of the part of the
        weight that the mask currently prunes, W (1 - mask)."""
        n, d = self.weight.shape
        k = int(self.SLoRB_k)
        assert d % k == 0, f"in_features ({d}) must be divisible by SLoRB_k ({k})."
        rows = d // k
        xp = self.x_proj.data
        xp.zero_()
        r = torch.arange(rows, device=xp.device)
        xp[r[:, None], (r * k)[:, None] + torch.arange(k, device=xp.device)] = 1
        if self.SLoRB_init_type == "xavier":
            nn.init.xavier_uniform_(self.x_proj)
        else:
            pruned = (self.weight.detach() * (1.0 - self.mask.detach())).view(n, rows, k)
            if self.SLoRB_init_type == "mean":
                init = pruned.mean(dim=2)
            elif self.SLoRB_init_type == "sum":
                init = pruned.sum(dim=2)
            else:
                raise ValueError(f"Invalid SLoRB_init_type: {self.SLoRB_init_type}")
            self.SLoRB_Weight.data.copy_(init)

    # -- grad / hessian EMA ----------------------------------------------------------------
    @torch.no_grad()
    def update_grad_hessian_ema(self, update_hessian_with_grad2: bool = True):
        """legacy/sparse_modeling.py:901-922 (including its early return for every metric but movement)."""
        if self._is_placeholder("grad_ema") or self.weight.grad is None:
            return
        g = self.weight.grad.detach()
        if g.shape != self.grad_ema.shape:
            if g.numel() != self.grad_ema.numel():
                return
            g = g.view_as(self.grad_ema)
        b = float(self.cfg.beta)
        with_h = update_hessian_with_grad2 and not self._is_placeholder("hessian_diag") and self.hessian_diag.shape == g.shape
        if g.numel() % 8 == 0 and g.dtype == self.grad_ema.dtype and g.is_contiguous():
            ops.grad_hessian_ema(g, self.grad_ema.data, self.hessian_diag.data if with_h else None, beta=b)
        else:  # sizes the 8-wide kernel does not take (never a SparseLinear weight with in_features % 8 == 0)
            self.grad_ema.mul_(b).add_(g.to(self.grad_ema.dtype), alpha=1 - b)
            if with_h:
                self.hessian_diag.mul_(b).add_((g * g).float(), alpha=1 - b)
        self._score_key = None  # the kernel wrote grad_ema / H behind autograd's version counters

    def update_importance_ema(self):
        pass

    @torch.no_grad()
    def accumulate_hutchinson(self, hvp: torch.Tensor, v: torch.Tensor, beta: Optional[float] = None):
        """H <- beta H + (1-beta) max(hvp * v, 0), fused with the score of the current weights
        (elementwise tail of update_hessian_hutchinson, legacy/utils.py:804-868)."""
        if self._is_placeholder("hessian_diag"):
            return
        self._buffers_ready()
        self._score_key = None
        if self._optimizer_score_target() is not None:
            # the optimizer pass of this step scores the weight it writes: only H is updated here
            ops.hutch_accumulate(self.hessian_diag.data, hvp.contiguous(), v.contiguous(),
                                 beta=float(self.cfg.beta if beta is None else beta))
            return
        if self.mask_metric in ("wanda", "movement"):
            # metrics that do not read H: the sample goes into H, the score is formed when it is wanted
            ops.hutch_accumulate(self.hessian_diag.data, hvp.contiguous(), v.contiguous(),
                                 beta=float(self.cfg.beta if beta is None else beta))
            return
        ops.hutch_score(self.weight.data, self.hessian_diag.data, self._score, self._norm, self._scratch,
                        hvp=hvp.contiguous(), v=v.contiguous(), beta=float(self.cfg.beta if beta is None else beta),
                        metric=self.mask_metric if self.mask_metric in _SUPPORTED_METRICS else "hessian_obd")
        self._combine_shard_norm()

    # -- schedules (host scalars) --------------------------------------------------------------
    def _mask_update_period(self, step: int) -> int:
        """legacy/sparse_modeling.py:944-952."""
        base = int(getattr(self.cfg, "mask_update_period", 10))
        sw = int(getattr(self.cfg, "mask_update_switch_step", 0) or 0)
        before = getattr(self.cfg, "mask_update_period_before", None)
        after = getattr(self.cfg, "mask_update_period_after", None)
        if sw > 0 and before is not None and after is not None:
            return int(before) if step < sw else int(after)
        return base

    def _temperature(self, step: int) -> float:
        """legacy/sparse_modeling.py:932-942."""
        k = max(1, int(self._mask_update_period(step)))
        init = float(self.cfg.temp_init)
        if self._block_size():
            init *= float(getattr(self.cfg, "block_sparse_temp_mult", 2.0))
        t = init * (float(self.cfg.temp_decay) ** (step // k))
        return float(max(float(self.cfg.temp_min), t))

    def _effective_sparsity(self, step: int) -> float:
        """legacy/sparse_modeling.py:954-964."""
        warm = int(self.cfg.sparsity_warmup_steps)
        if warm <= 0:
            return float(self.sparsity_ratio)
        r = min(1.0, max(0.0, step / max(1, warm)))
        if self._block_size():
            r = r * r * r
        return float(self.sparsity_ratio * r)

    def _beta_structural(self, step: int) -> float:
        """legacy/sparse_modeling.py:966-985."""
        start = int(getattr(self.cfg, "beta_structural_start", 0))
        end = int(getattr(self.cfg, "beta_structural_end", 0))
        if end <= start or step < start:
            return 0.0
        if step >= end:
            return 1.0
        t = float(step - start) / float(end - start)
        return float(3.0 * t * t - 2.0 * t * t * t)

    def _next_hardening_x(self, step: int) -> float:
        """legacy/sparse_modeling.py:1603-1619."""
        start = int(getattr(self.cfg, "mask_hardening_start", 0))
        duration = int(getattr(self.cfg, "mask_hardening_duration", 0))
        if duration <= 0:
            return 0.0 if (step >= start and start > 0) else 1.0
        if step < start:
            return 1.0
        if step >= start + duration:
            return 0.0
        return max(0.0, min(1.0, 1.0 - float(step - start) / float(max(1, duration))))

    # -- score and gate ---------------------------------------------------------------------
    @torch.no_grad()
    def _refresh_score(self):
        """Raw score of the current weights and its mean / std, without touching the Hessian."""
        self._buffers_ready()
        if self._score_key is not None and self._score_key == self._score_state():
            return  # written by the optimizer pass of this step; weight and Hessian untouched since
        self._score_key = None
        metric, H = self._resolved_metric()
        aux = None
        if metric == "wanda":
            ops.wanda_score(self.weight.data, self.scaler_row.data, self._score, self._norm, self._scratch)
            self._combine_shard_norm()
            return
        aux_scalar = float(self.cfg.temperature)
        if metric == "movement":
            aux = self.grad_ema.data
        elif metric == "weight_sq":
            # W * W in the weight dtype: the movement formula |W * aux| / 1 with aux = W
            metric, aux, aux_scalar = "movement", self.weight.data, 1.0
        ops.hutch_score(self.weight.data, H, self._score, self._norm, self._scratch, aux=aux,
                        aux_scalar=aux_scalar, metric=metric)
        self._combine_shard_norm()

    def _resolved_metric(self):
        """(metric, H) the score is computed with. A metric that lacks its tensor falls back as the
        reference does (legacy/sparse_modeling.py:1041-1079): to |W|, except ``hessian_obd`` without a
        Hessian tensor, which scores W * W ("weight_sq")."""
        metric = self.mask_metric
        if metric not in _SUPPORTED_METRICS:
            metric = "magnitude"
        H = None if self._is_placeholder("hessian_diag") else self.hessian_diag.data
        if H is None and metric == "hessian_obd":
            metric = "weight_sq"
        elif H is None and metric in ("hessian_ratio", "hessian"):
            metric = "magnitude"
        if metric == "wanda" and self._is_placeholder("scaler_row"):
            metric = "magnitude"
        if metric == "movement" and self._is_placeholder("grad_ema"):
            metric = "magnitude"
        return metric, H

    def _score_state(self):
        H = None if self._is_placeholder("hessian_diag") else self.hessian_diag
        return (self.weight.data_ptr(), self.weight._version, 0 if H is None else H.data_ptr(),
                0 if H is None else H._version, self.mask_metric)

    def _optimizer_score_target(self):
        """What this package's AdamW needs to write the score in its own pass, or None when the
        next step is not expected to update the mask (or the metric needs another tensor)."""
        if not (self.fuse_score_with_optimizer and self._fuse_score_next and self.change_mask):
            return None
        metric, H = self._resolved_metric()
        if metric in ("movement", "wanda", "weight_sq") or self.mode != "sparse_forward":
            return None
        self._check_2to4()
        self._buffers_ready()
        return metric, H

    def _optimizer_wrote_score(self):
        self._combine_shard_norm()
        self._score_key = self._score_state()
        self.weight._sf_wm_stale = True  # the masked weight is rewritten by the mask update that follows
        self.weight._sf_managed = True
        self._wm_key = None

    def _predict_mask_update(self, step: int) -> bool:
        if (not self.change_mask) or self.mask_type == "none" or step < int(self.cfg.sparsity_warmup_steps):
            return False
        return step % max(1, int(self._mask_update_period(step))) == 0

    def _combine_shard_norm(self):
        """Score mean / std are taken over the whole layer: when this module is one row shard, add up
        the shards' sums before forming them."""
        if not self._row_sharded:
            return
        from .sharding import combine_score_sums

        sums, n = combine_score_sums(self._scratch[:2], self.weight.numel(), self._row_shard_group)
        ops.score_norm_from_sums(sums, n, self._norm)

    def _score_is_bf16(self) -> bool:
        # the reference's score has dtype promote(weight, hessian): bf16 only when no fp32 Hessian enters
        return self.weight.dtype == torch.bfloat16 and self._resolved_metric()[0] in ("magnitude", "movement", "weight_sq")

    @torch.no_grad()
    def compute_gate_target(self, step: int) -> torch.Tensor:
        """Soft gate G of legacy/sparse_modeling.py:1018-1239 (structured and unstructured branches),
        as a tensor. Runs the fused update kernel on a copy of the mask with mask_lr = 1 and no
        penalty, which leaves exactly G in the copy."""
        if (not self.change_mask) or (self.mask_type == "none"):
            return torch.ones_like(self.mask)
        self._check_mask_modes()
        if self._block_size():
            bs = self._block_size()
            G = torch.ones_like(self.mask.data)
            gate = self._block_gate(step)
            ops.block_mask_apply(G, bs, torch.ones(gate.shape, dtype=torch.uint8, device=G.device), value=gate)
            return G
        self._check_2to4()
        self._refresh_score()
        G = torch.zeros_like(self.mask.data)
        stats = torch.zeros(_lib.MSTAT_COUNT, dtype=torch.float64, device=G.device)
        gate_args = dict(tau=self._gate_tau(step), temperature=self._temperature(step), mask_lr=1.0,
                         beta_s=self._beta_structural(step),
                         structured_exact=bool(getattr(self.cfg, "structured_exact", False)),
                         score_bf16=self._score_is_bf16())
        if self._general_nm():
            ops.mask_update_nm(self._score, self._norm, G, stats, int(self.N), int(self.M),
                               threshold_view=self._threshold_view(), **gate_args)
        else:
            ops.mask_update_nm24(self._score, self._norm, G, stats, **gate_args)
        if not self._is_placeholder("frozen_mask_flags"):
            # a frozen entry's gate is its own value (legacy/sparse_modeling.py:1227-1229)
            G = torch.where(self.frozen_mask_flags.data != 0, self.mask.data, G)
        return G

    def _check_mask_modes(self):
        """Gate / projection combinations the 2:4 kernels cover."""
        if self.mask_type not in ("structured", "unstructured"):
            raise ValueError(f"Invalid mask_type: {self.mask_type}")
        if self._block_size() or self._is_tile16():
            if self.mask_type != "unstructured":
                raise NotImplementedError("block hard masks are built for mask_type='unstructured'")
            return
        if self._resolved_hard_type() not in ("structured", "nm_2_4", "unstructured"):
            raise NotImplementedError(
                f"hard mask type {self._resolved_hard_type()!r} with mask_type={self.mask_type!r} is outside the "
                "kernel paths")

    @torch.no_grad()
    def _tau_unstructured(self, scores: torch.Tensor, sparsity: float, sample_idx: Optional[torch.Tensor] = None):
        """Quantile threshold of legacy/sparse_modeling.py:987-1015 on a random sample of the scores,
        averaged over data-parallel replicas (not over the row shards of one layer: each shard samples
        its own rows, as each FSDP rank does in the reference)."""
        flat = scores.flatten()
        n = flat.numel()
        m = int(self.cfg.tau_sample_size) if self.cfg.tau_sample_size is not None else n
        if m > 0 and n > m:
            idx = sample_idx if sample_idx is not None else torch.randint(0, n, (m,), device=flat.device)
            sample = flat[idx]
        else:
            sample = flat
        tau = torch.quantile(sample.float(), q=float(sparsity))
        if getattr(self, "_in_summon_context", False):
            return tau
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = tau.clone()
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            tau = t / dist.get_world_size()
        return tau

    def _gate_tau(self, step: int, score: Optional[torch.Tensor] = None):
        """Device scalar with the unstructured gate's threshold in normalised-score units, or None for
        the structured gate. The quantile of the raw score sample is mapped through the same affine
        normalisation as the scores (a quantile commutes with it)."""
        if self.mask_type != "unstructured":
            return None
        tau_raw = self._tau_unstructured(self._score if score is None else score, self._effective_sparsity(step),
                                         getattr(self, "_tau_sample_idx", None))
        return ((tau_raw - self._norm[0]) / self._norm[1]).to(torch.float32).reshape(1).contiguous()

    # -- periodic mask update ---------------------------------------------------------------
    @torch.no_grad()
    def update_mask(self, step: int, lambda_mid: float = 0.0, score_ready: bool = False):
        """legacy/sparse_modeling.py:1242-1666. One kernel: gate, penalty, EMA, hard projection,
        effective masked weight, metadata, flip count and mask sums. ``score_ready=True`` reuses
        the score left by ``accumulate_hutchinson`` in this step (weights unchanged since)."""
        if self.mask.numel() == 0:
            return
        if self.mask.dim() != 2 or self.weight.shape != self.mask.shape:
            return
        # the optimizer pass of the next step writes the score if that step updates the mask
        self._fuse_score_next = self._predict_mask_update(step + 1)
        if (not self.change_mask) or (self.mask_type == "none"):
            self.weight.flipped_mask = 0
            self.weight.init_flipped_mask = 0
            return
        if step < int(self.cfg.sparsity_warmup_steps):
            return
        if step % max(1, int(self._mask_update_period(step))) != 0:
            return
        self._check_mask_modes()
        if self._block_size():
            return self._update_mask_block(step, lambda_mid)
        if self._is_tile16():
            return self._update_mask_tile16(step, lambda_mid)
        self._check_2to4()
        if not score_ready:
            self._refresh_score()
        lam = 0.0 if lambda_mid is None else float(lambda_mid)
        mode = str(getattr(self.cfg, "mask_penalty_mode", "mid") or "mid")
        if lam != 0.0 and mode not in ("mid", "structured_topn", "nm_2_4"):
            raise NotImplementedError(f"mask_penalty_mode={mode!r} is outside the 2:4 kernel path")
        if lam != 0.0 and mode == "nm_2_4" and (int(self.N), int(self.M)) != (2, 4):
            raise NotImplementedError(f"mask_penalty_mode='nm_2_4' pulls towards top-2-of-4; the layer's groups are {self.N}:{self.M}")
        pmode = _lib.PENALTY_MID if mode == "mid" else _lib.PENALTY_TOPN
        self._launch_mask_update(self._score, self._norm, step, pen=float(self.mask_penalty_lr) * lam,
                                 pmode=pmode if lam != 0.0 else 0, tau=self._gate_tau(step), owner=self,
                                 score_bf16=self._score_is_bf16())

    def _update_mask_tile16(self, step: int, lambda_mid):
        """update_mask with hard_mask_type='block16': the unstructured gate, the per-tile top-k (or mid)
        penalty, binarise push, EMA, per-tile hard view, masked weight and flip count in one kernel."""
        self._check_tile16()
        if not self._is_placeholder("frozen_mask_flags"):
            raise NotImplementedError("freeze bands are built for the 2:4 mask update, not for block16 masks")
        if self._beta_structural(step) > 0.0:
            raise NotImplementedError("beta_structural mixing is an N:M target; it is not combined with block16 masks")
        self._buffers_ready()
        self._refresh_score()
        lam = 0.0 if lambda_mid is None else float(lambda_mid)
        mode = str(getattr(self.cfg, "mask_penalty_mode", "mid") or "mid")
        pmode = 0
        if lam != 0.0:
            if mode not in ("block16", "mid"):
                raise NotImplementedError(f"mask_penalty_mode={mode!r} is not combined with block16 masks")
            pmode = 1 if mode == "block16" else 2
        hx_new = self._next_hardening_x(step)
        ops.mask_update_tile16(self._score, self._norm, self._gate_tau(step), self.mask.data, self._stats,
                               keep_k=self._tile16_keep_k(), W=self.weight.data, wm=self._wm,
                               temperature=self._temperature(step), mask_lr=float(self.cfg.mask_lr),
                               pen=float(self.mask_penalty_lr) * lam, penalty_mode=pmode,
                               binarize_decay=float(getattr(self.cfg, "mask_binarize_decay", 0.0) or 0.0), hx=hx_new)
        self.hardening_x = hx_new
        self._fuse_score_next = self._predict_mask_update(step + 1)
        self.last_mask_stats = self._stats
        self.weight.flipped_mask = _LazyInt(self._stats, _lib.MSTAT_FLIPS)
        self.weight.init_flipped_mask = 0
        self.weight.mask = self.mask

    def _block_gate(self, step: int):
        """Per-block gate of legacy/sparse_modeling.py:1122-1157: RMS of the normalised score over each
        block, its quantile at the scheduled sparsity as threshold, a sigmoid at the temperature."""
        bs = self._block_size()
        self._refresh_score()
        _, sq = ops.block_sums(self._score, bs, norm=self._norm)
        rms = torch.sqrt(sq / float(bs * bs))
        tau = torch.quantile(rms.flatten().float(), q=float(self._effective_sparsity(step)))
        return torch.sigmoid((rms - tau) / (float(self._temperature(step)) + 1e-8)).contiguous()

    def _update_mask_block(self, step: int, lambda_mid):
        """update_mask in the block-sparse modes (legacy/sparse_modeling.py:1122-1157, 1395-1530, 1573-1663):
        block gate, pull towards the top blocks of the current mask, binarise push, EMA, block means
        written back over each block, hard view = top blocks by block RMS. Three passes over the layer
        beside the score (block sums of score and of mask, the EMA) and one that rewrites mask and
        masked weight; quantile and block ranking work on [out/bs, in/bs] arrays."""
        bs = self._block_size()
        if self.out_features < bs or self.in_features < bs or self.in_features % 4 != 0:
            raise NotImplementedError("block-sparse masks need at least one whole block and in_features % 4 == 0")
        if not self._is_placeholder("frozen_mask_flags"):
            raise NotImplementedError("freeze bands are built for the 2:4 mask update, not for block masks")
        if self._beta_structural(step) > 0.0:
            raise NotImplementedError("beta_structural mixing is an N:M target; it is not combined with block masks")
        self._buffers_ready()
        n = float(bs * bs)
        gate = self._block_gate(step)
        prev_sum, prev_sq = ops.block_sums(self.mask.data, bs)
        keep_prev = self._block_keep(torch.sqrt(prev_sq / n))
        lam = 0.0 if lambda_mid is None else float(lambda_mid)
        mode = str(getattr(self.cfg, "mask_penalty_mode", "mid") or "mid")
        pen, target = 0.0, None
        if lam != 0.0:
            scale = float(self.mask_penalty_lr) * lam
            if mode in ("block_sparse16", "block_sparse32"):
                if mode != self.hard_mask_type:
                    raise NotImplementedError("block penalty and block hard mask must use the same block size")
                # target: the top blocks by the MEAN of the current mask (:1420-1443)
                pen, target = scale, self._block_keep(prev_sum / n).float().contiguous()
            elif mode == "mid":
                # G - s (1 - 2m) = G - (-2s) (m - 1/2)
                pen, target = -2.0 * scale, torch.full_like(gate, 0.5)
            else:
                raise NotImplementedError(f"mask_penalty_mode={mode!r} is not combined with block masks")
        new_sum = ops.block_mask_update(self.mask.data, bs, gate, target, mask_lr=float(self.cfg.mask_lr), pen=pen,
                                        binarize_decay=float(getattr(self.cfg, "mask_binarize_decay", 0.0) or 0.0))
        hx_new = self._next_hardening_x(step)
        value = (new_sum / n).contiguous()
        keep_new = self._block_keep(value)  # the mask is block-constant now: its block RMS is the value itself
        ops.block_mask_apply(self.mask.data, bs, keep_new, value=value, W=self.weight.data, wm=self._wm, hx=hx_new)
        self.hardening_x = hx_new
        self._fuse_score_next = False
        self._stats.zero_()
        self._stats[_lib.MSTAT_FLIPS] = (keep_prev ^ keep_new).sum().double() * n
        self.last_mask_stats = self._stats
        self.weight.flipped_mask = _LazyInt(self._stats, _lib.MSTAT_FLIPS)
        self.weight.init_flipped_mask = 0
        self.weight.mask = self.mask

    def _launch_mask_update(self, score, norm, step, *, pen, pmode, tau, owner, score_bf16=False, pen_mask=None):
        """The fused update kernel on this layer's mask with the gate schedule (temperature, mask_lr,
        beta mixing, binarise push, hardening) of ``owner`` (the layer itself, or the gate layer of a
        GLU pair updated jointly)."""
        cfg = owner.cfg
        hx_new = owner._next_hardening_x(step)
        bands = {}
        if not self._is_placeholder("frozen_mask_flags"):
            if owner is not self or pen_mask is not None:
                raise NotImplementedError("freeze bands are not combined with the GLU joint mask update")
            # the low band snaps at every update, the high band from step 2000 on
            # (legacy/sparse_modeling.py:1621-1642)
            bands = dict(frozen=self.frozen_mask_flags.data, freeze_low=float(self.cfg.freeze_low),
                         freeze_high=float(self.cfg.freeze_high), freeze_apply_high=step >= 2000)
        common = dict(tau=tau, W=self.weight.data, wm=self._wm, temperature=owner._temperature(step),
                      mask_lr=float(cfg.mask_lr), pen=pen, penalty_mode=pmode, beta_s=owner._beta_structural(step),
                      binarize_decay=float(getattr(cfg, "mask_binarize_decay", 0.0) or 0.0), hx=hx_new,
                      structured_exact=bool(getattr(cfg, "structured_exact", False)), score_bf16=score_bf16)
        if self._general_nm():
            if bands:
                raise NotImplementedError(f"freeze bands are built for 2:4 groups (the layer has N:M = {self.N}:{self.M})")
            ops.mask_update_nm(score, norm, self.mask.data, self._stats, int(self.N), int(self.M), pen_mask=pen_mask,
                               threshold_view=self._threshold_view(), **common)
        else:
            ops.mask_update_nm24(score, norm, self.mask.data, self._stats, meta=self._meta, pen_mask=pen_mask,
                                 **common, **bands)
        self.hardening_x = hx_new
        self._fuse_score_next = self._predict_mask_update(step + 1)
        self.last_mask_stats = self._stats
        self._wm_key = self._current_key()
        self.weight._sf_wm_stale = False
        # The flip count stays on the device; reading the attribute costs one synchronisation.
        self.weight.flipped_mask = _LazyInt(self._stats, _lib.MSTAT_FLIPS)
        self.weight.init_flipped_mask = 0
        self.weight.mask = self.mask


class _LazyInt:
    """Integer that lives in a device tensor until somebody looks at it."""

    __slots__ = ("_t", "_i", "_v")

    def __init__(self, t, i):
        self._t, self._i, self._v = t.clone(), i, None

    def __int__(self):
        if self._v is None:
            self._v = int(self._t[self._i].item())
        return self._v

    __index__ = __int__

    def __repr__(self):
        return str(int(self))

    def __eq__(self, other):
        return int(self) == int(other)

    def __add__(self, other):
        return int(self) + int(other)

    __radd__ = __add__


# ----------------------------------------------------------------------------------------
# distillation wrapper
# ----------------------------------------------------------------------------------------
class _KLDivLoss(torch.autograd.Function):
    """Scalar distillation KL with the chunk rules of legacy/sparse_modeling.py:1749-1828: rows are
    summed in chunks of 2048 / 512 / 128 tokens (by vocabulary size), a chunk whose sum is not
    finite is dropped, the total is scaled by temperature^2 / tokens."""

    @staticmethod
    def forward(ctx, student_logits, teacher_logits, temperature):
        shape = student_logits.shape
        s2 = student_logits.reshape(-1, shape[-1]).contiguous()
        t2 = teacher_logits.reshape(-1, shape[-1]).to(s2.dtype).contiguous()
        rows, vocab = s2.shape
        chunk = 128 if vocab > 100000 else (512 if vocab > 50000 else 2048)
        row_kl, lse = ops.kl_div_fwd(s2, t2, temperature, 100.0)
        nchunks = (rows + chunk - 1) // chunk
        padded = torch.zeros(nchunks * chunk, dtype=torch.float64, device=s2.device)
        padded[:rows] = row_kl.double()
        sums = padded.view(nchunks, chunk).sum(1)
        keep = torch.isfinite(sums)
        total = torch.where(keep, sums, torch.zeros_like(sums)).sum()
        kl = (total * (float(temperature) ** 2) / rows).to(student_logits.dtype)
        ok = torch.isfinite(kl)
        kl = torch.where(ok, kl, torch.zeros_like(kl))
        row_keep = (keep & ok).repeat_interleave(chunk)[:rows].to(torch.float32)
        ctx.save_for_backward(s2, t2, lse, row_keep)
        ctx.temperature, ctx.shape, ctx.rows = float(temperature), shape, rows
        return kl

    @staticmethod
    def backward(ctx, g):
        s2, t2, lse, row_keep = ctx.saved_tensors
        scale = row_keep * (g.float() * (ctx.temperature ** 2) / ctx.rows)
        grad = ops.kl_div_bwd(s2, t2, lse, scale.contiguous(), ctx.temperature, 100.0)
        return grad.view(ctx.shape), None, None


class Distill_Model(torch.nn.Module):
    """Student / teacher wrapper of the reference (legacy/sparse_modeling.py:1668-1843): the models
    return ``(logits, loss, hidden_states)``; ``forward`` returns ``(student logits, task loss,
    layerwise loss or None, KL loss)``. The KL term is one fused kernel per direction."""

    def __init__(self, model, teacher=None, output_hidden_state=False):
        super().__init__()
        self.student = model
        self.teacher = teacher
        self.student.config.output_hidden_state = output_hidden_state
        self.teacher.config.output_hidden_state = output_hidden_state
        self.output_hidden_state = output_hidden_state
        self.teacher.eval()

    def forward(self, idx, targets=None):
        if self.teacher is None:
            student_logits, task_loss, _ = self.student(idx, targets)
            return student_logits, task_loss, None, torch.tensor(0.0, device=idx.device)
        student_logits, task_loss, student_hidden = self.student(idx, targets)
        with torch.no_grad():
            try:
                tdev = next(self.teacher.parameters()).device
            except Exception:
                tdev = idx.device
            idx_t = idx.to(tdev) if idx.device != tdev else idx
            targets_t = None if targets is None else (targets.to(tdev) if targets.device != tdev else targets)
            teacher_logits, _, teacher_hidden = self.teacher(idx_t, targets_t)
        if teacher_logits.device != student_logits.device:
            teacher_logits = teacher_logits.to(device=student_logits.device, dtype=student_logits.dtype)
        layerwise = None
        if self.output_hidden_state:
            if student_hidden is not None and teacher_hidden is not None:
                if len(teacher_hidden) == len(student_hidden):
                    teacher_hidden = [t.to(device=student_logits.device, dtype=student_logits.dtype) for t in teacher_hidden]
                layerwise = self.layerwise_loss(student_hidden, teacher_hidden)
            else:
                layerwise = 0.0
        return student_logits, task_loss, layerwise, self.kl_loss(student_logits, teacher_logits)

    def kl_loss(self, student_logits, teacher_logits, temperature=2):
        return _KLDivLoss.apply(student_logits, teacher_logits.detach(), float(temperature))

    def layerwise_loss(self, student_hidden_states, teacher_hidden_states):
        loss = 0.0
        eps = torch.finfo(torch.bfloat16).eps
        for s, t in zip(student_hidden_states, teacher_hidden_states):
            loss = loss + (s - t).pow(2).mean() / (t.pow(2).mean() + eps)
        return loss
