"""CPU oracle for the SparseLinear hot path.  TEST INFRASTRUCTURE ONLY.

A restatement, in plain torch-CPU tensor code, of the algorithms of the SparseForge
reference (liuhanzuo/SparseForge; citations are ``file:line`` inside that project). Only
``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline leg of ``bench.py`` may import
this module, and only as the checker; nothing in ``sparseforge_b200/`` imports it.

Parity status: the reference ships no tests or golden vectors, so the oracle is pinned
against outputs of the reference itself: ``tests/golden/make_golden.py`` imports the
reference (torch 2.11 CPU), runs it on seeded inputs with ``torch.topk`` made tie-stable
(lower index wins, as the specification of this path requires) and stores its inputs,
intermediates and outputs; ``tests/test_oracle_golden.py`` replays them through this module.

The arithmetic lives in PyTorch ATen (a dependency of the reference, ``requirements.txt:2``
``torch>=2.1.0``); rounding points below follow what ATen does for the dtype mix used
(bf16 weights and gradients, fp32 mask / Hessian / score).
"""
from __future__ import annotations

import math

import numpy as np
import torch


# --------------------------------------------------------------------------------------
# top-N of M with the tie rule "lower index wins"
# --------------------------------------------------------------------------------------
def stable_topk_indices(x: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries along the last dim; equal values keep index order.

    Stands in for ``torch.topk(..., largest=True).indices`` (used at
    legacy/sparse_modeling.py:597, 732, 1172, 1213, 1380, 1559), whose tie order is
    unspecified. NaN sorts as the largest value, as in torch.
    """
    return torch.sort(x, dim=-1, descending=True, stable=True).indices[..., :k]


def topn_indicator(x2d: torch.Tensor, n: int = 2, m: int = 4, dtype=None) -> torch.Tensor:
    """0/1 tensor marking the top-n of every group of m along the last dim (cols % m == 0)."""
    rows, cols = x2d.shape
    g = x2d.detach().float().view(rows, cols // m, m)
    idx = stable_topk_indices(g, n)
    out = torch.zeros_like(g, dtype=dtype or x2d.dtype)
    out.scatter_(-1, idx, 1.0)
    return out.view(rows, cols)


def hard_mask_from_soft(soft: torch.Tensor, mode: str = "structured", n: int = 2, m: int = 4) -> torch.Tensor:
    """legacy/sparse_modeling.py:510-735, modes 'structured' (:720-735), 'nm_2_4' (:578-603),
    'unstructured' (:526-527), 'none' (:523-524)."""
    if mode == "none":
        return torch.ones_like(soft)
    if mode == "unstructured" or soft.dim() != 2:
        return (soft > 0.5).to(soft.dtype)
    rows, cols = soft.shape
    if mode == "structured":
        if cols % m != 0:
            raise ValueError(f"in_features ({cols}) must be divisible by M ({m}).")
        return topn_indicator(soft, n, m)
    if mode == "nm_2_4":
        full = (cols // 4) * 4
        hard = torch.ones_like(soft)
        if full > 0:
            hard[:, :full] = topn_indicator(soft[:, :full].contiguous(), 2, 4)
        return hard
    raise ValueError(f"Invalid hard mask_type: {mode}")


def meta_from_hard(hard: torch.Tensor) -> torch.Tensor:
    """Logical 2:4 metadata of a 0/1 mask: per group nibble i0 | (i1 << 2) (i0 < i1 kept column
    offsets), two groups per byte (low nibble first), rows of ceil(cols/8) bytes. Groups of
    the ragged tail (beyond (cols//4)*4) get nibble 0. The reference has no metadata format;
    this is the canonical form the CUDA path is compared with."""
    rows, cols = hard.shape
    groups = cols // 4
    h = (hard[:, : groups * 4] > 0.5).view(rows, groups, 4).to(torch.int64)
    pos = torch.arange(4).view(1, 1, 4)
    big = torch.where(h > 0, pos, torch.full_like(pos, 99).expand_as(h))
    i0 = big.min(dim=-1).values
    small = torch.where(h > 0, pos, torch.full_like(pos, -1).expand_as(h))
    i1 = small.max(dim=-1).values
    nib = (i0 | (i1 << 2)).to(torch.uint8)
    bytes_per_row = (cols + 7) // 8
    padded = torch.zeros(rows, bytes_per_row * 2, dtype=torch.uint8)
    padded[:, :groups] = nib
    return (padded[:, 0::2] | (padded[:, 1::2] << 4)).contiguous()


# --------------------------------------------------------------------------------------
# Hutchinson accumulation and scores
# --------------------------------------------------------------------------------------
def hutchinson_accumulate(H: torch.Tensor, hvp: torch.Tensor, v: torch.Tensor, beta: float) -> torch.Tensor:
    """legacy/utils.py:804-868 (non-FSDP branch, world size 1): H <- beta H + (1-beta) clamp(hvp*v, 0)."""
    d = torch.clamp((hvp * v.to(hvp.dtype)).detach(), min=0.0)
    return H.clone().mul_(beta).add_(d, alpha=1 - beta)


def grad_hessian_ema(grad_ema, H, g, beta):
    """SparseLinear.update_grad_hessian_ema, legacy/sparse_modeling.py:901-922: the gradient EMA (kept
    for the movement metric) and, when the layer holds a Hessian tensor, the g^2 proxy folded into it.
    Returns (grad_ema, H) as new tensors; H may be None."""
    b = float(beta)
    e = grad_ema.clone().mul_(b).add_(g, alpha=1 - b)
    Hn = None if H is None else H.clone().mul_(b).add_(g * g, alpha=1 - b)
    return e, Hn


def wanda_add_batch(scaler_row, nsamples, inp):
    """SparseLinear.add_batch, legacy/sparse_modeling.py:884-898: running mean over samples of the
    squared L2 norm of every input channel. Returns the new scaler_row and sample count."""
    if inp.dim() == 2:
        inp = inp.unsqueeze(0)
    batch = inp.shape[0]
    if inp.dim() == 3:
        inp = inp.reshape(-1, inp.shape[-1])
    s = scaler_row.clone().mul_(nsamples / (nsamples + batch + 1e-8))
    nsamples += batch
    s.add_((torch.norm(inp.t().float(), p=2, dim=1) ** 2) / max(nsamples, 1))
    return s, nsamples


def importance_score(W, metric="hessian_obd", H=None, grad_ema=None, temperature=1.0, scaler_row=None):
    """legacy/sparse_modeling.py:1041-1079."""
    eps = 1e-8
    if metric == "wanda":
        return W.abs() * torch.sqrt(scaler_row.reshape(1, -1) + eps)
    if metric == "magnitude":
        return W.abs()
    if metric == "movement":
        return (W * grad_ema).abs() / max(float(temperature), eps)
    if metric == "hessian_obd":
        return (H + eps) * (W * W)
    if metric == "hessian_ratio":
        return W.abs() / torch.sqrt(H + eps)
    if metric == "hessian":
        return H
    raise ValueError(metric)


def score_norm_stats(scores: torch.Tensor):
    """mean and population std + 1e-6 of the fp32 scores, legacy/sparse_modeling.py:1085-1087."""
    s = scores.float()
    return s.mean(), s.std(unbiased=False) + 1e-6


def normalize_scores(scores: torch.Tensor) -> torch.Tensor:
    """legacy/sparse_modeling.py:1084-1088."""
    mu, sigma = score_norm_stats(scores)
    return ((scores.float() - mu) / sigma).to(scores.dtype)


# --------------------------------------------------------------------------------------
# gate target and mask update (structured N:M = 2:4)
# --------------------------------------------------------------------------------------
def gate_target_structured(scores_norm, temperature, *, exact=False, beta_s=0.0, n=2, m=4):
    """legacy/sparse_modeling.py:1164-1185 (+ beta mixing :1199-1225)."""
    rows, cols = scores_norm.shape
    s = scores_norm.float().view(rows, cols // m, m)
    idx = stable_topk_indices(s, n)
    tau = torch.gather(s, -1, idx[..., n - 1 : n])
    Tt = torch.tensor(float(temperature), dtype=torch.float32)
    if exact:
        G = torch.zeros_like(s, dtype=scores_norm.dtype)
        G.scatter_(-1, idx, 1.0)
        G = G.view(rows, cols)
    else:
        G = torch.sigmoid((s - tau) / (Tt + 1e-8)).view(rows, cols).to(scores_norm.dtype)
    if beta_s > 0.0:
        target = topn_indicator(scores_norm, n, m, dtype=G.dtype)
        G = ((1.0 - beta_s) * G.float() + beta_s * target.float()).to(G.dtype)
    return G


def tau_unstructured(scores_norm, sparsity, tau_sample_size=262144, sample_idx=None):
    """legacy/sparse_modeling.py:987-1015 (single process): quantile of a random sample of the
    normalised scores. The sample positions are an input here (the reference draws them with
    torch.randint on the tensor's device)."""
    flat = scores_norm.flatten()
    n = flat.numel()
    m = int(tau_sample_size) if tau_sample_size is not None else n
    sample = flat[sample_idx] if (m > 0 and n > m) else flat
    return torch.quantile(sample.float(), q=float(sparsity))


def gate_target_unstructured(scores_norm, tau, temperature, *, beta_s=0.0, n=2, m=4):
    """legacy/sparse_modeling.py:1099-1162 (non block-sparse branch, :1162) + beta mixing :1199-1225."""
    Tt = torch.tensor(float(temperature), dtype=torch.float32)
    G = torch.sigmoid((scores_norm.float() - tau) / (Tt + 1e-8)).to(scores_norm.dtype)
    if beta_s > 0.0:
        target = topn_indicator(scores_norm, n, m, dtype=G.dtype)
        G = ((1.0 - beta_s) * G.float() + beta_s * target.float()).to(G.dtype)
    return G


def mask_update(mask, G, *, mask_lr, lambda_mid=0.0, pen_lr=None, penalty_mode="mid", binarize_decay=0.0,
                n=2, m=4):
    """legacy/sparse_modeling.py:1288-1593 for the structured / nm_2_4 / mid penalty modes.
    Returns the new mask."""
    a = float(mask_lr)
    pen_lr = a if pen_lr is None else float(pen_lr)
    if float(lambda_mid) != 0.0:
        if penalty_mode in ("structured_topn", "nm_2_4"):
            target = topn_indicator(G, n, m, dtype=G.dtype)
            G = G - (pen_lr * float(lambda_mid)) * (mask.to(G.dtype) - target)
        elif penalty_mode == "mid":
            G = G - (pen_lr * float(lambda_mid)) * (1.0 - 2.0 * mask).to(G.dtype)
        else:
            raise ValueError(penalty_mode)
        G = G.clamp(0.0, 1.0)
    d = float(binarize_decay)
    if d != 0.0:
        G = G.clone()
        lt, gt = G < 0.5, G > 0.5
        G[lt] = G[lt] * (1.0 - d)
        G[gt] = G[gt] * (1.0 + d)
    return mask.clone().mul_(1 - a).add_(G, alpha=a).clamp_(0.0, 1.0)


# --------------------------------------------------------------------------------------
# block-sparse soft masks (hard_mask_type block_sparse16 / block_sparse32)
# --------------------------------------------------------------------------------------
def freeze_gate(G, mask, frozen):
    """legacy/sparse_modeling.py:1227-1229: a frozen entry's gate target is its own mask value."""
    return torch.where(frozen.bool(), mask, G)


def freeze_bands(mask, frozen, low, high, step):
    """Tail of update_mask, legacy/sparse_modeling.py:1621-1642: entries <= low snap to 0 at every
    update, entries >= high snap to 1 from step 2000 on; what was snapped is flagged."""
    mask, frozen = mask.clone(), frozen.clone()
    f0, f1 = mask <= low, mask >= high
    mask[f0] = 0.0
    applied = f0.clone()
    if step >= 2000:
        mask[f1] = 1.0
        applied |= f1
    return mask, torch.maximum(frozen, applied.to(frozen.dtype))


def harden_fraction(masks, flags, fraction=0.2, band_low=0.4, band_high=0.6):
    """legacy/utils.py:1236-1276 on lists of masks / flags; returns (masks, flags, count)."""
    masks, flags = [m.clone() for m in masks], [f.clone() for f in flags]
    sels = [(~f.bool()) & (m > band_low) & (m < band_high) for m, f in zip(masks, flags)]
    diffs = [(m[s] - 0.5).abs() for m, s in zip(masks, sels)]
    all_diff = torch.cat(diffs) if diffs else torch.zeros(0)
    k = int(all_diff.numel() * fraction)
    if k <= 0:
        return masks, flags, 0
    thr = torch.topk(all_diff, k, largest=False).values.max()
    count = 0
    for m, f, s, d in zip(masks, flags, sels, diffs):
        pick = torch.zeros_like(s)
        pick[s] = d <= thr
        m[pick] = (m[pick] > 0.5).to(m.dtype)
        f[pick] = 1.0
        count += int(pick.sum())
    return masks, flags, count


def _block_view(x, bs):
    rows, cols = x.shape
    ob, ib = rows // bs, cols // bs
    return x[: ob * bs, : ib * bs].float().reshape(ob, bs, ib, bs), ob, ib


def block_keep(block_values, sparsity_ratio):
    """0/1 [ob, ib]: the round((1 - sr) * blocks) largest blocks, ties to the lower flat index
    (legacy/sparse_modeling.py:621-637 with a tie-stable top-k)."""
    flat = block_values.flatten()
    total = flat.numel()
    k = max(0, min(total, int(round((1.0 - float(sparsity_ratio)) * total))))
    keep = torch.zeros(total)
    if k > 0:
        keep[stable_topk_indices(flat, k)] = 1.0
    return keep.view_as(block_values)


def _expand_blocks(block_values, like, bs, fill=1.0):
    ob, ib = block_values.shape
    out = torch.full(like.shape, float(fill), dtype=torch.float32)
    out[: ob * bs, : ib * bs] = block_values.float().repeat_interleave(bs, 0).repeat_interleave(bs, 1)
    return out


def blockify(x, bs):
    """legacy/sparse_modeling.py:461-508: block means broadcast over each whole block."""
    tiles, ob, ib = _block_view(x, bs)
    out = x.clone().float()
    out[: ob * bs, : ib * bs] = tiles.mean(dim=(1, 3)).repeat_interleave(bs, 0).repeat_interleave(bs, 1)
    return out.to(x.dtype)


def hard_mask_block(soft, bs, sparsity_ratio):
    """legacy/sparse_modeling.py:607-718: whole blocks kept by the RMS of the soft mask per block; the
    ragged tail stays 1."""
    tiles, ob, ib = _block_view(soft, bs)
    rms = (tiles ** 2).mean(dim=(1, 3)).sqrt()
    return _expand_blocks(block_keep(rms, sparsity_ratio), soft, bs).to(soft.dtype)


def gate_target_block(scores_norm, bs, sparsity, temperature):
    """legacy/sparse_modeling.py:1122-1157: RMS of the normalised scores per block, threshold at the
    quantile of the block values, sigmoid at the temperature; 1 in the ragged tail."""
    tiles, ob, ib = _block_view(scores_norm, bs)
    rms = (tiles ** 2).mean(dim=(1, 3)).sqrt()
    tau = torch.quantile(rms.flatten().float(), q=float(sparsity))
    Tt = torch.tensor(float(temperature), dtype=torch.float32)
    return _expand_blocks(torch.sigmoid((rms.float() - tau) / (Tt + 1e-8)), scores_norm, bs).to(scores_norm.dtype)


def mask_update_block(mask, G, bs, *, mask_lr, sparsity_ratio, lambda_mid=0.0, pen_lr=None, penalty_mode="mid",
                      binarize_decay=0.0):
    """legacy/sparse_modeling.py:1395-1530 (block penalty: pull towards the top blocks by the block
    MEAN of the current mask), :1567-1593 (mid pull, clamp, binarise push, EMA), :1600 (blockify)."""
    a = float(mask_lr)
    pen_lr = a if pen_lr is None else float(pen_lr)
    if float(lambda_mid) != 0.0:
        if penalty_mode in ("block_sparse16", "block_sparse32"):
            tiles, ob, ib = _block_view(mask, bs)
            target = _expand_blocks(block_keep(tiles.mean(dim=(1, 3)), sparsity_ratio), mask, bs)
            G = G - (pen_lr * float(lambda_mid)) * (mask.to(G.dtype) - target.to(G.dtype))
        elif penalty_mode == "mid":
            G = G - (pen_lr * float(lambda_mid)) * (1.0 - 2.0 * mask).to(G.dtype)
        else:
            raise ValueError(penalty_mode)
        G = G.clamp(0.0, 1.0)
    d = float(binarize_decay)
    if d != 0.0:
        G = G.clone()
        lt, gt = G < 0.5, G > 0.5
        G[lt] = G[lt] * (1.0 - d)
        G[gt] = G[gt] * (1.0 + d)
    return blockify(mask.clone().mul_(1 - a).add_(G, alpha=a).clamp_(0.0, 1.0), bs)


def _tile16_topk(x, keep_k):
    """0/1 tensor: the keep_k largest entries of every 16 x 16 tile, ties to the lower row-major
    position inside the tile (legacy/sparse_modeling.py:549-571 with a tie-stable top-k)."""
    rows, cols = x.shape
    ob, ib = rows // 16, cols // 16
    tiles = x.float().reshape(ob, 16, ib, 16).permute(0, 2, 1, 3).reshape(ob, ib, 256)
    keep = torch.zeros_like(tiles)
    if keep_k >= 256:
        keep.fill_(1.0)
    elif keep_k > 0:
        keep.scatter_(-1, stable_topk_indices(tiles, keep_k), 1.0)
    return keep.view(ob, ib, 16, 16).permute(0, 2, 1, 3).reshape(rows, cols)


def hard_mask_tile16(soft, sparsity_ratio):
    """legacy/sparse_modeling.py:537-574 for sizes that are multiples of 16."""
    keep_k = max(0, min(256, int(round((1.0 - float(sparsity_ratio)) * 256))))
    return _tile16_topk(soft, keep_k).to(soft.dtype)


def mask_update_tile16(mask, G, *, mask_lr, sparsity_ratio, lambda_mid=0.0, pen_lr=None, penalty_mode="block16",
                       binarize_decay=0.0):
    """legacy/sparse_modeling.py:1298-1348 ('block16' pull towards the per-tile top-k of the gate),
    :1567-1593 (mid pull, clamp, binarise push, EMA)."""
    a = float(mask_lr)
    pen_lr = a if pen_lr is None else float(pen_lr)
    if float(lambda_mid) != 0.0:
        if penalty_mode == "block16":
            keep_k = max(0, min(256, int(round((1.0 - float(sparsity_ratio)) * 256))))
            G = G - (pen_lr * float(lambda_mid)) * (mask.to(G.dtype) - _tile16_topk(G, keep_k).to(G.dtype))
        elif penalty_mode == "mid":
            G = G - (pen_lr * float(lambda_mid)) * (1.0 - 2.0 * mask).to(G.dtype)
        else:
            raise ValueError(penalty_mode)
        G = G.clamp(0.0, 1.0)
    d = float(binarize_decay)
    if d != 0.0:
        G = G.clone()
        lt, gt = G < 0.5, G > 0.5
        G[lt] = G[lt] * (1.0 - d)
        G[gt] = G[gt] * (1.0 + d)
    return mask.clone().mul_(1 - a).add_(G, alpha=a).clamp_(0.0, 1.0)


def glu_joint_update(gate_score, up_score, gate_mask, up_mask, *, temperature, mask_lr, lambda_mid=0.0,
                     pen_lr=None, penalty_mode="mid", binarize_decay=0.0, beta_s=0.0, exact=False, n=2, m=4):
    """Joint update of a GLU gate / up pair, legacy/utils.py:363-479: one gate target from the
    summed raw scores (:407-412, :536-613), the penalty pull taken from the GATE layer's mask
    (:616-643; modes other than structured_topn / mid only clamp), the binarise push (:423-431),
    then the same target moves both masks (:434-435). Returns (new gate mask, new up mask)."""
    joint = gate_score + up_score
    G = gate_target_structured(normalize_scores(joint).to(gate_mask.dtype), temperature, exact=exact, beta_s=beta_s, n=n, m=m)
    a = float(mask_lr)
    pen_lr = a if pen_lr is None else float(pen_lr)
    if float(lambda_mid) != 0.0:
        if penalty_mode == "structured_topn":
            G = G - (pen_lr * float(lambda_mid)) * (gate_mask.to(G.dtype) - topn_indicator(G, n, m, dtype=G.dtype))
        elif penalty_mode == "mid":
            G = G - (pen_lr * float(lambda_mid)) * (1.0 - 2.0 * gate_mask).to(G.dtype)
        G = G.clamp(0.0, 1.0)
    d = float(binarize_decay)
    if d != 0.0:
        G = G.clone()
        lt, gt = G < 0.5, G > 0.5
        G[lt] = G[lt] * (1.0 - d)
        G[gt] = G[gt] * (1.0 + d)
    return (gate_mask.clone().mul_(1 - a).add_(G, alpha=a).clamp_(0.0, 1.0),
            up_mask.clone().mul_(1 - a).add_(G, alpha=a).clamp_(0.0, 1.0))


def beta_structural(step, start, end):
    """legacy/sparse_modeling.py:966-985: smooth-step ramp of the structural mixing weight."""
    if end <= start or step < start:
        return 0.0
    if step >= end:
        return 1.0
    t = float(step - start) / float(end - start)
    return float(3.0 * t * t - 2.0 * t * t * t)


def hardening_x(step, start, duration):
    """legacy/sparse_modeling.py:1603-1619."""
    if duration <= 0:
        return 0.0 if (step >= start and start > 0) else 1.0
    if step < start:
        return 1.0
    if step >= start + duration:
        return 0.0
    return max(0.0, min(1.0, 1.0 - float(step - start) / float(max(1, duration))))


def temperature_at(step, temp_init, temp_decay, temp_min, period=1):
    """legacy/sparse_modeling.py:932-942 (non block-sparse)."""
    updates = step // max(1, int(period))
    return float(max(float(temp_min), float(temp_init) * (float(temp_decay) ** updates)))


def flip_count(prev_mask, new_mask, mode="structured", n=2, m=4):
    """legacy/sparse_modeling.py:1659-1661."""
    hp = hard_mask_from_soft(prev_mask, mode, n, m) > 0.5
    hn = hard_mask_from_soft(new_mask, mode, n, m) > 0.5
    return int((hp ^ hn).sum().item())


def effective_mask(mask, hx, mode="structured", finalized=False, n=2, m=4):
    """legacy/sparse_modeling.py:745-771."""
    if hx >= 1.0 - 1e-6 or finalized:
        return mask
    return (hx * mask) + ((1.0 - hx) * hard_mask_from_soft(mask, mode, n, m))


def masked_weight(W, eff_mask, scale=1.0):
    """legacy/sparse_modeling.py:74-81."""
    w = W * eff_mask.to(W.dtype)
    return w * scale if scale != 1.0 else w


def mask_stats(mask, n=2, m=4):
    """Per-layer sums behind mid_penalty (legacy/utils.py:913), nm_2_4_tile_stats (:1028-1234, sorted
    groups: top-2 / bottom-2 sums; top-n / rest of every group of m in general) and the threshold path
    of sparsity_penalty (:1003)."""
    rows, cols = mask.shape
    m64 = mask.double()
    g = torch.sort(m64.view(rows, cols // m, m), dim=-1, descending=True).values
    return {
        "sum_m": float(m64.sum()),
        "sum_m1m": float((m64 * (1 - m64)).sum()),
        "sum_top2": float(g[..., :n].sum()),
        "sum_bot2": float(g[..., n:].sum()),
        "count_lt_half": float((mask < 0.5).sum()),
    }


# --------------------------------------------------------------------------------------
# masked linear forward / backward
# --------------------------------------------------------------------------------------
def linear_forward(x, W, eff_mask, bias=None, scale=1.0):
    """legacy/sparse_modeling.py:72-93."""
    w = masked_weight(W, eff_mask, scale)
    x2 = x.reshape(-1, x.shape[-1])
    y = x2.matmul(w.t())
    if bias is not None:
        y = y + bias
    return y.view(*x.shape[:-1], W.shape[0])


def linear_backward(x, W, eff_mask, dy, has_bias=False):
    """legacy/sparse_modeling.py:96-132 (decay = 0): returns (dx, dW, db)."""
    cd = dy.dtype
    dy2 = dy.reshape(-1, dy.shape[-1])
    x2 = x.reshape(-1, x.shape[-1]).to(cd)
    w = W.to(cd) * eff_mask.to(cd)
    dx = dy2.matmul(w).view_as(x)
    dW = dy2.t().matmul(x2)
    db = dy2.sum(dim=0) if has_bias else None
    return dx, dW, db


# --------------------------------------------------------------------------------------
# mask-aware AdamW
# --------------------------------------------------------------------------------------
class MaskedLinearSTE(torch.autograd.Function):
    """Masked linear with a straight-through weight gradient, made of differentiable torch ops so
    that a second backward pass (Hutchinson) runs through it: legacy/sparse_modeling.py:72-132.
    ``eff_mask`` is the effective mask of the step (no gradient)."""

    @staticmethod
    def forward(ctx, x, W, b, eff_mask):
        ctx.save_for_backward(x, W, eff_mask)
        ctx.has_bias = b is not None
        return torch.nn.functional.linear(x, W * eff_mask.to(W.dtype), b)

    @staticmethod
    def backward(ctx, gy):
        x, W, M = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        gx = gy.matmul(W * M.to(W.dtype))                      # :112-115
        gW = gy2.t().matmul(x.reshape(-1, x.shape[-1]))        # :117-125, no mask (straight-through)
        gb = gy2.sum(0) if ctx.has_bias else None              # :127-129
        return gx, gW, gb, None


def hutchinson_hvps(loss, weights, probes):
    """hvp_i = d<g, v>/dW_i with g = dloss/dW (graph kept): legacy/utils.py:760-790."""
    grads = torch.autograd.grad(loss, weights, create_graph=True, retain_graph=True)
    dot = sum((g * v).sum() for g, v in zip(grads, probes))
    return torch.autograd.grad(dot, weights, retain_graph=True)


def mid_penalty_value(masks, lambda_mid):
    """lambda * sum(m (1 - m)) / count over all layers: legacy/utils.py:875-938."""
    if lambda_mid <= 0:
        return 0.0
    tot = sum(float((m.double() * (1 - m.double())).sum()) for m in masks)
    return lambda_mid * tot / sum(m.numel() for m in masks)


def clip_grad_norm(grads, max_norm):
    """torch.nn.utils.clip_grad_norm_ (2-norm over all gradients; coefficient clamped to 1)."""
    total = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g) for g in grads]))
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    return [g * coef for g in grads], float(total)


def adamw_step(p, g, m, v, *, step, lr, betas, eps, weight_decay, mask=None, decay=0.0, adaptive_l1=0.0, v_max=None):
    """legacy/adamw.py:79-174 for one tensor. `step` is the 1-based step number after the
    increment at :146. Returns (p, m, v) as new tensors; with `v_max` (amsgrad=True, :142-156)
    the denominator uses the running maximum of v and (p, m, v, v_max) is returned."""
    p, m, v = p.clone(), m.clone(), v.clone()
    beta1, beta2 = betas
    p.mul_(1 - lr * weight_decay)
    grad = g
    if mask is not None:
        grad = grad.add(p * (1 - mask), alpha=decay)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    m.mul_(beta1).add_(grad, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
    if v_max is not None:
        v_max = torch.max(v_max, v)
        denom = (v_max.sqrt() / math.sqrt(bc2)).add_(eps)
    else:
        denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-(lr / bc1))
    if adaptive_l1 > 0.0 and p.dim() >= 2 and mask is not None:
        p.add_(adaptive_l1 * torch.sign(p) / denom, alpha=-lr)
    return (p, m, v) if v_max is None else (p, m, v, v_max)


# --------------------------------------------------------------------------------------
# hard-2:4 compression and block-sparse-16 layout
# --------------------------------------------------------------------------------------
def sparse24_compress(W, soft):
    """Kept values [out, in/2] (column order) and packed metadata of top2(soft); semantics of the
    finalisation bake-in legacy/main_llama.py:2552-2563 (weight.mul_(hard))."""
    hard = topn_indicator(soft.float(), 2, 4, dtype=torch.float32)
    rows, cols = W.shape
    keep = hard.view(rows, cols // 4, 4) > 0.5
    idx = torch.sort(keep.to(torch.int8), dim=-1, descending=True, stable=True).indices[..., :2]
    idx = torch.sort(idx, dim=-1).values
    vals = torch.gather(W.view(rows, cols // 4, 4), -1, idx).reshape(rows, cols // 2)
    return vals, meta_from_hard(hard), hard


def block16_keep_mask(W, density=0.5, bs=16):
    """0/1 mask keeping the round(density * #blocks) 16x16 blocks of largest Frobenius norm (same
    ordering as the block RMS of legacy/sparse_modeling.py:686-710 applied to |W|); ties go to
    the lower flat block index."""
    out, inn = W.shape
    ob, ib = out // bs, inn // bs
    tiles = W.float().view(ob, bs, ib, bs).permute(0, 2, 1, 3).reshape(ob * ib, bs * bs)
    score = (tiles ** 2).sum(dim=-1)
    k = int(round(density * ob * ib))
    order = torch.sort(score, descending=True, stable=True).indices[:k]
    keep = torch.zeros(ob * ib, dtype=torch.bool)
    keep[order] = True
    return keep.view(ob, 1, ib, 1).expand(ob, bs, ib, bs).reshape(out, inn).to(W.dtype)


def bsr16_convert(W, mask, bs=16):
    """legacy/triton_block_sparse.py:46-103: (blocks[nnz,16,16], row_ptr int32, col_idx int32)."""
    out, inn = W.shape
    ob, ib = out // bs, inn // bs
    blocked = (W * mask).view(ob, bs, ib, bs).permute(0, 2, 1, 3)
    nz = blocked.abs().float().sum(dim=(-1, -2)) > 0
    row_ptr = torch.zeros(ob + 1, dtype=torch.int32)
    row_ptr[1:] = torch.cumsum(nz.sum(dim=1), 0).to(torch.int32)
    rows_i, cols_i = torch.nonzero(nz, as_tuple=True)
    blocks = blocked[rows_i, cols_i].contiguous()
    if blocks.shape[0] == 0:
        blocks = torch.zeros(1, bs, bs, dtype=W.dtype)
    return blocks, row_ptr, cols_i.to(torch.int32)


def mask_log_stats(masks, sample_idx, bins=100, eps=1e-8):
    """legacy/utils.py:2069-2280 for one process and no block-sparse layers: sums in fp64, the
    entropy of clamp(m, eps, 1 - eps) (the clamp runs in the mask's dtype), quantiles from the
    histogram of the sampled entries (the sample positions are an input)."""
    import math

    tot = sum_m = sum_m2 = ent = 0.0
    cnt = {k: 0.0 for k in ("lt05", "lt01", "lt001", "gt90", "gt99", "gt05")}
    s_lt = s_gt = 0.0
    hist = torch.zeros(bins, dtype=torch.float64)
    for m, idx in zip(masks, sample_idx):
        md = m.double()
        tot += m.numel()
        sum_m += float(md.sum())
        sum_m2 += float((md * md).sum())
        mm = m.clamp(eps, 1 - eps).double()
        ent += float((-(mm * mm.log()) - ((1 - mm) * (1 - mm).log())).sum())
        cnt["lt05"] += float((m < 0.5).sum()); cnt["lt01"] += float((m < 0.1).sum()); cnt["lt001"] += float((m < 0.01).sum())
        cnt["gt90"] += float((m > 0.9).sum()); cnt["gt99"] += float((m > 0.99).sum()); cnt["gt05"] += float((m > 0.5).sum())
        s_lt += float(md[m < 0.5].sum()); s_gt += float(md[m > 0.5].sum())
        hist += torch.histc(m.reshape(-1)[idx].float(), bins=bins, min=0.0, max=1.0).double()
    mean = sum_m / tot
    cdf = hist.cumsum(0) / (hist.sum() + 1e-12)

    def q(p):
        i = int(torch.searchsorted(cdf, torch.tensor([p], dtype=cdf.dtype)).item())
        return (max(0, min(bins - 1, i)) + 0.5) / bins

    return {"mask_mean": mean, "mask_std": math.sqrt(max(sum_m2 / tot - mean * mean, 0.0)), "mask_entropy": ent / tot,
            "mask_hard_sparsity@0.5": cnt["lt05"] / tot, "mask_frac_lt_0.1": cnt["lt01"] / tot,
            "mask_frac_lt_0.01": cnt["lt001"] / tot, "mask_frac_gt_0.9": cnt["gt90"] / tot,
            "mask_frac_gt_0.99": cnt["gt99"] / tot, "mask_frac_gt_0.5": cnt["gt05"] / tot,
            "mask_mean_lt_0.5": s_lt / cnt["lt05"] if cnt["lt05"] > 0 else 0.0,
            "mask_mean_gt_0.5": s_gt / cnt["gt05"] if cnt["gt05"] > 0 else 0.0,
            "mask_p10": q(0.10), "mask_p50": q(0.50), "mask_p90": q(0.90)}


def kl_distill_loss(student_logits, teacher_logits, temperature=2.0, max_logit=100.0):
    """Distill_Model.kl_loss, legacy/sparse_modeling.py:1749-1828, with differentiable torch ops:
    chunks of 2048 / 512 / 128 token rows by vocabulary size, fp32 log-softmax of the clamped and
    tempered logits, chunks with a non-finite sum dropped, total * temperature^2 / tokens."""
    shape = student_logits.shape
    s2 = student_logits.reshape(-1, shape[-1])
    t2 = teacher_logits.reshape(-1, shape[-1])
    rows, vocab = s2.shape
    chunk = 128 if vocab > 100000 else (512 if vocab > 50000 else 2048)
    total = torch.zeros((), dtype=torch.float32)
    for i in range(0, rows, chunk):
        a = torch.log_softmax(s2[i:i + chunk].float().clamp(-max_logit, max_logit) / temperature, dim=-1)
        b = torch.log_softmax(t2[i:i + chunk].float().clamp(-max_logit, max_logit) / temperature, dim=-1)
        if torch.isnan(a).any() or torch.isnan(b).any():
            continue
        c = ((b - a) * b.exp()).sum()
        if torch.isfinite(c):
            total = total + c
    kl = (total * (temperature ** 2) / rows).to(student_logits.dtype)
    return kl if torch.isfinite(kl) else torch.zeros((), dtype=student_logits.dtype)


def slorb_init(W, mask, k, init_type="mean"):
    """(x_proj, SLoRB_Weight) of legacy/sparse_modeling.py:830-872 (block-sum projection; the bypass
    weight starts from the block mean / sum of the pruned part W (1 - mask))."""
    n, d = W.shape
    rows = d // k
    x_proj = torch.zeros(rows, d, dtype=W.dtype)
    for r in range(rows):
        x_proj[r, r * k:(r + 1) * k] = 1
    pruned = (W * (1.0 - mask)).view(n, rows, k)
    return x_proj, (pruned.mean(dim=2) if init_type == "mean" else pruned.sum(dim=2))


def slorb_bypass(x, x_proj, slorb_weight):
    """out += (x x_proj^T) SLoRB_Weight^T, legacy/sparse_modeling.py:790-794."""
    return torch.nn.functional.linear(torch.nn.functional.linear(x, x_proj), slorb_weight)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    """bf16 tensors are stored as their raw uint16 bits."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()
