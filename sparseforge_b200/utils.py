"""Model-level drivers of the mask / Hessian path.

Host-side mirror of the functions the reference training loop imports from ``legacy/utils.py``
(``legacy/main_llama.py:32-50``) that belong to the SparseLinear hot path. Each walks the model's
``SparseLinear`` modules and calls their kernels; layer-wide scalars stay on the device until the
caller reads them. The perplexity evaluators of that file are outside this path: their names
exist here so that the training script's import list resolves, and raise when called.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from . import _lib, ops
from .sparse_modeling import SparseLinear


def get_raw_model(model):
    """Innermost student / base model (legacy/utils.py:59-88)."""
    if hasattr(model, "_fsdp_wrapped_module"):
        inner = model._fsdp_wrapped_module
        if hasattr(inner, "student"):
            student = inner.student
            return getattr(student, "_fsdp_wrapped_module", student)
        return inner
    if hasattr(model, "module"):
        return model.module.student if hasattr(model.module, "student") else model.module
    if hasattr(model, "student"):
        student = model.student
        return getattr(student, "_fsdp_wrapped_module", student)
    return model


def _sparse_modules(model):
    return [m for _, m in get_raw_model(model).named_modules() if isinstance(m, SparseLinear)]


@torch.no_grad()
def set_model_mode(model, mode: str):
    """legacy/utils.py:91-95."""
    for m in _sparse_modules(model):
        m.mode = mode


@torch.no_grad()
def sync_weight(model, device=None):
    """legacy/utils.py:99-106."""
    if device is not None:
        model = model.to(device)
    for m in _sparse_modules(model):
        m.sync_weight()
        m.invalidate_masked_weight()


@torch.no_grad()
def initialize_model(model):
    """legacy/utils.py:110-116."""
    for m in _sparse_modules(model):
        m.initialize()


@torch.no_grad()
def update_model_grad_ema(model, update_hessian_with_grad2: bool = True):
    """legacy/utils.py:122-134."""
    for m in _sparse_modules(model):
        m.update_grad_hessian_ema(update_hessian_with_grad2=update_hessian_with_grad2)


@torch.no_grad()
def update_mask_penalty_lr(model, step: int, max_steps: int, penalty_lr_min: float, penalty_lr_max: float,
                           schedule: str = "linear"):
    """legacy/utils.py:141-180."""
    if schedule == "linear":
        cur = penalty_lr_min + (penalty_lr_max - penalty_lr_min) * min(1.0, step / max(1, max_steps))
    elif schedule == "cosine":
        f = 0.5 * (1.0 - math.cos(math.pi * min(1.0, step / max(1, max_steps))))
        cur = penalty_lr_min + (penalty_lr_max - penalty_lr_min) * f
    else:
        cur = penalty_lr_max
    for m in _sparse_modules(model):
        m.mask_penalty_lr = cur
    return cur


@torch.no_grad()
def harden_fraction(model, fraction: float = 0.2, band_low: float = 0.4, band_high: float = 0.6) -> int:
    """legacy/utils.py:1236-1276: rounds the `fraction` of not-yet-frozen mask entries inside
    (band_low, band_high) that lie closest to 0.5, over all layers together, to 0 / 1 and freezes them.
    A rarely used maintenance step (the threshold is one order statistic over all layers), done
    with tensor operations on the device; layers without freeze bands have no flags and are skipped
    (the reference fails on them)."""
    raw = get_raw_model(model)
    cands = []
    for m in _sparse_modules(raw):
        if m._is_placeholder("frozen_mask_flags"):
            continue
        sel = (m.frozen_mask_flags.data == 0) & (m.mask.data > band_low) & (m.mask.data < band_high)
        if bool(sel.any()):
            cands.append((m, sel, (m.mask.data[sel] - 0.5).abs()))
    if not cands:
        return 0
    all_diff = torch.cat([c[2] for c in cands])
    k = int(all_diff.numel() * fraction)
    if k <= 0:
        return 0
    thr = torch.topk(all_diff, k, largest=False).values.max()
    hardened = 0
    for m, sel, diff in cands:
        pick = torch.zeros_like(sel)
        pick[sel] = diff <= thr
        n = int(pick.sum().item())
        if n:
            m.mask.data[pick] = (m.mask.data[pick] > 0.5).to(m.mask.dtype)
            m.frozen_mask_flags.data[pick] = 1.0
            m.invalidate_masked_weight()
            hardened += n
    return hardened


def all_ranks_ok(ok: bool, device=None) -> bool:
    """True only if every rank passes True (the ok-flag the reference all-reduces with MIN after
    steps that may fail on one rank only, legacy/main_llama.py:637-651, 771-788). A rank that caught
    an exception passes False and every rank learns of it before the next collective."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return bool(ok)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(int(flag.item()))


def loss_is_finite_on_all_ranks(loss: torch.Tensor) -> bool:
    """The training loop's guard (legacy/main_llama.py:2075-2108): if the loss of any rank is not
    finite, every rank skips backward and the optimizer step, so that the collectives of the
    sharded step stay matched."""
    return all_ranks_ok(bool(torch.isfinite(loss.detach()).all().item()), device=loss.device)


def grad_sync_context(model, is_last_micro: bool):
    """Gradient-accumulation control of the training loop (legacy/main_llama.py:1997-2008): inside the
    returned context the backward pass of a micro-step that is not the last one exchanges no gradients.
    A wrapper with ``no_sync()`` (FSDP, DistributedDataParallel) is entered for those micro-steps; a
    DistributedDataParallel wrapper also gets ``require_backward_grad_sync`` set, as the reference does.
    Anything else (one process) gets a null context."""
    import contextlib

    target = model.student if hasattr(model, "student") and hasattr(model.student, "no_sync") else model
    if hasattr(target, "require_backward_grad_sync"):
        target.require_backward_grad_sync = bool(is_last_micro)
        return contextlib.nullcontext()
    if (not is_last_micro) and hasattr(target, "no_sync"):
        return target.no_sync()
    return contextlib.nullcontext()


def _identify_glu_pairs(sparse_modules_dict):
    """{gate name: up name} of the GLU pairs whose gate layer asks for a joint mask
    (``...mlp.gate_proj`` / ``up_proj`` and ``...mlp.w1`` / ``w3``): legacy/utils.py:313-360."""
    import re

    pairs = {}
    for pat, other in ((re.compile(r"(.+\.mlp)\.gate_proj$"), "up_proj"), (re.compile(r"(.+\.mlp)\.w1$"), "w3")):
        for name, mod in sparse_modules_dict.items():
            m = pat.match(name)
            if m and f"{m.group(1)}.{other}" in sparse_modules_dict and getattr(mod.cfg, "glu_joint_mask", False):
                pairs[name] = f"{m.group(1)}.{other}"
    return pairs


@torch.no_grad()
def _update_glu_joint_mask(gate, up, step, lambda_mid):
    """One mask update for a gate / up pair from the SUM of their importance scores
    (legacy/utils.py:363-479): the gate layer's schedule (temperature, mask_lr, beta mixing,
    binarise push, hardening) drives both, the penalised target is formed once from the gate
    layer's mask, and both masks move towards it. Three kernels per pair beyond the two score
    passes: the joint score with its statistics, and one fused update per layer."""
    if (not gate.change_mask) or gate.mask_type == "none":
        for m in (gate, up):
            m.weight.flipped_mask = 0
            m.weight.init_flipped_mask = 0
        return
    if step < int(gate.cfg.sparsity_warmup_steps):
        return
    if step % max(1, int(gate._mask_update_period(step))) != 0:
        return
    if gate.mask.shape != up.mask.shape:
        import warnings

        warnings.warn(f"[GLU Joint] Shape mismatch: gate={tuple(gate.mask.shape)}, up={tuple(up.mask.shape)}. "
                      "Falling back to independent update.")
        gate.update_mask(step, lambda_mid=lambda_mid)
        up.update_mask(step, lambda_mid=lambda_mid)
        return
    for m in (gate, up):
        m._check_mask_modes()
        m._check_2to4()
        m._refresh_score()
    joint = getattr(gate, "_joint_score", None)
    if joint is None or joint.shape != gate._score.shape or joint.device != gate._score.device:
        joint = gate._joint_score = torch.empty_like(gate._score)
    ops.score_sum(gate._score, up._score, joint, gate._norm, gate._scratch)
    gate._combine_shard_norm()
    lam = 0.0 if lambda_mid is None else float(lambda_mid)
    mode = str(getattr(gate.cfg, "mask_penalty_mode", "mid") or "mid")
    # the joint path knows the top-N pull and the mid pull; any other mode leaves the gate as it is
    pmode = {"structured_topn": _lib.PENALTY_TOPN, "mid": _lib.PENALTY_MID}.get(mode, 0) if lam != 0.0 else 0
    pen = float(gate.mask_penalty_lr) * lam if pmode else 0.0
    tau = gate._gate_tau(step, joint)
    # `up` first: its penalty pull reads the gate layer's mask as it was before this update
    up._launch_mask_update(joint, gate._norm, step, pen=pen, pmode=pmode, tau=tau, owner=gate,
                           pen_mask=gate.mask.data if pmode else None)
    gate._launch_mask_update(joint, gate._norm, step, pen=pen, pmode=pmode, tau=tau, owner=gate)


@torch.no_grad()
def calculate_model_mask(model, step=0, lambda_mid: float = 0.0):
    """legacy/utils.py:183-310. The mask update of a layer is local to its rows, so no parameter is
    gathered first (the reference summons every FSDP parameter here). GLU gate / up pairs whose
    config sets ``glu_joint_mask`` get one joint update."""
    named = {n: m for n, m in get_raw_model(model).named_modules() if isinstance(m, SparseLinear)}
    handled = set()
    if any(getattr(m.cfg, "glu_joint_mask", False) for m in named.values()):
        for gname, uname in _identify_glu_pairs(named).items():
            _update_glu_joint_mask(named[gname], named[uname], step, lambda_mid)
            handled.update((gname, uname))
    for n, m in named.items():
        if n not in handled:
            m.update_mask(step, lambda_mid=lambda_mid)


@torch.no_grad()
def calculate_flip_rate(model):
    """legacy/utils.py:691-704."""
    flipped = init_flipped = total = 0
    for m in _sparse_modules(model):
        flipped += int(getattr(m.weight, "flipped_mask", 0))
        init_flipped += int(getattr(m.weight, "init_flipped_mask", 0))
        total += int(getattr(m.weight, "param_count", m.weight.numel()))
    return flipped, flipped / max(total, 1), init_flipped, init_flipped / max(total, 1)


def _rademacher_like(t: torch.Tensor) -> torch.Tensor:
    """+-1 probe in the dtype of ``t`` (legacy/utils.py:710-711)."""
    return (torch.randint_like(t, low=0, high=2, dtype=torch.int8).float() * 2 - 1).to(dtype=t.dtype, device=t.device)


def update_hessian_hutchinson(model, loss):
    """Hutchinson estimate diag(H) ~ E[(Hv) * v] for every SparseLinear weight
    (legacy/utils.py:714-868). The two autograd passes run through the differentiable tcgen05
    products; the accumulation, clamp and EMA are one fused kernel per layer, which also leaves
    the layer's importance score ready for the next mask update."""
    owners = _sparse_modules(model)
    if not owners:
        return
    params = [m.weight for m in owners]
    try:
        grads = torch.autograd.grad(loss, params, create_graph=True, retain_graph=True, allow_unused=True)
        dot, vs = None, []
        for g, p in zip(grads, params):
            if g is None:
                vs.append(None)
                continue
            v = _rademacher_like(p)
            vs.append(v)
            term = (g * v).sum()
            dot = term if dot is None else dot + term
        hvps = [None] * len(params) if dot is None else torch.autograd.grad(dot, params, retain_graph=True,
                                                                              allow_unused=True)
    except RuntimeError as e:
        raise RuntimeError(f"[Hutchinson] Double-backward failed: {e}") from e
    world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
    for m, hvp, v in zip(owners, hvps, vs):
        if hvp is None or v is None or m._is_placeholder("hessian_diag"):
            continue
        if world > 1 and hvp.shape == m.hessian_diag.shape and not getattr(m, "_row_sharded", False):
            # data-parallel replicas average clamp(hvp*v, 0) (legacy/utils.py:860-865); the clamp
            # commutes with nothing, so it is applied before the reduction as there.
            d = torch.clamp((hvp * v).detach(), min=0.0)
            dist.all_reduce(d, op=dist.ReduceOp.SUM)
            d.div_(world)
            m.accumulate_hutchinson(d, torch.ones_like(v))
        else:
            m.accumulate_hutchinson(hvp.detach(), v)


def _layer_stats(m: SparseLinear) -> torch.Tensor:
    stats = torch.zeros(_lib.MSTAT_COUNT, dtype=torch.float64, device=m.mask.device)
    ops.mask_stats(m.mask.data, stats)
    return stats


def _all_reduce(t: torch.Tensor) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t


@torch.no_grad()
def mid_penalty(model, lambda_mid: float = 0.0):
    """lambda * mean(m (1 - m)) over every mask (legacy/utils.py:875-938)."""
    mods = [m for m in _sparse_modules(model) if m.mask.numel() > 0]
    device = mods[0].mask.device if mods else torch.device("cuda")
    if lambda_mid <= 0 or not mods:
        return torch.tensor(0.0, device=device)
    acc = torch.zeros(2, dtype=torch.float64, device=device)
    for m in mods:
        s = _layer_stats(m)
        if not bool(torch.isfinite(s[_lib.MSTAT_SUM_M1M])):
            continue
        acc[0] += s[_lib.MSTAT_SUM_M1M]
        acc[1] += float(m.mask.numel())
    _all_reduce(acc)
    if float(acc[1]) <= 0:
        return torch.tensor(0.0, device=device)
    res = lambda_mid * acc[0] / acc[1]
    return res.to(torch.float32) if bool(torch.isfinite(res)) else torch.tensor(0.0, device=device)


@torch.no_grad()
def sparsity_penalty(model, target_sparsity: float = 0.5, alpha: float = 0.0):
    """Global hard sparsity and alpha * (sparsity - target)^2 (legacy/utils.py:941-1025); structured
    2-D masks count (M-N)/M analytically as there."""
    mods = [m for m in _sparse_modules(model) if m.mask.numel() > 0]
    device = mods[0].mask.device if mods else torch.device("cuda")
    acc = torch.zeros(2, dtype=torch.float64, device=device)
    for m in mods:
        mk = m.mask.detach()
        if getattr(m, "mask_type", "unstructured") == "structured" and mk.dim() == 2 and mk.shape[1] % int(m.M) == 0:
            acc[0] += float(mk.shape[0] * (mk.shape[1] // int(m.M)) * (int(m.M) - int(m.N)))
        else:
            acc[0] += (mk < 0.5).double().sum()
        acc[1] += float(mk.numel())
    _all_reduce(acc)
    cur = float(acc[0] / acc[1]) if float(acc[1]) > 0 else 0.0
    pen = torch.tensor(float(alpha * (cur - float(target_sparsity)) ** 2) if alpha != 0.0 else 0.0, device=device)
    return pen, cur


@torch.no_grad()
def nm_2_4_tile_stats(model, debug=False):
    """Average of the two largest / two smallest mask values per group of 4
    (legacy/utils.py:1028-1234)."""
    mods = [m for m in _sparse_modules(model) if m.mask.dim() == 2 and m.mask.shape[1] % 4 == 0 and m.mask.numel() > 0]
    zero = {"top2_avg": 0.0, "bot2_avg": 0.0, "top2_gap": 0.0, "bot2_gap": 0.0, "total_gap": 0.0}
    if not mods:
        return zero
    acc = torch.zeros(3, dtype=torch.float64, device=mods[0].mask.device)
    for m in mods:
        s = _layer_stats(m)
        acc[0] += s[_lib.MSTAT_SUM_TOP2]
        acc[1] += s[_lib.MSTAT_SUM_BOT2]
        acc[2] += float(m.mask.numel() // 4)
    _all_reduce(acc)
    tiles = float(acc[2])
    if tiles <= 0:
        return zero
    top2, bot2 = float(acc[0]) / (tiles * 2), float(acc[1]) / (tiles * 2)
    return {"top2_avg": top2, "bot2_avg": bot2, "top2_gap": 1.0 - top2, "bot2_gap": bot2,
            "total_gap": (1.0 - top2) + bot2}


@torch.no_grad()
@torch.no_grad()
def mask_stats(model, bins: int = 100, eps: float = 1e-8, sample_per_layer: int = 4096):
    """Global statistics of the continuous masks (legacy/utils.py:2069-2280): mean, std, entropy,
    fractions below / above thresholds, and p10 / p50 / p90 from a histogram of a random sample of
    every layer. One read of each mask (one kernel) plus a gather of the sample; the sums are
    all-reduced, so call it on every rank. Block-sparse layers add the mean mask value of the lower
    and upper half of their blocks."""
    mods = [m for m in _sparse_modules(model) if m.mask.numel() > 0]
    device = mods[0].mask.device if mods else torch.device("cuda")
    acc = torch.zeros(12, dtype=torch.float64, device=device)
    hist = torch.zeros(int(bins), dtype=torch.float64, device=device)
    blk = torch.zeros(5, dtype=torch.float64, device=device)  # blocks, lower-half sum / count, upper-half sum / count
    for m in mods:
        mk = m.mask.data
        ops.mask_summary(mk, acc, eps)
        bs = m._block_size() if hasattr(m, "_block_size") else 0
        if bs and mk.dim() == 2 and mk.shape[0] >= bs and mk.shape[1] >= bs and mk.shape[1] % 4 == 0:
            # block-sparse layers: mean mask value of the lower and of the upper half of the blocks (:2155-2188)
            sums, _ = ops.block_sums(mk, bs, want_sq=False)
            means = torch.sort((sums / float(bs * bs)).flatten()).values.double()
            half = means.numel() // 2
            blk[0] += means.numel()
            if half > 0:
                blk[1] += means[:half].sum(); blk[2] += half
                blk[3] += means[half:].sum(); blk[4] += means.numel() - half
        take = min(mk.numel(), int(sample_per_layer))
        if take > 0:
            idx = torch.randint(0, mk.numel(), (take,), device=device)
            ops.mask_sample_hist(mk, idx.to(torch.int64).contiguous(), hist)
    _all_reduce(acc)
    _all_reduce(hist)
    _all_reduce(blk)
    a = [float(x) for x in acc.cpu()]
    bk = [float(x) for x in blk.cpu()]
    tot = a[0]
    if tot <= 0:
        return {"mask_mean": 1.0, "mask_std": 0.0, "mask_entropy": 0.0, "mask_hard_sparsity@0.5": 0.0,
                "mask_frac_lt_0.1": 0.0, "mask_frac_lt_0.01": 0.0, "mask_p10": 1.0, "mask_p50": 1.0, "mask_p90": 1.0}
    mean = a[1] / tot
    std = math.sqrt(max(a[2] / tot - mean * mean, 0.0))
    h = hist.cpu()

    def q_from_hist(q):
        if float(h.sum()) <= 0:
            return mean
        cdf = h.cumsum(0) / (h.sum() + 1e-12)
        i = int(torch.searchsorted(cdf, torch.tensor([q], dtype=cdf.dtype)).item())
        return float((max(0, min(int(bins) - 1, i)) + 0.5) / int(bins))

    result = {
        "mask_mean": mean, "mask_std": std, "mask_entropy": a[3] / tot, "mask_hard_sparsity@0.5": a[4] / tot,
        "mask_frac_lt_0.1": a[5] / tot, "mask_frac_lt_0.01": a[6] / tot, "mask_frac_gt_0.9": a[7] / tot,
        "mask_frac_gt_0.99": a[8] / tot, "mask_frac_gt_0.5": a[9] / tot,
        "mask_mean_lt_0.5": a[10] / a[4] if a[4] > 0 else 0.0, "mask_mean_gt_0.5": a[11] / a[9] if a[9] > 0 else 0.0,
        "mask_p10": q_from_hist(0.10), "mask_p50": q_from_hist(0.50), "mask_p90": q_from_hist(0.90),
    }
    if bk[0] > 0:
        lower = bk[1] / bk[2] if bk[2] > 0 else 0.0
        upper = bk[3] / bk[4] if bk[4] > 0 else 0.0
        result.update({"blk_lower_half_mean": lower, "blk_upper_half_mean": upper, "blk_total_blocks": bk[0],
                       "blk_separation": upper - lower})
    return result


@torch.no_grad()
def log_mask_stats(model, step: int, wandb_run=None, prefix: str = "mask/", bins: int = 100,
                   sample_per_layer: int = 4096):
    """legacy/utils.py:2283-2340: global mask statistics plus the schedule scalars of the first layer,
    handed to ``wandb_run.log`` on rank 0. Returns the dictionary (on every rank)."""
    stats = mask_stats(model, bins=bins, sample_per_layer=sample_per_layer)
    log = {prefix + k: v for k, v in stats.items()}
    log["iter"] = step
    for m in _sparse_modules(model):
        log[prefix + "beta_structural"] = float(m._beta_structural(step))
        log[prefix + "hardening_x"] = float(getattr(m, "hardening_x", 1.0))
        break
    rank0 = not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
    if rank0 and wandb_run is not None and hasattr(wandb_run, "log"):
        try:
            wandb_run.log(log, step=step)
        except TypeError:
            wandb_run.log(log)
    return log


def finalize_hard_masks(model):
    """End-of-training bake-in (legacy/main_llama.py:2552-2563): mask <- top2(mask), weight *= mask,
    mask updates off, forward uses the mask as is."""
    for m in _sparse_modules(model):
        hard = m._hard_mask_from_soft(m.mask.data)
        m.mask.data.copy_(hard)
        m.weight.data.mul_(m.mask.data.to(m.weight.dtype))
        m.change_mask = False
        m._hardening_finalized = True
        m.hardening_x = 0.0
        m.invalidate_masked_weight()


@torch.no_grad()
def optimize_sparse_model_for_inference(model, use_slorb: bool = False, compressed: bool = False):
    """Inference bake-in (legacy/eval_wiki_ppl.py:548-651): every SparseLinear gets its HARD mask
    multiplied into the weight once and then runs ``dense_forward`` (a layer whose finalized
    weight already carries the zeros is not multiplied twice). With ``use_slorb`` the layer stays
    in ``sparse_forward`` and only its mask is made binary, as in the reference.
    ``compressed=True`` goes one step further than the reference: bf16 layers with a 2:4 hard view are stored in the
    2:4 compressed form and run on the sparse tensor cores (``SparseLinear.compress_for_inference``)."""
    optimized = total = 0
    for m in _sparse_modules(get_raw_model(model)):
        total += 1
        soft = m.mask.data
        binary = bool(torch.all((soft == 0) | (soft == 1)).item())
        hard = soft if binary else m._hard_mask_from_soft(soft)
        hard_w = hard.to(m.weight.dtype)
        can_dense = not use_slorb
        already = False
        if can_dense and getattr(m, "_hardening_finalized", False):
            wz = float((m.weight.data == 0).float().mean())
            mz = float((hard_w == 0).float().mean())
            already = wz >= mz - 1e-4
        if not already:
            if can_dense:
                m.weight.data.mul_(hard_w)
            else:
                m.mask.data.copy_(hard.to(m.mask.dtype))
        if can_dense:
            if compressed and m.weight.dtype == torch.bfloat16 and m.in_features % 16 == 0 and m._is_2to4_view():
                m.mask.data.copy_(hard.to(m.mask.dtype))
                m.compress_for_inference()
            else:
                m.mode = "dense_forward"
        m._inference_optimized = True
        m.invalidate_masked_weight()
        optimized += 1
    return model


@torch.no_grad()
def add_calibration(model, nsamples=128, device="cuda", calib_source="c4", synthetic_cache_path=None, dataloader=None):
    """WANDA calibration driver (legacy/utils.py:1989-2060): ``scaler_row`` of every SparseLinear
    starts at one, then ``nsamples`` calibration batches run through the model while a forward hook
    on each layer folds its input into ``scaler_row`` (``SparseLinear.add_batch``).

    The reference reads its batches from a pickled C4 (or synthetic) calibration set beside the
    script and walks ``model.transformer.h`` layer by layer; that data set is not part of this
    package. Pass ``dataloader``: an iterable whose items are the model's positional input (a tensor)
    or a tuple / list of positional inputs; the first ``nsamples`` items are used, each in one
    forward pass of the whole model. Without it the call raises."""
    raw = get_raw_model(model)
    mods = [m for m in _sparse_modules(raw) if not m._is_placeholder("scaler_row")]
    if dataloader is None:
        raise FileNotFoundError(
            f"add_calibration(calib_source={calib_source!r}): the pickled calibration set of the reference "
            "(data/c4_dataset/calibration_dataset.pkl, legacy/utils.py:2034) is not shipped with this package; "
            "pass dataloader=<iterable of model inputs>")
    for m in mods:
        m.scaler_row.data.fill_(1.0)
        m._score_key = None
    handles = [m.register_forward_hook(lambda mod, inp, out: mod.add_batch(inp[0].data, out.data)) for m in mods]
    try:
        for j, batch in enumerate(dataloader):
            if j >= int(nsamples):
                break
            args = batch if isinstance(batch, (tuple, list)) else (batch,)
            raw(*[a.to(device) if torch.is_tensor(a) else a for a in args])
    finally:
        for h in handles:
            h.remove()


def eval_ppl(model, bs=2, device="cuda:0", block_size=1024, model_name_or_path=None):
    """Name kept for ``from utils import eval_ppl`` (legacy/main_llama.py:32-50). WikiText-2 perplexity
    evaluation (legacy/utils.py:1284-1530) needs the data set and a tokenizer and is outside this package."""
    raise NotImplementedError("eval_ppl: perplexity evaluation (legacy/utils.py:1284-1530) is outside this package; "
                              "it covers the SparseLinear hot path only")


def eval_ppl_distributed(model, bs=2, device="cuda:0", block_size=1024, model_name_or_path=None, ptdtype=None):
    """Name kept for ``from utils import eval_ppl_distributed``; see ``eval_ppl``."""
    raise NotImplementedError("eval_ppl_distributed: perplexity evaluation (legacy/utils.py:1533-1980) is outside "
                              "this package; it covers the SparseLinear hot path only")
