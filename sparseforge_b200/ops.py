"""Tensor-level wrappers around the C ABI: each function validates its torch tensors, takes
their device pointers and enqueues one library call on the current CUDA stream.

torch is used here for device memory and streams only; the arithmetic is in the library.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import SF_BF16, SF_F32, SF_I8, check, lib

_DT = {torch.float32: SF_F32, torch.bfloat16: SF_BF16, torch.int8: SF_I8}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"sparseforge_b200: unsupported dtype {t.dtype} (float32 / bfloat16 only)") from None


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("sparseforge_b200: tensors must live on a CUDA device (there is no CPU path)")
        if not t.is_contiguous():
            raise RuntimeError("sparseforge_b200: tensors must be contiguous")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def hutch_score_scratch(device) -> torch.Tensor:
    return torch.empty(int(lib().sf_hutch_score_scratch_doubles(0)), dtype=torch.float64, device=device)


def hutch_score(W, H, score, norm, scratch, *, hvp=None, v=None, aux=None, aux_scalar=1.0, beta=0.99,
                metric="hessian_obd") -> None:
    """H <- beta H + (1-beta) max(hvp*v, 0) (when hvp is given); score <- metric(W, H); norm <- (mean, std+1e-6)."""
    _cuda(W, H, score, norm, scratch, hvp, v, aux)
    if score.dtype != torch.float32 or norm.dtype != torch.float32 or (H is not None and H.dtype != torch.float32):
        raise TypeError("hutch_score: H, score and norm must be float32")
    if hvp is not None and (hvp.dtype != W.dtype or hvp.numel() != W.numel()):
        raise TypeError("hutch_score: hvp must match W in dtype and size")
    if v is not None and v.dtype not in (torch.int8, W.dtype):
        raise TypeError("hutch_score: v must be int8 signs or have W's dtype")
    check(lib().sf_hutch_score(_p(hvp), _p(v), _dt(v) if v is not None else SF_I8, _p(H), _p(W), _dt(W), _p(aux),
                               float(aux_scalar), _p(score), _p(norm), _p(scratch), W.numel(), float(beta),
                               _lib.METRICS[metric], _stream()), "sf_hutch_score")


def hutch_accumulate(H, hvp, v, *, beta=0.99) -> None:
    """H <- beta H + (1-beta) max(hvp*v, 0) only: the score is left to a later pass (adamw_masked_score)."""
    _cuda(H, hvp, v)
    if H.dtype != torch.float32 or H.numel() != hvp.numel():
        raise TypeError("hutch_accumulate: H must be float32 with hvp's size")
    if v.dtype not in (torch.int8, hvp.dtype):
        raise TypeError("hutch_accumulate: v must be int8 signs or have hvp's dtype")
    check(lib().sf_hutch_score(_p(hvp), _p(v), _dt(v), _p(H), None, _dt(hvp), None, 1.0, None, None, None,
                               hvp.numel(), float(beta), _lib.METRICS["hessian_obd"], _stream()), "sf_hutch_score")


def grad_hessian_ema(g, grad_ema, H=None, *, beta=0.99) -> None:
    """grad_ema <- beta grad_ema + (1-beta) g and, with H, H <- beta H + (1-beta) g^2, in one pass
    (legacy/sparse_modeling.py:901-922)."""
    _cuda(g, grad_ema, H)
    if g.dtype != grad_ema.dtype or g.numel() != grad_ema.numel():
        raise TypeError("grad_hessian_ema: g and grad_ema must share dtype and size")
    if H is not None and (H.dtype != torch.float32 or H.numel() != g.numel()):
        raise TypeError("grad_hessian_ema: H must be float32 with g's size")
    check(lib().sf_grad_hessian_ema(_p(g), _p(grad_ema), _dt(g), _p(H), g.numel(), float(beta), _stream()),
          "sf_grad_hessian_ema")


def mask_update_nm24_from_weight(W, H, norm, mask, stats, wm, meta, *, metric="hessian_obd", tau=None, temperature=1.0,
                                 mask_lr=0.1, pen=0.0, penalty_mode=_lib.PENALTY_NONE, beta_s=0.0, binarize_decay=0.0,
                                 hx=1.0, structured_exact=False) -> None:
    """``mask_update_nm24`` with the score formed inside the pass from W and H (no score tensor)."""
    _cuda(W, H, norm, mask, stats, wm, meta, tau)
    if mask.dtype != torch.float32 or (H is not None and H.dtype != torch.float32) or stats.dtype != torch.float64:
        raise TypeError("mask_update_nm24_from_weight: mask / H float32, stats float64")
    if wm.dtype != W.dtype:
        raise TypeError("mask_update_nm24_from_weight: wm must have W's dtype")
    rows, cols = mask.shape
    check(lib().sf_mask_update_nm24_from_weight(_p(W), _dt(W), _p(H), _lib.METRICS[metric], _p(norm), _p(tau), _p(mask),
                                                _p(wm), _p(meta), _p(stats), rows, cols, float(temperature),
                                                float(mask_lr), float(pen), int(penalty_mode), float(beta_s),
                                                float(binarize_decay), float(hx), int(bool(structured_exact)),
                                                _stream()), "sf_mask_update_nm24_from_weight")


def score_sum(a, b, out, norm, scratch) -> None:
    """out <- a + b (fp32 scores of a gate / up pair); norm <- (mean, std + 1e-6) of out."""
    _cuda(a, b, out, norm, scratch)
    if not (a.dtype == b.dtype == out.dtype == torch.float32) or a.numel() != b.numel() or a.numel() != out.numel():
        raise TypeError("score_sum: a, b, out must be float32 tensors of one size")
    check(lib().sf_score_sum(_p(a), _p(b), _p(out), _p(norm), _p(scratch), a.numel(), _stream()), "sf_score_sum")


_WANDA_SCRATCH = {}


def wanda_add_batch(x2d, scaler_row, keep: float, denom: float) -> None:
    """scaler_row <- scaler_row * keep + ||x[:, c]||^2 / denom in place (WANDA calibration energy of
    the input channels, legacy/sparse_modeling.py:884-898); x2d is [tokens, in_features]."""
    _cuda(x2d, scaler_row)
    if x2d.dim() != 2 or scaler_row.dim() != 1 or scaler_row.numel() != x2d.shape[1]:
        raise ValueError("wanda_add_batch: x must be [tokens, in] and scaler_row [in]")
    if not (x2d.is_contiguous() and scaler_row.is_contiguous()):
        raise ValueError("wanda_add_batch: contiguous tensors expected")
    cols = x2d.shape[1]
    key = (x2d.device, cols)
    scratch = _WANDA_SCRATCH.get(key)
    if scratch is None:
        scratch = torch.empty(int(lib().sf_wanda_scratch_floats(cols)), dtype=torch.float32, device=x2d.device)
        _WANDA_SCRATCH[key] = scratch
    check(lib().sf_wanda_add_batch(_p(x2d), _dt(x2d), x2d.shape[0], cols, _p(scaler_row), _dt(scaler_row), float(keep),
                                   float(denom), _p(scratch), _stream()), "sf_wanda_add_batch")


def wanda_score(W, scaler_row, score, norm, scratch, eps: float = 1e-8) -> None:
    """score <- |W| * sqrt(scaler_row + eps) (fp32) with norm <- (mean, std + 1e-6)
    (legacy/sparse_modeling.py:1071-1088)."""
    _cuda(W, scaler_row, score, norm, scratch)
    if W.dim() != 2 or scaler_row.numel() != W.shape[1] or score.dtype != torch.float32 or score.numel() != W.numel():
        raise ValueError("wanda_score: W [out, in], scaler_row [in], score float32 of W's size expected")
    check(lib().sf_wanda_score(_p(W), _dt(W), _p(scaler_row), _dt(scaler_row), W.shape[0], W.shape[1], float(eps),
                               _p(score), _p(norm), _p(scratch), _stream()), "sf_wanda_score")


def mask_update_nm24(score, norm, mask, stats, *, tau=None, W=None, wm=None, meta=None, temperature=1.0, mask_lr=0.1,
                     pen=0.0, penalty_mode=_lib.PENALTY_NONE, beta_s=0.0, binarize_decay=0.0, hx=1.0,
                     structured_exact=False, score_bf16=False, pen_mask=None, frozen=None, freeze_low=0.0,
                     freeze_high=1.0, freeze_apply_high=False) -> None:
    _cuda(score, norm, mask, stats, W, wm, meta, tau, pen_mask, frozen)
    if pen_mask is not None and (pen_mask.dtype != torch.float32 or pen_mask.shape != mask.shape):
        raise TypeError("mask_update_nm24: pen_mask must be a float32 tensor of the mask's shape")
    if tau is not None and tau.dtype != torch.float32:
        raise TypeError("mask_update_nm24: tau must be a float32 device scalar")
    if mask.dim() != 2:
        raise ValueError("mask_update_nm24: mask must be 2-D [out, in]")
    if mask.dtype != torch.float32 or score.dtype != torch.float32 or stats.dtype != torch.float64:
        raise TypeError("mask_update_nm24: mask/score float32, stats float64")
    if wm is not None and (W is None or wm.dtype != W.dtype):
        raise TypeError("mask_update_nm24: wm needs W of the same dtype")
    rows, cols = mask.shape
    if frozen is not None:
        if pen_mask is not None:
            raise ValueError("mask_update_nm24: freeze bands and a joint penalty mask are not combined")
        if frozen.dtype != torch.float32 or frozen.shape != mask.shape:
            raise TypeError("mask_update_nm24: frozen must be a float32 tensor of the mask's shape")
        check(lib().sf_mask_update_nm24_frozen(_p(score), _p(norm), _p(tau), _p(frozen), float(freeze_low),
                                               float(freeze_high), int(bool(freeze_apply_high)), _p(mask), _p(W),
                                               _dt(W) if W is not None else SF_F32, _p(wm), _p(meta), _p(stats), rows,
                                               cols, float(temperature), float(mask_lr), float(pen), int(penalty_mode),
                                               float(beta_s), float(binarize_decay), float(hx),
                                               int(bool(structured_exact)), int(bool(score_bf16)), _stream()),
              "sf_mask_update_nm24_frozen")
        return
    if pen_mask is not None:
        check(lib().sf_mask_update_nm24_joint(_p(score), _p(norm), _p(tau), _p(pen_mask), _p(mask), _p(W),
                                              _dt(W) if W is not None else SF_F32, _p(wm), _p(meta), _p(stats), rows,
                                              cols, float(temperature), float(mask_lr), float(pen), int(penalty_mode),
                                              float(beta_s), float(binarize_decay), float(hx),
                                              int(bool(structured_exact)), int(bool(score_bf16)), _stream()),
              "sf_mask_update_nm24_joint")
        return
    check(lib().sf_mask_update_nm24(_p(score), _p(norm), _p(tau), _p(mask), _p(W), _dt(W) if W is not None else SF_F32,
                                    _p(wm), _p(meta), _p(stats), rows, cols, float(temperature), float(mask_lr),
                                    float(pen), int(penalty_mode), float(beta_s), float(binarize_decay), float(hx),
                                    int(bool(structured_exact)), int(bool(score_bf16)), _stream()),
          "sf_mask_update_nm24")


def project_nm24(soft, *, out_dtype=None, want_hard=True, want_meta=False):
    """Hard top-2-of-4 projection of a 2-D soft mask. Returns (hard or None, meta or None)."""
    if soft.dim() != 2:
        raise ValueError("project_nm24: soft must be 2-D")
    if not soft.is_cuda:
        raise RuntimeError("sparseforge_b200: tensors must live on a CUDA device (there is no CPU path)")
    if soft.stride(1) != 1 and soft.numel() > 0:
        soft = soft.contiguous()
    rows, cols = soft.shape
    out_dtype = out_dtype or soft.dtype
    hard = torch.empty((rows, cols), dtype=out_dtype, device=soft.device) if want_hard else None
    meta = torch.zeros((rows, (cols + 7) // 8), dtype=torch.uint8, device=soft.device) if want_meta else None
    if rows == 0 or cols == 0:
        return hard, meta
    check(lib().sf_project_nm24(_p(soft), _dt(soft), soft.stride(0), _p(hard), _DT[out_dtype], cols, _p(meta),
                                rows, cols, _stream()), "sf_project_nm24")
    return hard, meta


def mask_update_nm(score, norm, mask, stats, n_keep, m_group, *, tau=None, W=None, wm=None, temperature=1.0, mask_lr=0.1,
                   pen=0.0, penalty_mode=_lib.PENALTY_NONE, beta_s=0.0, binarize_decay=0.0, hx=1.0,
                   structured_exact=False, score_bf16=False, pen_mask=None, threshold_view=False) -> None:
    """``mask_update_nm24`` for a general N:M (M in 2, 4, 8, 16, 32); no metadata output. With
    ``threshold_view`` the hard view is ``mask > 0.5`` (hard_mask_type 'unstructured')."""
    _cuda(score, norm, mask, stats, W, wm, tau, pen_mask)
    if mask.dim() != 2:
        raise ValueError("mask_update_nm: mask must be 2-D [out, in]")
    if pen_mask is not None and (pen_mask.dtype != torch.float32 or pen_mask.shape != mask.shape):
        raise TypeError("mask_update_nm: pen_mask must be a float32 tensor of the mask's shape")
    if mask.dtype != torch.float32 or score.dtype != torch.float32 or stats.dtype != torch.float64:
        raise TypeError("mask_update_nm: mask/score float32, stats float64")
    if tau is not None and tau.dtype != torch.float32:
        raise TypeError("mask_update_nm: tau must be a float32 device scalar")
    if wm is not None and (W is None or wm.dtype != W.dtype):
        raise TypeError("mask_update_nm: wm needs W of the same dtype")
    rows, cols = mask.shape
    check(lib().sf_mask_update_nm(_p(score), _p(norm), _p(tau), _p(pen_mask), _p(mask), _p(W), _dt(W) if W is not None else SF_F32,
                                  _p(wm), _p(stats), rows, cols, int(n_keep), int(m_group), float(temperature),
                                  float(mask_lr), float(pen), int(penalty_mode), float(beta_s), float(binarize_decay),
                                  float(hx), int(bool(structured_exact)), int(bool(score_bf16)), int(bool(threshold_view)),
                                  _stream()), "sf_mask_update_nm")


def project_nm(soft, n_keep, m_group, *, out_dtype=None):
    """Hard top-N-of-M projection of a 2-D soft mask along its last dimension (0/1 tensor)."""
    if soft.dim() != 2:
        raise ValueError("project_nm: soft must be 2-D")
    if not soft.is_cuda:
        raise RuntimeError("sparseforge_b200: tensors must live on a CUDA device (there is no CPU path)")
    if soft.stride(1) != 1 and soft.numel() > 0:
        soft = soft.contiguous()
    rows, cols = soft.shape
    out_dtype = out_dtype or soft.dtype
    hard = torch.empty((rows, cols), dtype=out_dtype, device=soft.device)
    if rows == 0 or cols == 0:
        return hard
    check(lib().sf_project_nm(_p(soft), _dt(soft), soft.stride(0), _p(hard), _DT[out_dtype], cols, rows, cols,
                              int(n_keep), int(m_group), _stream()), "sf_project_nm")
    return hard


def effective_weight_nm(W, mask, wm, n_keep, m_group, *, hx=1.0, finalized=False, threshold_view=False) -> None:
    """wm <- W * cast(hx mask + (1 - hx) topN-of-M(mask)) for a general N:M."""
    _cuda(W, mask, wm)
    if mask.dtype != torch.float32:
        raise TypeError("effective_weight_nm: mask must be float32")
    rows, cols = W.shape
    check(lib().sf_effective_weight_nm(_p(W), _dt(W), _p(mask), _p(wm), rows, cols, int(n_keep), int(m_group), float(hx),
                                       int(bool(finalized)), int(bool(threshold_view)), _stream()), "sf_effective_weight_nm")


def effective_weight(W, mask, wm, *, meta=None, hx=1.0, finalized=False, scale=1.0) -> None:
    _cuda(W, mask, wm, meta)
    if mask.dtype != torch.float32:
        raise TypeError("effective_weight: mask must be float32")
    rows, cols = W.shape
    check(lib().sf_effective_weight(_p(W), _dt(W), _p(mask), _p(wm), _p(meta), rows, cols, float(hx),
                                    int(bool(finalized)), float(scale), _stream()), "sf_effective_weight")


def adamw_masked(p, g, m, v, *, mask=None, lr, beta1, beta2, eps, weight_decay, decay, step, adaptive_l1=0.0,
                 wm=None, hx=1.0, v_max=None) -> None:
    _cuda(p, g, m, v, mask, wm, v_max)
    if not (p.dtype == g.dtype == m.dtype == v.dtype):
        raise TypeError("adamw_masked: p, g, m, v must share a dtype")
    if mask is not None and mask.dtype != torch.float32:
        raise TypeError("adamw_masked: mask must be float32")
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if v_max is not None:  # AMSGrad: no masked-weight output in that variant
        if v_max.dtype != p.dtype or wm is not None:
            raise TypeError("adamw_masked: v_max must have the weight dtype and excludes wm")
        check(lib().sf_adamw_masked_amsgrad(_p(p), _p(g), _p(mask), _p(m), _p(v), _p(v_max), _dt(p), p.numel(), float(lr),
                                            float(beta1), float(beta2), float(eps), float(weight_decay), float(decay),
                                            float(bc1), float(bc2), float(adaptive_l1), _stream()),
              "sf_adamw_masked_amsgrad")
        return
    cols = p.shape[-1] if p.dim() >= 2 else 0
    check(lib().sf_adamw_masked(_p(p), _p(g), _p(mask), _p(m), _p(v), _dt(p), p.numel(), float(lr), float(beta1),
                                float(beta2), float(eps), float(weight_decay), float(decay), float(bc1), float(bc2),
                                float(adaptive_l1), _p(wm), float(hx), cols, _stream()), "sf_adamw_masked")


def adamw_masked_score(p, g, m, v, *, mask=None, lr, beta1, beta2, eps, weight_decay, decay, step, adaptive_l1=0.0,
                       H=None, score=None, norm, scratch, metric: str, hvp=None, probe=None, beta_h=0.99) -> None:
    """AdamW step and, in the same pass, the importance score of the updated weight with its mean/std.
    With hvp and probe the Hutchinson sample is folded into H first (as hutch_accumulate does)."""
    _cuda(p, g, m, v, mask, H, score, norm, scratch, hvp, probe)
    if hvp is not None:
        if probe is None or H is None or hvp.dtype != p.dtype or hvp.numel() != p.numel():
            raise TypeError("adamw_masked_score: hvp needs probe and H, and p's dtype and size")
        if probe.dtype not in (torch.int8, p.dtype):
            raise TypeError("adamw_masked_score: probe must be int8 signs or have p's dtype")
    if not (p.dtype == g.dtype == m.dtype == v.dtype):
        raise TypeError("adamw_masked_score: p, g, m, v must share a dtype")
    if mask is not None and mask.dtype != torch.float32:
        raise TypeError("adamw_masked_score: mask must be float32")
    if (score is not None and score.dtype != torch.float32) or (H is not None and H.dtype != torch.float32):
        raise TypeError("adamw_masked_score: H and score must be float32")
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    check(lib().sf_adamw_masked_score(_p(p), _p(g), _p(mask), _p(m), _p(v), _dt(p), p.numel(), float(lr), float(beta1),
                                      float(beta2), float(eps), float(weight_decay), float(decay), float(bc1),
                                      float(bc2), float(adaptive_l1), _p(hvp), _p(probe),
                                      _dt(probe) if probe is not None else SF_I8, float(beta_h), _p(H), _p(score),
                                      _p(norm), _p(scratch),
                                      _lib.METRICS[metric], _stream()), "sf_adamw_masked_score")


def mask_stats(mask, stats) -> None:
    _cuda(mask, stats)
    rows, cols = mask.shape
    check(lib().sf_mask_stats(_p(mask), _p(stats), rows, cols, _stream()), "sf_mask_stats")


def mask_update_tile16(score, norm, tau, mask, stats, *, keep_k, W=None, wm=None, temperature=1.0, mask_lr=0.1, pen=0.0,
                       penalty_mode=0, binarize_decay=0.0, hx=1.0) -> None:
    """Fused mask update of the 'block16' mode (top keep_k of every 16 x 16 tile)."""
    _cuda(score, norm, tau, mask, stats, W, wm)
    if mask.dtype != torch.float32 or score.dtype != torch.float32 or stats.dtype != torch.float64:
        raise TypeError("mask_update_tile16: mask / score float32, stats float64")
    rows, cols = mask.shape
    check(lib().sf_mask_update_tile16(_p(score), _p(norm), _p(tau), _p(mask), _p(W), _dt(W) if W is not None else SF_F32,
                                      _p(wm), _p(stats), rows, cols, int(keep_k), float(temperature), float(mask_lr),
                                      float(pen), int(penalty_mode), float(binarize_decay), float(hx), _stream()),
          "sf_mask_update_tile16")


def project_tile16(soft, keep_k, *, want_hard=True, W=None, wm=None, hx=1.0):
    """Per-tile hard view (float32 0/1) and / or masked weight of a float32 soft mask."""
    _cuda(soft, W, wm)
    if soft.dtype != torch.float32 or soft.dim() != 2:
        raise TypeError("project_tile16: soft must be a 2-D float32 tensor")
    rows, cols = soft.shape
    hard = torch.empty_like(soft) if want_hard else None
    check(lib().sf_project_tile16(_p(soft), _p(hard), _p(W), _dt(W) if W is not None else SF_F32, _p(wm), rows, cols,
                                  int(keep_k), float(hx), _stream()), "sf_project_tile16")
    return hard


def block_sums(x, bs, norm=None, want_sq=True):
    """(sum, sumsq) over every whole bs x bs block of a float32 matrix, each [rows // bs, cols // bs]."""
    _cuda(x, norm)
    if x.dtype != torch.float32 or x.dim() != 2:
        raise TypeError("block_sums: x must be a 2-D float32 tensor")
    rows, cols = x.shape
    ob, ib = rows // bs, cols // bs
    s = torch.empty((ob, ib), dtype=torch.float32, device=x.device)
    q = torch.empty((ob, ib), dtype=torch.float32, device=x.device) if want_sq else None
    check(lib().sf_block_sums(_p(x), rows, cols, int(bs), _p(norm), _p(s), _p(q), _stream()), "sf_block_sums")
    return s, q


def block_mask_update(mask, bs, gate, target=None, *, mask_lr, pen=0.0, binarize_decay=0.0):
    """EMA update of a block-mode soft mask; returns the per-block sums of the updated mask."""
    _cuda(mask, gate, target)
    rows, cols = mask.shape
    new_sum = torch.empty_like(gate)
    check(lib().sf_block_mask_update(_p(mask), rows, cols, int(bs), _p(gate), _p(target), float(mask_lr), float(pen),
                                     float(binarize_decay), _p(new_sum), _stream()), "sf_block_mask_update")
    return new_sum


def block_mask_apply(mask, bs, keep, *, value=None, W=None, wm=None, hx=1.0) -> None:
    _cuda(mask, keep, value, W, wm)
    if keep.dtype != torch.uint8:
        raise TypeError("block_mask_apply: keep must be uint8")
    rows, cols = mask.shape
    check(lib().sf_block_mask_apply(_p(mask), _p(W), _dt(W) if W is not None else SF_F32, _p(wm), rows, cols, int(bs),
                                    _p(value), _p(keep), float(hx), _stream()), "sf_block_mask_apply")


def mask_summary(mask, out, eps=1e-8) -> None:
    """Adds the twelve logging sums of one soft mask to ``out`` (float64[12])."""
    _cuda(mask, out)
    if mask.dtype != torch.float32 or out.dtype != torch.float64 or out.numel() < 12:
        raise TypeError("mask_summary: mask float32, out float64[12]")
    check(lib().sf_mask_summary(_p(mask), mask.numel(), float(eps), _p(out), _stream()), "sf_mask_summary")


def mask_sample_hist(mask, idx, hist) -> None:
    """Adds the histogram of mask.flatten()[idx] over len(hist) equal bins of [0, 1] to ``hist`` (float64)."""
    _cuda(mask, idx, hist)
    if mask.dtype != torch.float32 or idx.dtype != torch.int64 or hist.dtype != torch.float64:
        raise TypeError("mask_sample_hist: mask float32, idx int64, hist float64")
    check(lib().sf_mask_sample_hist(_p(mask), _p(idx), idx.numel(), hist.numel(), _p(hist), _stream()),
          "sf_mask_sample_hist")


def kl_div_fwd(student2d, teacher2d, temperature=2.0, max_logit=100.0):
    """(row_kl[rows], lse[rows, 2]) of the distillation KL; see ``sf_kl_div_fwd``."""
    _cuda(student2d, teacher2d)
    if student2d.shape != teacher2d.shape or student2d.dtype != teacher2d.dtype:
        raise TypeError("kl_div_fwd: student and teacher logits must share shape and dtype")
    rows, vocab = student2d.shape
    row_kl = torch.empty(rows, dtype=torch.float32, device=student2d.device)
    lse = torch.empty((rows, 2), dtype=torch.float32, device=student2d.device)
    check(lib().sf_kl_div_fwd(_p(student2d), _p(teacher2d), _dt(student2d), rows, vocab, float(temperature),
                              float(max_logit), _p(row_kl), _p(lse), _stream()), "sf_kl_div_fwd")
    return row_kl, lse


def kl_div_bwd(student2d, teacher2d, lse, row_scale, temperature=2.0, max_logit=100.0):
    _cuda(student2d, teacher2d, lse, row_scale)
    rows, vocab = student2d.shape
    grad = torch.empty_like(student2d)
    check(lib().sf_kl_div_bwd(_p(student2d), _p(teacher2d), _dt(student2d), _p(lse), _p(row_scale), rows, vocab,
                              float(temperature), float(max_logit), _p(grad), _stream()), "sf_kl_div_bwd")
    return grad


def _gemm_dtype(*ts) -> int:
    d = ts[0].dtype
    for t in ts:
        if t.dtype != d:
            raise TypeError(f"masked GEMM: operand dtypes differ ({[str(x.dtype) for x in ts]})")
    return _dt(ts[0])


def gemm_configure_stream(stream=None, *, max_ctas=0) -> None:
    """Bounds the thread blocks of every bf16 tensor-core product launched on ``stream`` (the current
    stream by default) to ``max_ctas``, so that two products on two streams can share the GPU; 0 lifts
    the bound (``sf_masked_gemm_configure_stream``)."""
    st = torch.cuda.current_stream() if stream is None else stream
    check(lib().sf_masked_gemm_configure_stream(st.cuda_stream, int(max_ctas)), "sf_masked_gemm_configure_stream")


def gemm_fwd(x2d, wm, bias=None, alpha=1.0, status=None):
    """y[T,out] = alpha * x2d[T,in] @ wm[out,in]^T (+ bias)."""
    _cuda(x2d, wm, bias, status)
    T, k = x2d.shape
    out, k2 = wm.shape
    if k != k2:
        raise ValueError(f"gemm_fwd: x has {k} features, weight has {k2}")
    dt = _gemm_dtype(x2d, wm) if bias is None else _gemm_dtype(x2d, wm, bias)
    y = torch.empty((T, out), dtype=x2d.dtype, device=x2d.device)
    if T == 0:
        return y
    check(lib().sf_masked_gemm_fwd(_p(x2d), _p(wm), _p(bias), _p(y), T, k, out, float(alpha), dt, _p(status),
                                   _stream()), "sf_masked_gemm_fwd")
    return y


def gemm_fwd_lowrank(x2d, wm, z2d, sw, bias=None, status=None):
    """y[T,out] = x2d @ wm^T + z2d @ sw^T (+ bias) in one launch (bf16, more than 128 rows)."""
    _cuda(x2d, wm, z2d, sw, bias, status)
    T, k = x2d.shape
    out, k2 = wm.shape
    if k != k2 or z2d.shape[0] != T or sw.shape != (out, z2d.shape[1]):
        raise ValueError(f"gemm_fwd_lowrank: shapes x{tuple(x2d.shape)} wm{tuple(wm.shape)} z{tuple(z2d.shape)} "
                         f"sw{tuple(sw.shape)} do not fit")
    dt = _gemm_dtype(x2d, wm, z2d, sw) if bias is None else _gemm_dtype(x2d, wm, z2d, sw, bias)
    y = torch.empty((T, out), dtype=x2d.dtype, device=x2d.device)
    check(lib().sf_masked_gemm_fwd_lowrank(_p(x2d), _p(wm), _p(z2d), _p(sw), _p(bias), _p(y), T, k, out, z2d.shape[1], dt,
                                           _p(status), _stream()), "sf_masked_gemm_fwd_lowrank")
    return y


def gemm_dgrad(dy2d, wm, status=None):
    """dx[T,in] = dy2d[T,out] @ wm[out,in]."""
    _cuda(dy2d, wm, status)
    T, out = dy2d.shape
    out2, k = wm.shape
    if out != out2:
        raise ValueError(f"gemm_dgrad: dy has {out} features, weight has {out2} rows")
    dt = _gemm_dtype(dy2d, wm)
    dx = torch.empty((T, k), dtype=dy2d.dtype, device=dy2d.device)
    if T == 0:
        return dx
    check(lib().sf_masked_gemm_dgrad(_p(dy2d), _p(wm), _p(dx), T, k, out, dt, _p(status), _stream()),
          "sf_masked_gemm_dgrad")
    return dx


def gemm_wgrad(dy2d, x2d, status=None):
    """dw[out,in] = dy2d[T,out]^T @ x2d[T,in]."""
    _cuda(dy2d, x2d, status)
    T, out = dy2d.shape
    T2, k = x2d.shape
    if T != T2:
        raise ValueError(f"gemm_wgrad: dy has {T} rows, x has {T2}")
    dt = _gemm_dtype(dy2d, x2d)
    if T == 0:
        return torch.zeros((out, k), dtype=dy2d.dtype, device=dy2d.device)
    dw = torch.empty((out, k), dtype=dy2d.dtype, device=dy2d.device)
    check(lib().sf_masked_gemm_wgrad(_p(dy2d), _p(x2d), _p(dw), T, k, out, dt, _p(status), _stream()),
          "sf_masked_gemm_wgrad")
    return dw


def mma_issue_cycles(n: int, *, a_from_tmem: bool = False, iters: int = 4096, ctas: int = 1, device=None) -> float:
    """SM cycles per ``tcgen05.mma`` of shape 128 x n x 16 (bf16) when one thread issues ``iters`` of them
    back to back (``sf_selftest_mma_issue_rate``); ``ctas`` blocks run at once, the slowest counts."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    cycles = torch.zeros(1, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    check(lib().sf_selftest_mma_issue_rate(int(n), int(bool(a_from_tmem)), int(iters), int(ctas), _p(cycles), _p(status),
                                           _stream()), "sf_selftest_mma_issue_rate")
    if int(status.item()) != 0:
        raise RuntimeError(f"mma_issue_cycles: the wait for the MMAs ran out (code {int(status)})")
    return float(cycles.item()) / iters


def bias_grad(dy2d):
    _cuda(dy2d)
    T, out = dy2d.shape
    db = torch.empty(out, dtype=torch.float32, device=dy2d.device)
    check(lib().sf_bias_grad(_p(dy2d), _dt(dy2d), _p(db), T, out, _stream()), "sf_bias_grad")
    return db


# ----------------------------------------------------------------------------------------
# hard-2:4 compressed weights
# ----------------------------------------------------------------------------------------
def sparse24_compress(W, soft):
    """(values[out,in/2] bf16, meta[out,in/8] uint8) of W pruned to top2(soft) per group of 4."""
    _cuda(W, soft)
    if W.dtype != torch.bfloat16 or soft.dtype != torch.float32:
        raise TypeError("sparse24_compress: W bfloat16, soft float32")
    out, k = W.shape
    values = torch.empty((out, k // 2), dtype=torch.bfloat16, device=W.device)
    meta = torch.empty((out, k // 8), dtype=torch.uint8, device=W.device)
    check(lib().sf_sparse24_compress(_p(W), _p(soft), _p(values), _p(meta), out, k, _stream()), "sf_sparse24_compress")
    return values, meta


def sparse24_decompress(values, meta):
    _cuda(values, meta)
    out, half = values.shape
    dense = torch.empty((out, half * 2), dtype=torch.bfloat16, device=values.device)
    check(lib().sf_sparse24_decompress(_p(values), _p(meta), _p(dense), out, half * 2, _stream()), "sf_sparse24_decompress")
    return dense


def sparse24_pack_meta(meta, out, k):
    """Logical metadata -> the order the sparse tensor-core GEMM loads."""
    _cuda(meta)
    n = int(lib().sf_sparse24_meta_tc_bytes(out, k))
    meta_tc = torch.empty(n, dtype=torch.uint8, device=meta.device)
    check(lib().sf_sparse24_pack_meta(_p(meta), _p(meta_tc), out, k, _stream()), "sf_sparse24_pack_meta")
    return meta_tc


_SPLITK_WS = {}  # (device index, stream) -> zeroed workspace, left zeroed by every call


def _splitk_workspace(device, nbytes):
    key = (device.index, _stream())
    ws = _SPLITK_WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _SPLITK_WS[key] = ws
    return ws


def sparse24_gemm(x2d, values, meta_tc, bias=None, status=None, splits=0):
    """y[T,out] = x2d[T,in] @ decompress(values, meta)^T (+ bias) on the sparse tensor cores.
    Up to 128 rows the K range of each weight tile is split over CTAs (``splits``: 0 = choose,
    1 = off) with fp32 partial sums in a cached, self-cleaning workspace."""
    _cuda(x2d, values, meta_tc, bias, status)
    if x2d.dtype != torch.bfloat16 or values.dtype != torch.bfloat16:
        raise TypeError("sparse24_gemm: bfloat16 only")
    T, k = x2d.shape
    out = values.shape[0]
    if values.shape[1] * 2 != k:
        raise ValueError(f"sparse24_gemm: x has {k} features, compressed weight has {values.shape[1] * 2}")
    y = torch.empty((T, out), dtype=torch.bfloat16, device=x2d.device)
    if T == 0:
        return y
    if T <= 128 and splits != 1:
        need = int(lib().sf_sparse24_splitk_workspace_bytes(T, out))
        ws = _splitk_workspace(x2d.device, need)
        check(lib().sf_sparse24_gemm_splitk(_p(x2d), _p(values), _p(meta_tc), _p(bias), _p(y), T, k, out, _p(ws),
                                            ws.numel(), int(splits), _p(status), _stream()), "sf_sparse24_gemm_splitk")
        return y
    check(lib().sf_sparse24_gemm(_p(x2d), _p(values), _p(meta_tc), _p(bias), _p(y), T, k, out, _p(status), _stream()),
          "sf_sparse24_gemm")
    return y


# ----------------------------------------------------------------------------------------
# row-sharded products whose epilogue delivers the result to the other GPUs
# ----------------------------------------------------------------------------------------
def _ptr_array(ptrs):
    import ctypes

    arr = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr


def gemm_fwd_allgather(x2d, wm, dest_ptrs, out_total, col_offset, bias=None, alpha=1.0, status=None) -> None:
    """Columns [col_offset, col_offset + wm.shape[0]) of the layer output, written by the GEMM
    epilogue into every destination (device pointers to [T, out_total] bf16 buffers, one per GPU)."""
    _cuda(x2d, wm, bias, status)
    T, k = x2d.shape
    out_local, k2 = wm.shape
    if k != k2:
        raise ValueError(f"gemm_fwd_allgather: x has {k} features, weight has {k2}")
    arr = _ptr_array(dest_ptrs)
    check(lib().sf_masked_gemm_fwd_allgather(_p(x2d), _p(wm), _p(bias), arr, len(dest_ptrs), T, k, out_local,
                                             int(out_total), int(col_offset), float(alpha), _gemm_dtype(x2d, wm),
                                             _p(status), _stream()), "sf_masked_gemm_fwd_allgather")


def gemm_fwd_multicast(x2d, wm, mc_ptr, out_total, col_offset, bias=None, alpha=1.0, status=None) -> None:
    """The same output all-gather through an NVSwitch multicast object: ``mc_ptr`` is the multicast
    address of the [T, out_total] bf16 output that every GPU holds at the same offset of its
    symmetric buffer; each piece is stored once and replicated by the switch."""
    _cuda(x2d, wm, bias, status)
    T, k = x2d.shape
    out_local, k2 = wm.shape
    if k != k2:
        raise ValueError(f"gemm_fwd_multicast: x has {k} features, weight has {k2}")
    import ctypes

    check(lib().sf_masked_gemm_fwd_multicast(_p(x2d), _p(wm), _p(bias), ctypes.c_void_p(int(mc_ptr)), T, k, out_local,
                                             int(out_total), int(col_offset), float(alpha), _gemm_dtype(x2d, wm),
                                             _p(status), _stream()), "sf_masked_gemm_fwd_multicast")


def gemm_dgrad_reducescatter(dy2d, wm, slot_ptrs, rank, status=None) -> None:
    """Partial input gradient of this shard, token rows of rank c written into slot_ptrs[c] (the
    [T/n, in] slot rank c keeps for this rank). The owner sums its slots with ``reduce_slots``."""
    _cuda(dy2d, wm, status)
    T, out_local = dy2d.shape
    if wm.shape[0] != out_local:
        raise ValueError(f"gemm_dgrad_reducescatter: dy has {out_local} columns, weight has {wm.shape[0]} rows")
    arr = _ptr_array(slot_ptrs)
    check(lib().sf_masked_gemm_dgrad_reducescatter(_p(dy2d), _p(wm), arr, len(slot_ptrs), int(rank), T, wm.shape[1], out_local,
                                                   _gemm_dtype(dy2d, wm), _p(status), _stream()),
          "sf_masked_gemm_dgrad_reducescatter")


def reduce_slots(slots, out=None):
    """Sum over the leading axis of ``slots`` ([G, ...]) in slot order, fp32 accumulation."""
    _cuda(slots, out)
    G = slots.shape[0]
    if out is None:
        out = torch.empty(slots.shape[1:], dtype=slots.dtype, device=slots.device)
    check(lib().sf_reduce_slots(_p(slots), _p(out), G, out.numel(), _dt(slots), _stream()), "sf_reduce_slots")
    return out


def multimem_reduce(mc_ptr: int, out, *, max_ctas=0) -> None:
    """out[i] <- sum over the GPUs of a multicast object of their copy of the bf16 element at
    ``mc_ptr + 2 i`` (``mc_ptr``: a multicast address, e.g. ``PeerArena.mc_ptr(offset)``)."""
    import ctypes

    _cuda(out)
    if out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise TypeError("multimem_reduce: out must be a contiguous bfloat16 tensor")
    if not mc_ptr:
        raise RuntimeError("multimem_reduce: no multicast address (the node offers no multicast object)")
    check(lib().sf_multimem_reduce(ctypes.c_void_p(int(mc_ptr)), _p(out), out.numel(), _dt(out), int(max_ctas), _stream()),
          "sf_multimem_reduce")


def peer_export(t: torch.Tensor):
    """(handle bytes, byte offset) that another process of this node passes to ``peer_open``."""
    import ctypes

    _cuda(t)
    buf = ctypes.create_string_buffer(int(lib().sf_peer_handle_bytes()))
    off = ctypes.c_int64(0)
    check(lib().sf_peer_export(_p(t), buf, ctypes.byref(off)), "sf_peer_export")
    return bytes(buf.raw), int(off.value)


def peer_open(handle: bytes, offset: int):
    """Maps a buffer exported by another process; returns (base, pointer) as integers."""
    import ctypes

    base, ptr = ctypes.c_void_p(0), ctypes.c_void_p(0)
    check(lib().sf_peer_open(ctypes.c_char_p(handle), int(offset), ctypes.byref(base), ctypes.byref(ptr)), "sf_peer_open")
    return int(base.value), int(ptr.value)


def peer_close(base: int) -> None:
    check(lib().sf_peer_close(int(base)), "sf_peer_close")


# ----------------------------------------------------------------------------------------
# block-sparse-16
# ----------------------------------------------------------------------------------------
def bsr16_build(W, mask=None):
    """(blocks[nnz,16,16], row_ptr int32, col_idx int32) of W*mask; a block is kept iff sum|W*mask| > 0."""
    _cuda(W, mask)
    out, k = W.shape
    row_ptr = torch.zeros(out // 16 + 1, dtype=torch.int32, device=W.device)
    nnz_t = torch.zeros(1, dtype=torch.int32, device=W.device)
    md = _dt(mask) if mask is not None else SF_F32
    check(lib().sf_bsr16_build(_p(W), _p(mask), _dt(W), md, None, _p(row_ptr), None, _p(nnz_t), out, k, _stream()),
          "sf_bsr16_build")
    nnz = int(nnz_t.item())
    blocks = torch.zeros((max(nnz, 1), 16, 16), dtype=W.dtype, device=W.device)
    col_idx = torch.zeros(nnz, dtype=torch.int32, device=W.device)
    if nnz > 0:
        check(lib().sf_bsr16_build(_p(W), _p(mask), _dt(W), md, _p(blocks), _p(row_ptr), _p(col_idx), None, out, k,
                                   _stream()), "sf_bsr16_build")
    return blocks, row_ptr, col_idx


def bsr16_to_dense(blocks, row_ptr, col_idx, out, k):
    _cuda(blocks, row_ptr, col_idx)
    dense = torch.empty((out, k), dtype=blocks.dtype, device=blocks.device)
    if col_idx.numel() == 0:
        return dense.zero_()
    check(lib().sf_bsr16_to_dense(_p(blocks), _p(row_ptr), _p(col_idx), _p(dense), k, out, _dt(blocks), _stream()),
          "sf_bsr16_to_dense")
    return dense


def _bsr_ws(workspace, out, k, like):
    if workspace is None:
        workspace = torch.empty((out, k), dtype=like.dtype, device=like.device)
    return workspace


def bsr16_fwd(x2d, blocks, row_ptr, col_idx, out, bias=None, workspace=None, status=None, dense_ready=False):
    """y = x . W^T for a block-CSR weight. The kept blocks are scattered into ``workspace`` ([out, in], the
    weight dtype) and the product runs on the dense tensor-core tiles; ``dense_ready=True`` says that
    ``workspace`` still holds the scattered weight of these very blocks (a layer whose blocks have not
    changed since its last call), and skips the scatter."""
    _cuda(x2d, blocks, row_ptr, col_idx, bias, workspace, status)
    T, k = x2d.shape
    ws = _bsr_ws(workspace, out, k, x2d)
    if dense_ready and workspace is not None:
        return gemm_fwd(x2d, ws, bias=bias, status=status)
    y = torch.empty((T, out), dtype=x2d.dtype, device=x2d.device)
    check(lib().sf_bsr16_fwd(_p(x2d), _p(blocks), _p(row_ptr), _p(col_idx), _p(bias), _p(y), _p(ws), T, k, out,
                             _gemm_dtype(x2d, blocks), _p(status), _stream()), "sf_bsr16_fwd")
    return y


def bsr16_dgrad(dy2d, blocks, row_ptr, col_idx, k, workspace=None, status=None, dense_ready=False):
    _cuda(dy2d, blocks, row_ptr, col_idx, workspace, status)
    T, out = dy2d.shape
    ws = _bsr_ws(workspace, out, k, dy2d)
    if dense_ready and workspace is not None:
        return gemm_dgrad(dy2d, ws, status=status)
    dx = torch.empty((T, k), dtype=dy2d.dtype, device=dy2d.device)
    check(lib().sf_bsr16_dgrad(_p(dy2d), _p(blocks), _p(row_ptr), _p(col_idx), _p(dx), _p(ws), T, k, out,
                               _gemm_dtype(dy2d, blocks), _p(status), _stream()), "sf_bsr16_dgrad")
    return dx


def bsr16_wgrad(dy2d, x2d, row_ptr, col_idx, workspace=None, status=None):
    _cuda(dy2d, x2d, row_ptr, col_idx, workspace, status)
    T, out = dy2d.shape
    k = x2d.shape[1]
    ws = _bsr_ws(workspace, out, k, x2d)
    dblocks = torch.zeros((max(col_idx.numel(), 1), 16, 16), dtype=x2d.dtype, device=x2d.device)
    check(lib().sf_bsr16_wgrad(_p(dy2d), _p(x2d), _p(row_ptr), _p(col_idx), _p(dblocks), _p(ws), T, k, out,
                               _gemm_dtype(dy2d, x2d), _p(status), _stream()), "sf_bsr16_wgrad")
    return dblocks


def score_norm_from_sums(sums, n, norm) -> None:
    """norm <- (mean, std + 1e-6) from device sums (sum s, sum s^2) over n elements."""
    _cuda(sums, norm)
    check(lib().sf_score_norm_from_sums(_p(sums), float(n), _p(norm), _stream()), "sf_score_norm_from_sums")
