"""Pins the CPU oracle against outputs of the reference itself (tests/golden/*.npz).

Each stage of the oracle is fed the reference's own inputs for that stage and must reproduce
the reference's output: bit-exact for hard masks, flip counts and block-CSR indices, and to
fp32 / bf16 rounding for floats (the same torch CPU ops are used, so most are bit-exact too).
"""
import math

import numpy as np
import pytest
import torch

from oracle import sparselinear_oracle as O
from tests.golden_io import Golden, rel_err

F32_TOL = 1e-5
BF16_TOL = 1e-2


def test_ties_projection_bit_exact():
    g = Golden("ties")
    for name in g["names"]:
        soft, hard = g[f"{name}_soft"], g[f"{name}_hard"]
        assert torch.equal(O.hard_mask_from_soft(soft, "structured"), hard), name
        # the stock topk only ever differs inside groups holding an exact 2nd/3rd tie
        assert g.scalar(f"{name}_stock_topk_diff_groups") <= g.scalar(f"{name}_tie_groups")
    assert g.scalar("ones_stock_topk_diff_groups") > 0  # the tie rule matters
    assert torch.equal(O.hard_mask_from_soft(g["tail_soft"], "nm_2_4"), g["tail_hard"])
    assert bool((g["tail_hard"][:, 28:] == 1).all())
    with pytest.raises(ValueError):
        O.hard_mask_from_soft(g["tail_soft"], "structured")


def test_metadata_round_trip():
    g = Golden("ties")
    for name in g["names"]:
        hard = g[f"{name}_hard"]
        meta = O.meta_from_hard(hard)
        rows, cols = hard.shape
        assert meta.shape == (rows, (cols + 7) // 8)
        nib = torch.stack([meta & 0xF, meta >> 4], dim=-1).view(rows, -1)[:, : cols // 4].long()
        i0, i1 = nib & 3, nib >> 2
        assert bool((i0 < i1).all())
        rebuilt = torch.zeros(rows, cols // 4, 4)
        rebuilt.scatter_(-1, i0.unsqueeze(-1), 1.0)
        rebuilt.scatter_(-1, i1.unsqueeze(-1), 1.0)
        assert torch.equal(rebuilt.view(rows, cols), hard)


@pytest.mark.parametrize("case,tol", [("chain_f32", F32_TOL), ("chain_bf16", BF16_TOL)])
def test_chain_stages(case, tol):
    g = Golden(case)
    W = g["W0"]
    H = torch.ones(W.shape)
    probe = 0
    m = torch.zeros_like(W)
    v = torch.zeros_like(W)
    mask = torch.ones(W.shape)
    X, dY = g["X"], g["dY"]
    lam = g.scalar("lambda_mid")
    for t in range(g.scalar("n_steps")):
        hx = g.scalar(f"s{t}_hx_fwd")
        assert torch.equal(mask, g[f"s{t}_mask_fwd"])
        # masked forward / backward
        eff = O.effective_mask(mask, hx)
        Y = O.linear_forward(X, W, eff)
        dx, dW, _ = O.linear_backward(X, W, eff, dY)
        assert rel_err(Y, g[f"s{t}_Y"]) <= tol
        assert rel_err(dx, g[f"s{t}_dX"]) <= tol
        assert rel_err(dW, g[f"s{t}_dW"]) <= tol
        # Hutchinson accumulation from the reference's hvp
        while probe < g.scalar(f"s{t}_probes_end"):
            H = O.hutchinson_accumulate(H, g[f"hvp_{probe}"], g[f"v_{probe}"].float(), 0.99)
            assert rel_err(H, g[f"H_{probe}"]) <= F32_TOL
            H = g[f"H_{probe}"].clone()
            probe += 1
        # AdamW on the reference's gradient
        W, m, v = O.adamw_step(W, g[f"s{t}_dW"], m, v, step=t + 1, lr=1e-4, betas=(0.9, 0.95), eps=1e-8,
                               weight_decay=0.1, mask=mask, decay=2e-4)
        assert rel_err(W, g[f"s{t}_W_opt"]) <= tol
        assert rel_err(m, g[f"s{t}_m"]) <= tol
        assert rel_err(v, g[f"s{t}_v"]) <= tol
        W, m, v = g[f"s{t}_W_opt"].clone(), g[f"s{t}_m"].clone(), g[f"s{t}_v"].clone()
        # score -> gate -> mask update -> projection
        raw = O.importance_score(W, "hessian_obd", H=H)
        assert rel_err(raw, g[f"s{t}_score_raw"]) <= F32_TOL
        G = O.gate_target_structured(O.normalize_scores(raw), g.scalar(f"s{t}_T"))
        assert rel_err(G, g[f"s{t}_G"]) <= F32_TOL
        new_mask = O.mask_update(mask, g[f"s{t}_G"], mask_lr=0.1, lambda_mid=lam, penalty_mode="structured_topn")
        assert rel_err(new_mask, g[f"s{t}_mask"]) <= F32_TOL
        assert O.flip_count(mask, g[f"s{t}_mask"]) == g.scalar(f"s{t}_flips")
        mask = g[f"s{t}_mask"].clone()
        assert torch.equal(O.hard_mask_from_soft(mask), g[f"s{t}_hard"])
        assert math.isclose(O.mask_stats(mask)["sum_m1m"], g.scalar(f"s{t}_mid_sum"), rel_tol=1e-9, abs_tol=1e-9)


def test_chain_paper_recipe():
    """Unstructured gate from a sampled quantile + nm_2_4 penalty and projection + |W|/sqrt(H) score."""
    g = Golden("chain_paper")
    lam = g.scalar("lambda_mid")
    mask = torch.ones(g["W0"].shape)
    for t in range(g.scalar("n_steps")):
        assert torch.equal(mask, g[f"s{t}_mask_fwd"])
        hx = g.scalar(f"s{t}_hx_fwd")
        eff = O.effective_mask(mask, hx, mode="nm_2_4")
        assert rel_err(O.linear_forward(g["X"], g[f"s{t}_W_fwd"], eff), g[f"s{t}_Y"]) <= BF16_TOL
        W, H = g[f"s{t}_W_opt"], g[f"H_{g.scalar(f's{t}_probes_end') - 1}"]
        raw = O.importance_score(W, "hessian_ratio", H=H)
        assert rel_err(raw, g[f"s{t}_score_raw"]) <= F32_TOL
        s = O.normalize_scores(raw)
        tau = O.tau_unstructured(s, 0.5, 1024, g[f"s{t}_tau_idx"])
        G = O.gate_target_unstructured(s, tau, g.scalar(f"s{t}_T"))
        assert rel_err(G, g[f"s{t}_G"]) <= F32_TOL
        new_mask = O.mask_update(mask, g[f"s{t}_G"], mask_lr=0.1, lambda_mid=lam, pen_lr=0.1, penalty_mode="nm_2_4")
        assert rel_err(new_mask, g[f"s{t}_mask"]) <= F32_TOL
        assert O.flip_count(mask, g[f"s{t}_mask"], "nm_2_4") == g.scalar(f"s{t}_flips")
        mask = g[f"s{t}_mask"].clone()
        assert torch.equal(O.hard_mask_from_soft(mask, "nm_2_4"), g[f"s{t}_hard"])


def test_training_loop_replay():
    """The oracle, free running, follows the reference's two-layer training loop step for step
    (forward, mid penalty, Hutchinson double backward, clip, AdamW with SR-STE decay, mask update
    with the top-N penalty pull, hardening) and ends in the same finalized state."""
    import json

    g = Golden("train_loop")
    hp, cfg = json.loads(str(g["hp_json"])), json.loads(str(g["cfg_json"]))
    W = {"fc1": g["init/fc1.weight"].clone(), "fc2": g["init/fc2.weight"].clone()}
    b1 = g["init/fc1.bias"].clone()
    mask = {k: torch.ones(W[k].shape) for k in W}
    H = {k: torch.ones(W[k].shape) for k in W}
    hx = {k: 1.0 for k in W}
    st = {k: (torch.zeros_like(t), torch.zeros_like(t)) for k, t in (("fc1", W["fc1"]), ("b1", b1), ("fc2", W["fc2"]))}
    tol = 1e-5
    for it in range(hp["steps"]):
        w1, w2, bb = W["fc1"].clone().requires_grad_(True), W["fc2"].clone().requires_grad_(True), b1.clone().requires_grad_(True)
        h = O.MaskedLinearSTE.apply(g["X"][it], w1, bb, O.effective_mask(mask["fc1"], hx["fc1"]))
        out = O.MaskedLinearSTE.apply(torch.nn.functional.gelu(h), w2, None, O.effective_mask(mask["fc2"], hx["fc2"]))
        lam = hp["lambda_mid_max"] * min(1.0, it / hp["lambda_mid_warmup"])
        loss = torch.nn.functional.mse_loss(out, g["Yt"][it]) + O.mid_penalty_value(list(mask.values()), lam)
        assert math.isclose(float(loss.detach()), g.scalar(f"s{it}_loss"), rel_tol=tol)
        probes = [g[f"s{it}_probe{j}"].float() for j in range(2)]
        hvps = O.hutchinson_hvps(loss, [w1, w2], probes)
        for k, hv, pv in zip(("fc1", "fc2"), hvps, probes):
            H[k] = O.hutchinson_accumulate(H[k], hv.detach(), pv, cfg["beta"])
            assert rel_err(H[k], g[f"s{it}_{k}_H"]) <= tol
        grads = torch.autograd.grad(loss, [w1, bb, w2])
        grads, gnorm = O.clip_grad_norm(list(grads), hp["grad_clip"])
        assert math.isclose(gnorm, g.scalar(f"s{it}_gnorm"), rel_tol=tol)
        decay = cfg["srste_decay"] * min(1.0, (it + 1) / hp["decay_ramp"])
        kw = dict(step=it + 1, lr=hp["lr"], betas=tuple(hp["betas"]), eps=1e-8, weight_decay=hp["weight_decay"])
        W["fc1"], *st["fc1"] = O.adamw_step(W["fc1"], grads[0], *st["fc1"], mask=mask["fc1"], decay=decay, **kw)
        b1, *st["b1"] = O.adamw_step(b1, grads[1], *st["b1"], **kw)
        W["fc2"], *st["fc2"] = O.adamw_step(W["fc2"], grads[2], *st["fc2"], mask=mask["fc2"], decay=decay, **kw)
        assert rel_err(b1, g[f"s{it}_fc1_b"]) <= tol
        flips = 0
        for k in ("fc1", "fc2"):
            assert rel_err(W[k], g[f"s{it}_{k}_W"]) <= tol
            T = O.temperature_at(it, cfg["temp_init"], cfg["temp_decay"], cfg["temp_min"])
            G = O.gate_target_structured(O.normalize_scores(O.importance_score(W[k], "hessian_obd", H=H[k])), T)
            new = O.mask_update(mask[k], G, mask_lr=cfg["mask_lr"], lambda_mid=lam, penalty_mode="structured_topn")
            assert rel_err(new, g[f"s{it}_{k}_mask"]) <= tol
            flips += O.flip_count(mask[k], new)
            mask[k] = new
            hx[k] = O.hardening_x(it, cfg["mask_hardening_start"], cfg["mask_hardening_duration"])
            assert math.isclose(hx[k], g.scalar(f"s{it}_{k}_hx"), abs_tol=1e-12)
        assert flips == int(g[f"s{it}_flip"][0])
    # bake-in: mask <- top2(mask), weight *= mask (legacy/main_llama.py:2552-2563)
    for k in ("fc1", "fc2"):
        hard = O.hard_mask_from_soft(mask[k])
        assert torch.equal(hard, g[f"final/{k}.mask"])
        assert rel_err(W[k] * hard, g[f"final/{k}.weight"]) <= tol
    h = O.linear_forward(g["eval_X"], g["final/fc1.weight"], g["final/fc1.mask"], bias=g["final/fc1.bias"])
    Ye = O.linear_forward(torch.nn.functional.gelu(h), g["final/fc2.weight"], g["final/fc2.mask"])
    assert rel_err(Ye, g["eval_Y"]) <= tol


def test_glu_joint_mask_update():
    """Gate / up pairs updated from the summed score, the third layer on its own."""
    import json

    g = Golden("glu_joint")
    base, variants = json.loads(str(g["base_json"])), json.loads(str(g["variants_json"]))
    for tag in [str(t) for t in g["variants"]]:
        cfg = dict(base, **variants[tag])
        W = {n: g[f"{tag}_{n}_W"] for n in ("gate", "up", "down")}
        H = {n: g[f"{tag}_{n}_H"] for n in ("gate", "up", "down")}
        mask = {n: g[f"{tag}_{n}_mask0"].clone() for n in ("gate", "up", "down")}
        for step in range(3):
            lam = g.scalar(f"{tag}_s{step}_lambda")
            T = O.temperature_at(step, cfg["temp_init"], cfg["temp_decay"], cfg["temp_min"])
            beta_s = O.beta_structural(step, cfg.get("beta_structural_start", 0), cfg.get("beta_structural_end", 0))
            bd = cfg.get("mask_binarize_decay", 0.0)
            sc = {n: O.importance_score(W[n], "hessian_obd", H=H[n]) for n in W}
            N, M = int(cfg["N"]), int(cfg["M"])
            new_gate, new_up = O.glu_joint_update(sc["gate"], sc["up"], mask["gate"], mask["up"], temperature=T,
                                                  mask_lr=cfg["mask_lr"], lambda_mid=lam, pen_lr=cfg["mask_penalty_lr"],
                                                  penalty_mode=cfg["mask_penalty_mode"], binarize_decay=bd, beta_s=beta_s,
                                                  n=N, m=M)
            G = O.gate_target_structured(O.normalize_scores(sc["down"]), T, beta_s=beta_s, n=N, m=M)
            new_down = O.mask_update(mask["down"], G, mask_lr=cfg["mask_lr"], lambda_mid=lam, pen_lr=cfg["mask_penalty_lr"],
                                     penalty_mode=cfg["mask_penalty_mode"], binarize_decay=bd, n=N, m=M)
            for n, new in (("gate", new_gate), ("up", new_up), ("down", new_down)):
                assert rel_err(new, g[f"{tag}_s{step}_{n}_mask"]) <= F32_TOL, (tag, step, n)
                assert O.flip_count(mask[n], g[f"{tag}_s{step}_{n}_mask"], "structured", N, M) == \
                    g.scalar(f"{tag}_s{step}_{n}_flips")
                mask[n] = g[f"{tag}_s{step}_{n}_mask"].clone()
                hx = O.hardening_x(step, cfg["mask_hardening_start"], cfg["mask_hardening_duration"])
                assert math.isclose(hx, g.scalar(f"{tag}_s{step}_{n}_hx"), abs_tol=1e-12)


def _same_stats(got, keys, values, rel):
    for k, v in zip(keys, values):
        if math.isnan(v):
            assert math.isnan(got[str(k)]), k
        else:
            assert math.isclose(got[str(k)], float(v), rel_tol=rel, abs_tol=1e-12), (k, got[str(k)], v)


def test_mask_log_stats():
    g = Golden("mask_stats")
    for tag in ("inside", "edges"):
        got = O.mask_log_stats([g[f"{tag}_fc1_mask"], g[f"{tag}_fc2_mask"]], [g[f"{tag}_idx0"], g[f"{tag}_idx1"]])
        _same_stats(got, g[f"{tag}_keys"], g[f"{tag}_values"].tolist(), 1e-12)
        # the per-step reductions over the same masks: mid penalty, sparsity penalty, 2:4 tile statistics
        masks = [g[f"{tag}_fc1_mask"], g[f"{tag}_fc2_mask"]]
        assert math.isclose(float(O.mid_penalty_value(masks, 0.7)), g.scalar(f"{tag}_mid_penalty"), rel_tol=1e-6)
        st = [O.mask_stats(m) for m in masks]
        n = sum(m.numel() for m in masks)
        assert g.scalar(f"{tag}_sparsity_cur") == 0.5  # structured layers: (M - N) / M by construction
        assert math.isclose(g.scalar(f"{tag}_sparsity_pen"), 2.0 * (0.5 - 0.4) ** 2, rel_tol=1e-6)
        cur = sum(s["count_lt_half"] for s in st) / n
        assert math.isclose(cur, g.scalar(f"{tag}_sparsity_cur_unstructured"), rel_tol=1e-12)
        assert math.isclose(2.0 * (cur - 0.4) ** 2, g.scalar(f"{tag}_sparsity_pen_unstructured"), rel_tol=1e-5)
        top2 = sum(s["sum_top2"] for s in st) / (n / 4 * 2)
        bot2 = sum(s["sum_bot2"] for s in st) / (n / 4 * 2)
        want = dict(zip([str(k) for k in g[f"{tag}_tile_keys"]], g[f"{tag}_tile_values"].tolist()))
        # the reference adds the sorted groups up in fp32: a few 1e-7 from the exact sums
        assert math.isclose(top2, want["top2_avg"], rel_tol=2e-6) and math.isclose(bot2, want["bot2_avg"], rel_tol=2e-6)
        assert math.isclose(1.0 - top2, want["top2_gap"], rel_tol=5e-6)
        assert math.isclose((1.0 - top2) + bot2, want["total_gap"], rel_tol=5e-6)


@pytest.mark.parametrize("tag,tol", [("f32", 1e-5), ("bf16", BF16_TOL), ("chunks", 1e-5)])
def test_kl_distill_loss(tag, tol):
    g = Golden("kl_loss")
    s = g[f"{tag}_student"].clone().requires_grad_(True)
    kl = O.kl_distill_loss(s, g[f"{tag}_teacher"])
    (kl * 1.5).backward()
    assert rel_err(kl.detach().float(), g[f"{tag}_kl"]) <= tol
    assert rel_err(s.grad.float(), g[f"{tag}_grad"].float()) <= tol


def test_slorb_bypass():
    g = Golden("slorb")
    for tag in ("mean", "sum"):
        W, mask, b = g[f"{tag}/weight"], g[f"{tag}/mask"], g[f"{tag}/bias"]
        xp, sw = O.slorb_init(W, mask, 8, tag)
        assert rel_err(sw, g[f"{tag}/SLoRB_Weight"]) <= F32_TOL
        if tag == "mean":
            assert torch.equal(xp, g[f"{tag}/x_proj"])
        x = g[f"{tag}_x"].clone().requires_grad_(True)
        w = W.clone().requires_grad_(True)
        s_w = g[f"{tag}/SLoRB_Weight"].clone().requires_grad_(True)
        y = O.MaskedLinearSTE.apply(x, w, b, O.effective_mask(mask, 1.0)) + O.slorb_bypass(x, g[f"{tag}/x_proj"], s_w)
        y.backward(g[f"{tag}_dy"])
        assert rel_err(y, g[f"{tag}_y"]) <= F32_TOL
        assert rel_err(x.grad, g[f"{tag}_dx"]) <= F32_TOL
        assert rel_err(w.grad, g[f"{tag}_dW"]) <= F32_TOL
        assert rel_err(s_w.grad, g[f"{tag}_dS"]) <= F32_TOL


@pytest.mark.parametrize("tag,tol", [("f32", F32_TOL), ("bf16", BF16_TOL)])
def test_wanda_metric(tag, tol):
    """add_batch over three batches, then the score |W| sqrt(scaler_row + eps) through two mask updates."""
    g = Golden("wanda")
    W = g[f"{tag}_W"]
    scaler, n = torch.zeros(W.shape[1], dtype=W.dtype), 0
    for i in range(3):
        scaler, n = O.wanda_add_batch(scaler, n, g[f"{tag}_x{i}"])
        assert n == g.scalar(f"{tag}_nsamples{i}")
        assert rel_err(scaler.float(), g[f"{tag}_scaler{i}"].float()) <= (0.0 if tag == "bf16" else 1e-6)
    mask = g[f"{tag}_mask0"]
    for j in range(2):
        s = O.normalize_scores(O.importance_score(W, "wanda", scaler_row=scaler))
        G = O.gate_target_structured(s, g.scalar(f"{tag}_T{j}"))
        assert rel_err(G.float(), g[f"{tag}_G{j}"].float()) <= tol
        new_mask = O.mask_update(mask, g[f"{tag}_G{j}"], mask_lr=0.2, lambda_mid=0.3, pen_lr=0.2,
                                 penalty_mode="structured_topn")
        assert rel_err(new_mask, g[f"{tag}_mask{j + 1}"]) <= F32_TOL
        assert O.flip_count(mask, g[f"{tag}_mask{j + 1}"]) == g.scalar(f"{tag}_flips{j}")
        mask = g[f"{tag}_mask{j + 1}"].clone()


def test_freeze_bands_and_harden_fraction():
    """Frozen entries keep their own value as gate target; the low band snaps at every update, the
    high band from step 2000 on; harden_fraction rounds the entries nearest 0.5 over two layers."""
    g = Golden("freeze")
    W, H = g["W"], g["H"]
    mask, flags = g["mask0"], torch.zeros(W.shape)
    raw = O.importance_score(W, "hessian_obd", H=H)
    for j, step in enumerate(int(s) for s in g["steps"]):
        G = O.freeze_gate(O.gate_target_structured(O.normalize_scores(raw), g.scalar(f"s{j}_T")), mask, flags)
        assert rel_err(G, g[f"s{j}_G"]) <= F32_TOL
        new = O.mask_update(mask, g[f"s{j}_G"], mask_lr=0.3, lambda_mid=0.4, pen_lr=0.3, penalty_mode="structured_topn")
        new, flags = O.freeze_bands(new, flags, 0.08, 0.93, step)
        assert rel_err(new, g[f"s{j}_mask"]) <= F32_TOL
        assert torch.equal(flags, g[f"s{j}_flags"])
        assert O.flip_count(mask, g[f"s{j}_mask"]) == g.scalar(f"s{j}_flips")
        mask = g[f"s{j}_mask"].clone()
    assert int(flags.sum()) > 200 and int((mask == 1).sum()) > 100  # the fixture does freeze on both sides
    masks, fl, n = O.harden_fraction([g["hf_mask_a0"], g["hf_mask_b0"]], [g["hf_flags_a0"], g["hf_flags_b0"]],
                                     fraction=0.3, band_low=0.35, band_high=0.7)
    assert n == g.scalar("hf_count")
    assert torch.equal(masks[0], g["hf_mask_a1"]) and torch.equal(masks[1], g["hf_mask_b1"])
    assert torch.equal(fl[0], g["hf_flags_a1"]) and torch.equal(fl[1], g["hf_flags_b1"])


@pytest.mark.parametrize("tag", ["bs16", "bs32", "tail"])
def test_block_sparse_soft_masks(tag):
    import json

    g = Golden("block_masks")
    spec = json.loads(str(g["cases_json"]))[tag]
    cfg = dict(json.loads(str(g["base_json"])), **spec["cfg"])
    bs = 16 if cfg["hard_mask_type"] == "block_sparse16" else 32
    W, H = g[f"{tag}_W"], g[f"{tag}_H"]
    mask = torch.ones(W.shape)
    hx = 1.0
    for step in range(5):
        T = O.temperature_at(step, cfg["temp_init"] * 2.0, cfg["temp_decay"], cfg["temp_min"])
        assert math.isclose(T, g.scalar(f"{tag}_s{step}_T"), rel_tol=1e-12)
        sparsity = cfg["sparsity_ratio"] * min(1.0, step / cfg["sparsity_warmup_steps"]) ** 3
        assert math.isclose(sparsity, g.scalar(f"{tag}_s{step}_sp"), rel_tol=1e-12, abs_tol=1e-15)
        s = O.normalize_scores(O.importance_score(W, "hessian_obd", H=H))
        G = O.blockify(O.gate_target_block(s, bs, sparsity, T), bs)
        assert rel_err(G, g[f"{tag}_s{step}_G"]) <= F32_TOL
        if step >= cfg["sparsity_warmup_steps"]:
            new = O.mask_update_block(mask, G, bs, mask_lr=cfg["mask_lr"], sparsity_ratio=cfg["sparsity_ratio"],
                                      lambda_mid=0.25, pen_lr=cfg["mask_penalty_lr"], penalty_mode=cfg["mask_penalty_mode"],
                                      binarize_decay=cfg.get("mask_binarize_decay", 0.0))
            flips = int(((O.hard_mask_block(mask, bs, 0.5) > 0.5) ^ (O.hard_mask_block(new, bs, 0.5) > 0.5)).sum())
            assert flips == g.scalar(f"{tag}_s{step}_flips")
            mask = new
            hx = O.hardening_x(step, cfg["mask_hardening_start"], cfg["mask_hardening_duration"])
        assert rel_err(mask, g[f"{tag}_s{step}_mask"]) <= F32_TOL
        assert math.isclose(hx, g.scalar(f"{tag}_s{step}_hx"), abs_tol=1e-12)
        hard = O.hard_mask_block(mask, bs, cfg["sparsity_ratio"])
        assert torch.equal(hard, g[f"{tag}_s{step}_hard"])
        eff = mask if hx >= 1.0 - 1e-6 else hx * mask + (1.0 - hx) * hard
        assert rel_err(O.linear_forward(g[f"{tag}_x"], W, eff), g[f"{tag}_s{step}_y"]) <= F32_TOL


@pytest.mark.parametrize("tag", ["tile16", "tile16mid"])
def test_block16_tile_masks(tag):
    """hard_mask_type='block16': unstructured gate, per-tile top-k penalty and hard view."""
    import json

    g = Golden("block_masks")
    spec = json.loads(str(g["cases_json"]))[tag]
    cfg = dict(json.loads(str(g["base_json"])), **spec["cfg"])
    sr = cfg["sparsity_ratio"]
    W, H = g[f"{tag}_W"], g[f"{tag}_H"]
    mask, hx = torch.ones(W.shape), 1.0
    for step in range(5):
        T = O.temperature_at(step, cfg["temp_init"], cfg["temp_decay"], cfg["temp_min"])
        assert math.isclose(T, g.scalar(f"{tag}_s{step}_T"), rel_tol=1e-12)
        sparsity = sr * min(1.0, step / cfg["sparsity_warmup_steps"])
        s = O.normalize_scores(O.importance_score(W, "hessian_obd", H=H))
        G = O.gate_target_unstructured(s, O.tau_unstructured(s, sparsity, None), T)
        assert rel_err(G, g[f"{tag}_s{step}_G"]) <= F32_TOL
        if step >= cfg["sparsity_warmup_steps"]:
            new = O.mask_update_tile16(mask, G, mask_lr=cfg["mask_lr"], sparsity_ratio=sr, lambda_mid=0.25,
                                       pen_lr=cfg["mask_penalty_lr"], penalty_mode=cfg["mask_penalty_mode"],
                                       binarize_decay=cfg.get("mask_binarize_decay", 0.0))
            flips = int(((O.hard_mask_tile16(mask, sr) > 0.5) ^ (O.hard_mask_tile16(new, sr) > 0.5)).sum())
            assert flips == g.scalar(f"{tag}_s{step}_flips")
            mask = new
            hx = O.hardening_x(step, cfg["mask_hardening_start"], cfg["mask_hardening_duration"])
        assert rel_err(mask, g[f"{tag}_s{step}_mask"]) <= F32_TOL
        hard = O.hard_mask_tile16(mask, sr)
        assert torch.equal(hard, g[f"{tag}_s{step}_hard"])
        eff = mask if hx >= 1.0 - 1e-6 else hx * mask + (1.0 - hx) * hard
        assert rel_err(O.linear_forward(g[f"{tag}_x"], W, eff), g[f"{tag}_s{step}_y"]) <= F32_TOL


def test_chain_bf16_schedule():
    g = Golden("chain_bf16")
    decay = 0.05 ** (1.0 / 9.0)
    for t in range(g.scalar("n_steps")):
        assert math.isclose(O.temperature_at(t, 1.0, decay, 0.05), g.scalar(f"s{t}_T"), rel_tol=1e-12)
        assert math.isclose(O.hardening_x(t, 1, 3), g.scalar(f"s{t}_hx"), rel_tol=1e-12, abs_tol=1e-12)


def test_penalty_variants():
    g = Golden("penalty")
    modes = {"topn": "structured_topn", "nm24": "nm_2_4", "mid": "mid", "bin": "structured_topn", "beta": "mid",
             "exact": "mid", "lowT": "structured_topn"}
    for tag in g["variants"]:
        W, H, mask0 = g[f"{tag}_W"], g[f"{tag}_H"], g[f"{tag}_mask0"]
        s = O.normalize_scores(O.importance_score(W, "hessian_obd", H=H))
        G = O.gate_target_structured(s, g.scalar(f"{tag}_T"), exact=(tag == "exact"), beta_s=g.scalar(f"{tag}_beta_s"))
        assert rel_err(G, g[f"{tag}_G"]) <= F32_TOL, tag
        new = O.mask_update(mask0, g[f"{tag}_G"], mask_lr=0.2, lambda_mid=g.scalar(f"{tag}_lambda"), pen_lr=0.15,
                            penalty_mode=modes[tag], binarize_decay=0.05 if tag == "bin" else 0.0)
        assert rel_err(new, g[f"{tag}_mask1"]) <= F32_TOL, tag
        mode = "nm_2_4" if tag == "nm24" else "structured"
        assert O.flip_count(mask0, g[f"{tag}_mask1"], mode) == g.scalar(f"{tag}_flips"), tag
        assert math.isclose(O.hardening_x(g.scalar(f"{tag}_step"), 2, 8), g.scalar(f"{tag}_hx"), rel_tol=1e-12)


NM_MODES = {"4of8_topn": "structured_topn", "1of4_mid": "mid", "3of4_bin": "structured_topn", "1of2_plain": "mid",
            "8of16_beta": "mid", "8of32_exact": "mid", "2of8_bf16": "structured_topn", "4of8_bf16_mag": "mid"}


def test_general_nm_variants():
    """N:M other than 2:4: gate, penalties, EMA, hard view, flip count and the masked forward /
    backward of the reference, replayed by the oracle."""
    g = Golden("nm_general")
    for tag in g["variants"]:
        n, m, metric = int(g.scalar(f"{tag}_N")), int(g.scalar(f"{tag}_M")), str(g[f"{tag}_metric"])
        W, mask0 = g[f"{tag}_W"], g[f"{tag}_mask0"]
        bf16 = W.dtype == torch.bfloat16
        tol = BF16_TOL if bf16 else F32_TOL
        H = g[f"{tag}_H"] if metric != "magnitude" else None
        assert torch.equal(O.hard_mask_from_soft(mask0, "structured", n, m), g[f"{tag}_hard0"]), tag
        s = O.normalize_scores(O.importance_score(W, metric, H=H))
        G = O.gate_target_structured(s, g.scalar(f"{tag}_T"), exact=tag.endswith("exact"), beta_s=g.scalar(f"{tag}_beta_s"),
                                     n=n, m=m)
        assert G.dtype == g[f"{tag}_G"].dtype
        assert rel_err(G.float(), g[f"{tag}_G"].float()) <= tol, tag
        new = O.mask_update(mask0, g[f"{tag}_G"], mask_lr=0.2, lambda_mid=g.scalar(f"{tag}_lambda"), pen_lr=0.15,
                            penalty_mode=NM_MODES[tag], binarize_decay=0.05 if tag == "3of4_bin" else 0.0, n=n, m=m)
        assert rel_err(new, g[f"{tag}_mask1"]) <= tol, tag
        hard1 = O.hard_mask_from_soft(g[f"{tag}_mask1"], "structured", n, m)
        assert torch.equal(hard1, g[f"{tag}_hard1"]), tag
        assert int(hard1.sum()) == hard1.numel() * n // m
        assert O.flip_count(mask0, g[f"{tag}_mask1"], "structured", n, m) == g.scalar(f"{tag}_flips"), tag
        hx = g.scalar(f"{tag}_hx")
        assert math.isclose(O.hardening_x(g.scalar(f"{tag}_step"), 2, 8), hx, rel_tol=1e-12)
        assert 0.0 < hx < 1.0  # the forward below mixes the soft mask with the hard view
        eff = O.effective_mask(g[f"{tag}_mask1"], hx, "structured", False, n, m)
        X, dY = g[f"{tag}_X"], g[f"{tag}_dY"]
        Y = O.linear_forward(X, W, eff)
        assert rel_err(Y.float(), g[f"{tag}_Y"].float()) <= tol, tag
        dX, dW, _ = O.linear_backward(X, W, eff, dY)
        assert rel_err(dX.float(), g[f"{tag}_dX"].float()) <= tol, tag
        assert rel_err(dW.float(), g[f"{tag}_dW"].float()) <= tol, tag


UH_MODES = {"mid": "mid", "topn": "structured_topn", "beta": "mid", "bin": "mid", "bf16": "mid"}


def test_unstructured_hard_view_variants():
    """mask_type='unstructured' with its own hard view (mask > 0.5): quantile gate, pulls, beta mixing, EMA,
    flip count by the threshold, masked forward / backward, replayed by the oracle."""
    g = Golden("unstructured_hard")
    for tag in g["variants"]:
        W, H, mask0 = g[f"{tag}_W"], g[f"{tag}_H"], g[f"{tag}_mask0"]
        tol = BF16_TOL if W.dtype == torch.bfloat16 else F32_TOL
        s = O.normalize_scores(O.importance_score(W, "hessian_obd", H=H))
        tau = O.tau_unstructured(s, g.scalar(f"{tag}_sparsity"), None)
        G = O.gate_target_unstructured(s, tau, g.scalar(f"{tag}_T"), beta_s=g.scalar(f"{tag}_beta_s"))
        assert rel_err(G.float(), g[f"{tag}_G"].float()) <= tol, tag
        new = O.mask_update(mask0, g[f"{tag}_G"], mask_lr=0.2, lambda_mid=g.scalar(f"{tag}_lambda"), pen_lr=0.15,
                            penalty_mode=UH_MODES[tag], binarize_decay=0.05 if tag == "bin" else 0.0)
        assert rel_err(new, g[f"{tag}_mask1"]) <= tol, tag
        assert torch.equal(O.hard_mask_from_soft(g[f"{tag}_mask1"], "unstructured"), g[f"{tag}_hard1"]), tag
        assert O.flip_count(mask0, g[f"{tag}_mask1"], "unstructured") == g.scalar(f"{tag}_flips"), tag
        hx = g.scalar(f"{tag}_hx")
        assert 0.0 < hx < 1.0
        eff = O.effective_mask(g[f"{tag}_mask1"], hx, "unstructured")
        X, dY = g[f"{tag}_X"], g[f"{tag}_dY"]
        assert rel_err(O.linear_forward(X, W, eff).float(), g[f"{tag}_Y"].float()) <= tol, tag
        dX, dW, _ = O.linear_backward(X, W, eff, dY)
        assert rel_err(dX.float(), g[f"{tag}_dX"].float()) <= tol, tag
        assert rel_err(dW.float(), g[f"{tag}_dW"].float()) <= tol, tag


@pytest.mark.parametrize("tag,tol,l1", [("f32", F32_TOL, 0.0), ("bf16", BF16_TOL, 0.0), ("l1", F32_TOL, 0.02)])
def test_adamw(tag, tol, l1):
    g = Golden("adamw")
    p = g[f"{tag}_p0"]
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    for t in range(3):
        p, m, v = O.adamw_step(p, g[f"{tag}_g{t}"], m, v, step=t + 1, lr=1e-3, betas=(0.9, 0.95), eps=1e-8,
                               weight_decay=0.1, mask=g[f"{tag}_mask"], decay=5e-4 * (t + 1), adaptive_l1=l1)
        assert rel_err(p, g[f"{tag}_p{t + 1}"]) <= tol
        assert rel_err(m, g[f"{tag}_m{t + 1}"]) <= tol
        assert rel_err(v, g[f"{tag}_v{t + 1}"]) <= tol


@pytest.mark.parametrize("tag,tol", [("f32", F32_TOL), ("bf16", BF16_TOL)])
def test_adamw_amsgrad(tag, tol):
    g = Golden("adamw_ams")
    p = g[f"{tag}_p0"]
    m, v, vmax = torch.zeros_like(p), torch.zeros_like(p), torch.zeros_like(p)
    for t in range(4):
        p, m, v, vmax = O.adamw_step(p, g[f"{tag}_g{t}"], m, v, step=t + 1, lr=1e-3, betas=(0.9, 0.95), eps=1e-8,
                                     weight_decay=0.1, mask=g[f"{tag}_mask"], decay=5e-4 * (t + 1), v_max=vmax)
        for got, name in ((p, "p"), (m, "m"), (v, "v"), (vmax, "vmax")):
            assert rel_err(got.float(), g[f"{tag}_{name}{t + 1}"].float()) <= tol
    assert not torch.equal(vmax, v)  # the maximum is doing something in this fixture


def test_block_sparse_layout():
    g = Golden("block_sparse")
    W = g["W"]
    assert torch.equal(O.block16_keep_mask(W, 0.5), g["mask"])
    blocks, row_ptr, col_idx = O.bsr16_convert(W, g["mask"])
    assert torch.equal(blocks, g["blocks"])
    assert torch.equal(row_ptr, g["row_ptr"]) and torch.equal(col_idx, g["col_idx"])
    Y = g["X"].matmul((W * g["mask"]).t())
    assert rel_err(Y, g["Y"]) <= F32_TOL


def test_sparse24_compress_round_trip():
    torch.manual_seed(0)
    W = torch.randn(16, 64)
    vals, meta, hard = O.sparse24_compress(W, W.abs())
    assert torch.equal(hard, O.hard_mask_from_soft(W.abs()))
    nib = torch.stack([meta & 0xF, meta >> 4], dim=-1).view(16, -1).long()
    idx = torch.stack([nib & 3, nib >> 2], dim=-1)
    dense = torch.zeros(16, 16, 4)
    dense.scatter_(-1, idx, vals.view(16, 16, 2))
    assert torch.equal(dense.view(16, 64), W * hard)


def test_c_oracle_matches_reference_fixtures_and_python_oracle():
    """The C restatement of the projection (oracle/nm24_oracle.c) against the reference's outputs."""
    from oracle import nm24_c

    g = Golden("ties")
    for name in list(g["names"]) + ["tail"]:
        soft, want = g[f"{name}_soft"], g[f"{name}_hard"]
        hard, meta = nm24_c.project(soft.numpy())
        assert np.array_equal(hard, want.numpy()), name
        assert np.array_equal(meta, O.meta_from_hard(want).numpy()), name
    x = np.array([[np.nan, 1.0, 2.0, 3.0, 1.0, np.nan, np.nan, 0.0]], dtype=np.float32)
    assert np.array_equal(nm24_c.project(x)[0], O.hard_mask_from_soft(torch.from_numpy(x)).numpy())
    torch.manual_seed(3)
    big = torch.rand(256, 1024)
    hard, meta = nm24_c.project(big.numpy())
    assert np.array_equal(hard, O.hard_mask_from_soft(big).numpy())
    assert np.array_equal(meta, O.meta_from_hard(O.hard_mask_from_soft(big)).numpy())


def test_c1_full_size_chain():
    """The fp32 GPT-2-small MLP case at its full size ([3072, 768] weight, 8192 tokens): the oracle's
    whole chain (four Hutchinson probes through its own double backward, score, gate, mask update,
    projection, masked forward / backward) against the reference's recorded run (tests/golden/c1.npz)."""
    import numpy as np

    from tests import baseline_cases as B

    g = Golden("c1")
    W, X, dY = B.c1_inputs()
    for name, t in (("W", W), ("X", X), ("dY", dY)):
        assert torch.allclose(B.fingerprint(t), g[f"fp_{name}"], rtol=1e-12, atol=0), f"seeded input {name} differs"
    res = B.c1_oracle(W, X, dY)
    rows_w, rows_y, rows_x = g["rows_w"], g["rows_y"], g["rows_x"]

    def check(name, t, rows, rtol, atol_scale):
        t2 = t.reshape(-1, t.shape[-1])
        want = g[f"{name}_rows"]
        B.assert_elementwise(t2[rows], want, rtol, atol_scale * B.rms(want), name)
        s = g[f"{name}_sum"]
        assert abs(float(t2.double().sum()) - float(s[0])) <= 1e-4 * float(s[1]) ** 0.5 * t2.numel() ** 0.5 + 1e-9, name
        assert abs(float((t2.double() ** 2).sum()) - float(s[1])) <= 1e-4 * float(s[1]), name

    # second-order products of fp32 GEMMs: the summation order inside the host BLAS is the only difference
    for i in range(4):
        check(f"hvp_{i}", res["hvp"][i], rows_w, 1e-4, 1e-4)
        check(f"H_{i}", res["H"][i], rows_w, 1e-5, 1e-7)
    check("score_raw", res["score_raw"], rows_w, 1e-5, 1e-7)
    assert torch.allclose(res["score_mean_std"], g["score_mean_std"], rtol=1e-5, atol=0)
    check("G", res["G"], rows_w, 1e-5, 1e-7)
    check("mask", res["mask"], rows_w, 1e-5, 1e-7)
    want_hard = torch.from_numpy(np.unpackbits(g["hard_bits"].numpy(), axis=1)[:, : W.shape[1]].astype(np.float32))
    diff, groups = B.hard_mismatch(res["hard"], want_hard)
    ties = B.near_tie_groups(res["mask"], 1e-5)
    assert bool((groups & ~ties).sum() == 0), "a hard-mask group differs outside the near-ties of the soft mask"
    assert diff <= 2 * int(ties.sum())
    # given the same soft mask the projection is exact: flips follow from it
    if diff == 0:
        assert res["flips"] == g.scalar("flips")
    check("Y", res["Y"], rows_y, 1e-5, 1e-5)
    check("dX", res["dX"], rows_x, 1e-5, 1e-5)
    check("dW", res["dW"], rows_w, 1e-5, 1e-5)


@pytest.mark.parametrize("tag,tol", [("f32", F32_TOL), ("bf16", BF16_TOL)])
def test_movement_metric_and_grad_ema(tag, tol):
    """Gradient EMA + g^2 Hessian proxy and the movement score against the reference's run
    (tests/golden/movement.npz): the same ATen ops, so the EMA tensors are bit-identical."""
    g = Golden("movement")
    W0 = g[f"{tag}_W0"]
    ema, H = torch.zeros_like(W0), torch.zeros(W0.shape)
    mask = torch.ones(W0.shape)
    for t in range(3):
        ema, H = O.grad_hessian_ema(ema, H, g[f"{tag}_g{t}"], 0.9)
        assert torch.equal(ema, g[f"{tag}_ema{t}"])
        assert torch.equal(H, g[f"{tag}_H{t}"])
        raw = O.importance_score(g[f"{tag}_W{t + 1}"], "movement", grad_ema=ema, temperature=0.7)
        G = O.gate_target_structured(O.normalize_scores(raw), O.temperature_at(t, 1.0, 0.8, 0.05))
        assert rel_err(G.float(), g[f"{tag}_G{t}"].float()) <= tol
        new_mask = O.mask_update(mask, g[f"{tag}_G{t}"].float(), mask_lr=0.2)
        assert rel_err(new_mask, g[f"{tag}_mask{t + 1}"]) <= F32_TOL
        assert O.flip_count(mask, g[f"{tag}_mask{t + 1}"]) == g.scalar(f"{tag}_flips{t}")
        mask = g[f"{tag}_mask{t + 1}"].clone()
