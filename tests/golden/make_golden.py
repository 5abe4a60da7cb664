"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE ITSELF.

Run where the SparseForge reference is available (it is imported, unmodified, from
``$SPARSEFORGE_REFERENCE/legacy``):

    SPARSEFORGE_REFERENCE=<checkout of liuhanzuo/SparseForge> WANDB_MODE=disabled python tests/golden/make_golden.py

The reference runs on torch CPU with ``torch.topk`` replaced by a tie-stable version (equal
values: lower index first), the tie rule this path is specified with; ``ties.npz`` also
records how many 2:4 groups the stock ``torch.topk`` decides differently and how many groups
hold an exact 2nd/3rd tie. Every fixture stores inputs, intermediates and outputs, so each
stage can be replayed on its own. bf16 tensors are stored as raw uint16 bits under keys
ending in ``__bf16``. Nothing here is needed at test time except the ``.npz`` files.
"""
from __future__ import annotations

import collections
import json
import os
import sys

os.environ.setdefault("WANDB_MODE", "disabled")
import numpy as np
import torch

REF = os.environ.get("SPARSEFORGE_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "legacy")):
    raise SystemExit("set SPARSEFORGE_REFERENCE to a checkout of the SparseForge reference (the directory holding legacy/)")
sys.path.insert(0, os.path.join(REF, "legacy"))
HERE = os.path.dirname(os.path.abspath(__file__))

_orig_topk = torch.topk
_TopK = collections.namedtuple("topk", ["values", "indices"])


def stable_topk(x, k, dim=-1, largest=True, sorted=True):  # noqa: A002
    # the k smallest are only used through their values (harden_fraction's threshold), where ties do not matter
    s = torch.sort(x, dim=dim, descending=bool(largest), stable=True)
    sl = [slice(None)] * x.dim()
    sl[dim] = slice(0, k)
    return _TopK(s.values[tuple(sl)], s.indices[tuple(sl)])


torch.topk = stable_topk
import adamw as ref_adamw  # noqa: E402
import sparse_modeling as ref_sm  # noqa: E402
import triton_block_sparse as ref_bs  # noqa: E402
import utils as ref_utils  # noqa: E402


def put(d, name, t):
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().contiguous().clone()
        if t.dtype == torch.bfloat16:
            d[name + "__bf16"] = t.view(torch.int16).numpy().view(np.uint16)
        else:
            d[name] = t.numpy()
    else:
        d[name] = np.asarray(t)


def save(name, d):
    d["torch_version"] = np.asarray(torch.__version__)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
    print(name, {k: getattr(v, "shape", None) for k, v in d.items() if k != "torch_version"})


def rademacher(shape, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 2, shape, generator=g, dtype=torch.int8).float() * 2 - 1).to(dtype)


def make_layer(out_f, in_f, W, dtype, **cfg_kw):
    cfg = ref_sm.SparseLinearConfig(**cfg_kw)
    layer = ref_sm.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False)
    layer = layer.to(dtype)
    layer.weight.data.copy_(W.to(dtype))
    layer.initialize()
    # fp32 mask / Hessian next to (possibly bf16) weights, the dtype mix of the LLaMA-shaped runs
    layer.mask.data = layer.mask.data.float()
    layer.hessian_diag.data = layer.hessian_diag.data.float()
    layer.sync_weight()
    return layer


def hutchinson_once(layer, X, dY, v, d, tag):
    """One update_hessian_hutchinson call with an injected probe; records hvp and H."""
    T = X.shape[0] * X.shape[1]

    def loss_fn():
        Y = layer(X)
        return (torch.nn.functional.gelu(Y.float()) * dY.float()).sum() / T

    # the same double backward the reference performs, only to record hvp
    loss = loss_fn()
    (g,) = torch.autograd.grad(loss, [layer.weight], create_graph=True, retain_graph=True)
    (hvp,) = torch.autograd.grad((g * v).sum(), [layer.weight], retain_graph=False)
    put(d, f"hvp_{tag}", hvp)
    ref_utils._rademacher_like = lambda t: v.clone()
    ref_utils.update_hessian_hutchinson(layer, loss_fn())
    put(d, f"H_{tag}", layer.hessian_diag.data)


_orig_randint = torch.randint


def case_chain(name, out_f, in_f, batch, seq, dtype, steps, cfg_kw, lambda_mid=0.0, seed=0, tau_idx_seed=None):
    """Score -> mask update -> projection -> masked fwd/bwd -> AdamW, `steps` times."""
    torch.manual_seed(seed)
    W = torch.randn(out_f, in_f) * 0.02
    X = torch.randn(batch, seq, in_f).to(dtype)
    dY = torch.randn(batch, seq, out_f).to(dtype)
    d = {}
    put(d, "W0", W.to(dtype)); put(d, "X", X); put(d, "dY", dY)
    layer = make_layer(out_f, in_f, W, dtype, **cfg_kw)
    opt = ref_adamw.AdamW([layer.weight], lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
    d["n_steps"] = np.asarray(steps)
    d["lambda_mid"] = np.asarray(lambda_mid)
    probe = 0
    for t in range(steps):
        Xr = X.clone().requires_grad_(True)
        # forward / backward with the current mask and hardening state
        put(d, f"s{t}_hx_fwd", float(layer.hardening_x))
        put(d, f"s{t}_mask_fwd", layer.mask.data)
        put(d, f"s{t}_W_fwd", layer.weight.data)
        layer.weight.grad = None
        Y = layer(Xr)
        Y.backward(dY)
        put(d, f"s{t}_Y", Y); put(d, f"s{t}_dX", Xr.grad); put(d, f"s{t}_dW", layer.weight.grad)
        # Hutchinson probes (one per step; the first step takes four, as in the fp32 config)
        for _ in range(4 if t == 0 else 1):
            v = rademacher((out_f, in_f), 1 + probe, dtype)
            put(d, f"v_{probe}", v.to(torch.int8))
            hutchinson_once(layer, X, dY, v, d, str(probe))
            probe += 1
        d[f"s{t}_probes_end"] = np.asarray(probe)
        # optimizer
        opt.step(decay=2e-4)
        st = opt.state[layer.weight]
        put(d, f"s{t}_W_opt", layer.weight.data); put(d, f"s{t}_m", st["exp_avg"]); put(d, f"s{t}_v", st["exp_avg_sq"])
        # mask update
        put(d, f"s{t}_T", layer._temperature(t))
        if tau_idx_seed is not None:
            # the unstructured gate samples score positions with torch.randint: inject recorded ones
            gi = torch.Generator().manual_seed(tau_idx_seed + t)
            idx = _orig_randint(0, out_f * in_f, (int(layer.cfg.tau_sample_size),), generator=gi)
            put(d, f"s{t}_tau_idx", idx)
            torch.randint = lambda *a, **k: idx.clone()
        G = layer.compute_gate_target(t)
        put(d, f"s{t}_G", G)
        if layer.mask_metric == "hessian_ratio":
            raw = layer.weight.data.abs() / torch.sqrt(layer.hessian_diag.data + 1e-8)
        else:
            raw = (layer.hessian_diag.data + 1e-8) * (layer.weight.data * layer.weight.data)
        put(d, f"s{t}_score_raw", raw)
        ref_utils.calculate_model_mask(layer, step=t, lambda_mid=lambda_mid)
        torch.randint = _orig_randint
        put(d, f"s{t}_mask", layer.mask.data)
        put(d, f"s{t}_hx", float(layer.hardening_x))
        put(d, f"s{t}_flips", int(layer.weight.flipped_mask))
        put(d, f"s{t}_hard", layer._hard_mask_from_soft(layer.mask.data))
        put(d, f"s{t}_mid_sum", float((layer.mask.data.double() * (1 - layer.mask.data.double())).sum()))
    save(name, d)


def case_penalty():
    """update_mask with the penalty pulls, binarize push and beta mixing switched on."""
    torch.manual_seed(7)
    out_f, in_f = 40, 64
    d = {}
    variants = [
        ("topn", dict(mask_penalty_mode="structured_topn"), 0.7, 0.0),
        ("nm24", dict(mask_penalty_mode="nm_2_4", hard_mask_type="nm_2_4"), 0.4, 0.0),
        ("mid", dict(mask_penalty_mode="mid"), 0.9, 0.0),
        ("bin", dict(mask_penalty_mode="structured_topn", mask_binarize_decay=0.05), 0.3, 0.0),
        ("beta", dict(mask_penalty_mode="mid", beta_structural_start=0, beta_structural_end=10), 0.0, 0.0),
        ("exact", dict(structured_exact=True), 0.0, 0.0),
        ("lowT", dict(temp_init=0.01, temp_min=0.01, mask_penalty_mode="structured_topn"), 0.5, 0.0),
    ]
    d["variants"] = np.asarray([v[0] for v in variants])
    for tag, kw, lam, _ in variants:
        W = torch.randn(out_f, in_f) * 0.02
        layer = make_layer(out_f, in_f, W, torch.float32, mask_type="structured", mask_metric="hessian_obd",
                           mask_update_period=1, sparsity_warmup_steps=0, mask_lr=0.2, mask_penalty_lr=0.15,
                           mask_hardening_start=2, mask_hardening_duration=8, **kw)
        layer.mask.data = torch.rand(out_f, in_f)
        layer.hessian_diag.data = torch.rand(out_f, in_f) + 0.1
        step = 4
        put(d, f"{tag}_W", W); put(d, f"{tag}_H", layer.hessian_diag.data); put(d, f"{tag}_mask0", layer.mask.data)
        put(d, f"{tag}_lambda", lam); put(d, f"{tag}_step", step)
        put(d, f"{tag}_T", layer._temperature(step)); put(d, f"{tag}_beta_s", layer._beta_structural(step))
        put(d, f"{tag}_G", layer.compute_gate_target(step))
        layer.update_mask(step, lambda_mid=lam)
        put(d, f"{tag}_mask1", layer.mask.data); put(d, f"{tag}_hx", float(layer.hardening_x))
        put(d, f"{tag}_flips", int(layer.weight.flipped_mask))
    save("penalty", d)


def case_ties():
    """Hard projection on inputs full of ties, plus the disagreement count of the stock topk."""
    torch.manual_seed(11)
    d = {}
    cfg = dict(mask_type="structured", mask_metric="magnitude")
    layer = make_layer(8, 16, torch.randn(8, 16), torch.float32, **cfg)
    inputs = {
        "ones": torch.ones(24, 32),
        "bf16q": torch.rand(64, 128).to(torch.bfloat16).float(),
        "coarse": (torch.randint(0, 4, (48, 64)).float() / 4.0),
        "rand": torch.rand(64, 64),
        "special": torch.tensor([[0.0, -0.0, 0.0, -0.0, 1.0, 1.0, 0.5, 1.0],
                                 [0.5, 0.5, 0.5, 0.7, 2.0, 1.0, 1.0, 1.0]]),
    }
    d["names"] = np.asarray(list(inputs))
    for k, soft in inputs.items():
        put(d, f"{k}_soft", soft)
        put(d, f"{k}_hard", layer._hard_mask_from_soft(soft))
        torch.topk = _orig_topk
        stock = layer._hard_mask_from_soft(soft)
        torch.topk = stable_topk
        g = soft.view(soft.shape[0], -1, 4)
        srt = torch.sort(g, dim=-1, descending=True).values
        tie_groups = int((srt[..., 1] == srt[..., 2]).sum())
        diff_groups = int(((stock != layer._hard_mask_from_soft(soft)).view(soft.shape[0], -1, 4).any(-1)).sum())
        d[f"{k}_tie_groups"] = np.asarray(tie_groups)
        d[f"{k}_stock_topk_diff_groups"] = np.asarray(diff_groups)
    # nm_2_4 projection keeps a ragged tail (in % 4 != 0) at 1
    layer.hard_mask_type = "nm_2_4"
    tail = torch.rand(12, 30)
    put(d, "tail_soft", tail); put(d, "tail_hard", layer._hard_mask_from_soft(tail))
    save("ties", d)


def case_adamw():
    torch.manual_seed(5)
    d = {}
    for tag, dtype, l1 in (("f32", torch.float32, 0.0), ("bf16", torch.bfloat16, 0.0), ("l1", torch.float32, 0.02)):
        p = torch.nn.Parameter((torch.randn(32, 64) * 0.02).to(dtype))
        p.mask = torch.rand(32, 64)
        opt = ref_adamw.AdamW([p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, adaptive_l1_decay=l1)
        put(d, f"{tag}_p0", p.data); put(d, f"{tag}_mask", p.mask)
        for t in range(3):
            g = (torch.randn(32, 64) * 0.1).to(dtype)
            p.grad = g.clone()
            opt.step(decay=5e-4 * (t + 1))
            st = opt.state[p]
            put(d, f"{tag}_g{t}", g); put(d, f"{tag}_p{t + 1}", p.data)
            put(d, f"{tag}_m{t + 1}", st["exp_avg"]); put(d, f"{tag}_v{t + 1}", st["exp_avg_sq"])
    save("adamw", d)


def case_adamw_ams():
    """AdamW with amsgrad=True (legacy/adamw.py:126-128, 142-156): gradients shrink and grow again, so
    the running maximum of the second moment differs from the second moment itself."""
    torch.manual_seed(6)
    d = {}
    scales = (0.1, 0.01, 0.05, 0.002)
    d["scales"] = np.asarray(scales)
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        p = torch.nn.Parameter((torch.randn(32, 64) * 0.02).to(dtype))
        p.mask = torch.rand(32, 64)
        opt = ref_adamw.AdamW([p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=True)
        put(d, f"{tag}_p0", p.data); put(d, f"{tag}_mask", p.mask)
        for t, sc in enumerate(scales):
            g = (torch.randn(32, 64) * sc).to(dtype)
            p.grad = g.clone()
            opt.step(decay=5e-4 * (t + 1))
            st = opt.state[p]
            put(d, f"{tag}_g{t}", g); put(d, f"{tag}_p{t + 1}", p.data)
            put(d, f"{tag}_m{t + 1}", st["exp_avg"]); put(d, f"{tag}_v{t + 1}", st["exp_avg_sq"])
            put(d, f"{tag}_vmax{t + 1}", st["max_exp_avg_sq"])
    save("adamw_ams", d)


def case_block_sparse():
    torch.manual_seed(3)
    out_f, in_f, T = 64, 96, 24
    W = torch.randn(out_f, in_f) * 0.02
    ob, ib = out_f // 16, in_f // 16
    score = (W.view(ob, 16, ib, 16).permute(0, 2, 1, 3).reshape(ob * ib, 256) ** 2).sum(-1)
    keep = torch.zeros(ob * ib, dtype=torch.bool)
    keep[torch.sort(score, descending=True, stable=True).indices[: (ob * ib) // 2]] = True
    mask = keep.view(ob, 1, ib, 1).expand(ob, 16, ib, 16).reshape(out_f, in_f).float()
    blocks, row_ptr, col_idx = ref_bs.convert_to_block_sparse(W, mask, 16)
    layer = ref_bs.BlockSparseLinear(blocks, row_ptr, col_idx, in_f, out_f, None, 16)
    X = torch.randn(T, in_f)
    d = {}
    put(d, "W", W); put(d, "mask", mask); put(d, "blocks", blocks); put(d, "row_ptr", row_ptr)
    put(d, "col_idx", col_idx); put(d, "X", X); put(d, "Y", layer._torch_forward(X))
    save("block_sparse", d)


class TinyMLP(torch.nn.Module):
    """Two SparseLinear layers around a GELU (the shape of a GPT-2 MLP block, legacy/model.py:95-113)."""

    def __init__(self, linear_cls, cfg, d_in=64, d_hid=128, d_out=64):
        super().__init__()
        self.fc1 = linear_cls(d_in, d_hid, sparselinear_config=cfg, bias=True)
        self.fc2 = linear_cls(d_hid, d_out, sparselinear_config=cfg, bias=False)

    def forward(self, x):
        return self.fc2(torch.nn.functional.gelu(self.fc1(x)))


TRAIN_LOOP_CFG = dict(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, mask_update_period=1,
                      sparsity_warmup_steps=0, mask_lr=0.2, beta=0.9, temp_init=1.0, temp_min=0.05,
                      temp_decay=0.6, mask_hardening_start=2, mask_hardening_duration=3,
                      mask_penalty_mode="structured_topn", srste_decay=2e-4)
TRAIN_LOOP = dict(steps=6, lr=5e-3, betas=(0.9, 0.95), weight_decay=0.1, grad_clip=1.0, lambda_mid_max=0.3,
                  lambda_mid_warmup=4, decay_ramp=3)


def case_train_loop():
    """Free-running training loop over a two-layer model in the reference's order
    (legacy/main_llama.py:1997-2211): forward, loss + mid penalty, Hutchinson, backward, clip,
    grad EMA, GradScaler.step(optimizer, decay=), calculate_model_mask; then the end-of-training
    bake-in (legacy/main_llama.py:2552-2563) and the state dict a checkpoint would hold."""
    torch.manual_seed(321)
    hp = TRAIN_LOOP
    cfg = ref_sm.SparseLinearConfig(**TRAIN_LOOP_CFG)
    model = TinyMLP(ref_sm.SparseLinear, cfg)
    with torch.no_grad():
        model.fc1.weight.copy_(torch.randn(128, 64) * 0.15)
        model.fc1.bias.copy_(torch.randn(128) * 0.05)
        model.fc2.weight.copy_(torch.randn(64, 128) * 0.15)
    ref_utils.initialize_model(model)
    d = {}
    for n, t in model.state_dict().items():
        put(d, "init/" + n, t)
    params = [model.fc1.weight, model.fc1.bias, model.fc2.weight]
    opt = ref_adamw.AdamW(params, lr=hp["lr"], betas=hp["betas"], weight_decay=hp["weight_decay"],
                          srste_decay=TRAIN_LOOP_CFG["srste_decay"])
    scaler = torch.amp.GradScaler("cpu", enabled=False)
    steps = hp["steps"]
    X = torch.randn(steps, 4, 16, 64)
    Yt = torch.randn(steps, 4, 16, 64)
    put(d, "X", X); put(d, "Yt", Yt)
    for it in range(steps):
        out = model(X[it])
        task = torch.nn.functional.mse_loss(out, Yt[it])
        lam = hp["lambda_mid_max"] * min(1.0, it / hp["lambda_mid_warmup"])
        loss = task + ref_utils.mid_penalty(model, lam)
        probes = [rademacher(tuple(w.shape), 5000 + 10 * it + j, torch.float32) for j, w in
                  enumerate((model.fc1.weight, model.fc2.weight))]
        for j, v in enumerate(probes):
            put(d, f"s{it}_probe{j}", v.to(torch.int8))
        queue = [v.clone() for v in probes]
        ref_utils._rademacher_like = lambda t, q=queue: q.pop(0)
        ref_utils.update_hessian_hutchinson(model, loss)
        scaler.scale(loss).backward()
        scaler.unscale_(opt)
        gnorm = torch.nn.utils.clip_grad_norm_(model.parameters(), hp["grad_clip"])
        ref_utils.update_model_grad_ema(model, update_hessian_with_grad2=False)
        decay = TRAIN_LOOP_CFG["srste_decay"] * min(1.0, (it + 1) / hp["decay_ramp"])
        scaler.step(opt, decay=decay)
        scaler.update()
        opt.zero_grad(set_to_none=True)
        ref_utils.calculate_model_mask(model, it, lambda_mid=lam)
        put(d, f"s{it}_loss", float(loss.detach())); put(d, f"s{it}_task", float(task.detach())); put(d, f"s{it}_gnorm", float(gnorm))
        put(d, f"s{it}_lambda_mid", lam); put(d, f"s{it}_decay", decay)
        put(d, f"s{it}_flip", np.asarray(ref_utils.calculate_flip_rate(model), dtype=np.float64))
        for ln, layer in (("fc1", model.fc1), ("fc2", model.fc2)):
            put(d, f"s{it}_{ln}_W", layer.weight.data); put(d, f"s{it}_{ln}_mask", layer.mask.data)
            put(d, f"s{it}_{ln}_H", layer.hessian_diag.data); put(d, f"s{it}_{ln}_hx", float(layer.hardening_x))
        put(d, f"s{it}_fc1_b", model.fc1.bias.data)
    # end-of-training bake-in, the non-sharded branch
    with torch.no_grad():
        for layer in (model.fc1, model.fc2):
            hard = layer._hard_mask_from_soft(layer.mask).detach()
            layer.mask.copy_(hard)
            layer.weight.mul_(layer.mask)
            layer.change_mask = False
            layer._hardening_finalized = True
        Xe = torch.randn(3, 8, 64)
        put(d, "eval_X", Xe); put(d, "eval_Y", model(Xe))
    sd = model.state_dict()
    d["state_keys"] = np.asarray(list(sd.keys()))
    for n, t in sd.items():
        put(d, "final/" + n, t)
    opt_sd = opt.state_dict()
    d["opt_state_keys"] = np.asarray(sorted(opt_sd["state"][0].keys()))
    d["opt_group_keys"] = np.asarray(sorted(k for k in opt_sd["param_groups"][0].keys()))
    d["cfg_json"] = np.asarray(json.dumps(TRAIN_LOOP_CFG))
    d["hp_json"] = np.asarray(json.dumps(TRAIN_LOOP))
    save("train_loop", d)


class _GLUMLP(torch.nn.Module):
    def __init__(self, linear_cls, cfg, d=64, h=96):
        super().__init__()
        self.gate_proj = linear_cls(d, h, sparselinear_config=cfg, bias=False)
        self.up_proj = linear_cls(d, h, sparselinear_config=cfg, bias=False)
        self.down_proj = linear_cls(h, d, sparselinear_config=cfg, bias=False)


class TinyGLU(torch.nn.Module):
    """Module names as in a LLaMA block (``mlp.gate_proj / up_proj / down_proj``), which is what the
    pair detection keys on (legacy/utils.py:313-360)."""

    def __init__(self, linear_cls, cfg):
        super().__init__()
        self.block = torch.nn.Module()
        self.block.mlp = _GLUMLP(linear_cls, cfg)
        self.mlp = self.block.mlp


GLU_VARIANTS = {
    "topn": dict(mask_penalty_mode="structured_topn", mask_binarize_decay=0.05, beta_structural_start=0,
                 beta_structural_end=4),
    "mid": dict(mask_penalty_mode="mid"),
    "nm24": dict(mask_penalty_mode="nm_2_4"),
    "topn48": dict(N=4, M=8, mask_penalty_mode="structured_topn", beta_structural_start=0, beta_structural_end=4),
}
GLU_BASE = dict(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, mask_update_period=1, sparsity_warmup_steps=0,
                mask_lr=0.25, temp_init=0.8, temp_min=0.05, temp_decay=0.7, mask_hardening_start=1,
                mask_hardening_duration=2, mask_penalty_lr=0.2, glu_joint_mask=True)


def case_glu_joint():
    """calculate_model_mask on a gate / up / down triple with glu_joint_mask: the pair gets one
    joint update from the summed scores (legacy/utils.py:363-479), down its own."""
    d = {"variants": np.asarray(list(GLU_VARIANTS)), "base_json": np.asarray(json.dumps(GLU_BASE)),
         "variants_json": np.asarray(json.dumps(GLU_VARIANTS))}
    for tag, extra in GLU_VARIANTS.items():
        torch.manual_seed(11 + len(tag))
        cfg = ref_sm.SparseLinearConfig(**dict(GLU_BASE, **extra))
        model = TinyGLU(ref_sm.SparseLinear, cfg)
        ref_utils.initialize_model(model)
        with torch.no_grad():
            for n, m in (("gate", model.mlp.gate_proj), ("up", model.mlp.up_proj), ("down", model.mlp.down_proj)):
                m.weight.copy_(torch.randn_like(m.weight) * 0.05)
                m.hessian_diag.copy_(torch.rand_like(m.hessian_diag) + 0.1)
                m.mask.copy_(torch.rand_like(m.mask))  # gate and up start from different masks
                put(d, f"{tag}_{n}_W", m.weight.data); put(d, f"{tag}_{n}_H", m.hessian_diag.data)
                put(d, f"{tag}_{n}_mask0", m.mask.data)
        for step in range(3):
            lam = 0.3 * (step + 1) / 3
            ref_utils.calculate_model_mask(model, step, lambda_mid=lam)
            put(d, f"{tag}_s{step}_lambda", lam)
            for n, m in (("gate", model.mlp.gate_proj), ("up", model.mlp.up_proj), ("down", model.mlp.down_proj)):
                put(d, f"{tag}_s{step}_{n}_mask", m.mask.data); put(d, f"{tag}_s{step}_{n}_hx", float(m.hardening_x))
                put(d, f"{tag}_s{step}_{n}_flips", int(m.weight.flipped_mask))
    save("glu_joint", d)


def case_mask_stats():
    """mask_stats (legacy/utils.py:2069-2280) of a two-layer model, once with masks strictly inside
    (0, 1) and once with entries at exactly 0 and 1 (the entropy term is then NaN in the reference:
    the fp32 clamp bound 1 - 1e-8 is 1)."""
    torch.manual_seed(77)
    cfg = ref_sm.SparseLinearConfig(**TRAIN_LOOP_CFG)
    model = TinyMLP(ref_sm.SparseLinear, cfg)
    ref_utils.initialize_model(model)
    d = {}
    for tag in ("inside", "edges"):
        with torch.no_grad():
            for m in (model.fc1, model.fc2):
                if tag == "inside":
                    m.mask.copy_(torch.rand_like(m.mask) * 0.98 + 0.01)
                else:
                    m.mask.copy_((torch.randn_like(m.mask) * 0.5 + 0.5).clamp(0.0, 1.0))
        put(d, f"{tag}_fc1_mask", model.fc1.mask.data); put(d, f"{tag}_fc2_mask", model.fc2.mask.data)
        gi = torch.Generator().manual_seed(5 + len(tag))
        idxs = [_orig_randint(0, 128 * 64, (512,), generator=gi) for _ in range(2)]
        put(d, f"{tag}_idx0", idxs[0]); put(d, f"{tag}_idx1", idxs[1])
        q = [i.clone() for i in idxs]
        torch.randint = lambda *a, **k: q.pop(0)
        st = ref_utils.mask_stats(model, bins=100, sample_per_layer=512)
        torch.randint = _orig_randint
        d[f"{tag}_keys"] = np.asarray(list(st.keys()))
        d[f"{tag}_values"] = np.asarray([float(v) for v in st.values()], dtype=np.float64)
        # the per-step reductions of the loop over the same masks (legacy/utils.py:875-1234): mid penalty,
        # sparsity penalty (structured layers count (M - N) / M analytically; then with the layers switched to
        # the threshold count of the unstructured mask type), 2:4 tile statistics
        put(d, f"{tag}_mid_penalty", float(ref_utils.mid_penalty(model, 0.7)))
        pen, cur = ref_utils.sparsity_penalty(model, 0.4, 2.0)
        put(d, f"{tag}_sparsity_pen", float(pen)); put(d, f"{tag}_sparsity_cur", float(cur))
        for m in (model.fc1, model.fc2):
            m.mask_type = "unstructured"
        pen, cur = ref_utils.sparsity_penalty(model, 0.4, 2.0)
        put(d, f"{tag}_sparsity_pen_unstructured", float(pen)); put(d, f"{tag}_sparsity_cur_unstructured", float(cur))
        for m in (model.fc1, model.fc2):
            m.mask_type = "structured"
        ts = ref_utils.nm_2_4_tile_stats(model)
        d[f"{tag}_tile_keys"] = np.asarray(list(ts.keys()))
        d[f"{tag}_tile_values"] = np.asarray([float(v) for v in ts.values()], dtype=np.float64)
    save("mask_stats", d)


def case_kl_loss():
    """Distill_Model.kl_loss (legacy/sparse_modeling.py:1749-1828) and its gradient with respect
    to the student logits, fp32 and bf16, with a few logits beyond the +-100 clamp and one row made
    of NaN (its chunk is dropped)."""
    torch.manual_seed(42)
    d = {}
    for tag, dtype, rows, vocab in (("f32", torch.float32, 40, 512), ("bf16", torch.bfloat16, 24, 1024),
                                    ("chunks", torch.float32, 2100, 16)):
        s = (torch.randn(2, rows // 2, vocab) * 3.0).to(dtype)
        t = (torch.randn(2, rows // 2, vocab) * 3.0).to(dtype)
        s[0, 0, :4] = torch.tensor([150.0, -140.0, 99.0, -99.5]).to(dtype)
        t[0, 1, :2] = torch.tensor([120.0, -130.0]).to(dtype)
        if tag == "chunks":
            s[1, -1, 3] = float("nan")  # the last chunk (rows 2048..2099) is dropped
        s.requires_grad_(True)
        # logits come out of a model, i.e. they are not a leaf (the reference clamps in place)
        kl = ref_sm.Distill_Model.kl_loss(None, s * 1.0, t.clone())
        (kl * 1.5).backward()
        put(d, f"{tag}_student", s.detach()); put(d, f"{tag}_teacher", t); put(d, f"{tag}_kl", kl.detach().float())
        put(d, f"{tag}_grad", s.grad)
    save("kl_loss", d)


def case_slorb():
    """SparseLinear with the SLoRB bypass (legacy/sparse_modeling.py:388-408, 790-794, 830-872):
    init_SLoRB from a soft mask, then forward / backward with gradients of x, weight, SLoRB_Weight
    and (trainable) x_proj."""
    d = {}
    for tag, init, trainable in (("mean", "mean", False), ("sum", "sum", True)):
        torch.manual_seed(17 + len(tag) + int(trainable))
        cfg = ref_sm.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, SLoRB=True, SLoRB_k=8,
                                        SLoRB_init_type=init, trainable_projection=trainable, mask_hardening_start=1000)
        layer = ref_sm.SparseLinear(64, 48, sparselinear_config=cfg, bias=True)
        layer.initialize()
        with torch.no_grad():
            layer.weight.copy_(torch.randn(48, 64) * 0.1)
            layer.bias.copy_(torch.randn(48) * 0.1)
            layer.mask.copy_(torch.rand(48, 64))
        layer.init_SLoRB()
        if trainable:
            with torch.no_grad():
                layer.x_proj.add_(torch.randn_like(layer.x_proj) * 0.05)
        x = torch.randn(3, 8, 64, requires_grad=True)
        dy = torch.randn(3, 8, 48)
        y = layer(x)
        y.backward(dy)
        d[f"{tag}_state_keys"] = np.asarray(list(layer.state_dict().keys()))
        for n, t in layer.state_dict().items():
            put(d, f"{tag}/" + n, t)
        put(d, f"{tag}_x", x.detach()); put(d, f"{tag}_dy", dy); put(d, f"{tag}_y", y.detach())
        put(d, f"{tag}_dx", x.grad); put(d, f"{tag}_dW", layer.weight.grad); put(d, f"{tag}_dS", layer.SLoRB_Weight.grad)
        if trainable:
            put(d, f"{tag}_dP", layer.x_proj.grad)
    save("slorb", d)


BLOCK_CASES = {
    "bs16": dict(shape=(128, 160), cfg=dict(hard_mask_type="block_sparse16", mask_penalty_mode="block_sparse16",
                                            mask_binarize_decay=0.05)),
    "bs32": dict(shape=(128, 160), cfg=dict(hard_mask_type="block_sparse32", mask_penalty_mode="block_sparse32")),
    "tail": dict(shape=(72, 104), cfg=dict(hard_mask_type="block_sparse16", mask_penalty_mode="mid")),
    # per-tile top-k (hard_mask_type block16), the second recipe of the paper's LLaMA table
    "tile16": dict(shape=(64, 96), cfg=dict(hard_mask_type="block16", mask_penalty_mode="block16",
                                            mask_binarize_decay=0.05)),
    "tile16mid": dict(shape=(32, 48), cfg=dict(hard_mask_type="block16", mask_penalty_mode="mid", sparsity_ratio=0.75)),
}
BLOCK_BASE = dict(mask_type="unstructured", mask_metric="hessian_obd", sparsity_ratio=0.5, mask_update_period=1,
                  sparsity_warmup_steps=1, mask_lr=0.3, temp_init=0.5, temp_min=0.05, temp_decay=0.7,
                  mask_hardening_start=2, mask_hardening_duration=2, mask_penalty_lr=0.2, tau_sample_size=1 << 30)


def case_wanda():
    """WANDA metric: add_batch folds the activation energy of three batches (3-D, 3-D, 2-D input)
    into scaler_row (legacy/sparse_modeling.py:884-898); the score |W| * sqrt(scaler_row + eps)
    (:1071-1077) then drives two mask updates."""
    d = {}
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        torch.manual_seed(21)
        out_f, in_f = 24, 64
        W = torch.randn(out_f, in_f) * 0.02
        layer = make_layer(out_f, in_f, W, dtype, mask_type="structured", mask_metric="wanda", mask_update_period=1,
                           sparsity_warmup_steps=0, mask_lr=0.2, mask_penalty_mode="structured_topn",
                           mask_hardening_start=2, mask_hardening_duration=8)
        put(d, f"{tag}_W", layer.weight.data)
        batches = [torch.randn(3, 10, in_f), torch.randn(2, 7, in_f) * 2.0, torch.randn(5, in_f) * 0.5]
        for i, x in enumerate(batches):
            x = x.to(dtype)
            put(d, f"{tag}_x{i}", x)
            layer.add_batch(x, None)
            put(d, f"{tag}_scaler{i}", layer.scaler_row.data)
            put(d, f"{tag}_nsamples{i}", int(layer.nsamples))
        layer.mask.data = torch.rand(out_f, in_f)
        put(d, f"{tag}_mask0", layer.mask.data)
        for j, step in enumerate((3, 4)):
            put(d, f"{tag}_G{j}", layer.compute_gate_target(step))
            put(d, f"{tag}_T{j}", layer._temperature(step))
            layer.update_mask(step, lambda_mid=0.3)
            put(d, f"{tag}_mask{j + 1}", layer.mask.data)
            put(d, f"{tag}_flips{j}", int(layer.weight.flipped_mask))
            put(d, f"{tag}_hx{j}", float(layer.hardening_x))
    save("wanda", d)


def case_freeze():
    """Freeze bands (freeze_low / freeze_high): frozen entries keep their own value as gate target
    (legacy/sparse_modeling.py:1227-1229), the snap and the flags at the end of update_mask
    (:1621-1642) before and after step 2000, and harden_fraction over two layers (legacy/utils.py:1236-1276)."""
    d = {}
    torch.manual_seed(33)
    out_f, in_f = 32, 64
    W = torch.randn(out_f, in_f) * 0.02
    layer = make_layer(out_f, in_f, W, torch.float32, mask_type="structured", mask_metric="hessian_obd",
                       mask_update_period=1, sparsity_warmup_steps=0, mask_lr=0.3, mask_penalty_mode="structured_topn",
                       mask_hardening_start=2, mask_hardening_duration=8, temp_init=0.3, temp_min=0.3,
                       freeze_low=0.08, freeze_high=0.93)
    layer.hessian_diag.data = torch.rand(out_f, in_f) + 0.1
    layer.mask.data = torch.rand(out_f, in_f)
    put(d, "W", W); put(d, "H", layer.hessian_diag.data); put(d, "mask0", layer.mask.data)
    steps = [5, 6, 7, 2000, 2001, 2002]
    d["steps"] = np.asarray(steps)
    for j, step in enumerate(steps):
        put(d, f"s{j}_G", layer.compute_gate_target(step))
        put(d, f"s{j}_T", layer._temperature(step))
        layer.update_mask(step, lambda_mid=0.4)
        put(d, f"s{j}_mask", layer.mask.data); put(d, f"s{j}_flags", layer.frozen_mask_flags.data.float())
        put(d, f"s{j}_flips", int(layer.weight.flipped_mask)); put(d, f"s{j}_hx", float(layer.hardening_x))
    # harden_fraction over two layers
    other = make_layer(16, 32, torch.randn(16, 32) * 0.02, torch.float32, mask_type="structured",
                       mask_metric="hessian_obd", freeze_low=0.08, freeze_high=0.93)
    other.mask.data = torch.rand(16, 32)
    other.frozen_mask_flags.data = (torch.rand(16, 32) < 0.1).float()
    model = torch.nn.Sequential(layer, other)
    put(d, "hf_mask_a0", layer.mask.data); put(d, "hf_flags_a0", layer.frozen_mask_flags.data.float())
    put(d, "hf_mask_b0", other.mask.data); put(d, "hf_flags_b0", other.frozen_mask_flags.data.float())
    n = ref_utils.harden_fraction(model, fraction=0.3, band_low=0.35, band_high=0.7)
    put(d, "hf_count", int(n))
    put(d, "hf_mask_a1", layer.mask.data); put(d, "hf_flags_a1", layer.frozen_mask_flags.data.float())
    put(d, "hf_mask_b1", other.mask.data); put(d, "hf_flags_b1", other.frozen_mask_flags.data.float())
    save("freeze", d)


def case_block_masks():
    """Block-sparse soft masks (hard_mask_type block_sparse16 / 32): block gate, block penalty, EMA,
    blockified mask, block hard view, masked forward (legacy/sparse_modeling.py:461-508, 607-718,
    1122-1157, 1395-1530)."""
    d = {"cases_json": np.asarray(json.dumps(BLOCK_CASES)), "base_json": np.asarray(json.dumps(BLOCK_BASE))}
    for tag, spec in BLOCK_CASES.items():
        torch.manual_seed(31 + len(tag))
        out_f, in_f = spec["shape"]
        cfg = ref_sm.SparseLinearConfig(**dict(BLOCK_BASE, **spec["cfg"]))
        layer = ref_sm.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False)
        layer.initialize()
        with torch.no_grad():
            layer.weight.copy_(torch.randn(out_f, in_f) * 0.05)
            layer.hessian_diag.copy_(torch.rand(out_f, in_f) + 0.05)
        put(d, f"{tag}_W", layer.weight.data); put(d, f"{tag}_H", layer.hessian_diag.data)
        x = torch.randn(6, in_f)
        put(d, f"{tag}_x", x)
        for step in range(5):
            lam = 0.25
            put(d, f"{tag}_s{step}_G", layer.compute_gate_target(step))
            layer.update_mask(step, lambda_mid=lam)
            put(d, f"{tag}_s{step}_mask", layer.mask.data); put(d, f"{tag}_s{step}_hx", float(layer.hardening_x))
            put(d, f"{tag}_s{step}_flips", int(layer.weight.flipped_mask))
            put(d, f"{tag}_s{step}_hard", layer._hard_mask_from_soft(layer.mask.data))
            put(d, f"{tag}_s{step}_T", layer._temperature(step)); put(d, f"{tag}_s{step}_sp", layer._effective_sparsity(step))
            put(d, f"{tag}_s{step}_y", layer(x).detach())
    save("block_masks", d)


C1_ROWS = dict(w_rows=64, y_rows=32, dx_rows=64)


def c1_inputs():
    """The fp32 GPT-2-small MLP case: W [3072, 768] ~ N(0, 0.02), X [8, 1024, 768] ~ N(0, 1),
    dY [8, 1024, 3072] ~ N(0, 1) drawn in that order from the CPU generator seeded with 0."""
    torch.manual_seed(0)
    W = torch.randn(3072, 768) * 0.02
    X = torch.randn(8, 1024, 768)
    dY = torch.randn(8, 1024, 3072)
    return W, X, dY


def c1_sample_rows(n_rows, count, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.sort(torch.randperm(n_rows, generator=g)[:count]).values


def case_c1():
    """The whole fp32 chain at its full size: four Hutchinson probes, one mask update at step 0, the hard
    2:4 projection, then a masked forward / backward with the hard mask (hardening_x = 0). The inputs
    are regenerated from the seed at test time (fingerprints stored); the hard mask is stored as packed
    bits, the float tensors as full-tensor sums plus a sample of rows."""
    W, X, dY = c1_inputs()
    out_f, in_f = W.shape
    T = X.shape[0] * X.shape[1]
    d = {}
    for name, t in (("W", W), ("X", X), ("dY", dY)):
        put(d, f"fp_{name}", torch.stack([t.double().sum(), (t.double() ** 2).sum(), t.flatten()[12345].double()]))
    layer = make_layer(out_f, in_f, W, torch.float32, mask_type="structured", mask_metric="hessian_obd", N=2, M=4,
                       temp_init=1.0, mask_update_period=1, sparsity_warmup_steps=0)
    rows_w = c1_sample_rows(out_f, C1_ROWS["w_rows"], 11)
    rows_y = c1_sample_rows(T, C1_ROWS["y_rows"], 12)
    rows_x = c1_sample_rows(T, C1_ROWS["dx_rows"], 13)
    put(d, "rows_w", rows_w); put(d, "rows_y", rows_y); put(d, "rows_x", rows_x)

    def summary(name, t, rows):
        t2 = t.detach().reshape(-1, t.shape[-1])
        put(d, f"{name}_sum", torch.stack([t2.double().sum(), (t2.double() ** 2).sum(), t2.double().abs().max()]))
        put(d, f"{name}_rows", t2[rows])

    for i in range(4):
        v = rademacher((out_f, in_f), 1 + i, torch.float32)
        dd = {}
        hutchinson_once(layer, X, dY, v, dd, str(i))
        summary(f"hvp_{i}", torch.from_numpy(dd[f"hvp_{i}"]), rows_w)
        summary(f"H_{i}", layer.hessian_diag.data, rows_w)
    put(d, "T0", layer._temperature(0))
    raw = (layer.hessian_diag.data + 1e-8) * (layer.weight.data * layer.weight.data)
    summary("score_raw", raw, rows_w)
    put(d, "score_mean_std", torch.stack([raw.float().mean(), raw.float().std(unbiased=False) + 1e-6]))
    summary("G", layer.compute_gate_target(0), rows_w)
    ref_utils.calculate_model_mask(layer, step=0, lambda_mid=0.0)
    summary("mask", layer.mask.data, rows_w)
    put(d, "flips", int(layer.weight.flipped_mask))
    put(d, "hx_after_update", float(layer.hardening_x))
    hard = layer._hard_mask_from_soft(layer.mask.data)
    d["hard_bits"] = np.packbits(hard.numpy().astype(np.uint8), axis=1)
    # near-ties of the soft mask: groups whose 2nd and 3rd largest values are closer than 1e-5 relative
    srt = torch.sort(layer.mask.data.view(out_f, in_f // 4, 4), dim=-1, descending=True).values
    put(d, "near_tie_groups", int(((srt[..., 1] - srt[..., 2]).abs() <= 1e-5 * srt[..., 1].abs()).sum()))
    layer.hardening_x = 0.0
    Xr = X.clone().requires_grad_(True)
    layer.weight.grad = None
    Y = layer(Xr)
    Y.backward(dY)
    summary("Y", Y, rows_y); summary("dX", Xr.grad, rows_x); summary("dW", layer.weight.grad, rows_w)
    save("c1", d)


def case_movement():
    """mask_metric='movement': update_grad_hessian_ema (legacy/sparse_modeling.py:901-922) fed by real
    backward passes, AdamW, and mask updates scored by |W * grad_ema| / temperature. A second layer is
    built with ``enable_hutchinson`` set on its config so that the g^2 branch into hessian_diag runs."""
    d = {}
    for tag, dtype in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        torch.manual_seed(41)
        out_f, in_f = 48, 64
        W = torch.randn(out_f, in_f) * 0.05
        kw = dict(mask_type="structured", mask_metric="movement", N=2, M=4, mask_update_period=1, sparsity_warmup_steps=0,
                  mask_lr=0.2, beta=0.9, temperature=0.7, temp_init=1.0, temp_decay=0.8, mask_hardening_start=2,
                  mask_hardening_duration=4)
        cfg = ref_sm.SparseLinearConfig(**kw)
        cfg.enable_hutchinson = True  # hessian_diag becomes a full tensor, fed by g^2
        layer = ref_sm.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False).to(dtype)
        layer.weight.data.copy_(W.to(dtype))
        layer.initialize()
        layer.mask.data = layer.mask.data.float()
        layer.hessian_diag.data = layer.hessian_diag.data.float()
        layer.sync_weight()
        opt = ref_adamw.AdamW([layer.weight], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
        put(d, f"{tag}_W0", layer.weight.data)
        X = torch.randn(3, 10, in_f).to(dtype)
        put(d, f"{tag}_X", X)
        for t in range(3):
            dY = torch.randn(3, 10, out_f).to(dtype)
            put(d, f"{tag}_dY{t}", dY)
            layer.weight.grad = None
            layer(X).backward(dY)
            put(d, f"{tag}_g{t}", layer.weight.grad)
            ref_utils.update_model_grad_ema(layer, update_hessian_with_grad2=True)
            put(d, f"{tag}_ema{t}", layer.grad_ema.data); put(d, f"{tag}_H{t}", layer.hessian_diag.data)
            opt.step(decay=1e-4)
            put(d, f"{tag}_W{t + 1}", layer.weight.data)
            put(d, f"{tag}_G{t}", layer.compute_gate_target(t))
            ref_utils.calculate_model_mask(layer, step=t, lambda_mid=0.0)
            put(d, f"{tag}_mask{t + 1}", layer.mask.data); put(d, f"{tag}_hx{t}", float(layer.hardening_x))
            put(d, f"{tag}_flips{t}", int(layer.weight.flipped_mask))
    save("movement", d)


def case_nm():
    """mask_type='structured' with N:M other than 2:4 (legacy/sparse_modeling.py:720-735, :1164-1225,
    :1532-1570): gate, penalty pulls, beta mixing, exact gate, EMA, hard view, flip count, and a masked
    forward / backward with hardening active. The previous masks are rounded to two decimals so that
    groups hold exact ties."""
    torch.manual_seed(53)
    out_f, in_f = 48, 128
    d = {}
    variants = [
        ("4of8_topn", 4, 8, torch.float32, "hessian_obd", dict(mask_penalty_mode="structured_topn"), 0.6),
        ("1of4_mid", 1, 4, torch.float32, "hessian_obd", dict(mask_penalty_mode="mid"), 0.8),
        ("3of4_bin", 3, 4, torch.float32, "hessian_ratio", dict(mask_penalty_mode="structured_topn", mask_binarize_decay=0.05), 0.3),
        ("1of2_plain", 1, 2, torch.float32, "hessian_obd", dict(), 0.0),
        ("8of16_beta", 8, 16, torch.float32, "hessian_obd",
         dict(mask_penalty_mode="mid", beta_structural_start=0, beta_structural_end=10), 0.2),
        ("8of32_exact", 8, 32, torch.float32, "hessian_obd", dict(structured_exact=True), 0.0),
        ("2of8_bf16", 2, 8, torch.bfloat16, "hessian_obd", dict(mask_penalty_mode="structured_topn"), 0.5),
        ("4of8_bf16_mag", 4, 8, torch.bfloat16, "magnitude", dict(), 0.0),
    ]
    d["variants"] = np.asarray([v[0] for v in variants])
    for tag, n, m, dtype, metric, kw, lam in variants:
        W = torch.randn(out_f, in_f) * 0.02
        layer = make_layer(out_f, in_f, W, dtype, mask_type="structured", mask_metric=metric, N=n, M=m,
                           mask_update_period=1, sparsity_warmup_steps=0, mask_lr=0.2, mask_penalty_lr=0.15,
                           mask_hardening_start=2, mask_hardening_duration=8, **kw)
        layer.mask.data = (torch.rand(out_f, in_f) * 100).round() / 100
        if metric != "magnitude":
            layer.hessian_diag.data = torch.rand(out_f, in_f) + 0.1
        step = 4
        put(d, f"{tag}_N", n); put(d, f"{tag}_M", m); put(d, f"{tag}_metric", metric)
        put(d, f"{tag}_W", layer.weight.data); put(d, f"{tag}_mask0", layer.mask.data)
        if metric != "magnitude":
            put(d, f"{tag}_H", layer.hessian_diag.data)
        put(d, f"{tag}_lambda", lam); put(d, f"{tag}_step", step)
        put(d, f"{tag}_T", layer._temperature(step)); put(d, f"{tag}_beta_s", layer._beta_structural(step))
        put(d, f"{tag}_hard0", layer._hard_mask_from_soft(layer.mask.data))
        put(d, f"{tag}_G", layer.compute_gate_target(step))
        layer.update_mask(step, lambda_mid=lam)
        put(d, f"{tag}_mask1", layer.mask.data); put(d, f"{tag}_hx", float(layer.hardening_x))
        put(d, f"{tag}_flips", int(layer.weight.flipped_mask))
        put(d, f"{tag}_hard1", layer._hard_mask_from_soft(layer.mask.data))
        X = torch.randn(2, 12, in_f).to(dtype).requires_grad_(True)
        dY = torch.randn(2, 12, out_f).to(dtype)
        layer.weight.grad = None
        Y = layer(X)
        Y.backward(dY)
        put(d, f"{tag}_X", X); put(d, f"{tag}_dY", dY); put(d, f"{tag}_Y", Y); put(d, f"{tag}_dX", X.grad)
        put(d, f"{tag}_dW", layer.weight.grad)
    save("nm_general", d)


def case_unstructured_hard():
    """mask_type='unstructured' with the matching hard view ``mask > 0.5`` (legacy/sparse_modeling.py:526-527):
    quantile gate, penalty pulls, beta mixing (N:M groups only shape the pull and the mixing), EMA, flip count
    by the threshold, and a masked forward / backward with hardening active."""
    torch.manual_seed(59)
    out_f, in_f = 48, 128
    d = {}
    variants = [
        ("mid", torch.float32, dict(mask_penalty_mode="mid"), 0.6),
        ("topn", torch.float32, dict(mask_penalty_mode="structured_topn"), 0.5),
        ("beta", torch.float32, dict(mask_penalty_mode="mid", beta_structural_start=0, beta_structural_end=10), 0.2),
        ("bin", torch.float32, dict(mask_penalty_mode="mid", mask_binarize_decay=0.05), 0.0),
        ("bf16", torch.bfloat16, dict(mask_penalty_mode="mid"), 0.4),
    ]
    d["variants"] = np.asarray([v[0] for v in variants])
    for tag, dtype, kw, lam in variants:
        W = torch.randn(out_f, in_f) * 0.02
        layer = make_layer(out_f, in_f, W, dtype, mask_type="unstructured", mask_metric="hessian_obd", N=2, M=4,
                           sparsity_ratio=0.5, mask_update_period=1, sparsity_warmup_steps=0, mask_lr=0.2, mask_penalty_lr=0.15,
                           mask_hardening_start=2, mask_hardening_duration=8, **kw)
        layer.mask.data = torch.rand(out_f, in_f)
        layer.hessian_diag.data = torch.rand(out_f, in_f) + 0.1
        step = 4
        put(d, f"{tag}_W", layer.weight.data); put(d, f"{tag}_mask0", layer.mask.data); put(d, f"{tag}_H", layer.hessian_diag.data)
        put(d, f"{tag}_lambda", lam); put(d, f"{tag}_step", step)
        put(d, f"{tag}_T", layer._temperature(step)); put(d, f"{tag}_beta_s", layer._beta_structural(step))
        put(d, f"{tag}_sparsity", layer._effective_sparsity(step))
        put(d, f"{tag}_G", layer.compute_gate_target(step))
        layer.update_mask(step, lambda_mid=lam)
        put(d, f"{tag}_mask1", layer.mask.data); put(d, f"{tag}_hx", float(layer.hardening_x))
        put(d, f"{tag}_flips", int(layer.weight.flipped_mask))
        put(d, f"{tag}_hard1", layer._hard_mask_from_soft(layer.mask.data))
        X = torch.randn(2, 12, in_f).to(dtype).requires_grad_(True)
        dY = torch.randn(2, 12, out_f).to(dtype)
        layer.weight.grad = None
        Y = layer(X)
        Y.backward(dY)
        put(d, f"{tag}_X", X); put(d, f"{tag}_dY", dY); put(d, f"{tag}_Y", Y); put(d, f"{tag}_dX", X.grad)
        put(d, f"{tag}_dW", layer.weight.grad)
    save("unstructured_hard", d)


SCHEDULE_CONFIGS = {
    "anneal": dict(temp_init=1.0, temp_min=0.05, temp_decay=0.7, mask_update_period=3, mask_hardening_start=5,
                   mask_hardening_duration=10, sparsity_warmup_steps=20, beta_structural_start=4, beta_structural_end=12),
    "switch": dict(temp_init=2.0, temp_min=0.1, temp_decay=0.9, mask_update_switch_step=10, mask_update_period_before=2,
                   mask_update_period_after=5, mask_hardening_start=0, mask_hardening_duration=1, sparsity_warmup_steps=0),
    "block": dict(mask_type="unstructured", hard_mask_type="block_sparse16", sparsity_ratio=0.6, temp_init=1.0, temp_min=0.05,
                  temp_decay=0.8, mask_update_period=1, sparsity_warmup_steps=40, mask_hardening_start=100,
                  mask_hardening_duration=50),
}
SCHEDULE_STEPS = [0, 1, 2, 3, 4, 5, 7, 8, 9, 10, 11, 12, 15, 19, 20, 21, 30, 40, 41, 100, 125, 150, 151, 1000]


def case_schedules():
    """Host-side schedules of a layer (legacy/sparse_modeling.py:932-985, 1603-1619) and of the loop
    (update_mask_penalty_lr legacy/utils.py:141-180): values of the reference over a grid of steps. The
    hardening value is read after an update_mask call at that step on a fresh layer (it is set there)."""
    d = {"configs_json": np.asarray(json.dumps(SCHEDULE_CONFIGS)), "steps": np.asarray(SCHEDULE_STEPS)}
    for tag, kw in SCHEDULE_CONFIGS.items():
        rows = []
        for step in SCHEDULE_STEPS:
            torch.manual_seed(3)
            cfg = ref_sm.SparseLinearConfig(**dict(dict(mask_type="structured", mask_metric="magnitude"), **kw))
            layer = ref_sm.SparseLinear(32, 16, sparselinear_config=cfg, bias=False)
            layer.initialize()
            layer.mask.data = torch.rand(16, 32)
            vals = [float(layer._temperature(step)), float(layer._mask_update_period(step)),
                    float(layer._effective_sparsity(step)), float(layer._beta_structural(step))]
            # force an update at this step so that the hardening schedule is evaluated there
            layer.cfg.mask_update_period = 1
            layer.cfg.mask_update_switch_step = None
            layer.cfg.sparsity_warmup_steps = 0
            layer.update_mask(step, lambda_mid=0.0)
            vals.append(float(layer.hardening_x))
            rows.append(vals)
        d[f"{tag}_values"] = np.asarray(rows, dtype=np.float64)  # temperature, period, sparsity, beta, hardening_x
    lin = ref_sm.SparseLinear(8, 8, sparselinear_config=ref_sm.SparseLinearConfig(), bias=False)
    pl = [[float(ref_utils.update_mask_penalty_lr(lin, s, 50, 0.02, 0.3, sched)) for s in (0, 1, 10, 25, 49, 50, 80)]
          for sched in ("constant", "linear", "cosine", "other")]
    import dataclasses

    ref_cfg = ref_sm.SparseLinearConfig()
    d["config_defaults_json"] = np.asarray(json.dumps({f.name: getattr(ref_cfg, f.name)
                                                       for f in dataclasses.fields(ref_sm.SparseLinearConfig)}))
    d["penalty_lr_steps"] = np.asarray([0, 1, 10, 25, 49, 50, 80])
    d["penalty_lr"] = np.asarray(pl, dtype=np.float64)
    save("schedules", d)


if __name__ == "__main__":
    # `make_golden.py wanda ...` regenerates only the named single-function cases
    only = [a for a in sys.argv[1:] if not a.startswith("-")]
    if only:
        for name in only:
            globals()["case_" + name]()
        raise SystemExit(0)
    base = dict(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, mask_update_period=1,
                sparsity_warmup_steps=0, mask_lr=0.1, beta=0.99)
    # scaled-down copy of the fp32 GPT-2-MLP case (temperature 1, no hardening before the update)
    case_chain("chain_f32", 96, 64, 2, 20, torch.float32, 1,
               dict(base, temp_init=1.0, mask_hardening_start=1000, mask_hardening_duration=10000))
    # scaled-down copy of the bf16 LLaMA-shaped tempering run: temperature 1.0 -> 0.05, hardening from step 1
    case_chain("chain_bf16", 64, 128, 2, 32, torch.bfloat16, 4,
               dict(base, temp_init=1.0, temp_min=0.05, temp_decay=0.05 ** (1.0 / 9.0), mask_hardening_start=1,
                    mask_hardening_duration=3, mask_penalty_mode="structured_topn"), lambda_mid=0.25, seed=100)
    # the launcher's default recipe (train_llama.sh:223-262): unstructured gate from a sampled quantile,
    # nm_2_4 projection and penalty, |W| / sqrt(H) score
    case_chain("chain_paper", 64, 128, 2, 32, torch.bfloat16, 3,
               dict(mask_type="unstructured", hard_mask_type="nm_2_4", mask_metric="hessian_ratio", N=2, M=4,
                    mask_update_period=1, sparsity_warmup_steps=0, mask_lr=0.1, beta=0.98, temp_init=1.0, temp_min=0.05,
                    temp_decay=0.5, mask_hardening_start=1, mask_hardening_duration=2, mask_penalty_lr=0.1,
                    mask_penalty_mode="nm_2_4", tau_sample_size=1024, sparsity_ratio=0.5),
               lambda_mid=0.1, seed=200, tau_idx_seed=900)
    case_train_loop()
    case_glu_joint()
    case_mask_stats()
    case_kl_loss()
    case_slorb()
    case_block_masks()
    case_c1()
    case_movement()
    case_wanda()
    case_freeze()
    case_penalty()
    case_ties()
    case_adamw()
    case_adamw_ams()
    case_block_sparse()
