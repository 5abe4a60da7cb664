"""A free-running training loop over a two-layer model, the end-of-training bake-in, the checkpoint
state dict and the inference bake-in, against a trajectory recorded from the reference
(tests/golden/train_loop.npz; generator: tests/golden/make_golden.py, case_train_loop).

The loop is the reference's (legacy/main_llama.py:1997-2211): forward, loss + mid penalty,
Hutchinson, backward, clip, grad EMA, GradScaler.step(optimizer, decay=), calculate_model_mask.
Nothing is reset between steps, so the tolerance is that of six accumulated fp32 steps.
"""
import json

import pytest
import torch

from golden_io import Golden, rel_err
from oracle import sparselinear_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
LOOP_TOL = 2e-4  # six free-running fp32 steps through GEMMs with another summation order


class TinyMLP(torch.nn.Module):
    def __init__(self, linear_cls, cfg, d_in=64, d_hid=128, d_out=64):
        super().__init__()
        self.fc1 = linear_cls(d_in, d_hid, sparselinear_config=cfg, bias=True)
        self.fc2 = linear_cls(d_hid, d_out, sparselinear_config=cfg, bias=False)

    def forward(self, x):
        return self.fc2(torch.nn.functional.gelu(self.fc1(x)))


def _build(g, prefix):
    import sparseforge_b200 as sf

    cfg = sf.SparseLinearConfig(**json.loads(str(g["cfg_json"])))
    model = TinyMLP(sf.SparseLinear, cfg).to(DEV)
    sd = {k: g[prefix + k].to(DEV) for k in [str(k) for k in g["state_keys"]]}
    # the reference's keys, shapes and dtypes load with strict=True
    missing, unexpected = model.load_state_dict(sd, strict=True)
    assert not missing and not unexpected
    assert list(model.state_dict().keys()) == [str(k) for k in g["state_keys"]]
    for k, v in model.state_dict().items():
        assert tuple(v.shape) == tuple(g[prefix + k].shape), k
    return model, cfg


def _hard_agreement(a, b):
    return float((a.cpu() == b.cpu()).float().mean())


def test_training_loop_follows_the_reference():
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden("train_loop")
    hp = json.loads(str(g["hp_json"]))
    cfgd = json.loads(str(g["cfg_json"]))
    model, _ = _build(g, "init/")
    U.initialize_model(model)
    opt = sf.AdamW([model.fc1.weight, model.fc1.bias, model.fc2.weight], lr=hp["lr"], betas=tuple(hp["betas"]),
                   weight_decay=hp["weight_decay"], srste_decay=cfgd["srste_decay"])
    scaler = torch.amp.GradScaler("cuda", enabled=False)
    X, Yt = g["X"].to(DEV), g["Yt"].to(DEV)
    for it in range(hp["steps"]):
        out = model(X[it])
        task = torch.nn.functional.mse_loss(out, Yt[it])
        lam = hp["lambda_mid_max"] * min(1.0, it / hp["lambda_mid_warmup"])
        assert lam == pytest.approx(g.scalar(f"s{it}_lambda_mid"))
        loss = task + U.mid_penalty(model, lam)
        queue = [g[f"s{it}_probe{j}"].to(DEV).float() for j in range(2)]
        U._rademacher_like = lambda t, q=queue: q.pop(0)
        U.update_hessian_hutchinson(model, loss)
        scaler.scale(loss).backward()
        scaler.unscale_(opt)
        gnorm = torch.nn.utils.clip_grad_norm_(model.parameters(), hp["grad_clip"])
        U.update_model_grad_ema(model, update_hessian_with_grad2=False)
        decay = cfgd["srste_decay"] * min(1.0, (it + 1) / hp["decay_ramp"])
        scaler.step(opt, decay=decay)
        scaler.update()
        opt.zero_grad(set_to_none=True)
        U.calculate_model_mask(model, it, lambda_mid=lam)

        assert float(loss.detach()) == pytest.approx(g.scalar(f"s{it}_loss"), rel=LOOP_TOL)
        assert float(gnorm) == pytest.approx(g.scalar(f"s{it}_gnorm"), rel=LOOP_TOL)
        for ln, layer in (("fc1", model.fc1), ("fc2", model.fc2)):
            assert layer.hardening_x == pytest.approx(g.scalar(f"s{it}_{ln}_hx"))
            assert rel_err(layer.weight.data, g[f"s{it}_{ln}_W"]) <= LOOP_TOL, (it, ln)
            assert rel_err(layer.hessian_diag.data, g[f"s{it}_{ln}_H"]) <= 5 * LOOP_TOL, (it, ln)
            assert rel_err(layer.mask.data, g[f"s{it}_{ln}_mask"]) <= 5 * LOOP_TOL, (it, ln)
        assert rel_err(model.fc1.bias.data, g[f"s{it}_fc1_b"]) <= LOOP_TOL
        # flips: equal unless a near-tie of the soft mask is decided the other way
        flipped = U.calculate_flip_rate(model)[0]
        assert abs(flipped - g[f"s{it}_flip"][0].item()) <= 4, (it, flipped)

    # optimizer state layout a resumed run would read
    osd = opt.state_dict()
    assert sorted(osd["state"][0].keys()) == [str(k) for k in g["opt_state_keys"]]
    assert set(str(k) for k in g["opt_group_keys"]) <= set(osd["param_groups"][0].keys())

    # end-of-training bake-in
    U.finalize_hard_masks(model)
    for ln, layer in (("fc1", model.fc1), ("fc2", model.fc2)):
        assert _hard_agreement(layer.mask.data, g[f"final/{ln}.mask"]) >= 0.999
        grp = layer.mask.data.view(layer.out_features, -1, 4).sum(-1)
        assert torch.all(grp == 2)
        assert torch.all((layer.weight.data == 0) | (layer.mask.data == 1))
    with torch.no_grad():
        Ye = model(g["eval_X"].to(DEV))
    assert rel_err(Ye, g["eval_Y"]) <= 50 * LOOP_TOL  # a flipped near-tie moves one small weight in or out


def test_reference_checkpoint_loads_and_bakes_in():
    """The reference's finalized state dict loads key for key; the loaded model reproduces the
    reference's output in all three inference forms: masked forward, dense bake-in
    (legacy/eval_wiki_ppl.py:548-651) and the compressed 2:4 tensor-core form."""
    from sparseforge_b200 import utils as U

    g = Golden("train_loop")
    Xe, want = g["eval_X"].to(DEV), g["eval_Y"]

    def load():
        model, _ = _build(g, "final/")
        for m in model.modules():
            if hasattr(m, "hardening_x"):  # what the reference's loader sets (eval_wiki_ppl.py:828-831)
                m.hardening_x = 0.0
                m._hardening_finalized = True
        return model.eval()

    model = load()
    with torch.no_grad():
        assert rel_err(model(Xe), want) <= 1e-5
    W_before = model.fc1.weight.data.clone()
    U.optimize_sparse_model_for_inference(model)
    assert model.fc1.mode == "dense_forward" and model.fc2.mode == "dense_forward"
    assert torch.equal(model.fc1.weight.data, W_before)  # the finalized weight is not masked twice
    with torch.no_grad():
        assert rel_err(model(Xe), want) <= 1e-5

    # a checkpoint saved before the bake-in (soft masks, unmasked weights) gets the hard mask once
    soft, _ = _build(g, "init/")
    soft.fc1.mask.data.copy_(g["s3_fc1_mask"].to(DEV))
    soft.fc1.weight.data.copy_(g["s3_fc1_W"].to(DEV))
    hard = soft.fc1._hard_mask_from_soft(soft.fc1.mask.data)
    U.optimize_sparse_model_for_inference(soft)
    assert torch.equal(soft.fc1.weight.data, g["s3_fc1_W"].to(DEV) * hard)

    # compressed form: bf16 weights on the sparse tensor cores
    model16 = load().to(torch.bfloat16)
    with torch.no_grad():
        dense16 = model16(Xe.to(torch.bfloat16)).float()
    U.optimize_sparse_model_for_inference(model16, compressed=True)
    assert model16.fc1.mode == "sparse24_forward" and model16.fc2.mode == "sparse24_forward"
    assert model16.fc1._sp_values.shape == (128, 32) and model16.fc1._sp_values.dtype == torch.bfloat16
    with torch.no_grad():
        sparse16 = model16(Xe.to(torch.bfloat16)).float()
    assert rel_err(sparse16, dense16) <= 1e-2
    assert rel_err(sparse16, want) <= 2e-2
    with pytest.raises(RuntimeError):
        model16.train()
        model16(Xe.to(torch.bfloat16).requires_grad_(True))


class _GLUMLP(torch.nn.Module):
    def __init__(self, linear_cls, cfg, d=64, h=96):
        super().__init__()
        self.gate_proj = linear_cls(d, h, sparselinear_config=cfg, bias=False)
        self.up_proj = linear_cls(d, h, sparselinear_config=cfg, bias=False)
        self.down_proj = linear_cls(h, d, sparselinear_config=cfg, bias=False)


class TinyGLU(torch.nn.Module):
    def __init__(self, linear_cls, cfg):
        super().__init__()
        self.block = torch.nn.Module()
        self.block.mlp = _GLUMLP(linear_cls, cfg)
        self.mlp = self.block.mlp


@pytest.mark.parametrize("tag", ["topn", "mid", "nm24", "topn48"])
def test_glu_joint_mask_follows_the_reference(tag):
    """calculate_model_mask with glu_joint_mask: gate_proj / up_proj get one update from the summed
    score (penalty pull from the gate layer's mask), down_proj its own (legacy/utils.py:183-479)."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden("glu_joint")
    cfgd = dict(json.loads(str(g["base_json"])), **json.loads(str(g["variants_json"]))[tag])
    model = TinyGLU(sf.SparseLinear, sf.SparseLinearConfig(**cfgd)).to(DEV)
    U.initialize_model(model)
    layers = {"gate": model.mlp.gate_proj, "up": model.mlp.up_proj, "down": model.mlp.down_proj}
    for n, m in layers.items():
        m.weight.data.copy_(g[f"{tag}_{n}_W"].to(DEV))
        m.hessian_diag.data.copy_(g[f"{tag}_{n}_H"].to(DEV))
        m.mask.data.copy_(g[f"{tag}_{n}_mask0"].to(DEV))
        m.invalidate_masked_weight()
    assert U._identify_glu_pairs({n: m for n, m in model.named_modules() if isinstance(m, sf.SparseLinear)}) == \
        {"block.mlp.gate_proj": "block.mlp.up_proj"}
    for step in range(3):
        prev = {n: m.mask.data.clone() for n, m in layers.items()}
        U.calculate_model_mask(model, step, lambda_mid=g.scalar(f"{tag}_s{step}_lambda"))
        for n, m in layers.items():
            want = g[f"{tag}_s{step}_{n}_mask"]
            assert rel_err(m.mask.data, want) <= 1e-5, (tag, step, n)
            assert m.hardening_x == pytest.approx(g.scalar(f"{tag}_s{step}_{n}_hx"))
            # the kernel's flip count is exact for the mask it produced; the reference's differs only
            # where a near-tie of the new soft mask is decided the other way
            hard_prev = m._hard_mask_from_soft(prev[n]) > 0.5
            hard_now = m._hard_mask_from_soft(m.mask.data) > 0.5
            assert int(m.weight.flipped_mask) == int((hard_prev ^ hard_now).sum())
            assert abs(int(m.weight.flipped_mask) - g.scalar(f"{tag}_s{step}_{n}_flips")) <= 4
            # continue from the reference's mask so that each step checks one update
            m.mask.data.copy_(want.to(DEV))
            m.invalidate_masked_weight()
            # the masked weight written by the update belongs to the mask before the reset; rebuild
            wm = m.masked_weight()
            eff = m.mask.data * m.hardening_x + (1 - m.hardening_x) * m._hard_mask_from_soft(m.mask.data) \
                if m.hardening_x < 1.0 else m.mask.data
            assert rel_err(wm, m.weight.data * eff) <= 1e-5


@pytest.mark.parametrize("tag", ["inside", "edges"])
def test_mask_stats_follow_the_reference(tag):
    """mask_stats / log_mask_stats (legacy/utils.py:2069-2340) with the reference's sample positions."""
    import math

    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g, gl = Golden("mask_stats"), Golden("train_loop")
    model = TinyMLP(sf.SparseLinear, sf.SparseLinearConfig(**json.loads(str(gl["cfg_json"])))).to(DEV)
    model.fc1.mask.data.copy_(g[f"{tag}_fc1_mask"].to(DEV))
    model.fc2.mask.data.copy_(g[f"{tag}_fc2_mask"].to(DEV))
    queue = [g[f"{tag}_idx0"].to(DEV), g[f"{tag}_idx1"].to(DEV)]
    orig = torch.randint
    torch.randint = lambda *a, **k: queue.pop(0)
    try:
        logged = {}

        class Run:
            def log(self, d, step=None):
                logged.update(d)

        out = U.log_mask_stats(model, 7, wandb_run=Run(), sample_per_layer=512)
    finally:
        torch.randint = orig
    assert logged == out and out["iter"] == 7 and out["mask/hardening_x"] == 1.0
    for k, v in zip(g[f"{tag}_keys"], g[f"{tag}_values"].tolist()):
        got = out["mask/" + str(k)]
        if math.isnan(v):
            assert math.isnan(got), k
        else:
            assert got == pytest.approx(v, rel=1e-5, abs=1e-12), k  # entropy terms use fp32 logarithms
    # the per-step reductions of the loop over the same masks (legacy/utils.py:875-1234)
    assert float(U.mid_penalty(model, 0.7)) == pytest.approx(g.scalar(f"{tag}_mid_penalty"), rel=1e-5)
    pen, cur = U.sparsity_penalty(model, 0.4, 2.0)
    assert cur == g.scalar(f"{tag}_sparsity_cur") and float(pen) == pytest.approx(g.scalar(f"{tag}_sparsity_pen"), rel=1e-6)
    for m in (model.fc1, model.fc2):
        m.mask_type = "unstructured"
    pen, cur = U.sparsity_penalty(model, 0.4, 2.0)
    assert cur == pytest.approx(g.scalar(f"{tag}_sparsity_cur_unstructured"), rel=1e-12)
    assert float(pen) == pytest.approx(g.scalar(f"{tag}_sparsity_pen_unstructured"), rel=1e-5)
    for m in (model.fc1, model.fc2):
        m.mask_type = "structured"
    tiles = U.nm_2_4_tile_stats(model)
    for k, v in zip(g[f"{tag}_tile_keys"], g[f"{tag}_tile_values"].tolist()):
        assert tiles[str(k)] == pytest.approx(v, rel=5e-6, abs=1e-9), k  # the reference's sums are fp32


@pytest.mark.parametrize("tag,tol", [("f32", 1e-5), ("bf16", 1e-2), ("chunks", 1e-5)])
def test_kl_distillation_loss(tag, tol):
    """The fused KL kernels against Distill_Model.kl_loss of the reference (loss and the gradient of
    the student logits; logits beyond the clamp get no gradient; a chunk with NaN is dropped)."""
    import sparseforge_b200 as sf

    g = Golden("kl_loss")
    s = g[f"{tag}_student"].to(DEV).requires_grad_(True)
    t = g[f"{tag}_teacher"].to(DEV)
    kl = sf.Distill_Model.kl_loss(None, s, t)
    (kl * 1.5).backward()
    assert kl.dtype == s.dtype
    assert rel_err(kl.detach().float(), g[f"{tag}_kl"]) <= tol
    assert rel_err(s.grad.float(), g[f"{tag}_grad"].float()) <= tol
    assert not torch.isnan(s.grad).any()
    # a vocabulary of LLaMA's size: rows against a float64 evaluation on the device
    if tag == "f32":
        torch.manual_seed(3)
        s2 = (torch.randn(64, 32000, device=DEV) * 4).to(torch.bfloat16)
        t2 = (torch.randn(64, 32000, device=DEV) * 4).to(torch.bfloat16)
        from sparseforge_b200 import ops

        row_kl, lse = ops.kl_div_fwd(s2, t2, 2.0, 100.0)
        a = torch.log_softmax(s2.double() / 2, -1)
        b = torch.log_softmax(t2.double() / 2, -1)
        assert rel_err(row_kl, ((b - a) * b.exp()).sum(-1)) <= 1e-5
        assert rel_err(lse[:, 0], torch.logsumexp(s2.double() / 2, -1)) <= 1e-6


@pytest.mark.parametrize("tag,trainable", [("mean", False), ("sum", True)])
def test_slorb_bypass_follows_the_reference(tag, trainable):
    """SLoRB low-rank bypass (legacy/sparse_modeling.py:388-408, 790-794, 830-872): state-dict keys,
    init_SLoRB, forward and all gradients."""
    import sparseforge_b200 as sf

    g = Golden("slorb")
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, SLoRB=True, SLoRB_k=8,
                                SLoRB_init_type=tag, trainable_projection=trainable, mask_hardening_start=1000)
    layer = sf.SparseLinear(64, 48, sparselinear_config=cfg, bias=True).to(DEV)
    keys = [str(k) for k in g[f"{tag}_state_keys"]]
    assert list(layer.state_dict().keys()) == keys
    layer.load_state_dict({k: g[f"{tag}/{k}"].to(DEV) for k in keys}, strict=True)
    assert layer.x_proj.requires_grad == trainable and layer.SLoRB_Weight.requires_grad
    if not trainable:
        # init_SLoRB rebuilds projection and bypass weight from W and the soft mask
        want_p, want_s = layer.x_proj.data.clone(), layer.SLoRB_Weight.data.clone()
        layer.x_proj.data.zero_(); layer.SLoRB_Weight.data.zero_()
        layer.init_SLoRB()
        assert torch.equal(layer.x_proj.data, want_p)
        assert rel_err(layer.SLoRB_Weight.data, want_s) <= 1e-5
    x = g[f"{tag}_x"].to(DEV).requires_grad_(True)
    y = layer(x)
    y.backward(g[f"{tag}_dy"].to(DEV))
    assert rel_err(y, g[f"{tag}_y"]) <= 1e-5
    assert rel_err(x.grad, g[f"{tag}_dx"]) <= 1e-5
    assert rel_err(layer.weight.grad, g[f"{tag}_dW"]) <= 1e-5
    assert rel_err(layer.SLoRB_Weight.grad, g[f"{tag}_dS"]) <= 1e-5
    if trainable:
        assert rel_err(layer.x_proj.grad, g[f"{tag}_dP"]) <= 1e-5
    else:
        assert layer.x_proj.grad is None


@pytest.mark.parametrize("trainable", [False, True])
def test_slorb_inside_the_main_product_at_layer_size(trainable):
    """bf16, more than 128 rows: the bypass term runs inside the main product's launch. Output and all
    gradients equal a dense fp32 autograd model of legacy/sparse_modeling.py:759-794 with the same
    effective mask; a Hessian-vector product through the layer runs (second-order path)."""
    import sparseforge_b200 as sf

    torch.manual_seed(23)
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, SLoRB=True, SLoRB_k=16,
                                SLoRB_init_type="mean", trainable_projection=trainable)
    layer = sf.SparseLinear(512, 384, sparselinear_config=cfg, bias=True).to(DEV).to(torch.bfloat16)
    layer.initialize()
    layer.mask.data.copy_(torch.rand(384, 512, device=DEV))
    layer.init_SLoRB()
    layer.hardening_x = 0.5
    layer.invalidate_masked_weight()
    x = torch.randn(4, 96, 512, device=DEV).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(4, 96, 384, device=DEV).to(torch.bfloat16)
    y = layer(x)
    y.backward(dy)

    eff = O.effective_mask(layer.mask.data.cpu(), 0.5).double()
    W = layer.weight.data.cpu().double().requires_grad_(True)
    P = layer.x_proj.data.cpu().double().requires_grad_(True)
    S = layer.SLoRB_Weight.data.cpu().double().requires_grad_(True)
    xd = x.detach().cpu().double().requires_grad_(True)

    class Ste(torch.autograd.Function):
        @staticmethod
        def forward(ctx, a, w):
            ctx.save_for_backward(a, w)
            return a @ (w * eff).t()

        @staticmethod
        def backward(ctx, g):
            a, w = ctx.saved_tensors
            return g @ (w * eff), g.reshape(-1, g.shape[-1]).t() @ a.reshape(-1, a.shape[-1])

    yd = Ste.apply(xd, W) + layer.bias.data.cpu().double() + (xd @ P.t()) @ S.t()
    yd.backward(dy.cpu().double())
    assert rel_err(y.detach().cpu().double(), yd.detach()) <= 1e-2
    assert rel_err(x.grad.cpu().double(), xd.grad) <= 1e-2
    assert rel_err(layer.weight.grad.cpu().double(), W.grad) <= 1e-2
    assert rel_err(layer.SLoRB_Weight.grad.cpu().double(), S.grad) <= 1e-2
    if trainable:
        assert rel_err(layer.x_proj.grad.cpu().double(), P.grad) <= 1e-2
    else:
        assert layer.x_proj.grad is None
    # without the bypass the output is visibly different: the term is really inside the product
    with torch.no_grad():
        plain = torch.nn.functional.linear(x.detach().float(), (layer.weight.data.float() * eff.float().to(DEV)),
                                           layer.bias.data.float())
    assert rel_err(plain.cpu().double(), yd.detach()) > 1e-2
    # second order: d/dW of <dL/dW, v> through a loss that is not linear in the output
    layer.weight.grad = None
    loss = torch.nn.functional.gelu(layer(x.detach()).float()).square().mean()
    (g1,) = torch.autograd.grad(loss, [layer.weight], create_graph=True)
    v = (torch.randint(0, 2, g1.shape, device=DEV).float() * 2 - 1).to(g1.dtype)
    (hvp,) = torch.autograd.grad((g1 * v).sum(), [layer.weight])
    assert torch.isfinite(hvp.float()).all() and float(hvp.float().abs().max()) > 0


def test_slorb_survives_compressed_inference():
    """A layer with the low-rank bypass that is compressed to hard 2:4 keeps the bypass: its output
    equals the masked dense path (binary mask) plus the bypass term (legacy/eval_wiki_ppl.py:560-575, 623
    keeps such layers in sparse_forward because the bypass is needed at inference)."""
    import sparseforge_b200 as sf

    torch.manual_seed(17)
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, SLoRB=True, SLoRB_k=16,
                                SLoRB_init_type="mean")
    layer = sf.SparseLinear(256, 128, sparselinear_config=cfg, bias=True).to(DEV).to(torch.bfloat16)
    layer.initialize()
    layer.mask.data.copy_(torch.rand(128, 256, device=DEV))
    layer.init_SLoRB()
    assert float(layer.SLoRB_Weight.data.abs().max()) > 0
    x = torch.randn(3, 40, 256, device=DEV).to(torch.bfloat16)
    hard = layer._hard_mask_from_soft(layer.mask.data)
    with torch.no_grad():
        dense = torch.nn.functional.linear(x.float(), layer.weight.data.float() * hard, layer.bias.data.float())
        bypass = (x.float() @ layer.x_proj.data.float().t()) @ layer.SLoRB_Weight.data.float().t()
        layer.eval()
        layer.compress_for_inference()
        assert layer.mode == "sparse24_forward"
        y = layer(x)
    assert float(bypass.abs().max()) > 0.01 * float(dense.abs().max())  # the term is not negligible here
    assert rel_err(y.float(), dense + bypass) <= 1e-2
    assert rel_err(y.float(), dense) > 1e-2


def test_add_calibration_runs_the_hooks():
    """utils.add_calibration with a caller-supplied loader (legacy/utils.py:1989-2060): scaler_row starts
    at one and every batch is folded in through SparseLinear.add_batch, as calling add_batch by hand does."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    torch.manual_seed(19)
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="wanda")
    model = torch.nn.Sequential(sf.SparseLinear(64, 32, sparselinear_config=cfg, bias=False),
                                sf.SparseLinear(32, 16, sparselinear_config=cfg, bias=False)).to(DEV)
    for m in model:
        m.initialize()
    batches = [torch.randn(2, 5, 64) for _ in range(4)]
    U.add_calibration(model, nsamples=3, device=DEV, dataloader=batches)
    first = model[0]
    assert first.nsamples == 6
    want, ns = torch.ones(64), 0
    for b in batches[:3]:
        want, ns = O.wanda_add_batch(want, ns, b)
    assert rel_err(first.scaler_row.data, want) <= 1e-5
    assert model[1].nsamples == 6 and float(model[1].scaler_row.data.min()) > 0


def test_score_fusion_with_the_optimizer_changes_nothing():
    """The module path with the score written by the optimizer pass (and the Hutchinson step
    updating H only) against the same loop with separate score passes: the same weights, masks,
    Hessians and flip counts after every step. The two score kernels sum eight values at a time in
    fp32 in another grouping, so mean and std of the score agree to fp32 rounding, not bit for bit."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden("train_loop")
    hp = json.loads(str(g["hp_json"]))
    cfgd = json.loads(str(g["cfg_json"]))
    X, Yt = g["X"].to(DEV), g["Yt"].to(DEV)
    runs = []
    for fuse in (False, True):
        model, _ = _build(g, "init/")
        U.initialize_model(model)
        for m in (model.fc1, model.fc2):
            m.fuse_score_with_optimizer = fuse
        opt = sf.AdamW([model.fc1.weight, model.fc1.bias, model.fc2.weight], lr=hp["lr"], betas=tuple(hp["betas"]),
                       weight_decay=hp["weight_decay"], srste_decay=cfgd["srste_decay"])
        trace = []
        for it in range(4):
            loss = torch.nn.functional.mse_loss(model(X[it]), Yt[it]) + U.mid_penalty(model, 0.1)
            queue = [g[f"s{it}_probe{j}"].to(DEV).float() for j in range(2)]
            U._rademacher_like = lambda t, q=queue: q.pop(0)
            U.update_hessian_hutchinson(model, loss)
            loss.backward()
            opt.step(decay=1e-4)
            opt.zero_grad(set_to_none=True)
            if it == 2:  # a forward between the optimizer and the mask update sees the new weight
                with torch.no_grad():
                    trace.append(model(X[it]).clone())
            U.calculate_model_mask(model, it, lambda_mid=0.1)
            for m in (model.fc1, model.fc2):
                trace += [m.weight.data.clone(), m.mask.data.clone(), m.hessian_diag.data.clone(),
                          torch.tensor(int(m.weight.flipped_mask)), m.masked_weight().clone()]
        assert model.fc1._fuse_score_next  # every step updates the mask in this recipe
        runs.append(trace)
    assert len(runs[0]) == len(runs[1])
    for a, b in zip(*runs):
        assert torch.allclose(a.float(), b.float(), rtol=1e-5, atol=1e-6)
