"""mask_type='structured' with N:M other than 2:4 (legacy/sparse_modeling.py:720-735, :1164-1225,
:1532-1570): the one-thread-per-group kernels and the SparseLinear paths built on them, against a
fixture recorded from the reference (tests/golden/nm_general.npz; generator: case_nm of
tests/golden/make_golden.py) and against the CPU oracle at layer size.

Bars: hard views and flip counts bit-exact; soft masks, gates and products 1e-5 (fp32) / 1e-2 (bf16)
relative to the largest reference magnitude.
"""
import pytest
import torch

from golden_io import Golden, rel_err
from oracle import sparselinear_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
F32_TOL = 1e-5
BF16_TOL = 1e-2

PEN_MODE = {"4of8_topn": 1, "1of4_mid": 2, "3of4_bin": 1, "1of2_plain": 0, "8of16_beta": 2, "8of32_exact": 0,
            "2of8_bf16": 1, "4of8_bf16_mag": 0}


@pytest.fixture(scope="module")
def ops():
    from sparseforge_b200 import ops as _ops

    return _ops


def dev(t):
    return t.to(DEV).contiguous()


def _variant(g, tag):
    n, m, metric = int(g.scalar(f"{tag}_N")), int(g.scalar(f"{tag}_M")), str(g[f"{tag}_metric"])
    H = g[f"{tag}_H"] if metric != "magnitude" else None
    return n, m, metric, g[f"{tag}_W"], H, g[f"{tag}_mask0"]


def _score(ops, W, H, metric):
    score = torch.empty(W.shape, dtype=torch.float32, device=DEV)
    norm = torch.zeros(2, dtype=torch.float32, device=DEV)
    ops.hutch_score(dev(W), None if H is None else dev(H), score, norm, ops.hutch_score_scratch(DEV), metric=metric)
    return score, norm


def test_kernels_follow_the_reference(ops):
    from sparseforge_b200 import _lib

    g = Golden("nm_general")
    for tag in g["variants"]:
        n, m, metric, W, H, mask0 = _variant(g, tag)
        bf16 = W.dtype == torch.bfloat16
        tol = BF16_TOL if bf16 else F32_TOL
        score_bf16 = bf16 and metric == "magnitude"  # the reference's score then has the weight's dtype
        score, norm = _score(ops, W, H, metric)
        common = dict(temperature=g.scalar(f"{tag}_T"), beta_s=g.scalar(f"{tag}_beta_s"),
                      structured_exact=tag.endswith("exact"), score_bf16=score_bf16)
        # hard view of the incoming mask: exact, ties included (the fixture's masks are full of them)
        assert torch.equal(ops.project_nm(dev(mask0), n, m).cpu(), g[f"{tag}_hard0"]), tag
        # mask_lr = 1 on a zero mask leaves exactly the gate
        G = torch.zeros(W.shape, dtype=torch.float32, device=DEV)
        stats = torch.zeros(8, dtype=torch.float64, device=DEV)
        ops.mask_update_nm(score, norm, G, stats, n, m, mask_lr=1.0, **common)
        assert rel_err(G.cpu(), g[f"{tag}_G"].float()) <= tol, tag
        # the update itself
        lam = g.scalar(f"{tag}_lambda")
        hx = g.scalar(f"{tag}_hx")
        mask = dev(mask0)
        wm = torch.empty_like(dev(W))
        ops.mask_update_nm(score, norm, mask, stats, n, m, W=dev(W), wm=wm, mask_lr=0.2, pen=0.15 * lam,
                           penalty_mode=PEN_MODE[tag] if lam else 0, binarize_decay=0.05 if tag == "3of4_bin" else 0.0,
                           hx=hx, **common)
        mask = mask.cpu()
        # bf16 scores: the reference rounds the gate to bf16 as well, and so does the kernel
        assert rel_err(mask, g[f"{tag}_mask1"]) <= tol, tag
        hard = O.hard_mask_from_soft(mask, "structured", n, m)
        assert torch.equal(ops.project_nm(dev(mask), n, m).cpu(), hard), tag
        assert int(hard.sum()) == hard.numel() * n // m
        # flips are an exact function of the masks the kernel itself produced ...
        assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(mask0, mask, "structured", n, m), tag
        # ... and agree with the reference wherever its new mask has no near-tie decided the other way
        if torch.equal(hard, g[f"{tag}_hard1"]):
            assert int(stats[_lib.MSTAT_FLIPS]) == g.scalar(f"{tag}_flips"), tag
        assert (hard != g[f"{tag}_hard1"]).float().mean() <= 2e-3, tag
        st = O.mask_stats(mask, n, m)
        s = stats.cpu()
        assert abs(float(s[_lib.MSTAT_SUM_M]) - st["sum_m"]) <= 1e-5 * st["sum_m"]
        assert abs(float(s[_lib.MSTAT_SUM_M1M]) - st["sum_m1m"]) <= 1e-5 * st["sum_m1m"] + 1e-9
        assert abs(float(s[_lib.MSTAT_SUM_TOP2]) - st["sum_top2"]) <= 1e-5 * st["sum_top2"]
        assert abs(float(s[_lib.MSTAT_SUM_BOT2]) - st["sum_bot2"]) <= 1e-5 * st["sum_m"]
        assert float(s[_lib.MSTAT_COUNT_LT_HALF]) == st["count_lt_half"]
        want_wm = O.masked_weight(W, O.effective_mask(mask, hx, "structured", False, n, m))
        assert rel_err(wm.cpu().float(), want_wm.float()) <= tol, tag
        # the stand-alone product pass writes the same masked weight
        wm2 = torch.empty_like(wm)
        ops.effective_weight_nm(dev(W), dev(mask), wm2, n, m, hx=hx)
        assert torch.equal(wm2, wm), tag
        ops.effective_weight_nm(dev(W), dev(mask), wm2, n, m, hx=hx, finalized=True)
        assert rel_err(wm2.cpu().float(), O.masked_weight(W, mask).float()) <= tol, tag


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_general_kernel_with_2_of_4_equals_the_2to4_kernel(ops, dtype):
    """Same arithmetic, other thread layout: bit-identical masks, products, flip counts."""
    torch.manual_seed(11)
    rows, cols = 96, 256
    W = (torch.randn(rows, cols) * 0.02).to(dtype)
    H = torch.rand(rows, cols) + 0.1
    mask0 = (torch.rand(rows, cols) * 50).round() / 50
    score, norm = _score(ops, W, H, "hessian_obd")
    for kw in (dict(), dict(pen=0.05, penalty_mode=1), dict(pen=0.07, penalty_mode=2, binarize_decay=0.03),
               dict(beta_s=0.3), dict(structured_exact=True), dict(hx=0.35, pen=0.02, penalty_mode=1)):
        args = dict(dict(temperature=0.3, mask_lr=0.15), **kw)
        a, b = dev(mask0), dev(mask0)
        sa = torch.zeros(8, dtype=torch.float64, device=DEV)
        sb = torch.zeros(8, dtype=torch.float64, device=DEV)
        wa, wb = torch.empty_like(dev(W)), torch.empty_like(dev(W))
        meta = torch.zeros(rows, cols // 8, dtype=torch.uint8, device=DEV)
        ops.mask_update_nm24(score, norm, a, sa, W=dev(W), wm=wa, meta=meta, **args)
        ops.mask_update_nm(score, norm, b, sb, 2, 4, W=dev(W), wm=wb, **args)
        assert torch.equal(a, b), kw
        assert torch.equal(wa, wb), kw
        assert int(sa[0]) == int(sb[0]), kw
        assert torch.allclose(sa[1:6], sb[1:6], rtol=1e-5, atol=1e-5), kw
    assert torch.equal(ops.project_nm(dev(mask0), 2, 4), ops.project_nm24(dev(mask0))[0])


@pytest.mark.parametrize("n,m", [(4, 8), (1, 4), (5, 16), (8, 32), (1, 2)])
def test_layer_size_against_the_oracle(ops, n, m):
    """A [1024, 4096] bf16 layer through one update: hard view exact outside near-ties of the soft mask."""
    torch.manual_seed(100 + m)
    rows, cols = 1024, 4096
    W = (torch.randn(rows, cols) * 0.02).to(torch.bfloat16)
    H = torch.rand(rows, cols) * 0.5 + 0.75
    mask0 = torch.rand(rows, cols)
    T, mask_lr, hx = 0.264, 0.1, 0.6
    score, norm = _score(ops, W, H, "hessian_obd")
    mask = dev(mask0)
    stats = torch.zeros(8, dtype=torch.float64, device=DEV)
    wm = torch.empty_like(dev(W))
    ops.mask_update_nm(score, norm, mask, stats, n, m, W=dev(W), wm=wm, temperature=T, mask_lr=mask_lr, hx=hx)
    s = O.normalize_scores(O.importance_score(W, "hessian_obd", H=H))
    want = O.mask_update(mask0, O.gate_target_structured(s, T, n=n, m=m), mask_lr=mask_lr, n=n, m=m)
    got = mask.cpu()
    assert rel_err(got, want) <= F32_TOL
    hard_got = ops.project_nm(mask, n, m).cpu()
    assert torch.equal(hard_got, O.hard_mask_from_soft(got, "structured", n, m))
    assert torch.all(hard_got.view(rows, cols // m, m).sum(-1) == n)
    # the reference's hard view of ITS mask differs only where two entries of a group are within rounding
    diff_groups = (hard_got != O.hard_mask_from_soft(want, "structured", n, m)).view(rows, cols // m, m).any(-1)
    if bool(diff_groups.any()):
        srt = torch.sort(want.view(rows, cols // m, m)[diff_groups], dim=-1, descending=True).values
        assert float((srt[:, n - 1] - srt[:, n]).abs().max()) <= 1e-5
    assert float(diff_groups.float().mean()) <= 1e-4
    from sparseforge_b200 import _lib

    assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(mask0, got, "structured", n, m)
    want_wm = O.masked_weight(W, O.effective_mask(got, hx, "structured", False, n, m))
    assert rel_err(wm.cpu().float(), want_wm.float()) <= BF16_TOL


@pytest.mark.parametrize("rows,cols,n,m", [(3, 12, 1, 4), (5, 6, 1, 2), (7, 20, 3, 4), (3, 24, 5, 8), (1, 2, 1, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_group_counts_that_do_not_fill_a_thread(ops, rows, cols, n, m, dtype):
    """Small groups are handled several per thread; a layer whose group count is not a multiple of that
    falls back to one group per thread. Same results as the oracle either way."""
    from sparseforge_b200 import _lib

    torch.manual_seed(rows * 100 + cols)
    W = (torch.randn(rows, cols) * 0.02).to(dtype)
    H = torch.rand(rows, cols) + 0.2
    mask0 = torch.rand(rows, cols)
    # the score pass takes multiples of eight elements; these sizes come with a score made on the host
    raw = O.importance_score(W, "hessian_obd", H=H).float()
    mu, sigma = O.score_norm_stats(raw)
    score, norm = dev(raw), torch.tensor([float(mu), float(sigma)], dtype=torch.float32, device=DEV)
    mask = dev(mask0)
    stats = torch.zeros(8, dtype=torch.float64, device=DEV)
    wm = torch.empty_like(dev(W))
    ops.mask_update_nm(score, norm, mask, stats, n, m, W=dev(W), wm=wm, temperature=0.4, mask_lr=0.3, pen=0.05,
                       penalty_mode=1, hx=0.5)
    s = O.normalize_scores(O.importance_score(W, "hessian_obd", H=H))
    want = O.mask_update(mask0, O.gate_target_structured(s, 0.4, n=n, m=m), mask_lr=0.3, lambda_mid=1.0, pen_lr=0.05,
                         penalty_mode="structured_topn", n=n, m=m)
    got = mask.cpu()
    assert rel_err(got, want) <= 1e-5
    assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(mask0, got, "structured", n, m)
    tol = BF16_TOL if dtype == torch.bfloat16 else F32_TOL
    want_wm = O.masked_weight(W, O.effective_mask(got, 0.5, "structured", False, n, m))
    assert rel_err(wm.cpu().float(), want_wm.float()) <= tol
    wm2 = torch.empty_like(wm)
    ops.effective_weight_nm(dev(W), mask, wm2, n, m, hx=0.5)
    assert torch.equal(wm2, wm)
    assert torch.equal(ops.project_nm(mask, n, m).cpu(), O.hard_mask_from_soft(got, "structured", n, m))


def test_projection_strides_dtypes_and_nan(ops):
    torch.manual_seed(3)
    big = torch.rand(20, 96, device=DEV)
    view = big[:, 16:80]  # row stride 96, 64 columns
    for n, m in ((3, 8), (1, 4), (2, 16)):
        got = ops.project_nm(view, n, m).cpu()
        assert torch.equal(got, O.hard_mask_from_soft(view.cpu().contiguous(), "structured", n, m))
    soft = torch.rand(8, 32)
    soft[0, 3] = float("nan")  # sorts as the largest value, as in torch
    soft[1, :8] = 0.5
    got = ops.project_nm(dev(soft), 2, 8).cpu()
    assert torch.equal(got, O.hard_mask_from_soft(soft, "structured", 2, 8))
    assert got[0, 3] == 1 and got[1, :8].tolist() == [1, 1, 0, 0, 0, 0, 0, 0]
    sb = soft.nan_to_num(0.0).to(torch.bfloat16)
    got = ops.project_nm(dev(sb), 4, 8)
    assert got.dtype == torch.bfloat16
    assert torch.equal(got.cpu().float(), O.hard_mask_from_soft(sb.float(), "structured", 4, 8))
    got32 = ops.project_nm(dev(sb), 4, 8, out_dtype=torch.float32)
    assert torch.equal(got32.cpu(), got.cpu().float())


def test_bad_arguments_are_refused(ops):
    soft = torch.rand(4, 24, device=DEV)
    for n, m in ((2, 3), (4, 4), (0, 4), (2, 64)):
        with pytest.raises(RuntimeError):
            ops.project_nm(soft, n, m)
    with pytest.raises(RuntimeError):
        ops.project_nm(soft, 4, 16)  # 24 columns are not a multiple of 16
    W = torch.randn(4, 24, device=DEV)
    with pytest.raises(RuntimeError):
        ops.effective_weight_nm(W, soft, torch.empty_like(W), 2, 16)


def _layer(g, tag):
    import sparseforge_b200 as sf

    n, m, metric, W, H, mask0 = _variant(g, tag)
    kw = {"4of8_topn": dict(mask_penalty_mode="structured_topn"), "1of4_mid": dict(mask_penalty_mode="mid"),
          "3of4_bin": dict(mask_penalty_mode="structured_topn", mask_binarize_decay=0.05), "1of2_plain": dict(),
          "8of16_beta": dict(mask_penalty_mode="mid", beta_structural_start=0, beta_structural_end=10),
          "8of32_exact": dict(structured_exact=True), "2of8_bf16": dict(mask_penalty_mode="structured_topn"),
          "4of8_bf16_mag": dict()}[tag]
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric=metric, N=n, M=m, mask_update_period=1,
                                sparsity_warmup_steps=0, mask_lr=0.2, mask_penalty_lr=0.15, mask_hardening_start=2,
                                mask_hardening_duration=8, **kw)
    layer = sf.SparseLinear(W.shape[1], W.shape[0], sparselinear_config=cfg, bias=False).to(DEV).to(W.dtype)
    layer.weight.data.copy_(W.to(DEV))
    layer.initialize()
    layer.mask.data.copy_(mask0.to(DEV))
    if H is not None:
        layer.hessian_diag.data.copy_(H.to(DEV))
    layer.invalidate_masked_weight()
    return layer, n, m


def test_sparse_linear_follows_the_reference():
    g = Golden("nm_general")
    for tag in g["variants"]:
        layer, n, m = _layer(g, tag)
        bf16 = layer.weight.dtype == torch.bfloat16
        tol = BF16_TOL if bf16 else F32_TOL
        step = int(g.scalar(f"{tag}_step"))
        assert torch.equal(layer._hard_mask_from_soft(layer.mask.data).cpu(), g[f"{tag}_hard0"]), tag
        assert rel_err(layer.compute_gate_target(step).cpu().float(), g[f"{tag}_G"].float()) <= tol, tag
        layer.update_mask(step, lambda_mid=g.scalar(f"{tag}_lambda"))
        assert layer.hardening_x == pytest.approx(g.scalar(f"{tag}_hx"))
        assert rel_err(layer.mask.data.cpu(), g[f"{tag}_mask1"]) <= tol, tag
        hard = layer._hard_mask_from_soft(layer.mask.data).cpu()
        if torch.equal(hard, g[f"{tag}_hard1"]):
            assert int(layer.weight.flipped_mask) == g.scalar(f"{tag}_flips"), tag
        X = g[f"{tag}_X"].to(DEV).requires_grad_(True)
        Y = layer(X)
        Y.backward(g[f"{tag}_dY"].to(DEV))
        assert rel_err(Y.detach().cpu().float(), g[f"{tag}_Y"].float()) <= tol, tag
        assert rel_err(X.grad.cpu().float(), g[f"{tag}_dX"].float()) <= tol, tag
        assert rel_err(layer.weight.grad.cpu().float(), g[f"{tag}_dW"].float()) <= tol, tag
        # compressed inference is the sparse tensor cores' 2:4 format only
        with pytest.raises(NotImplementedError):
            layer.compress_for_inference()


class _TwoLayers(torch.nn.Module):
    def __init__(self, cfg, d=64, h=128):
        import sparseforge_b200 as sf

        super().__init__()
        self.fc1 = sf.SparseLinear(d, h, sparselinear_config=cfg, bias=False)
        self.fc2 = sf.SparseLinear(h, d, sparselinear_config=cfg, bias=False)

    def forward(self, x):
        return self.fc2(torch.nn.functional.gelu(self.fc1(x)))


@pytest.mark.parametrize("hard_type,n,m", [("match", 4, 8), ("block16", 2, 4), ("block_sparse16", 2, 4)])
def test_second_order_products_use_the_layers_own_hard_view(hard_type, n, m):
    """With hardening active the Hessian-vector product of the first layer passes through the second
    layer's masked weight: its backward must apply the layer's own effective mask (N:M, per-tile or
    block), which a dense autograd model with the oracle's effective masks checks."""
    import sparseforge_b200 as sf

    torch.manual_seed(5)
    mask_type = "structured" if hard_type == "match" else "unstructured"
    cfg = sf.SparseLinearConfig(mask_type=mask_type, hard_mask_type=hard_type, mask_metric="hessian_obd", N=n, M=m,
                                sparsity_ratio=0.5, mask_update_period=1, sparsity_warmup_steps=0)
    model = _TwoLayers(cfg).to(DEV)
    for layer in (model.fc1, model.fc2):
        layer.initialize()
        layer.mask.data.copy_(torch.rand_like(layer.mask.data))
        layer.hardening_x = 0.4
        layer.invalidate_masked_weight()
    X = torch.randn(24, 64, device=DEV)
    target = torch.randn(24, 64, device=DEV)
    v = torch.randint(0, 2, model.fc1.weight.shape, device=DEV).float() * 2 - 1
    loss = ((model(X) - target) ** 2).mean()
    (g1,) = torch.autograd.grad(loss, [model.fc1.weight], create_graph=True)
    (hvp,) = torch.autograd.grad((g1 * v).sum(), [model.fc1.weight])

    # dense model with the same effective masks
    def eff(layer):
        mask = layer.mask.data.cpu()
        if hard_type == "match":
            hard = O.hard_mask_from_soft(mask, "structured", n, m)
        elif hard_type == "block16":
            hard = O.hard_mask_tile16(mask, 0.5)
        else:
            hard = O.hard_mask_block(mask, 16, 0.5)
        return 0.4 * mask + (1.0 - 0.4) * hard

    W1 = model.fc1.weight.data.cpu().double().requires_grad_(True)
    W2 = model.fc2.weight.data.cpu().double()
    e1, e2 = eff(model.fc1).double(), eff(model.fc2).double()

    class Ste(torch.autograd.Function):  # masked forward, gradient straight to the dense weight
        @staticmethod
        def forward(ctx, x, W, e):
            ctx.save_for_backward(x, W, e)
            return x @ (W * e).t()

        @staticmethod
        def backward(ctx, gy):
            x, W, e = ctx.saved_tensors
            return gy @ (W * e), gy.t() @ x, None

    Xd = X.cpu().double()
    out = Ste.apply(torch.nn.functional.gelu(Ste.apply(Xd, W1, e1)), W2, e2)
    loss_d = ((out - target.cpu().double()) ** 2).mean()
    (g1d,) = torch.autograd.grad(loss_d, [W1], create_graph=True)
    (hvp_d,) = torch.autograd.grad((g1d * v.cpu().double()).sum(), [W1])
    assert rel_err(g1.detach().cpu().double(), g1d.detach()) <= 1e-4
    assert float(hvp_d.abs().max()) > 0
    assert rel_err(hvp.cpu().double(), hvp_d) <= 1e-4


def test_adamw_keeps_the_masked_weight_of_a_general_layer_current():
    """The optimizer kernel writes the masked weight only for 2:4 layers; for other N:M the layer
    rebuilds it on the next forward."""
    import sparseforge_b200 as sf

    torch.manual_seed(9)
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=4, M=8, mask_update_period=2,
                                sparsity_warmup_steps=0, mask_lr=0.3)
    layer = sf.SparseLinear(64, 32, sparselinear_config=cfg, bias=False).to(DEV)
    layer.initialize()
    layer.mask.data.copy_(torch.rand_like(layer.mask.data))
    layer.hardening_x = 0.5
    layer.invalidate_masked_weight()
    opt = sf.AdamW([layer.weight], lr=1e-2, weight_decay=0.0)
    X = torch.randn(16, 64, device=DEV)
    for step in range(4):
        Y = layer(X)
        eff = O.effective_mask(layer.mask.data.cpu(), float(layer.hardening_x), "structured", False, 4, 8)
        want = X.cpu() @ (layer.weight.data.cpu() * eff).t()
        assert rel_err(Y.detach().cpu(), want) <= 1e-4, step
        Y.square().mean().backward()
        opt.step(decay=0.0)
        opt.zero_grad(set_to_none=True)
        layer.update_mask(step)
        layer.hardening_x = 0.5


UH_KW = {"mid": dict(mask_penalty_mode="mid"), "topn": dict(mask_penalty_mode="structured_topn"),
         "beta": dict(mask_penalty_mode="mid", beta_structural_start=0, beta_structural_end=10),
         "bin": dict(mask_penalty_mode="mid", mask_binarize_decay=0.05), "bf16": dict(mask_penalty_mode="mid")}


def test_unstructured_hard_view_follows_the_reference():
    """mask_type='unstructured' with its own hard view (mask > 0.5, legacy/sparse_modeling.py:526-527):
    gate, update, flip count, masked forward / backward of SparseLinear against the recorded reference run."""
    import sparseforge_b200 as sf

    g = Golden("unstructured_hard")
    for tag in g["variants"]:
        W, H, mask0 = g[f"{tag}_W"], g[f"{tag}_H"], g[f"{tag}_mask0"]
        tol = BF16_TOL if W.dtype == torch.bfloat16 else F32_TOL
        cfg = sf.SparseLinearConfig(mask_type="unstructured", mask_metric="hessian_obd", N=2, M=4, sparsity_ratio=0.5,
                                    mask_update_period=1, sparsity_warmup_steps=0, mask_lr=0.2, mask_penalty_lr=0.15,
                                    mask_hardening_start=2, mask_hardening_duration=8, **UH_KW[tag])
        layer = sf.SparseLinear(W.shape[1], W.shape[0], sparselinear_config=cfg, bias=False).to(DEV).to(W.dtype)
        layer.weight.data.copy_(W.to(DEV))
        layer.initialize()
        layer.mask.data.copy_(mask0.to(DEV))
        layer.hessian_diag.data.copy_(H.to(DEV))
        layer.invalidate_masked_weight()
        assert layer._threshold_view() and layer._general_nm() and not layer._is_2to4_view()
        step = int(g.scalar(f"{tag}_step"))
        assert rel_err(layer.compute_gate_target(step).cpu().float(), g[f"{tag}_G"].float()) <= tol, tag
        layer.update_mask(step, lambda_mid=g.scalar(f"{tag}_lambda"))
        assert layer.hardening_x == pytest.approx(g.scalar(f"{tag}_hx"))
        got = layer.mask.data.cpu()
        assert rel_err(got, g[f"{tag}_mask1"]) <= tol, tag
        # flips: an exact function of the masks the kernel produced; equal to the reference's unless an entry
        # sits within rounding of 0.5
        assert int(layer.weight.flipped_mask) == O.flip_count(mask0, got, "unstructured"), tag
        hard = layer._hard_mask_from_soft(layer.mask.data).cpu()
        if torch.equal(hard, g[f"{tag}_hard1"]):
            assert int(layer.weight.flipped_mask) == g.scalar(f"{tag}_flips"), tag
        assert (hard != g[f"{tag}_hard1"]).float().mean() <= 2e-3, tag
        X = g[f"{tag}_X"].to(DEV).requires_grad_(True)
        Y = layer(X)
        Y.backward(g[f"{tag}_dY"].to(DEV))
        assert rel_err(Y.detach().cpu().float(), g[f"{tag}_Y"].float()) <= tol, tag
        assert rel_err(X.grad.cpu().float(), g[f"{tag}_dX"].float()) <= tol, tag
        assert rel_err(layer.weight.grad.cpu().float(), g[f"{tag}_dW"].float()) <= tol, tag
        with pytest.raises(NotImplementedError):
            layer.compress_for_inference()
