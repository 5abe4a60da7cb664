"""GPU parity of every kernel against the CPU oracle and the reference-generated fixtures.

All calls go through the C ABI (``sparseforge_b200.ops`` is a pointer-passing wrapper).
Bars: bit-exact for hard masks, metadata and flip counts; 1e-5 (fp32) / 1e-2 (bf16) relative to
the largest reference magnitude for scores, soft masks, GEMM outputs and optimizer state.
"""
import pytest
import torch

from oracle import sparselinear_oracle as O
from tests.golden_io import Golden, rel_err

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
BF16_TOL = 1e-2
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from sparseforge_b200 import ops as _ops

    return _ops


def dev(t):
    return t.to(DEV).contiguous()


def unpack_meta(meta, cols):
    """[rows, cols/8] packed bytes -> 0/1 mask [rows, cols]."""
    meta = meta.cpu()
    rows = meta.shape[0]
    nib = torch.stack([meta & 0xF, meta >> 4], dim=-1).view(rows, -1)[:, : cols // 4].long()
    out = torch.zeros(rows, cols // 4, 4)
    out.scatter_(-1, (nib & 3).unsqueeze(-1), 1.0)
    out.scatter_(-1, (nib >> 2).unsqueeze(-1), 1.0)
    return out.view(rows, cols)


# ---------------------------------------------------------------------------------------
# hard projection
# ---------------------------------------------------------------------------------------
def test_project_ties_bit_exact(ops):
    g = Golden("ties")
    for name in g["names"]:
        soft, want = g[f"{name}_soft"], g[f"{name}_hard"]
        hard, meta = ops.project_nm24(dev(soft), want_meta=True)
        assert torch.equal(hard.cpu(), want), name
        assert torch.equal(meta.cpu(), O.meta_from_hard(want)), name
        assert torch.equal(unpack_meta(meta, soft.shape[1]), want), name
        hb, _ = ops.project_nm24(dev(soft), out_dtype=torch.bfloat16)
        assert torch.equal(hb.float().cpu(), want), name


def test_project_ragged_tail_and_strides(ops):
    g = Golden("ties")
    soft, want = g["tail_soft"], g["tail_hard"]
    hard, meta = ops.project_nm24(dev(soft), want_meta=True)
    assert torch.equal(hard.cpu(), want)
    assert torch.equal(meta.cpu(), O.meta_from_hard(want))
    # a column slice of a wider tensor (row stride != cols)
    wide = torch.rand(16, 96)
    view = dev(wide)[:, 8:72]
    h2, _ = ops.project_nm24(view)
    assert torch.equal(h2.cpu(), O.hard_mask_from_soft(wide[:, 8:72].contiguous()))
    # empty inputs
    h3, m3 = ops.project_nm24(torch.empty(0, 64, device=DEV), want_meta=True)
    assert h3.shape == (0, 64) and m3.shape == (0, 8)


def test_project_nan_and_bf16_input(ops):
    x = torch.tensor([[float("nan"), 1.0, 2.0, 3.0, 1.0, float("nan"), float("nan"), 0.0]])
    hard, _ = ops.project_nm24(dev(x))
    assert torch.equal(hard.cpu(), O.hard_mask_from_soft(x))
    xb = torch.rand(32, 64).to(torch.bfloat16)
    hb, _ = ops.project_nm24(dev(xb))
    assert torch.equal(hb.float().cpu(), O.hard_mask_from_soft(xb.float()))


@pytest.mark.parametrize("shape", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_project_llama_shapes_properties(ops, shape):
    torch.manual_seed(100)
    w = (torch.randn(shape) * 0.02).abs()
    hard, meta = ops.project_nm24(dev(w), want_meta=True)
    # exactly two kept per group, idempotent, metadata decodes to the mask, equal to the oracle
    assert bool((hard.view(shape[0], -1, 4).sum(-1) == 2).all())
    again, _ = ops.project_nm24(hard)
    assert torch.equal(again, hard)
    assert torch.equal(unpack_meta(meta, shape[1]), hard.cpu())
    assert torch.equal(hard.cpu(), O.hard_mask_from_soft(w))


# ---------------------------------------------------------------------------------------
# Hutchinson accumulate + score
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["chain_f32", "chain_bf16"])
def test_hutch_score_chain(ops, case):
    g = Golden(case)
    probe = 0
    H = torch.ones(g["W0"].shape)
    for t in range(g.scalar("n_steps")):
        W = g[f"s{t}_W_fwd"]
        while probe < g.scalar(f"s{t}_probes_end"):
            Hd = dev(H)
            score = torch.empty(W.shape, dtype=torch.float32, device=DEV)
            norm = torch.zeros(2, dtype=torch.float32, device=DEV)
            scratch = ops.hutch_score_scratch(DEV)
            # int8 probe and weight-dtype probe must agree
            ops.hutch_score(dev(W), Hd, score, norm, scratch, hvp=dev(g[f"hvp_{probe}"]), v=dev(g[f"v_{probe}"]), beta=0.99)
            Hd2 = dev(H)
            ops.hutch_score(dev(W), Hd2, score, norm, scratch, hvp=dev(g[f"hvp_{probe}"]),
                            v=dev(g[f"v_{probe}"].to(W.dtype)), beta=0.99)
            assert torch.equal(Hd, Hd2)
            assert rel_err(Hd, g[f"H_{probe}"]) <= F32_TOL
            want = O.importance_score(W, "hessian_obd", H=g[f"H_{probe}"])
            assert rel_err(score, want) <= F32_TOL
            mu, sigma = O.score_norm_stats(want)
            assert abs(float(norm[0]) - float(mu)) <= F32_TOL * abs(float(mu))
            assert abs(float(norm[1]) - float(sigma)) <= F32_TOL * abs(float(sigma))
            H = g[f"H_{probe}"].clone()
            probe += 1


@pytest.mark.parametrize("metric", ["hessian_obd", "hessian_ratio", "magnitude", "hessian", "movement"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_score_metrics(ops, metric, dtype):
    torch.manual_seed(1)
    W = (torch.randn(64, 128) * 0.02).to(dtype)
    H = torch.rand(64, 128) + 0.05
    ge = (torch.randn(64, 128) * 0.01).to(dtype)
    score = torch.empty(W.shape, dtype=torch.float32, device=DEV)
    norm = torch.zeros(2, dtype=torch.float32, device=DEV)
    ops.hutch_score(dev(W), dev(H), score, norm, ops.hutch_score_scratch(DEV), aux=dev(ge), aux_scalar=0.7, metric=metric)
    want = O.importance_score(W, metric, H=H, grad_ema=ge, temperature=0.7)
    tol = F32_TOL if (dtype == torch.float32 or metric in ("hessian",)) else BF16_TOL
    assert rel_err(score, want.float()) <= tol
    mu, sigma = O.score_norm_stats(score.cpu())
    assert abs(float(norm[0]) - float(mu)) <= 1e-5 * abs(float(mu)) + 1e-12
    assert abs(float(norm[1]) - float(sigma)) <= 1e-5 * abs(float(sigma))


# ---------------------------------------------------------------------------------------
# mask update
# ---------------------------------------------------------------------------------------
def run_mask_update(ops, W, H, mask0, *, T, mask_lr, pen, pmode, beta_s=0.0, bin_d=0.0, hx=1.0, exact=False):
    Wd, Hd = dev(W), dev(H)
    score = torch.empty(W.shape, dtype=torch.float32, device=DEV)
    norm = torch.zeros(2, dtype=torch.float32, device=DEV)
    ops.hutch_score(Wd, Hd, score, norm, ops.hutch_score_scratch(DEV))
    mask = dev(mask0)
    stats = torch.zeros(8, dtype=torch.float64, device=DEV)
    wm = torch.empty_like(Wd)
    meta = torch.zeros(W.shape[0], W.shape[1] // 8, dtype=torch.uint8, device=DEV)
    ops.mask_update_nm24(score, norm, mask, stats, W=Wd, wm=wm, meta=meta, temperature=T, mask_lr=mask_lr, pen=pen,
                         penalty_mode=pmode, beta_s=beta_s, binarize_decay=bin_d, hx=hx, structured_exact=exact)
    return mask.cpu(), stats.cpu(), wm.cpu(), meta.cpu()


@pytest.mark.parametrize("case,tol", [("chain_f32", F32_TOL), ("chain_bf16", BF16_TOL)])
def test_mask_update_chain(ops, case, tol):
    from sparseforge_b200 import _lib

    g = Golden(case)
    lam = g.scalar("lambda_mid")
    for t in range(g.scalar("n_steps")):
        W, H = g[f"s{t}_W_opt"], g[f"H_{g.scalar(f's{t}_probes_end') - 1}"]
        mask0 = g[f"s{t}_mask_fwd"]
        hx = g.scalar(f"s{t}_hx")
        mask, stats, wm, meta = run_mask_update(ops, W, H, mask0, T=g.scalar(f"s{t}_T"), mask_lr=0.1, pen=0.1 * lam,
                                                pmode=_lib.PENALTY_TOPN if lam else 0, hx=hx)
        want = g[f"s{t}_mask"]
        assert rel_err(mask, want) <= F32_TOL
        hard_now = O.hard_mask_from_soft(mask)
        # flips and metadata are exact functions of the masks the kernel itself produced
        assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(mask0, mask)
        assert torch.equal(unpack_meta(meta, W.shape[1]), hard_now)
        # and they agree with the reference wherever the reference's mask has no near-tie
        if torch.equal(hard_now, g[f"s{t}_hard"]):
            assert int(stats[_lib.MSTAT_FLIPS]) == g.scalar(f"s{t}_flips")
        assert (hard_now != g[f"s{t}_hard"]).float().mean() <= 1e-3
        st = O.mask_stats(mask)
        assert abs(float(stats[_lib.MSTAT_SUM_M]) - st["sum_m"]) <= 1e-5 * st["sum_m"]
        assert abs(float(stats[_lib.MSTAT_SUM_M1M]) - st["sum_m1m"]) <= 1e-5 * st["sum_m1m"] + 1e-9
        assert abs(float(stats[_lib.MSTAT_SUM_TOP2]) - st["sum_top2"]) <= 1e-5 * st["sum_top2"]
        assert abs(float(stats[_lib.MSTAT_SUM_BOT2]) - st["sum_bot2"]) <= 1e-5 * st["sum_bot2"] + 1e-9
        assert float(stats[_lib.MSTAT_COUNT_LT_HALF]) == st["count_lt_half"]
        want_wm = O.masked_weight(W, O.effective_mask(mask, hx))
        assert rel_err(wm.float(), want_wm.float()) <= tol


def test_mask_update_penalty_variants(ops):
    from sparseforge_b200 import _lib

    g = Golden("penalty")
    pm = {"topn": 1, "nm24": 1, "mid": 2, "bin": 1, "beta": 2, "exact": 2, "lowT": 1}
    for tag in g["variants"]:
        lam = g.scalar(f"{tag}_lambda")
        mask, stats, wm, meta = run_mask_update(
            ops, g[f"{tag}_W"], g[f"{tag}_H"], g[f"{tag}_mask0"], T=g.scalar(f"{tag}_T"), mask_lr=0.2, pen=0.15 * lam,
            pmode=pm[tag] if lam else 0, beta_s=g.scalar(f"{tag}_beta_s"), bin_d=0.05 if tag == "bin" else 0.0,
            hx=g.scalar(f"{tag}_hx"), exact=(tag == "exact"))
        assert rel_err(mask, g[f"{tag}_mask1"]) <= F32_TOL, tag
        assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(g[f"{tag}_mask0"], mask), tag
        if torch.equal(O.hard_mask_from_soft(mask), O.hard_mask_from_soft(g[f"{tag}_mask1"])):
            assert int(stats[_lib.MSTAT_FLIPS]) == g.scalar(f"{tag}_flips"), tag


def test_gate_from_update_kernel(ops):
    """mask_lr = 1 on a zero mask leaves exactly the gate G."""
    g = Golden("penalty")
    for tag in ("topn", "beta", "exact", "lowT"):
        mask, _, _, _ = run_mask_update(ops, g[f"{tag}_W"], g[f"{tag}_H"], torch.zeros(g[f"{tag}_W"].shape),
                                        T=g.scalar(f"{tag}_T"), mask_lr=1.0, pen=0.0, pmode=0,
                                        beta_s=g.scalar(f"{tag}_beta_s"), exact=(tag == "exact"))
        assert rel_err(mask, g[f"{tag}_G"]) <= F32_TOL, tag


def test_effective_weight(ops):
    torch.manual_seed(2)
    for dtype, tol in ((torch.float32, F32_TOL), (torch.bfloat16, BF16_TOL)):
        W = (torch.randn(48, 64) * 0.02).to(dtype)
        mask = torch.rand(48, 64)
        for hx, fin in ((1.0, False), (0.4, False), (0.0, False), (0.3, True)):
            wm = torch.empty_like(dev(W))
            meta = torch.zeros(48, 8, dtype=torch.uint8, device=DEV)
            ops.effective_weight(dev(W), dev(mask), wm, meta=meta, hx=hx, finalized=fin)
            want = O.masked_weight(W, O.effective_mask(mask, hx, finalized=fin))
            assert rel_err(wm.float(), want.float()) <= tol
            assert torch.equal(unpack_meta(meta, 64), O.hard_mask_from_soft(mask))


# ---------------------------------------------------------------------------------------
# AdamW
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag,tol,l1", [("f32", F32_TOL, 0.0), ("bf16", BF16_TOL, 0.0), ("l1", F32_TOL, 0.02)])
def test_adamw_golden(ops, tag, tol, l1):
    g = Golden("adamw")
    p = dev(g[f"{tag}_p0"])
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    mask = dev(g[f"{tag}_mask"])
    for t in range(3):
        wm = torch.empty_like(p)
        ops.adamw_masked(p, dev(g[f"{tag}_g{t}"]), m, v, mask=mask, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                         weight_decay=0.1, decay=5e-4 * (t + 1), step=t + 1, adaptive_l1=l1, wm=wm, hx=0.5)
        assert rel_err(p.float(), g[f"{tag}_p{t + 1}"].float()) <= tol
        assert rel_err(m.float(), g[f"{tag}_m{t + 1}"].float()) <= tol
        assert rel_err(v.float(), g[f"{tag}_v{t + 1}"].float()) <= tol
        want_wm = O.masked_weight(p.cpu(), O.effective_mask(mask.cpu(), 0.5))
        assert rel_err(wm.float(), want_wm.float()) <= tol


@pytest.mark.parametrize("tag,tol", [("f32", F32_TOL), ("bf16", BF16_TOL)])
def test_adamw_amsgrad_golden(ops, tag, tol):
    """amsgrad=True through the optimizer class against the reference's trajectory (tests/golden/adamw_ams.npz)."""
    import sparseforge_b200 as sf

    g = Golden("adamw_ams")
    p = torch.nn.Parameter(dev(g[f"{tag}_p0"]))
    p.mask = dev(g[f"{tag}_mask"])
    opt = sf.AdamW([p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, amsgrad=True)
    for t in range(4):
        p.grad = dev(g[f"{tag}_g{t}"]).clone()
        opt.step(decay=5e-4 * (t + 1))
        st = opt.state[p]
        for got, name in ((p.data, "p"), (st["exp_avg"], "m"), (st["exp_avg_sq"], "v"), (st["max_exp_avg_sq"], "vmax")):
            assert rel_err(got.float(), g[f"{tag}_{name}{t + 1}"].float()) <= tol, (name, t)


def test_adamw_no_mask(ops):
    torch.manual_seed(4)
    p0, g0 = torch.randn(1024) * 0.1, torch.randn(1024) * 0.01
    p = dev(p0)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    ops.adamw_masked(p, dev(g0), m, v, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, decay=0.0, step=1)
    wp, wm_, wv = O.adamw_step(p0, g0, torch.zeros(1024), torch.zeros(1024), step=1, lr=1e-3, betas=(0.9, 0.999),
                               eps=1e-8, weight_decay=0.01)
    assert rel_err(p, wp) <= F32_TOL and rel_err(m, wm_) <= F32_TOL and rel_err(v, wv) <= F32_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("metric", ["hessian_obd", "hessian_ratio", "magnitude", "hessian"])
def test_adamw_with_score_equals_separate_calls(ops, dtype, metric):
    """The fused optimizer+score pass and the H-only accumulation give, bit for bit, what the
    separate calls give: H update, AdamW step, then the score of the new weight."""
    torch.manual_seed(11)
    rows, cols = 96, 264  # 25344 elements: not a multiple of a 256-element span
    p0 = (torch.randn(rows, cols) * 0.05).to(dtype)
    g0 = (torch.randn(rows, cols) * 0.01).to(dtype)
    hvp = (torch.randn(rows, cols) * 0.1).to(dtype)
    sign = (torch.randint(0, 2, (rows, cols)) * 2 - 1).to(torch.int8)
    mask = torch.rand(rows, cols)
    H0 = torch.rand(rows, cols) * 1e-3
    kw = dict(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, decay=2e-4, step=3, adaptive_l1=1e-5)

    # separate calls
    pa, ma, va, Ha = dev(p0), dev(torch.full_like(p0, 1e-3)), dev(torch.full_like(p0, 1e-5)), dev(H0)
    sa, na, scr = torch.empty(rows, cols, device=DEV), torch.empty(2, device=DEV), ops.hutch_score_scratch(DEV)
    ops.hutch_score(pa, Ha, sa, na, scr, hvp=dev(hvp), v=dev(sign), beta=0.98, metric=metric)
    ops.adamw_masked(pa, dev(g0), ma, va, mask=dev(mask), **kw)
    ops.hutch_score(pa, Ha, sa, na, scr, metric=metric)
    sums_a = scr[:2].clone()

    # H only, then optimizer + score in one pass
    pb, mb, vb, Hb = dev(p0), dev(torch.full_like(p0, 1e-3)), dev(torch.full_like(p0, 1e-5)), dev(H0)
    sb, nb, scr2 = torch.empty(rows, cols, device=DEV), torch.empty(2, device=DEV), ops.hutch_score_scratch(DEV)
    ops.hutch_accumulate(Hb, dev(hvp), dev(sign), beta=0.98)
    ops.adamw_masked_score(pb, dev(g0), mb, vb, mask=dev(mask), H=Hb, score=sb, norm=nb, scratch=scr2,
                           metric=metric, **kw)
    assert torch.equal(Ha, Hb)
    assert torch.equal(pa, pb) and torch.equal(ma, mb) and torch.equal(va, vb)
    assert torch.equal(sa, sb)
    # all three in one pass (the probe once as int8 signs, once in the weight dtype)
    for probe in (dev(sign), dev(sign.to(dtype))):
        pc, mc, vc, Hc = dev(p0), dev(torch.full_like(p0, 1e-3)), dev(torch.full_like(p0, 1e-5)), dev(H0)
        sc_, nc = torch.empty(rows, cols, device=DEV), torch.empty(2, device=DEV)
        ops.adamw_masked_score(pc, dev(g0), mc, vc, mask=dev(mask), H=Hc, score=sc_, norm=nc, scratch=scr2,
                               metric=metric, hvp=dev(hvp), probe=probe, beta_h=0.98, **kw)
        assert torch.equal(Ha, Hc) and torch.equal(pa, pc) and torch.equal(ma, mc) and torch.equal(va, vc)
        assert torch.equal(sa, sc_) and torch.allclose(na, nc, rtol=1e-6, atol=0)
    # eight values at a time are summed in fp32, and the two kernels group the eight differently
    assert torch.allclose(sums_a, scr2[:2], rtol=1e-6, atol=0)
    assert torch.allclose(na, nb, rtol=1e-6, atol=0)
    # and against the oracle's score of the new weight
    want = O.importance_score(pb.cpu(), metric, H=Hb.cpu())
    assert rel_err(sb, want.float()) <= (F32_TOL if dtype == torch.float32 else BF16_TOL)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("metric,extra", [("hessian_obd", {}), ("hessian_ratio", dict(pen=0.03, penalty_mode=2)),
                                          ("magnitude", dict(beta_s=0.3, binarize_decay=0.05)), ("hessian", {})])
def test_mask_update_from_weight_equals_update_from_score(ops, dtype, metric, extra):
    """Forming the score inside the mask update from W and H gives, bit for bit, the update from the
    score tensor the optimizer pass would have written; that pass then only needs the statistics."""
    torch.manual_seed(21)
    rows, cols = 80, 136
    W = dev((torch.randn(rows, cols) * 0.05).to(dtype))
    g0 = dev((torch.randn(rows, cols) * 0.01).to(dtype))
    H = dev(torch.rand(rows, cols) * 1e-2)
    mask0 = torch.rand(rows, cols)
    kw = dict(lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, decay=2e-4, step=2)
    upd = dict(temperature=0.3, mask_lr=0.2, hx=0.4, **extra)

    def run(with_score):
        p, m, v = W.clone(), torch.zeros_like(W), torch.zeros_like(W)
        mask, stats = dev(mask0), torch.zeros(8, dtype=torch.float64, device=DEV)
        norm, scr = torch.empty(2, device=DEV), ops.hutch_score_scratch(DEV)
        wm, meta = torch.empty_like(p), torch.zeros(rows, cols // 8, dtype=torch.uint8, device=DEV)
        score = torch.empty(rows, cols, device=DEV) if with_score else None
        ops.adamw_masked_score(p, g0, m, v, mask=mask, H=H, score=score, norm=norm, scratch=scr, metric=metric, **kw)
        if with_score:
            ops.mask_update_nm24(score, norm, mask, stats, W=p, wm=wm, meta=meta, **upd)
        else:
            ops.mask_update_nm24_from_weight(p, H, norm, mask, stats, wm, meta, metric=metric, **upd)
        return p, mask, wm, meta, stats, norm

    a, b = run(True), run(False)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_passes_agree_for_16_and_32_byte_aligned_tensors(ops):
    """The optimizer+score and mask-update passes move the fp32 mask and Hessian with 32-byte accesses
    when their addresses allow it and with 16-byte accesses otherwise: same results either way."""
    torch.manual_seed(23)
    rows, cols = 64, 264
    n = rows * cols
    W0 = (torch.randn(rows, cols) * 0.05).to(torch.bfloat16)
    g0 = (torch.randn(rows, cols) * 0.01).to(torch.bfloat16)
    hvp = (torch.randn(rows, cols) * 0.1).to(torch.bfloat16)
    sign = (torch.randint(0, 2, (rows, cols)) * 2 - 1).to(torch.int8)
    H0, mask0 = torch.rand(rows, cols) * 1e-2, torch.rand(rows, cols)

    def fp32(t, shift):  # a copy that starts `shift` floats into a 32-byte aligned buffer
        buf = torch.empty(n + 8, device=DEV)
        view = buf[shift:shift + n].view(rows, cols)
        view.copy_(t)
        assert view.data_ptr() % 32 == (4 * shift) % 32
        return view

    def run(shift):
        p, m, v = dev(W0), torch.zeros(rows, cols, dtype=torch.bfloat16, device=DEV), torch.zeros(rows, cols, dtype=torch.bfloat16, device=DEV)
        H, mask = fp32(H0, shift), fp32(mask0, shift)
        norm, scr = torch.empty(2, device=DEV), ops.hutch_score_scratch(DEV)
        stats = torch.zeros(8, dtype=torch.float64, device=DEV)
        wm, meta = torch.empty_like(p), torch.zeros(rows, cols // 8, dtype=torch.uint8, device=DEV)
        ops.adamw_masked_score(p, dev(g0), m, v, mask=mask, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                               decay=2e-4, step=2, hvp=dev(hvp), probe=dev(sign), beta_h=0.98, H=H, score=None, norm=norm,
                               scratch=scr, metric="hessian_obd")
        ops.mask_update_nm24_from_weight(p, H, norm, mask, stats, wm, meta, metric="hessian_obd", temperature=0.4,
                                         mask_lr=0.2, hx=0.6)
        score = torch.empty(rows, cols, device=DEV)
        ops.hutch_score(p, H, score, norm, scr, metric="hessian_obd")
        mask2, stats2 = mask.clone() if shift == 0 else fp32(mask, shift), torch.zeros(8, dtype=torch.float64, device=DEV)
        ops.mask_update_nm24(fp32(score, shift), norm, mask2, stats2, W=p, wm=wm.clone(), meta=meta.clone(),
                             temperature=0.3, mask_lr=0.2, hx=0.6, pen=0.02, penalty_mode=1)
        return [t.clone() for t in (p, m, v, H, mask, wm, meta, stats, norm, mask2, stats2)]

    for a, b in zip(run(0), run(4)):
        assert torch.equal(a, b)


# ---------------------------------------------------------------------------------------
# argument checks: bad calls are refused on the host, nothing is launched
# ---------------------------------------------------------------------------------------
def test_bad_arguments_are_refused(ops):
    with pytest.raises(RuntimeError):
        ops.project_nm24(torch.rand(8, 8))  # CPU tensor
    score = torch.zeros(8, 12, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        ops.mask_update_nm24(score, torch.zeros(2, device=DEV), torch.ones(8, 12, device=DEV),
                             torch.zeros(8, dtype=torch.float64, device=DEV))
    with pytest.raises(RuntimeError, match="multiples of 8"):
        ops.gemm_fwd(torch.zeros(8, 12, device=DEV, dtype=torch.bfloat16), torch.zeros(16, 12, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        ops.gemm_fwd(torch.zeros(8, 16, device=DEV), torch.zeros(16, 24, device=DEV))
    with pytest.raises(TypeError):
        ops.gemm_fwd(torch.zeros(8, 16, device=DEV), torch.zeros(16, 16, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        ops.project_nm24(torch.zeros(8, 8, device=DEV, dtype=torch.float16))


# ---------------------------------------------------------------------------------------
# sizes that do not fill the last 256-element warp span
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(24, 40), (3, 8), (33, 72)])
def test_ragged_sizes_against_oracle(ops, shape):
    from sparseforge_b200 import _lib

    torch.manual_seed(shape[0] * 100 + shape[1])
    rows, cols = shape
    W = torch.randn(rows, cols) * 0.02
    H0 = torch.rand(rows, cols) + 0.1
    hvp = torch.randn(rows, cols) * 0.01
    v = (torch.randint(0, 2, (rows, cols), dtype=torch.int8) * 2 - 1)
    mask0 = torch.rand(rows, cols)
    Hd = dev(H0)
    score = torch.full((rows, cols), -7.0, device=DEV)
    norm = torch.zeros(2, device=DEV)
    ops.hutch_score(dev(W), Hd, score, norm, ops.hutch_score_scratch(DEV), hvp=dev(hvp), v=dev(v), beta=0.9)
    H1 = O.hutchinson_accumulate(H0, hvp, v.float(), 0.9)
    want = O.importance_score(W, "hessian_obd", H=H1)
    assert rel_err(Hd, H1) <= F32_TOL and rel_err(score, want) <= F32_TOL
    mu, sigma = O.score_norm_stats(want)
    assert abs(float(norm[0]) - float(mu)) <= F32_TOL * abs(float(mu))
    assert abs(float(norm[1]) - float(sigma)) <= F32_TOL * abs(float(sigma))
    mask, stats, wm, meta = run_mask_update(ops, W, H1, mask0, T=0.3, mask_lr=0.25, pen=0.05, pmode=_lib.PENALTY_TOPN, hx=0.5)
    G = O.gate_target_structured(O.normalize_scores(want), 0.3)
    want_mask = O.mask_update(mask0, G, mask_lr=0.25, lambda_mid=1.0, pen_lr=0.05, penalty_mode="structured_topn")
    assert rel_err(mask, want_mask) <= F32_TOL
    assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(mask0, mask)
    st = O.mask_stats(mask)
    assert abs(float(stats[_lib.MSTAT_SUM_M]) - st["sum_m"]) <= 1e-5 * st["sum_m"]
    assert float(stats[_lib.MSTAT_COUNT_LT_HALF]) == st["count_lt_half"]
    assert torch.equal(unpack_meta(meta, cols), O.hard_mask_from_soft(mask))
    assert rel_err(wm, O.masked_weight(W, O.effective_mask(mask, 0.5))) <= F32_TOL
    p = dev(W)
    m, vv = torch.zeros_like(p), torch.zeros_like(p)
    g = torch.randn(rows, cols) * 0.1
    wm2 = torch.empty_like(p)
    ops.adamw_masked(p, dev(g), m, vv, mask=dev(mask0), lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                     decay=1e-3, step=1, wm=wm2, hx=0.25)
    wp, wm_, wv = O.adamw_step(W, g, torch.zeros(rows, cols), torch.zeros(rows, cols), step=1, lr=1e-3, betas=(0.9, 0.95),
                               eps=1e-8, weight_decay=0.1, mask=mask0, decay=1e-3)
    assert rel_err(p, wp) <= F32_TOL and rel_err(m, wm_) <= F32_TOL and rel_err(vv, wv) <= F32_TOL
    assert rel_err(wm2, O.masked_weight(wp, O.effective_mask(mask0, 0.25))) <= F32_TOL


@pytest.mark.parametrize("tag,tol", [("f32", F32_TOL), ("bf16", BF16_TOL)])
def test_wanda_metric_follows_the_reference(ops, tag, tol):
    """SparseLinear with mask_metric='wanda' against the trajectory recorded from the reference
    (tests/golden/wanda.npz): add_batch over three batches, two mask updates."""
    import sparseforge_b200 as sf

    g = Golden("wanda")
    W = g[f"{tag}_W"]
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="wanda", mask_update_period=1, sparsity_warmup_steps=0,
                                mask_lr=0.2, mask_penalty_mode="structured_topn", mask_hardening_start=2,
                                mask_hardening_duration=8)
    layer = sf.SparseLinear(W.shape[1], W.shape[0], sparselinear_config=cfg, bias=False).to(DEV).to(W.dtype)
    layer.initialize()
    layer.mask.data = layer.mask.data.float()
    layer.weight.data.copy_(W.to(DEV))
    assert tuple(layer.scaler_row.shape) == (W.shape[1],) and not layer._is_placeholder("scaler_row")
    for i in range(3):
        layer.add_batch(g[f"{tag}_x{i}"].to(DEV), None)
        assert layer.nsamples == g.scalar(f"{tag}_nsamples{i}")
        assert rel_err(layer.scaler_row.data.float(), g[f"{tag}_scaler{i}"].float()) <= (1e-2 if tag == "bf16" else 1e-5)
    # the fixture's scaler from here on, so that a last-bit difference in a bf16 sum does not move the scores
    layer.scaler_row.data.copy_(g[f"{tag}_scaler2"].to(DEV))
    layer.mask.data.copy_(g[f"{tag}_mask0"].to(DEV))
    layer.invalidate_masked_weight()
    for j, step in enumerate((3, 4)):
        assert rel_err(layer.compute_gate_target(step).float(), g[f"{tag}_G{j}"].float()) <= tol
        prev = layer.mask.data.clone().cpu()
        layer.update_mask(step, lambda_mid=0.3)
        assert rel_err(layer.mask.data, g[f"{tag}_mask{j + 1}"]) <= tol, (tag, j)
        assert layer.hardening_x == pytest.approx(g.scalar(f"{tag}_hx{j}"))
        assert int(layer.weight.flipped_mask) == O.flip_count(prev, layer.mask.data.cpu())
        if torch.equal(O.hard_mask_from_soft(layer.mask.data.cpu()), O.hard_mask_from_soft(g[f"{tag}_mask{j + 1}"])):
            assert int(layer.weight.flipped_mask) == g.scalar(f"{tag}_flips{j}")
        layer.mask.data.copy_(g[f"{tag}_mask{j + 1}"].to(DEV))
        layer.invalidate_masked_weight()


@pytest.mark.parametrize("tag,tol", [("f32", F32_TOL), ("bf16", BF16_TOL)])
def test_movement_metric_and_grad_ema_follow_the_reference(ops, tag, tol):
    """update_model_grad_ema (one fused pass: gradient EMA + g^2 into H) and the movement score against
    the reference's trajectory (tests/golden/movement.npz)."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden("movement")
    W0 = g[f"{tag}_W0"]
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="movement", N=2, M=4, mask_update_period=1,
                                sparsity_warmup_steps=0, mask_lr=0.2, beta=0.9, temperature=0.7, temp_init=1.0,
                                temp_decay=0.8, mask_hardening_start=2, mask_hardening_duration=4)
    cfg.enable_hutchinson = True
    layer = sf.SparseLinear(W0.shape[1], W0.shape[0], sparselinear_config=cfg, bias=False).to(DEV).to(W0.dtype)
    layer.weight.data.copy_(W0.to(DEV))
    layer.initialize()
    assert not layer._is_placeholder("grad_ema") and not layer._is_placeholder("hessian_diag")
    for t in range(3):
        layer.weight.grad = dev(g[f"{tag}_g{t}"])
        U.update_model_grad_ema(layer, update_hessian_with_grad2=True)
        assert rel_err(layer.grad_ema.data.float(), g[f"{tag}_ema{t}"].float()) <= tol
        assert rel_err(layer.hessian_diag.data, g[f"{tag}_H{t}"]) <= (F32_TOL if tag == "f32" else tol)
        if tag == "f32":
            assert torch.equal(layer.grad_ema.data.cpu(), g[f"{tag}_ema{t}"])  # same roundings as ATen
        layer.grad_ema.data.copy_(g[f"{tag}_ema{t}"].to(DEV))
        layer.weight.data.copy_(g[f"{tag}_W{t + 1}"].to(DEV))
        layer.invalidate_masked_weight()
        assert rel_err(layer.compute_gate_target(t).float(), g[f"{tag}_G{t}"].float()) <= tol
        prev = layer.mask.data.clone().cpu()
        U.calculate_model_mask(layer, step=t, lambda_mid=0.0)
        assert rel_err(layer.mask.data, g[f"{tag}_mask{t + 1}"]) <= tol
        assert layer.hardening_x == pytest.approx(g.scalar(f"{tag}_hx{t}"))
        assert int(layer.weight.flipped_mask) == O.flip_count(prev, layer.mask.data.cpu())
        layer.mask.data.copy_(g[f"{tag}_mask{t + 1}"].to(DEV))
        layer.invalidate_masked_weight()
    # a layer without a Hessian tensor only keeps the gradient EMA; other metrics return early
    plain = sf.SparseLinear(64, 48, sparselinear_config=sf.SparseLinearConfig(mask_metric="movement"), bias=False).to(DEV)
    plain.weight.grad = torch.ones_like(plain.weight)
    plain.update_grad_hessian_ema()
    assert float(plain.grad_ema.data.min()) == pytest.approx(0.01)
    obd = sf.SparseLinear(64, 48, sparselinear_config=sf.SparseLinearConfig(mask_metric="hessian_obd"), bias=False).to(DEV)
    obd.initialize()
    obd.weight.grad = torch.ones_like(obd.weight)
    obd.update_grad_hessian_ema()
    assert float(obd.hessian_diag.data.min()) == 1.0  # the reference's early return: H keeps its initial value


def test_wanda_kernels_at_layer_size(ops):
    """Column energy and score at a LLaMA-sized matrix against torch on the device (fp32 sums in
    another order: 1e-5), bf16 activations and weights."""
    torch.manual_seed(31)
    T, out_f, in_f = 4096, 1024, 11008
    x = torch.randn(T, in_f, device=DEV).to(torch.bfloat16)
    scaler = torch.rand(in_f, device=DEV)
    want = scaler * 0.25 + (x.float() ** 2).sum(0) / 7.0
    ops.wanda_add_batch(x, scaler, 0.25, 7.0)
    assert rel_err(scaler, want) <= 1e-5
    W = (torch.randn(out_f, in_f, device=DEV) * 0.02).to(torch.bfloat16)
    score = torch.empty(out_f, in_f, device=DEV)
    norm = torch.empty(2, device=DEV)
    scratch = ops.hutch_score_scratch(DEV)
    ops.wanda_score(W, scaler, score, norm, scratch)
    ref = W.abs().float() * torch.sqrt(scaler.reshape(1, -1) + 1e-8)
    assert rel_err(score, ref) <= 1e-6
    assert float(norm[0]) == pytest.approx(float(ref.mean()), rel=1e-5)
    assert float(norm[1]) == pytest.approx(float(ref.std(unbiased=False)) + 1e-6, rel=1e-4)


def test_freeze_bands_follow_the_reference(ops):
    """SparseLinear with freeze_low / freeze_high against the trajectory recorded from the reference
    (tests/golden/freeze.npz): six updates across step 2000, then harden_fraction over two layers.
    Entries whose pre-snap value lies within 1e-5 of a band edge may snap differently (the kernel's
    sigmoid is not ATen's to the last bit) and are left out of the comparison."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden("freeze")
    W = g["W"]
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", mask_update_period=1,
                                sparsity_warmup_steps=0, mask_lr=0.3, mask_penalty_mode="structured_topn",
                                mask_hardening_start=2, mask_hardening_duration=8, temp_init=0.3, temp_min=0.3,
                                freeze_low=0.08, freeze_high=0.93)
    layer = sf.SparseLinear(W.shape[1], W.shape[0], sparselinear_config=cfg, bias=False).to(DEV)
    layer.initialize()
    assert tuple(layer.frozen_mask_flags.shape) == tuple(W.shape) and not layer._is_placeholder("frozen_mask_flags")
    layer.weight.data.copy_(W.to(DEV))
    layer.hessian_diag.data.copy_(g["H"].to(DEV))
    layer.mask.data.copy_(g["mask0"].to(DEV))
    layer.invalidate_masked_weight()
    prev = g["mask0"]
    for j, step in enumerate(int(s) for s in g["steps"]):
        assert layer._temperature(step) == pytest.approx(g.scalar(f"s{j}_T"), rel=1e-12)
        assert rel_err(layer.compute_gate_target(step), g[f"s{j}_G"]) <= F32_TOL
        layer.update_mask(step, lambda_mid=0.4)
        pre = O.mask_update(prev, g[f"s{j}_G"], mask_lr=0.3, lambda_mid=0.4, pen_lr=0.3, penalty_mode="structured_topn")
        sure = ((pre - 0.08).abs() > 1e-5) & ((pre - 0.93).abs() > 1e-5)
        assert int((~sure).sum()) <= 4
        got, flags = layer.mask.data.cpu(), layer.frozen_mask_flags.data.cpu()
        assert rel_err(got[sure], g[f"s{j}_mask"][sure]) <= F32_TOL, j
        assert torch.equal(flags[sure], g[f"s{j}_flags"][sure]), j
        assert layer.hardening_x == pytest.approx(g.scalar(f"s{j}_hx"))
        assert int(layer.weight.flipped_mask) == O.flip_count(prev, got)
        # masked weight and metadata were formed from the snapped mask
        hx = layer.hardening_x
        want_wm = O.masked_weight(W, O.effective_mask(got, hx))
        assert rel_err(layer._wm.cpu(), want_wm) <= F32_TOL
        assert torch.equal(unpack_meta(layer._meta, W.shape[1]), O.hard_mask_from_soft(got))
        prev = g[f"s{j}_mask"]
        layer.mask.data.copy_(prev.to(DEV))
        layer.frozen_mask_flags.data.copy_(g[f"s{j}_flags"].to(DEV))
        layer.invalidate_masked_weight()
    other = sf.SparseLinear(32, 16, sparselinear_config=sf.SparseLinearConfig(
        mask_type="structured", mask_metric="hessian_obd", freeze_low=0.08, freeze_high=0.93), bias=False).to(DEV)
    layer.mask.data.copy_(g["hf_mask_a0"].to(DEV)); layer.frozen_mask_flags.data.copy_(g["hf_flags_a0"].to(DEV))
    other.mask.data.copy_(g["hf_mask_b0"].to(DEV)); other.frozen_mask_flags.data.copy_(g["hf_flags_b0"].to(DEV))
    n = U.harden_fraction(torch.nn.Sequential(layer, other), fraction=0.3, band_low=0.35, band_high=0.7)
    assert n == g.scalar("hf_count")
    assert torch.equal(layer.mask.data.cpu(), g["hf_mask_a1"]) and torch.equal(other.mask.data.cpu(), g["hf_mask_b1"])
    assert torch.equal(layer.frozen_mask_flags.data.cpu(), g["hf_flags_a1"])
    assert torch.equal(other.frozen_mask_flags.data.cpu(), g["hf_flags_b1"])
