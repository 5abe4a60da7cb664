"""GPU parity of the masked GEMMs (tcgen05 bf16 path and fp32 FMA path) and of the module-level
chain against the reference-generated fixtures. The reference for a GEMM is the fp32 product of the
same (already rounded) inputs; tolerance 1e-2 for bf16 results, 1e-5 for fp32, relative to the
largest reference magnitude."""
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


def ref_products(x, w, dy):
    """fp64 products of the given tensors, computed on the GPU by torch (the checker only)."""
    xd, wd, dyd = x.double(), w.double(), dy.double()
    return xd @ wd.t(), dyd @ wd, dyd.t() @ xd


def check_status(status):
    assert int(status[0]) == 0, f"a device-side wait ran out, code {int(status[0])}"


# ragged sizes exercise partial tiles in M, N and K; the last rows are LLaMA-2-7B layer shapes
BF16_SHAPES = [
    (128, 64, 256),
    (8, 8, 8),
    (136, 72, 264),
    (1000, 200, 520),
    (256, 4096, 512),
    (2048, 1024, 1280),
    (8192, 4096, 4096),
    (8192, 4096, 11008),
    (8192, 11008, 4096),
]


@pytest.mark.parametrize("T,k,n", BF16_SHAPES)
def test_bf16_products(ops, T, k, n):
    torch.manual_seed(T + k + n)
    x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.02).to(torch.bfloat16)
    dy = torch.randn(T, n, device=DEV).to(torch.bfloat16)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    y = ops.gemm_fwd(x, w, status=status)
    dx = ops.gemm_dgrad(dy, w, status=status)
    dw = ops.gemm_wgrad(dy, x, status=status)
    torch.cuda.synchronize()
    check_status(status)
    if T * k * n <= 2048 * 1024 * 1280:
        ry, rdx, rdw = ref_products(x, w, dy)
    else:
        ry, rdx, rdw = (x.float() @ w.float().t()), (dy.float() @ w.float()), (dy.float().t() @ x.float())
    assert rel_err(y, ry) <= BF16_TOL
    assert rel_err(dx, rdx) <= BF16_TOL
    assert rel_err(dw, rdw) <= BF16_TOL


@pytest.mark.parametrize("T,k,n", [(8192, 4096, 512), (2048, 1024, 2048), (1024, 4096, 520), (1000, 264, 1064)])
def test_bf16_products_under_a_cta_limit(ops, T, k, n):
    """A stream limited to a part of the SMs (`sf_masked_gemm_configure_stream`, what lets two products
    share the GPU) gives, bit for bit, the products of an unlimited launch: every output tile is computed
    by one CTA pair with the same K order, whoever gets it."""
    torch.manual_seed(T + k + n + 1)
    bf = torch.bfloat16
    x = torch.randn(T, k, device=DEV).to(bf)
    w = (torch.randn(n, k, device=DEV) * 0.02).to(bf)
    dy = torch.randn(T, n, device=DEV).to(bf)
    b = torch.randn(n, device=DEV).to(bf)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)

    def run():
        return (ops.gemm_fwd(x, w, bias=b, alpha=0.75, status=status), ops.gemm_dgrad(dy, w, status=status),
                ops.gemm_wgrad(dy, x, status=status))

    try:
        full = run()
        ops.gemm_configure_stream(max_ctas=2)
        one_pair = run()
        ops.gemm_configure_stream(max_ctas=46)
        some = run()
    finally:
        ops.gemm_configure_stream(max_ctas=0)
    torch.cuda.synchronize()
    check_status(status)
    want = (0.75 * (x.float() @ w.float().t()) + b.float(), dy.float() @ w.float(), dy.float().t() @ x.float())
    for got, a, c, ref in zip(full, one_pair, some, want):
        assert rel_err(got, ref) <= BF16_TOL
        assert torch.equal(got, a) and torch.equal(got, c)


def test_bf16_bias_and_scale(ops):
    torch.manual_seed(0)
    x = torch.randn(200, 128, device=DEV).to(torch.bfloat16)
    w = (torch.randn(320, 128, device=DEV) * 0.05).to(torch.bfloat16)
    b = torch.randn(320, device=DEV).to(torch.bfloat16)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    y = ops.gemm_fwd(x, w, bias=b, alpha=1.5, status=status)
    check_status(status)
    assert rel_err(y, 1.5 * (x.double() @ w.double().t()) + b.double()) <= BF16_TOL


@pytest.mark.parametrize("T,k,n,r,bias", [(384, 256, 512, 64, True), (1024, 4096, 4096, 64, False), (1000, 264, 1064, 40, True),
                                          (8192, 4096, 11008, 256, False), (136, 64, 48, 8, True)])
def test_forward_with_a_low_rank_pair(ops, T, k, n, r, bias):
    """y = x wm^T + z sw^T (+ bias) in one launch: the second operand pair's K blocks run on in the same
    accumulator (a rank that is not a multiple of the 64-deep K block is zero-filled)."""
    torch.manual_seed(T + r)
    x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    wm = (torch.randn(n, k, device=DEV) * 0.02).to(torch.bfloat16)
    z = torch.randn(T, r, device=DEV).to(torch.bfloat16)
    sw = (torch.randn(n, r, device=DEV) * 0.05).to(torch.bfloat16)
    b = torch.randn(n, device=DEV).to(torch.bfloat16) if bias else None
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    y = ops.gemm_fwd_lowrank(x, wm, z, sw, b, status=status)
    assert int(status[0]) == 0
    want = x.float() @ wm.float().t() + z.float() @ sw.float().t()
    if bias:
        want = want + b.float()
    assert rel_err(y.float(), want) <= BF16_TOL
    # the second pair matters in this case, and leaving it out is seen
    assert rel_err(ops.gemm_fwd(x, wm, b).float(), want) > BF16_TOL


def test_low_rank_pair_refuses_what_it_cannot_do(ops):
    x = torch.randn(64, 64, device=DEV).to(torch.bfloat16)
    wm = torch.randn(32, 64, device=DEV).to(torch.bfloat16)
    z = torch.randn(64, 16, device=DEV).to(torch.bfloat16)
    sw = torch.randn(32, 16, device=DEV).to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.gemm_fwd_lowrank(x, wm, z, sw)  # 64 rows: below the CTA-pair kernel's range
    xb = torch.randn(256, 64, device=DEV).to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.gemm_fwd_lowrank(xb, wm, torch.randn(256, 12, device=DEV).to(torch.bfloat16),
                             torch.randn(32, 12, device=DEV).to(torch.bfloat16))  # rank not a multiple of 8
    with pytest.raises(RuntimeError):
        ops.gemm_fwd_lowrank(xb.float(), wm.float(), torch.randn(256, 16, device=DEV), torch.randn(32, 16, device=DEV))


def test_bf16_linearity_at_full_size(ops):
    """A size-independent property at the LLaMA gate/up shape: products are linear in x."""
    torch.manual_seed(1)
    T, k, n = 8192, 4096, 11008
    x1 = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.02).to(torch.bfloat16)
    y1 = ops.gemm_fwd(x1, w).float()
    y2 = ops.gemm_fwd((x1.float() * 2).to(torch.bfloat16), w).float()  # exact doubling in bf16
    assert rel_err(y2, 2 * y1) <= BF16_TOL
    # row permutation of x permutes rows of y exactly
    perm = torch.randperm(T, device=DEV)
    yp = ops.gemm_fwd(x1[perm].contiguous(), w)
    assert torch.equal(yp.float(), y1[perm])


@pytest.mark.parametrize("T,k,n", [(40, 64, 96), (100, 72, 50), (8192, 768, 3072)])
def test_f32_products(ops, T, k, n):
    torch.manual_seed(T)
    x = torch.randn(T, k, device=DEV)
    w = torch.randn(n, k, device=DEV) * 0.02
    dy = torch.randn(T, n, device=DEV)
    ry, rdx, rdw = ref_products(x, w, dy)
    assert rel_err(ops.gemm_fwd(x, w), ry) <= F32_TOL
    assert rel_err(ops.gemm_dgrad(dy, w), rdx) <= F32_TOL
    assert rel_err(ops.gemm_wgrad(dy, x), rdw) <= F32_TOL


def test_bias_grad(ops):
    torch.manual_seed(3)
    for dtype, tol in ((torch.float32, F32_TOL), (torch.bfloat16, 1e-4)):
        dy = torch.randn(1000, 328, device=DEV).to(dtype)
        assert rel_err(ops.bias_grad(dy), dy.double().sum(0)) <= tol


# ---------------------------------------------------------------------------------------
# module-level chain against the reference run (same sequence as tests/golden/make_golden.py)
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("case,dtype,tol,steps_cfg", [
    ("chain_f32", torch.float32, F32_TOL, dict(temp_init=1.0, mask_hardening_start=1000, mask_hardening_duration=10000)),
    ("chain_bf16", torch.bfloat16, BF16_TOL, dict(temp_init=1.0, temp_min=0.05, temp_decay=0.05 ** (1.0 / 9.0),
                                                   mask_hardening_start=1, mask_hardening_duration=3,
                                                   mask_penalty_mode="structured_topn")),
])
def test_sparse_linear_chain(case, dtype, tol, steps_cfg):
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden(case)
    W0, X, dY = g["W0"], g["X"].to(DEV), g["dY"].to(DEV)
    out_f, in_f = W0.shape
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, mask_update_period=1,
                                sparsity_warmup_steps=0, mask_lr=0.1, beta=0.99, **steps_cfg)
    layer = sf.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False).to(DEV).to(dtype)
    layer.mask.data = layer.mask.data.float()
    layer.hessian_diag.data = layer.hessian_diag.data.float()
    layer.weight.data.copy_(W0.to(DEV))
    layer.initialize()
    opt = sf.AdamW([layer.weight], lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
    lam = g.scalar("lambda_mid")
    T = X.shape[0] * X.shape[1]
    probe = 0
    # Float outputs are compared at the tolerance; whatever the next stage consumes is then reset
    # to the reference's value so that each step checks one stage at a time.
    for t in range(g.scalar("n_steps")):
        assert layer.hardening_x == pytest.approx(g.scalar(f"s{t}_hx_fwd"))
        Xr = X.clone().requires_grad_(True)
        layer.weight.grad = None
        Y = layer(Xr)
        Y.backward(dY)
        assert rel_err(Y.float(), g[f"s{t}_Y"].float()) <= tol
        assert rel_err(Xr.grad.float(), g[f"s{t}_dX"].float()) <= tol
        assert rel_err(layer.weight.grad.float(), g[f"s{t}_dW"].float()) <= tol
        while probe < g.scalar(f"s{t}_probes_end"):
            v = g[f"v_{probe}"].to(DEV).to(dtype)
            U._rademacher_like = lambda tt, v=v: v.clone()
            loss = (torch.nn.functional.gelu(layer(X).float()) * dY.float()).sum() / T
            U.update_hessian_hutchinson(layer, loss)
            # hvp comes out of second-order products of bf16/fp32 GEMMs: compare H, which the
            # reference forms from it
            assert rel_err(layer.hessian_diag.data, g[f"H_{probe}"]) <= (1e-4 if dtype == torch.float32 else tol)
            layer.hessian_diag.data.copy_(g[f"H_{probe}"].to(DEV))
            probe += 1
        layer.weight.grad = g[f"s{t}_dW"].to(DEV)
        opt.step(decay=2e-4)
        st = opt.state[layer.weight]
        assert rel_err(layer.weight.data.float(), g[f"s{t}_W_opt"].float()) <= tol
        assert rel_err(st["exp_avg"].float(), g[f"s{t}_m"].float()) <= tol
        assert rel_err(st["exp_avg_sq"].float(), g[f"s{t}_v"].float()) <= tol
        layer.weight.data.copy_(g[f"s{t}_W_opt"].to(DEV))
        layer.invalidate_masked_weight()  # a .data edit: the score left by the optimizer pass is stale
        st["exp_avg"].copy_(g[f"s{t}_m"].to(DEV)); st["exp_avg_sq"].copy_(g[f"s{t}_v"].to(DEV))
        assert layer._temperature(t) == pytest.approx(g.scalar(f"s{t}_T"), rel=1e-12)
        G = layer.compute_gate_target(t)
        assert rel_err(G, g[f"s{t}_G"]) <= F32_TOL
        prev = layer.mask.data.clone()
        U.calculate_model_mask(layer, step=t, lambda_mid=lam)
        assert rel_err(layer.mask.data, g[f"s{t}_mask"]) <= F32_TOL
        assert layer.hardening_x == pytest.approx(g.scalar(f"s{t}_hx"))
        assert int(layer.weight.flipped_mask) == O.flip_count(prev.cpu(), layer.mask.data.cpu())
        layer.mask.data.copy_(g[f"s{t}_mask"].to(DEV))
        layer.invalidate_masked_weight()
        hard = layer._hard_mask_from_soft(layer.mask.data)
        assert torch.equal(hard.cpu(), g[f"s{t}_hard"])
        pen = U.mid_penalty(layer, 1.0)
        assert float(pen) * layer.mask.numel() == pytest.approx(g.scalar(f"s{t}_mid_sum"), rel=1e-5)
    flipped, ratio, _, _ = U.calculate_flip_rate(layer)
    assert 0 <= ratio <= 1
    _, cur = U.sparsity_penalty(layer, 0.5, 1.0)
    assert cur == pytest.approx(0.5)
    stats = U.nm_2_4_tile_stats(layer)
    want = O.mask_stats(layer.mask.data.cpu())
    assert stats["top2_avg"] == pytest.approx(want["sum_top2"] / (layer.mask.numel() / 2), rel=1e-5)


def test_gemm_from_a_fresh_thread(ops):
    """The tensor-core GEMM is callable as the first CUDA action of a new host thread (autograd runs
    backward passes on such threads)."""
    import threading

    x = torch.randn(64, 64, device=DEV).to(torch.bfloat16)
    w = torch.randn(64, 64, device=DEV).to(torch.bfloat16)
    out = {}

    def run():
        try:
            out["y"] = ops.gemm_dgrad(x, w)
            torch.cuda.synchronize()
        except Exception as e:  # surfaced below
            out["err"] = e

    t = threading.Thread(target=run)
    t.start()
    t.join()
    assert "err" not in out, out.get("err")
    assert rel_err(out["y"], x.float() @ w.float()) <= BF16_TOL


def test_paper_recipe_mask_path():
    """The launcher's default recipe (unstructured gate from a sampled quantile, nm_2_4 projection and
    penalty, |W|/sqrt(H) score) against the reference run: every stage is fed the reference's inputs."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden("chain_paper")
    W0 = g["W0"]
    out_f, in_f = W0.shape
    cfg = sf.SparseLinearConfig(mask_type="unstructured", hard_mask_type="nm_2_4", mask_metric="hessian_ratio", N=2, M=4,
                                mask_update_period=1, sparsity_warmup_steps=0, mask_lr=0.1, beta=0.98, temp_init=1.0,
                                temp_min=0.05, temp_decay=0.5, mask_hardening_start=1, mask_hardening_duration=2,
                                mask_penalty_lr=0.1, mask_penalty_mode="nm_2_4", tau_sample_size=1024, sparsity_ratio=0.5)
    layer = sf.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False).to(DEV).to(torch.bfloat16)
    layer.initialize()
    lam = g.scalar("lambda_mid")
    X, dY = g["X"].to(DEV), g["dY"].to(DEV)
    for t in range(g.scalar("n_steps")):
        # forward / backward with the reference's weight, mask and hardening state
        layer.weight.data.copy_(g[f"s{t}_W_fwd"].to(DEV))
        layer.mask.data.copy_(g[f"s{t}_mask_fwd"].to(DEV))
        layer.hardening_x = g.scalar(f"s{t}_hx_fwd")
        layer.invalidate_masked_weight()
        Xr = X.clone().requires_grad_(True)
        layer.weight.grad = None
        Y = layer(Xr)
        Y.backward(dY)
        assert rel_err(Y.float(), g[f"s{t}_Y"].float()) <= BF16_TOL
        assert rel_err(Xr.grad.float(), g[f"s{t}_dX"].float()) <= BF16_TOL
        assert rel_err(layer.weight.grad.float(), g[f"s{t}_dW"].float()) <= BF16_TOL
        # mask update from the reference's post-optimizer weight and Hessian
        layer.weight.data.copy_(g[f"s{t}_W_opt"].to(DEV))
        layer.hessian_diag.data.copy_(g[f"H_{g.scalar(f's{t}_probes_end') - 1}"].to(DEV))
        layer._tau_sample_idx = g[f"s{t}_tau_idx"].to(DEV)
        assert layer._temperature(t) == pytest.approx(g.scalar(f"s{t}_T"), rel=1e-12)
        G = layer.compute_gate_target(t)
        assert rel_err(G, g[f"s{t}_G"]) <= F32_TOL
        prev = layer.mask.data.clone()
        U.calculate_model_mask(layer, step=t, lambda_mid=lam)
        assert rel_err(layer.mask.data, g[f"s{t}_mask"]) <= F32_TOL
        assert layer.hardening_x == pytest.approx(g.scalar(f"s{t}_hx"))
        assert int(layer.weight.flipped_mask) == O.flip_count(prev.cpu(), layer.mask.data.cpu(), "nm_2_4")
        layer.mask.data.copy_(g[f"s{t}_mask"].to(DEV))
        assert torch.equal(layer._hard_mask_from_soft(layer.mask.data).cpu(), g[f"s{t}_hard"])


@pytest.mark.parametrize("T,in_f,out_local,G", [(512, 192, 256, 2), (1024, 328, 136, 4), (2048, 264, 136, 4), (768, 64, 136, 2),
                                                 (4096, 256, 1376, 8), (1024, 4096, 512, 2), (1024, 512, 4096, 2)])
def test_sharded_epilogues_on_one_gpu(ops, T, in_f, out_local, G):
    """The all-gather and reduce-scatter epilogues with every "rank" played in turn on one GPU: the
    destinations are ordinary buffers of this GPU, so only the addressing is under test."""
    torch.manual_seed(T + G)
    bf = torch.bfloat16
    out_total = out_local * G
    x = torch.randn(T, in_f, device=DEV).to(bf)
    wms = [(torch.randn(out_local, in_f, device=DEV) * 0.05).to(bf) for _ in range(G)]
    dys = [torch.randn(T, out_local, device=DEV).to(bf) for _ in range(G)]
    bias = [(torch.randn(out_local, device=DEV) * 0.1).to(bf) for _ in range(G)]
    status = torch.zeros(4, dtype=torch.int32, device=DEV)

    # output all-gather: every rank's full output buffer ends up with all column blocks
    y_all = [torch.full((T, out_total), float("nan"), device=DEV, dtype=bf) for _ in range(G)]
    for r in range(G):
        ops.gemm_fwd_allgather(x, wms[r], [y.data_ptr() for y in y_all], out_total, r * out_local, bias=bias[r],
                               alpha=0.5, status=status)
    want = torch.cat([ops.gemm_fwd(x, wms[r], bias[r], alpha=0.5) for r in range(G)], dim=1)
    for y in y_all:
        assert torch.equal(y, want)

    # input-gradient reduce-scatter: slots[c][r] is rank c's slot for rank r's partial sums
    rows = T // G
    slots = [torch.full((G, rows, in_f), float("nan"), device=DEV, dtype=bf) for _ in range(G)]
    for r in range(G):
        ops.gemm_dgrad_reducescatter(dys[r], wms[r], [slots[c][r].data_ptr() for c in range(G)], r, status=status)
    partial = [ops.gemm_dgrad(dys[r], wms[r]) for r in range(G)]
    for c in range(G):
        for r in range(G):
            assert torch.equal(slots[c][r], partial[r][c * rows:(c + 1) * rows])
        got = ops.reduce_slots(slots[c])
        ref = sum(p[c * rows:(c + 1) * rows].float() for p in partial)
        assert rel_err(got.float(), ref) <= 1e-2
    assert int(status[0]) == 0
    with pytest.raises(RuntimeError):
        ops.gemm_fwd_allgather(x[:64], wms[0], [y_all[0].data_ptr()], out_total, 0)  # too few rows for the pair kernel
    with pytest.raises(RuntimeError):
        ops.gemm_fwd_allgather(x, wms[0], [y_all[0].data_ptr()], out_total, out_total)  # columns out of range


def test_a_wait_that_runs_out_reports_and_returns(ops):
    """The bounded wait of the pipeline roles, on a barrier nobody arrives at: the kernel returns,
    the status word holds the code, and the next product on the same context is correct."""
    from sparseforge_b200 import _lib

    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _lib.check(_lib.lib().sf_selftest_bounded_wait(5.0, status.data_ptr(), torch.cuda.current_stream().cuda_stream),
               "sf_selftest_bounded_wait")
    torch.cuda.synchronize()
    assert int(status[0]) == 99
    x = torch.randn(256, 64, device=DEV).to(torch.bfloat16)
    w = torch.randn(128, 64, device=DEV).to(torch.bfloat16)
    assert rel_err(ops.gemm_fwd(x, w).float(), x.float() @ w.float().t()) <= 1e-2


def test_mma_issue_rate_probe(ops):
    """The probe behind the block-sparse-16 design: the cost of one 128 x N x 16 MMA does not fall below a
    floor of a few dozen cycles, so sixteen-wide MMAs (one per 16 x 16 weight block) run far below the
    rate of the 128- and 256-wide ones. Sanity bounds only; the figures are in profiles/."""
    c16, c64, c128, c256 = (ops.mma_issue_cycles(n) for n in (16, 64, 128, 256))
    assert 100 <= c256 <= 400        # 128 cycles at the full rate of 8192 FLOP per clock and SM
    assert c128 <= 0.75 * c256
    assert c16 >= 0.5 * c64          # narrowing below 64 columns buys (almost) nothing
    t16 = ops.mma_issue_cycles(16, a_from_tmem=True)
    assert t16 >= 0.5 * c64

