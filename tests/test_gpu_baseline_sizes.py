"""Parity at the benchmark's own sizes (the small cases elsewhere cannot reach: grids of one resident
wave with many spans per thread, 32-byte vector accesses, fp64 partial sums over thousands of blocks).

* the fp32 GPT-2-small MLP case, end to end through ``SparseLinear``, against the oracle run on the
  CPU at test time and against the reference's recorded run (tests/golden/c1.npz);
* the bf16 LLaMA-2-7B q-projection matrix [4096, 4096]: two consecutive steps of the exact pair of
  passes the benchmark times, against the oracle's chain in the reference's order.

Bars. Integer outputs (hard masks, 2:4 metadata, flip counts) are exact functions of the soft mask:
they are compared bit for bit on the same soft mask, and where the soft masks themselves differ in
the last bits the number of differing hard entries is printed and must stay inside the groups whose
2nd / 3rd soft values are closer than the float tolerance. Floats: every entry within
rtol |reference| + atol with rtol 1e-5 (fp32) / 1e-2 (bf16). atol is stated at each check as a fraction
of the tensor's RMS: next to nothing for fp32 element-wise results, 1e-5 of the RMS for fp32 GEMM
outputs (sums with cancellation), and 1e-2 of the RMS for tensors STORED in bf16, whose entries come
out of a sum of two rounded terms (ATen rounds beta * m and the decayed gradient to bf16 before adding
them; an entry where the two nearly cancel carries the rounding of the larger term).
"""
import numpy as np
import pytest
import torch

from oracle import sparselinear_oracle as O
from tests import baseline_cases as B
from tests.golden_io import Golden, rel_err

pytestmark = pytest.mark.gpu

DEV = "cuda"
F32, BF16 = 1e-5, 1e-2


def unpack_meta(meta, cols):
    meta = meta.cpu()
    rows = meta.shape[0]
    nib = torch.stack([meta & 0xF, meta >> 4], dim=-1).view(rows, -1)[:, : cols // 4].long()
    out = torch.zeros(rows, cols // 4, 4)
    out.scatter_(-1, (nib & 3).unsqueeze(-1), 1.0)
    out.scatter_(-1, (nib >> 2).unsqueeze(-1), 1.0)
    return out.view(rows, cols)


def report_hard(tag, hard_gpu, hard_ref, soft_ref, rtol, atol=0.0):
    """Prints and bounds the hard-mask disagreement between two chains whose soft masks agree to rtol."""
    diff, groups = B.hard_mismatch(hard_gpu, hard_ref)
    ties = B.near_tie_groups(soft_ref, rtol, atol)
    print(f"[parity] {tag}: {diff} of {hard_ref.numel()} hard-mask entries differ from the oracle's; "
          f"{int(ties.sum())} of {ties.numel()} groups hold a 2nd/3rd near-tie at rtol {rtol:g}")
    assert int((groups & ~ties).sum()) == 0, f"{tag}: a hard-mask group differs outside the near-ties"
    assert diff <= 2 * int(ties.sum())
    return diff


# ---------------------------------------------------------------------------------------------
# fp32 GPT-2-small MLP case, whole chain
# ---------------------------------------------------------------------------------------------
def test_c1_whole_chain_fp32():
    import sparseforge_b200 as sf
    from sparseforge_b200 import ops
    from sparseforge_b200 import utils as U

    g = Golden("c1")
    W, X, dY = B.c1_inputs()
    for name, t in (("W", W), ("X", X), ("dY", dY)):
        assert torch.allclose(B.fingerprint(t), g[f"fp_{name}"], rtol=1e-12, atol=0), f"seeded input {name} differs"
    want = B.c1_oracle(W, X, dY)
    out_f, in_f = W.shape
    T = X.shape[0] * X.shape[1]
    rows_w, rows_y, rows_x = g["rows_w"], g["rows_y"], g["rows_x"]

    def check(name, got, ref_full, rows, rtol, atol_scale):
        """Against the oracle on every entry and against the reference's recorded rows."""
        got2 = got.detach().reshape(-1, got.shape[-1]).cpu()
        ref2 = ref_full.reshape(-1, ref_full.shape[-1])
        atol = atol_scale * B.rms(ref2)
        B.assert_elementwise(got2, ref2, rtol, atol, name + " vs oracle")
        B.assert_elementwise(got2[rows], g[f"{name}_rows"], rtol, atol, name + " vs reference fixture")

    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, temp_init=1.0,
                                mask_update_period=1, sparsity_warmup_steps=0)
    layer = sf.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False).to(DEV)
    layer.weight.data.copy_(W.to(DEV))
    layer.initialize()
    Xd, dYd = X.to(DEV), dY.to(DEV)

    # four Hutchinson probes through the real double backward (three GEMM-shaped second-order products
    # per probe on the fp32 kernels): H within 1e-4 of the host BLAS result, entry by entry
    for i in range(4):
        v = B.c1_probe(i, W.shape).to(DEV)
        if i == 0:
            # the Hessian-vector product itself (it only moves H by a thousandth, so H alone says little)
            loss = (torch.nn.functional.gelu(layer(Xd).float()) * dYd).sum() / T
            (g1,) = torch.autograd.grad(loss, [layer.weight], create_graph=True)
            (hvp,) = torch.autograd.grad((g1 * v).sum(), [layer.weight])
            check("hvp_0", hvp, want["hvp"][0], rows_w, 1e-4, 1e-4)
            del g1, hvp, loss
        U._rademacher_like = lambda tt, v=v: v.clone()
        loss = (torch.nn.functional.gelu(layer(Xd).float()) * dYd).sum() / T
        U.update_hessian_hutchinson(layer, loss)
        check(f"H_{i}", layer.hessian_diag.data, want["H"][i], rows_w, 1e-4, 1e-6)
    # from here on every stage starts from the oracle's H, so that each is checked on the same input
    layer.hessian_diag.data.copy_(want["H"][3].to(DEV))
    layer.invalidate_masked_weight()
    score = torch.empty(out_f, in_f, device=DEV)
    norm = torch.zeros(2, device=DEV)
    ops.hutch_score(layer.weight.data, layer.hessian_diag.data, score, norm, ops.hutch_score_scratch(DEV))
    check("score_raw", score, want["score_raw"], rows_w, F32, 1e-9)
    assert torch.allclose(norm.cpu(), want["score_mean_std"], rtol=F32, atol=0)
    assert torch.allclose(norm.cpu(), g["score_mean_std"], rtol=F32, atol=0)
    check("G", layer.compute_gate_target(0), want["G"], rows_w, F32, 1e-7)
    prev = layer.mask.data.clone()
    U.calculate_model_mask(layer, step=0, lambda_mid=0.0)
    check("mask", layer.mask.data, want["mask"], rows_w, F32, 1e-7)
    mask_gpu = layer.mask.data.cpu()
    assert int(layer.weight.flipped_mask) == O.flip_count(prev.cpu(), mask_gpu)

    # mask indices: bit-exact on the same soft mask (the oracle's and the kernel's own) ...
    ref_hard = torch.from_numpy(np.unpackbits(g["hard_bits"].numpy(), axis=1)[:, :in_f].astype(np.float32))
    hard_of_oracle_mask, meta = ops.project_nm24(want["mask"].to(DEV), want_meta=True)
    assert torch.equal(hard_of_oracle_mask.cpu(), want["hard"])
    assert torch.equal(meta.cpu(), O.meta_from_hard(want["hard"]))
    hard_gpu = layer._hard_mask_from_soft(layer.mask.data).cpu()
    assert torch.equal(hard_gpu, O.hard_mask_from_soft(mask_gpu))
    assert torch.equal(unpack_meta(layer.metadata(), in_f), hard_gpu)
    # ... and between the two chains only inside near-ties of the soft mask (count printed)
    report_hard("fp32 MLP case, kernel chain vs oracle", hard_gpu, want["hard"], want["mask"], F32)
    report_hard("fp32 MLP case, kernel chain vs reference fixture", hard_gpu, ref_hard, want["mask"], F32)
    if torch.equal(hard_gpu, ref_hard):
        assert int(layer.weight.flipped_mask) == g.scalar("flips")

    # masked forward / backward with the hard mask (hardening_x = 0) on the oracle's soft mask
    layer.mask.data.copy_(want["mask"].to(DEV))
    layer.hardening_x = 0.0
    layer.invalidate_masked_weight()
    Xr = Xd.clone().requires_grad_(True)
    layer.weight.grad = None
    Y = layer(Xr)
    Y.backward(dYd)
    check("Y", Y, want["Y"], rows_y, F32, 1e-5)
    check("dX", Xr.grad, want["dX"], rows_x, F32, 1e-5)
    check("dW", layer.weight.grad, want["dW"], rows_w, F32, 1e-5)


# ---------------------------------------------------------------------------------------------
# bf16 LLaMA-2-7B q-projection: the optimizer + score pass and the mask update the benchmark times
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shift", [0, 4], ids=["mask_H_32B_aligned", "mask_H_16B_aligned"])
def test_c2_bench_pair_two_steps(shift):
    from sparseforge_b200 import _lib, ops

    rows = cols = 4096
    hp = B.C2_HYPER
    st = B.c2_state(rows, cols)
    dev = lambda t: t.to(DEV).contiguous()  # noqa: E731
    W, m, v = dev(st["W"]), dev(st["m"]), dev(st["v"])
    H, mask = B.fp32_at_offset(st["H"], shift, DEV), B.fp32_at_offset(st["mask"], shift, DEV)
    norm, scratch = torch.zeros(2, device=DEV), ops.hutch_score_scratch(DEV)
    stats = torch.zeros(8, dtype=torch.float64, device=DEV)
    wm = torch.empty_like(W)
    meta = torch.zeros(rows, cols // 8, dtype=torch.uint8, device=DEV)
    total_diff = 0
    for it in (3, 4):  # annealed temperature (0.37, 0.26) and a hardening factor strictly inside (0, 1)
        inp = B.c2_step_inputs(rows, cols, it)
        want = B.c2_oracle_step(st, inp, it)
        assert 0.05 < want["temp"] < 1.0 and 0.0 < want["hx"] < 1.0
        ops.adamw_masked_score(W, dev(inp["g"]), m, v, mask=mask, lr=hp["lr"], beta1=hp["beta1"], beta2=hp["beta2"],
                               eps=hp["eps"], weight_decay=hp["weight_decay"], decay=hp["decay"], step=it + 1,
                               hvp=dev(inp["hvp"]), probe=dev(inp["probe"]), beta_h=hp["beta_h"], H=H, score=None,
                               norm=norm, scratch=scratch, metric="hessian_obd")
        B.assert_elementwise(H, want["H"], F32, 1e-12, f"step {it}: H")
        # bf16 state: one unit in the last place is 2^-8 = 0.4 % of the value
        B.assert_elementwise(W.float(), want["W"].float(), BF16, BF16 * B.rms(want["W"].float()), f"step {it}: W")
        B.assert_elementwise(m.float(), want["m"].float(), BF16, BF16 * B.rms(want["m"].float()), f"step {it}: exp_avg")
        B.assert_elementwise(v.float(), want["v"].float(), BF16, BF16 * B.rms(want["v"].float()), f"step {it}: exp_avg_sq")
        n_w_diff = int((W.cpu() != want["W"]).sum())
        print(f"[parity] step {it}: {n_w_diff} of {W.numel()} bf16 weights differ from the oracle's (by one unit in the last place)")
        # the score statistics belong to the weight the kernel itself produced: compare with the oracle's
        # statistics of that weight
        mu, sigma = O.score_norm_stats(O.importance_score(W.cpu(), "hessian_obd", H=H.cpu()))
        assert torch.allclose(norm.cpu(), torch.stack([mu, sigma]), rtol=F32, atol=0)
        assert torch.allclose(norm.cpu(), want["norm"], rtol=1e-3, atol=0)

        # the mask update is checked on the state the kernel left (so that this stage sees the same
        # inputs on both sides): oracle gate and EMA from the kernel's W and H
        raw = O.importance_score(W.cpu(), "hessian_obd", H=H.cpu())
        G = O.gate_target_structured(O.normalize_scores(raw), want["temp"])
        want_mask = O.mask_update(st["mask"], G, mask_lr=hp["mask_lr"])
        prev_mask = mask.cpu().clone()
        ops.mask_update_nm24_from_weight(W, H, norm, mask, stats, wm, meta, metric="hessian_obd",
                                         temperature=want["temp"], mask_lr=hp["mask_lr"], hx=want["hx"])
        B.assert_elementwise(mask, want_mask, F32, 1e-7, f"step {it}: soft mask")
        mask_cpu = mask.cpu()
        hard_own = O.hard_mask_from_soft(mask_cpu)
        # integer outputs against the projection of the kernel's own soft mask: bit for bit
        assert torch.equal(unpack_meta(meta, cols), hard_own)
        assert torch.equal(meta.cpu(), O.meta_from_hard(hard_own))
        assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(prev_mask, mask_cpu)
        # and against the oracle's own chain: only inside near-ties
        total_diff += report_hard(f"bf16 q-projection step {it}", hard_own, O.hard_mask_from_soft(want_mask), want_mask,
                                  F32, 1e-7)
        want_wm = O.masked_weight(W.cpu(), O.effective_mask(mask_cpu, want["hx"]))
        B.assert_elementwise(wm.float(), want_wm.float(), BF16, BF16 * B.rms(want_wm.float()), f"step {it}: masked weight")
        ms = O.mask_stats(mask_cpu)
        assert abs(float(stats[_lib.MSTAT_SUM_M]) - ms["sum_m"]) <= 1e-6 * ms["sum_m"]
        assert abs(float(stats[_lib.MSTAT_SUM_M1M]) - ms["sum_m1m"]) <= 1e-6 * ms["sum_m1m"]
        assert float(stats[_lib.MSTAT_COUNT_LT_HALF]) == ms["count_lt_half"]
        # the oracle's free-running chain (its own W after its own AdamW): a weight that rounds to the
        # neighbouring bf16 value moves that entry's score by 0.8 % and, through the group threshold, the
        # gate of the four entries of its group; nothing else may differ
        within, _ = B.elementwise_violations(mask, want["mask"], F32, 1e-7)
        print(f"[parity] step {it}: {within} of {mask.numel()} soft-mask entries differ from the free-running oracle "
              f"chain by more than 1e-5 (largest difference {float((mask.cpu() - want['mask']).abs().max()):.3g})")
        assert within <= 4 * n_w_diff
        # next step: both sides continue from the kernel's state
        st = {"W": W.cpu().clone(), "m": m.cpu().clone(), "v": v.cpu().clone(), "mask": mask_cpu.clone(), "H": H.cpu().clone()}
    print(f"[parity] bf16 q-projection, two steps: {total_diff} hard-mask entries differ in total")


def test_c2_three_pass_path_one_step():
    """The same q-shaped step through the three separate passes the module path uses when the score is not
    folded into the optimizer: Hutchinson accumulate + score (`sf_hutch_score`), mask-aware AdamW that also
    emits the masked weight (`sf_adamw_masked`), score of the new weight, mask update from the score tensor
    (`sf_mask_update_nm24`). Against the oracle, entry by entry, at the size the benchmark runs."""
    from sparseforge_b200 import _lib, ops

    rows = cols = 4096
    hp = B.C2_HYPER
    it = 5
    st = B.c2_state(rows, cols, seed=101)
    inp = B.c2_step_inputs(rows, cols, it, seed=101)
    temp, hx = B.c2_schedule(it)
    dev = lambda t: t.to(DEV).contiguous()  # noqa: E731
    W, m, v, H, mask = dev(st["W"]), dev(st["m"]), dev(st["v"]), dev(st["H"]), dev(st["mask"])
    score = torch.empty(rows, cols, device=DEV)
    norm, scratch = torch.zeros(2, device=DEV), ops.hutch_score_scratch(DEV)
    # pass 1: H <- EMA of clamp(hvp * v, 0); score of the CURRENT weight
    ops.hutch_score(W, H, score, norm, scratch, hvp=dev(inp["hvp"]), v=dev(inp["probe"]), beta=hp["beta_h"])
    want_H = O.hutchinson_accumulate(st["H"], inp["hvp"], inp["probe"].to(inp["hvp"].dtype), hp["beta_h"])
    B.assert_elementwise(H, want_H, F32, 1e-12, "H")
    want_score = O.importance_score(st["W"], "hessian_obd", H=want_H)
    B.assert_elementwise(score, want_score, F32, 1e-9 * B.rms(want_score), "score of the current weight")
    mu, sigma = O.score_norm_stats(want_score)
    assert torch.allclose(norm.cpu(), torch.stack([mu, sigma]), rtol=F32, atol=0)
    # pass 2: AdamW with the mask term, masked weight emitted at the step's hardening factor
    wm = torch.empty_like(W)
    ops.adamw_masked(W, dev(inp["g"]), m, v, mask=mask, lr=hp["lr"], beta1=hp["beta1"], beta2=hp["beta2"], eps=hp["eps"],
                     weight_decay=hp["weight_decay"], decay=hp["decay"], step=it + 1, wm=wm, hx=hx)
    wW, wm_, wv = O.adamw_step(st["W"], inp["g"], st["m"], st["v"], step=it + 1, lr=hp["lr"], betas=(hp["beta1"], hp["beta2"]),
                               eps=hp["eps"], weight_decay=hp["weight_decay"], mask=st["mask"], decay=hp["decay"])
    for name, got, want in (("W", W, wW), ("exp_avg", m, wm_), ("exp_avg_sq", v, wv)):
        B.assert_elementwise(got.float(), want.float(), BF16, BF16 * B.rms(want.float()), name)
    want_wm = O.masked_weight(W.cpu(), O.effective_mask(st["mask"], hx))
    B.assert_elementwise(wm.float(), want_wm.float(), BF16, BF16 * B.rms(want_wm.float()), "masked weight from the optimizer pass")
    # pass 3: score of the NEW weight, then the mask update from the score tensor
    ops.hutch_score(W, H, score, norm, scratch)
    raw = O.importance_score(W.cpu(), "hessian_obd", H=H.cpu())
    B.assert_elementwise(score, raw, F32, 1e-9 * B.rms(raw), "score of the new weight")
    G = O.gate_target_structured(O.normalize_scores(raw), temp)
    want_mask = O.mask_update(st["mask"], G, mask_lr=hp["mask_lr"])
    stats = torch.zeros(8, dtype=torch.float64, device=DEV)
    meta = torch.zeros(rows, cols // 8, dtype=torch.uint8, device=DEV)
    ops.mask_update_nm24(score, norm, mask, stats, W=W, wm=wm, meta=meta, temperature=temp, mask_lr=hp["mask_lr"], hx=hx)
    B.assert_elementwise(mask, want_mask, F32, 1e-7, "soft mask")
    mask_cpu = mask.cpu()
    hard_own = O.hard_mask_from_soft(mask_cpu)
    assert torch.equal(meta.cpu(), O.meta_from_hard(hard_own))
    assert int(stats[_lib.MSTAT_FLIPS]) == O.flip_count(st["mask"], mask_cpu)
    report_hard("bf16 q-projection, three-pass path", hard_own, O.hard_mask_from_soft(want_mask), want_mask, F32, 1e-7)
    want_wm = O.masked_weight(W.cpu(), O.effective_mask(mask_cpu, hx))
    B.assert_elementwise(wm.float(), want_wm.float(), BF16, BF16 * B.rms(want_wm.float()), "masked weight from the mask update")

