"""Inputs and oracle chains of the two benchmark-sized parity cases (not a test module).

* the fp32 GPT-2-small MLP case: W [3072, 768], X [8, 1024, 768], four Hutchinson probes, one mask
  update at step 0, hard 2:4 projection, masked forward / backward with the hard mask;
* the bf16 LLaMA-2-7B q-projection case: one [4096, 4096] matrix, the optimizer + score pass and
  the 2:4 mask update exactly as the benchmark runs them.

The oracle chains are plain calls into ``oracle/sparselinear_oracle.py`` in the order of the
reference's training step (legacy/main_llama.py:1997-2211); they run on the CPU in seconds.
"""
import torch

from oracle import sparselinear_oracle as O


# ---------------------------------------------------------------------------------------------
# element-wise comparison
# ---------------------------------------------------------------------------------------------
def elementwise_violations(a: torch.Tensor, b: torch.Tensor, rtol: float, atol: float):
    """(count of entries with |a - b| > rtol |b| + atol, largest |a - b| / (rtol |b| + atol))."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    bound = rtol * b.abs() + atol
    ratio = (a - b).abs() / bound
    return int((ratio > 1.0).sum()), float(ratio.max())


def assert_elementwise(a, b, rtol, atol, what=""):
    bad, worst = elementwise_violations(a, b, rtol, atol)
    assert bad == 0, f"{what}: {bad} entries beyond |a-b| <= {rtol}|b| + {atol:g} (worst at {worst:.2f} of the bound)"


def rms(t: torch.Tensor) -> float:
    return float(t.detach().double().pow(2).mean().sqrt())


def near_tie_groups(soft: torch.Tensor, rtol: float, atol: float = 0.0) -> torch.Tensor:
    """Boolean [rows, cols / 4]: 2:4 groups whose 2nd and 3rd largest soft values are so close that a
    perturbation of every value by rtol |value| + atol can swap them (each of the two may move)."""
    rows, cols = soft.shape
    s = torch.sort(soft.detach().float().cpu().view(rows, cols // 4, 4), dim=-1, descending=True).values
    return (s[..., 1] - s[..., 2]) <= 2.0 * (rtol * s[..., 1].abs() + atol)


def hard_mismatch(hard_a: torch.Tensor, hard_b: torch.Tensor):
    """(entries that differ, boolean [rows, cols / 4] of the groups holding them)."""
    diff = hard_a.cpu() != hard_b.cpu()
    rows, cols = diff.shape
    return int(diff.sum()), diff.view(rows, cols // 4, 4).any(-1)


def fp32_at_offset(t: torch.Tensor, shift_floats: int, device) -> torch.Tensor:
    """A float32 copy of ``t`` on ``device`` that starts ``shift_floats`` floats into a 256-byte aligned
    buffer: shift 0 gives a 32-byte aligned tensor, shift 4 one that is only 16-byte aligned."""
    n = t.numel()
    buf = torch.empty(n + 64, dtype=torch.float32, device=device)
    view = buf[shift_floats:shift_floats + n].view(t.shape)
    view.copy_(t)
    assert view.data_ptr() % 32 == (4 * shift_floats) % 32
    return view


# ---------------------------------------------------------------------------------------------
# fp32 GPT-2-small MLP case
# ---------------------------------------------------------------------------------------------
def c1_inputs():
    torch.manual_seed(0)
    W = torch.randn(3072, 768) * 0.02
    X = torch.randn(8, 1024, 768)
    dY = torch.randn(8, 1024, 3072)
    return W, X, dY


def fingerprint(t: torch.Tensor) -> torch.Tensor:
    return torch.stack([t.double().sum(), (t.double() ** 2).sum(), t.flatten()[12345].double()])


def c1_probe(i: int, shape) -> torch.Tensor:
    g = torch.Generator().manual_seed(1 + i)
    return torch.randint(0, 2, shape, generator=g, dtype=torch.int8).float() * 2 - 1


def c1_oracle(W, X, dY, n_probes=4, beta=0.99, mask_lr=0.1):
    """The whole chain through the oracle. Returns a dict of full tensors."""
    out_f, in_f = W.shape
    T = X.shape[0] * X.shape[1]
    mask0 = torch.ones_like(W)
    H = torch.ones_like(W)
    res = {"hvp": [], "H": []}
    Wp = W.clone().requires_grad_(True)
    for i in range(n_probes):
        v = c1_probe(i, W.shape)
        Y = O.MaskedLinearSTE.apply(X, Wp, None, O.effective_mask(mask0, 1.0))
        loss = (torch.nn.functional.gelu(Y.float()) * dY.float()).sum() / T
        (hvp,) = O.hutchinson_hvps(loss, [Wp], [v])
        hvp = hvp.detach()
        H = O.hutchinson_accumulate(H, hvp, v, beta)
        res["hvp"].append(hvp)
        res["H"].append(H)
    raw = O.importance_score(W, "hessian_obd", H=H)
    res["score_raw"] = raw
    mu, sigma = O.score_norm_stats(raw)
    res["score_mean_std"] = torch.stack([mu, sigma])
    G = O.gate_target_structured(O.normalize_scores(raw), 1.0)
    res["G"] = G
    mask = O.mask_update(mask0, G, mask_lr=mask_lr)
    res["mask"] = mask
    res["flips"] = O.flip_count(mask0, mask)
    hard = O.hard_mask_from_soft(mask)
    res["hard"] = hard
    res["Y"] = O.linear_forward(X, W, hard)
    res["dX"], res["dW"], _ = O.linear_backward(X, W, hard, dY)
    return res


# ---------------------------------------------------------------------------------------------
# bf16 LLaMA-2-7B q-projection case: the pair of passes the benchmark times
# ---------------------------------------------------------------------------------------------
C2_HYPER = dict(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, decay=2e-4, beta_h=0.99, mask_lr=0.1)


def c2_schedule(it: int):
    """Temperature annealed 1.0 -> 0.05 over ten steps and the hardening factor, as the benchmark sets them."""
    decay_t = 0.05 ** (1.0 / 9.0)
    temp = max(0.05, decay_t ** (it % 10))
    hx = max(0.0, min(1.0, 1.0 - ((it % 10) - 1) / 9.0)) if (it % 10) >= 1 else 1.0
    return temp, hx


def c2_state(rows=4096, cols=4096, seed=100):
    """Seeded state of one matrix in the middle of a tempering run: bf16 weight and Adam moments,
    fp32 soft mask in (0, 1) and Hessian diagonal."""
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    st = {
        "W": (torch.randn(rows, cols, generator=g) * 0.02).to(bf),
        "m": (torch.randn(rows, cols, generator=g) * 0.05).to(bf),
        "v": (torch.rand(rows, cols, generator=g) * 0.01).to(bf),
        "mask": torch.rand(rows, cols, generator=g),
        "H": torch.rand(rows, cols, generator=g) * 1e-3 + 1e-5,
    }
    return st


def c2_step_inputs(rows, cols, it, seed=100):
    g = torch.Generator().manual_seed(seed * 1000 + it)
    bf = torch.bfloat16
    return {
        "g": torch.randn(rows, cols, generator=g).to(bf),
        "hvp": (torch.randn(rows, cols, generator=g) * 1e-3).to(bf),
        "probe": (torch.randint(0, 2, (rows, cols), generator=g, dtype=torch.int8) * 2 - 1),
    }


def c2_oracle_step(st, inp, it):
    """One step in the reference's order: Hutchinson sample into H, AdamW, score of the NEW weight,
    normalisation, structured gate, mask EMA, projection, metadata, masked weight."""
    hp = C2_HYPER
    temp, hx = c2_schedule(it)
    H = O.hutchinson_accumulate(st["H"], inp["hvp"], inp["probe"].to(inp["hvp"].dtype), hp["beta_h"])
    W, m, v = O.adamw_step(st["W"], inp["g"], st["m"], st["v"], step=it + 1, lr=hp["lr"], betas=(hp["beta1"], hp["beta2"]),
                           eps=hp["eps"], weight_decay=hp["weight_decay"], mask=st["mask"], decay=hp["decay"])
    raw = O.importance_score(W, "hessian_obd", H=H)
    mu, sigma = O.score_norm_stats(raw)
    G = O.gate_target_structured(O.normalize_scores(raw), temp)
    mask = O.mask_update(st["mask"], G, mask_lr=hp["mask_lr"])
    hard = O.hard_mask_from_soft(mask)
    return {"H": H, "W": W, "m": m, "v": v, "norm": torch.stack([mu, sigma]), "mask": mask, "hard": hard,
            "meta": O.meta_from_hard(hard), "flips": O.flip_count(st["mask"], mask),
            "wm": O.masked_weight(W, O.effective_mask(mask, hx)), "temp": temp, "hx": hx}
