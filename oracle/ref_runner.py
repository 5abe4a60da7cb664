"""Runs the reference's OWN code (compiled into ``oracle/_ref/`` by ``oracle/build_ref.py``) on the host
cores: one tempering step of one LLaMA-shaped matrix, in the order of the reference's training loop
(legacy/main_llama.py:1997-2211). TEST / BENCHMARK INFRASTRUCTURE: used by ``bench.py --impl reference``
and the ``cpu_baseline`` leg only.

What runs reference code: ``SparseLinear.forward`` and its autograd backward (masked GEMMs,
legacy/sparse_modeling.py:72-132), ``AdamW.step(decay=)`` (legacy/adamw.py:65-176) and
``utils.calculate_model_mask`` (legacy/utils.py:183-310: score, normalisation, 2:4 gate, mask EMA, hard
projection, flip count). The Hutchinson sample is folded into H by the three tensor ops of the tail of
``update_hessian_hutchinson`` (legacy/utils.py:804-868, restated in ``sparselinear_oracle``) from a
synthetic Hessian-vector product, exactly what the GPU arm of the benchmark does: the double backward
that produces a real one is not part of the timed step on either side.

``torch.topk`` is made tie-stable (lower index wins) while the reference runs, the tie rule this path
is specified with.
"""
from __future__ import annotations

import collections
import importlib
import importlib.machinery
import importlib.util
import os
import sys
import time

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

_TopK = collections.namedtuple("topk", ["values", "indices"])
_orig_topk = torch.topk


def _stable_topk(x, k, dim=-1, largest=True, sorted=True):  # noqa: A002
    s = torch.sort(x, dim=dim, descending=bool(largest), stable=True)
    sl = [slice(None)] * x.dim()
    sl[dim] = slice(0, k)
    return _TopK(s.values[tuple(sl)], s.indices[tuple(sl)])


def _path(name):
    return os.path.join(REF_DIR, name + ".bytecode")


def available() -> bool:
    return all(os.path.exists(_path(m)) for m in ("sparse_modeling", "utils", "adamw"))


def load():
    """(sparse_modeling, utils, adamw) of the reference, loaded from the bytecode in oracle/_ref under
    their own module names (``utils`` imports ``sparse_modeling`` by that name)."""
    if not available():
        raise RuntimeError("oracle/_ref is empty: run `SPARSEFORGE_REFERENCE=<checkout> python oracle/build_ref.py`")
    os.environ.setdefault("WANDB_MODE", "disabled")
    mods = []
    for name in ("sparse_modeling", "adamw", "utils"):
        m = sys.modules.get(name)
        if m is None or getattr(m, "__file__", None) != _path(name):
            loader = importlib.machinery.SourcelessFileLoader(name, _path(name))
            spec = importlib.util.spec_from_file_location(name, _path(name), loader=loader)
            m = importlib.util.module_from_spec(spec)
            sys.modules[name] = m
            try:
                loader.exec_module(m)
            except BaseException:
                sys.modules.pop(name, None)
                raise
        mods.append(m)
    return mods[0], mods[2], mods[1]


class RefMatrix:
    """One SparseLinear of the reference with the dtype mix of the LLaMA runs (bf16 weight and Adam
    moments, fp32 mask and Hessian diagonal) and its synthetic step inputs."""

    def __init__(self, mods, rows, cols, tokens, seed):
        sm, _, adamw = mods
        g = torch.Generator().manual_seed(seed)
        bf = torch.bfloat16
        cfg = sm.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, mask_update_period=1,
                                    sparsity_warmup_steps=0, mask_lr=0.1, beta=0.99, temp_init=1.0, temp_min=0.05,
                                    temp_decay=0.05 ** (1.0 / 9.0), mask_hardening_start=1, mask_hardening_duration=9)
        layer = sm.SparseLinear(cols, rows, sparselinear_config=cfg, bias=False).to(bf)
        layer.weight.data.copy_((torch.randn(rows, cols, generator=g) * 0.02).to(bf))
        layer.initialize()
        layer.mask.data = layer.mask.data.float()
        layer.hessian_diag.data = layer.hessian_diag.data.float()
        layer.sync_weight()
        self.layer = layer
        self.opt = adamw.AdamW([layer.weight], lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        self.x = torch.randn(tokens, cols, generator=g).to(bf)
        self.dy = torch.randn(tokens, rows, generator=g).to(bf)
        self.hvp = (torch.randn(rows, cols, generator=g) * 1e-3).to(bf)
        self.probe = (torch.randint(0, 2, (rows, cols), generator=g, dtype=torch.int8) * 2 - 1).to(bf)
        self.flops = 6.0 * tokens * rows * cols


def step(mods, mat: RefMatrix, it: int) -> None:
    """One tempering step of one matrix: masked forward / backward, Hutchinson tail, AdamW, mask update."""
    _, utils, _ = mods
    layer = mat.layer
    layer.weight.grad = None
    x = mat.x.clone().requires_grad_(True)
    layer(x).backward(mat.dy)
    with torch.no_grad():  # tail of update_hessian_hutchinson, legacy/utils.py:804-868 (world size 1)
        d = torch.clamp(mat.hvp * mat.probe, min=0.0)
        layer.hessian_diag.data.mul_(0.99).add_(d, alpha=0.01)
    mat.opt.step(decay=2e-4)
    utils.calculate_model_mask(layer, step=it % 10, lambda_mid=0.0)


def timed_steps(shapes, tokens, steps, warmup, threads=None):
    """Runs `warmup` + `steps` sample steps (one step = one tempering step of each matrix in `shapes`) and
    returns (seconds per step (list), flops per step, threads used)."""
    threads = int(threads or os.cpu_count() or 1)
    torch.set_num_threads(threads)  # torchrun exports OMP_NUM_THREADS=1: set the count explicitly
    mods = load()
    torch.topk = _stable_topk
    try:
        mats = [RefMatrix(mods, r, c, tokens, 100 + i) for i, (_, r, c) in enumerate(shapes)]
        times = []
        for it in range(warmup + steps):
            t0 = time.perf_counter()
            for m in mats:
                step(mods, m, it)
            if it >= warmup:
                times.append(time.perf_counter() - t0)
    finally:
        torch.topk = _orig_topk
    return times, sum(m.flops for m in mats), torch.get_num_threads()
