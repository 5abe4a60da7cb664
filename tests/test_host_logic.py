"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, host
schedules and shard arithmetic match the reference formulas, and the product refuses CPU tensors
(there is no fallback path)."""
import math
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "sparseforge_b200.h")).read()
    return sorted(set(re.findall(r"SF_API\s+[\w\s\*]+?\b(sf_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sparseforge_b200 import _lib

    lib = _lib.lib()
    declared = header_symbols()
    assert len(declared) >= 25
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, missing
    # the ctypes table covers the header, nothing more, nothing less
    assert sorted(_lib.declared_symbols()) == declared
    assert lib.sf_version() >= 100
    assert int(lib.sf_hutch_score_scratch_doubles(1 << 20)) == 4096
    assert int(lib.sf_sparse24_meta_tc_bytes(256, 384)) == 2 * 3 * 2048


def test_argument_errors_come_back_as_codes_without_a_gpu():
    from sparseforge_b200 import _lib

    lib = _lib.lib()
    # null pointers / bad sizes are refused on the host before anything touches a device
    assert lib.sf_project_nm24(None, 0, 8, None, 0, 8, None, 4, 8, None) == -1
    assert b"soft must be non-null" in lib.sf_last_error_string()
    assert lib.sf_masked_gemm_fwd(1 << 12, 1 << 12, None, 1 << 12, 8, 12, 8, 1.0, 1, None, None) == -2
    assert b"multiples of 8" in lib.sf_last_error_string()
    assert lib.sf_sparse24_gemm(16, 16, 16, None, 16, 8, 24, 8, None, None) == -2
    assert lib.sf_bsr16_build(16, None, 1, 1, None, 16, None, None, 24, 32, None) == -1


def test_ops_refuse_cpu_tensors():
    from sparseforge_b200 import ops
    import sparseforge_b200 as sf

    with pytest.raises(RuntimeError, match="CUDA"):
        ops.project_nm24(torch.rand(4, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.gemm_fwd(torch.zeros(8, 8), torch.zeros(8, 8))
    layer = sf.SparseLinear(16, 16, sparselinear_config=sf.SparseLinearConfig(), bias=False)
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(torch.zeros(2, 16))
    p = torch.nn.Parameter(torch.zeros(8, 8))
    p.grad = torch.zeros(8, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        sf.AdamW([p]).step()


def test_config_fields_match_the_reference_dataclass():
    import dataclasses

    import sparseforge_b200 as sf

    want = ["change_mask", "mode", "mask_type", "mask_metric", "sparsity_ratio", "N", "M", "beta", "score_ema_beta",
            "mask_update_period", "mask_update_switch_step", "mask_update_period_before", "mask_update_period_after",
            "mask_lr", "mask_penalty_lr", "mask_penalty_mode", "temp_init", "temp_min", "temp_decay",
            "mask_binarize_decay", "mask_hardening_start", "mask_hardening_duration", "sparsity_warmup_steps",
            "tau_sample_size", "temperature", "freeze_low", "freeze_high", "SLoRB", "SLoRB_k", "SLoRB_init_type",
            "trainable_projection", "structured_exact", "hard_mask_type", "beta_structural_start",
            "beta_structural_end", "gradient_checkpointing", "srste_decay", "glu_joint_mask", "weight_scaling"]
    assert [f.name for f in dataclasses.fields(sf.SparseLinearConfig)] == want
    cfg = sf.SparseLinearConfig()
    assert (cfg.mask_lr, cfg.temp_decay, cfg.mask_update_period, cfg.sparsity_warmup_steps) == (0.10, 0.97, 10, 100)
    # every field and its default, as recorded from the reference's dataclass (legacy/sparse_modeling.py:136-239)
    import json

    from golden_io import Golden

    ref = json.loads(str(Golden("schedules")["config_defaults_json"]))
    assert list(ref) == want
    assert {f.name: getattr(cfg, f.name) for f in dataclasses.fields(sf.SparseLinearConfig)} == ref


def test_host_schedules_match_reference_formulas():
    import sparseforge_b200 as sf
    from oracle import sparselinear_oracle as O

    cfg = sf.SparseLinearConfig(temp_init=1.0, temp_min=0.05, temp_decay=0.7, mask_update_period=3,
                                mask_hardening_start=5, mask_hardening_duration=10, sparsity_warmup_steps=20,
                                beta_structural_start=4, beta_structural_end=12)
    layer = sf.SparseLinear(16, 8, sparselinear_config=cfg, bias=False)
    for step in (0, 1, 2, 3, 7, 30, 100):
        assert layer._temperature(step) == pytest.approx(O.temperature_at(step, 1.0, 0.7, 0.05, period=3), rel=1e-12)
        assert layer._next_hardening_x(step) == pytest.approx(O.hardening_x(step, 5, 10), abs=1e-12)
    assert layer._effective_sparsity(10) == pytest.approx(0.25)
    assert layer._beta_structural(3) == 0.0 and layer._beta_structural(12) == 1.0
    t = (8 - 4) / 8
    assert layer._beta_structural(8) == pytest.approx(3 * t * t - 2 * t ** 3)
    cfg2 = sf.SparseLinearConfig(mask_update_switch_step=10, mask_update_period_before=2, mask_update_period_after=5)
    l2 = sf.SparseLinear(16, 8, sparselinear_config=cfg2, bias=False)
    assert (l2._mask_update_period(9), l2._mask_update_period(10)) == (2, 5)
    # state-dict keys of the reference layer
    assert set(layer.state_dict()) == {"weight", "mask", "grad_ema", "hessian_diag", "frozen_mask_flags", "scaler_row"}
    assert layer.mask.dtype == torch.float32 and layer.grad_ema.numel() == 1 and layer._is_placeholder("grad_ema")


def test_host_schedules_follow_the_reference_over_a_grid_of_steps():
    """Temperature, update period, effective sparsity, beta mixing and hardening of a layer, and the penalty
    learning-rate schedule of the loop, against values recorded from the reference
    (tests/golden/schedules.npz; legacy/sparse_modeling.py:932-985, 1603-1619, legacy/utils.py:141-180)."""
    import json

    import sparseforge_b200 as sf
    from golden_io import Golden
    from sparseforge_b200 import utils as U

    g = Golden("schedules")
    steps = [int(x) for x in g["steps"]]
    for tag, kw in json.loads(str(g["configs_json"])).items():
        cfg = sf.SparseLinearConfig(**dict(dict(mask_type="structured", mask_metric="magnitude"), **kw))
        layer = sf.SparseLinear(32, 16, sparselinear_config=cfg, bias=False)
        want = g[f"{tag}_values"]
        for i, step in enumerate(steps):
            got = [layer._temperature(step), float(layer._mask_update_period(step)), layer._effective_sparsity(step),
                   layer._beta_structural(step), layer._next_hardening_x(step)]
            for name, a, b in zip(("temperature", "period", "sparsity", "beta", "hardening_x"), got, want[i].tolist()):
                assert a == pytest.approx(b, rel=1e-12, abs=1e-15), (tag, step, name)
    lin = sf.SparseLinear(8, 8, sparselinear_config=sf.SparseLinearConfig(), bias=False)
    for row, sched in zip(g["penalty_lr"].tolist(), ("constant", "linear", "cosine", "other")):
        for s_, v in zip([int(x) for x in g["penalty_lr_steps"]], row):
            assert U.update_mask_penalty_lr(lin, s_, 50, 0.02, 0.3, sched) == pytest.approx(v, rel=1e-12), (sched, s_)
            assert lin.mask_penalty_lr == pytest.approx(v, rel=1e-12)


def test_unsupported_configurations_raise():
    import sparseforge_b200 as sf

    wanda = sf.SparseLinear(16, 8, sparselinear_config=sf.SparseLinearConfig(mask_metric="wanda"))
    assert tuple(wanda.scaler_row.shape) == (16,) and not wanda._is_placeholder("scaler_row") and wanda.nsamples == 0
    bands = sf.SparseLinear(16, 8, sparselinear_config=sf.SparseLinearConfig(freeze_low=0.1))
    assert tuple(bands.frozen_mask_flags.shape) == (8, 16) and not bands._is_placeholder("frozen_mask_flags")
    slorb = sf.SparseLinear(64, 8, sparselinear_config=sf.SparseLinearConfig(SLoRB=True, SLoRB_k=16))
    assert tuple(slorb.x_proj.shape) == (4, 64) and tuple(slorb.SLoRB_Weight.shape) == (8, 4)
    assert list(slorb.state_dict().keys())[-2:] == ["x_proj", "SLoRB_Weight"]
    assert sf.AdamW([torch.nn.Parameter(torch.zeros(2))], amsgrad=True).param_groups[0]["amsgrad"] is True
    with pytest.raises(ValueError):
        sf.AdamW([torch.nn.Parameter(torch.zeros(2))], lr=-1.0)


def test_general_nm_configurations_are_checked_on_the_host():
    """N:M other than 2:4: which group sizes the kernels take, which combinations are refused, and the
    argument checks of the entry points (no device needed for any of it)."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import _lib

    def layer(n, m, in_f=64, **kw):
        return sf.SparseLinear(in_f, 8, sparselinear_config=sf.SparseLinearConfig(mask_type="structured", N=n, M=m, **kw),
                               bias=False)

    assert not layer(2, 4)._general_nm() and layer(4, 8)._general_nm() and layer(1, 4)._general_nm()
    for n, m in ((4, 8), (1, 2), (3, 4), (5, 16), (31, 32)):
        layer(n, m)._check_2to4()
    for n, m in ((2, 3), (8, 8), (0, 4), (2, 64)):
        with pytest.raises(NotImplementedError):
            layer(n, m)._check_2to4()
    with pytest.raises(ValueError, match="divisible by M"):
        layer(4, 16, in_f=72)._check_2to4()
    with pytest.raises(NotImplementedError, match="must agree"):
        layer(4, 8, hard_mask_type="nm_2_4")._check_2to4()
    with pytest.raises(NotImplementedError, match="2:4"):
        layer(4, 8).compress_for_inference()
    layer(2, 4)._check_strict_2to4("x")
    thr = sf.SparseLinear(64, 8, sparselinear_config=sf.SparseLinearConfig(mask_type="unstructured"), bias=False)
    assert thr._threshold_view() and thr._general_nm() and not thr._is_2to4_view()
    thr._check_2to4()
    thr._check_mask_modes()

    lib = _lib.lib()
    assert lib.sf_project_nm(16, 0, 96, 16, 0, 96, 4, 96, 2, 3, None) == -2  # M = 3
    assert b"M=3" in lib.sf_last_error_string()
    assert lib.sf_project_nm(16, 0, 64, 16, 0, 64, 4, 60, 4, 8, None) == -1  # 60 columns, M = 8
    assert lib.sf_project_nm(None, 0, 64, 16, 0, 64, 4, 64, 4, 8, None) == -1
    assert lib.sf_effective_weight_nm(16, 1, 16, 16, 4, 64, 8, 8, 0.5, 0, 0, None) == -1  # N = M
    assert lib.sf_effective_weight_nm(16, 1, 16, 16, 4, 64, 4, 8, 0.5, 0, 2, None) == -1  # hard view 2
    assert lib.sf_mask_update_nm(16, 16, None, None, 16, None, 0, None, 16, 4, 64, 4, 8, 1.0, 0.1, 0.0, 3, 0.0, 0.0, 1.0, 0,
                                 0, 0, None) == -1  # penalty mode 3
    assert lib.sf_mask_update_nm(16, 16, None, None, 24, None, 0, None, 16, 4, 64, 4, 8, 1.0, 0.1, 0.0, 0, 0.0, 0.0, 1.0, 0,
                                 0, 0, None) == -3  # mask not 16-byte aligned
    # the low-rank forward: rank and dtype checks
    assert lib.sf_masked_gemm_fwd_lowrank(16, 16, 16, 16, None, 16, 256, 64, 64, 12, 1, None, None) == -2
    assert lib.sf_masked_gemm_fwd_lowrank(16, 16, None, 16, None, 16, 256, 64, 64, 16, 1, None, None) == -1
    assert lib.sf_masked_gemm_fwd_lowrank(16, 16, 16, 16, None, 16, 256, 64, 64, 16, 0, None, None) == -2


def test_peer_sharded_layer_buffers_and_checks_without_a_gpu():
    """Landing-buffer bookkeeping and input checks of PeerShardedLinear with a stand-in arena."""
    import sparseforge_b200 as sf
    from sparseforge_b200.sharding import PeerShardedLinear

    class Arena:
        world, rank, mc_base, group = 2, 1, 0, None

        def close(self):
            self.closed = True

    shard = sf.SparseLinear(64, 32, sparselinear_config=sf.SparseLinearConfig(), bias=False).to(torch.bfloat16)
    arena = Arena()
    layer = PeerShardedLinear(shard, out_total=64, max_tokens=512, arena=arena)
    assert shard._row_sharded and layer.arena is arena
    y_bytes, s_bytes = 512 * 64 * 2, 512 * 64 * 2
    spans = []
    for par in range(PeerShardedLinear.N_BUFFERS):
        y_off, s_off = layer._offsets(par)
        spans += [(y_off, y_off + y_bytes), (s_off, s_off + s_bytes)]
        assert y_off % 16 == 0 and s_off % 16 == 0
    spans.sort()
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))  # the four regions do not overlap
    assert [layer._next_parity() for _ in range(4)] == [1, 0, 1, 0]
    layer._check(torch.zeros(256, 64, dtype=torch.bfloat16))
    for bad in (torch.zeros(128, 64, dtype=torch.bfloat16), torch.zeros(260, 64, dtype=torch.bfloat16),
                torch.zeros(1024, 64, dtype=torch.bfloat16)):
        with pytest.raises(ValueError):
            layer._check(bad)
    with pytest.raises(TypeError):
        layer._check(torch.zeros(256, 64))
    with pytest.raises(ValueError):
        PeerShardedLinear(shard, out_total=96, max_tokens=512, arena=Arena())
    layer.close()
    assert arena.closed and layer.arena is None


def test_shard_bounds():
    from sparseforge_b200.sharding import shard_bounds

    for out in (4096, 11008):
        for world in (1, 2, 4, 8):
            spans = [shard_bounds(out, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == out
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all((hi - lo) % 16 == 0 for lo, hi in spans)
    with pytest.raises(ValueError):
        shard_bounds(11008, 3, 0)
    with pytest.raises(ValueError):
        shard_bounds(4096, 4, 4)


def test_get_raw_model_unwraps():
    from sparseforge_b200 import utils as U

    class Box(torch.nn.Module):
        def __init__(self, inner, attr):
            super().__init__()
            setattr(self, attr, inner)

    core = torch.nn.Linear(2, 2)
    assert U.get_raw_model(core) is core
    assert U.get_raw_model(Box(core, "module")) is core
    assert U.get_raw_model(Box(core, "student")) is core
    assert U.get_raw_model(Box(Box(core, "student"), "module")) is core
    assert math.isclose(U.update_mask_penalty_lr(core, 5, 10, 0.0, 1.0, "linear"), 0.5)


def test_every_name_the_training_script_imports_exists():
    """``from utils import (...)`` of legacy/main_llama.py:32-50 must resolve against this package, and so
    must its imports from sparse_modeling and adamw; the evaluators raise a clear error when called."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import adamw, sparse_modeling
    from sparseforge_b200 import utils as U

    for name in ("calculate_model_mask", "calculate_flip_rate", "set_model_mode", "initialize_model", "add_calibration",
                 "eval_ppl", "eval_ppl_distributed", "sync_weight", "update_model_grad_ema", "update_hessian_hutchinson",
                 "mid_penalty", "harden_fraction", "log_mask_stats", "get_raw_model", "sparsity_penalty",
                 "nm_2_4_tile_stats", "update_mask_penalty_lr"):
        assert callable(getattr(U, name)), name
    for name in ("Distill_Model", "SparseLinearConfig", "SparseLinear", "STE", "SRSTE", "FusedMaskedLinearSTE"):
        assert hasattr(sparse_modeling, name), name
    assert adamw.AdamW is sf.AdamW
    with pytest.raises(NotImplementedError, match="outside this package"):
        U.eval_ppl(torch.nn.Linear(2, 2))
    with pytest.raises(NotImplementedError, match="outside this package"):
        U.eval_ppl_distributed(torch.nn.Linear(2, 2))
    with pytest.raises(FileNotFoundError, match="dataloader"):
        U.add_calibration(torch.nn.Linear(2, 2))


def test_prepared_calls_convert_once_and_read_cells_at_call_time():
    """``_lib.prepare`` wraps the arguments of a library call in ctypes once; a ctypes instance among them is a
    cell whose current value is read at every call; a non-zero return code raises with the library's message."""
    import ctypes

    from sparseforge_b200 import _lib

    with pytest.raises(TypeError, match="arguments expected"):
        _lib.prepare("sf_masked_gemm_configure_stream", None)
    limit = ctypes.c_int(-1)
    call = _lib.prepare("sf_masked_gemm_configure_stream", None, limit)
    with pytest.raises(RuntimeError, match="max_ctas must be >= 0"):
        call()
    limit.value = 0  # the same prepared call, the cell changed: now valid (forgets the stream)
    call()
    rows = ctypes.c_int64(4)
    bad = _lib.prepare("sf_project_nm24", None, 0, 8, None, 0, 8, None, rows, 8, None)
    with pytest.raises(RuntimeError, match="soft must be non-null"):
        bad()


def test_bench_schedules_and_host_threads():
    import bench

    temps = [bench.schedule(it)[0] for it in range(10)]
    assert temps[0] == 1.0 and temps[9] == pytest.approx(0.05) and all(a > b for a, b in zip(temps, temps[1:]))
    assert bench.schedule(0)[1] == 1.0 and bench.schedule(1)[1] == 1.0 and bench.schedule(10)[1] == 1.0
    assert bench.schedule(5)[1] == pytest.approx(1.0 - 4 / 9)
    assert 1 <= bench.host_threads() <= (os.cpu_count() or 1)
    assert bench.layer_flops(8192, 4096, 4096) == pytest.approx(824.63e9, rel=1e-4)
