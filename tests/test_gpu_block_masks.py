"""Block-sparse soft masks (hard_mask_type block_sparse16 / block_sparse32) against a trajectory
recorded from the reference (tests/golden/block_masks.npz; generator case_block_masks):
block gate, block penalty / mid pull, binarise push, EMA, blockified mask, block hard view, flip
counts and the masked forward pass (legacy/sparse_modeling.py:461-508, 607-718, 1122-1157, 1395-1530).
"""
import json

import pytest
import torch

from golden_io import Golden, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("tag", ["bs16", "bs32", "tail", "tile16", "tile16mid"])
def test_block_sparse_soft_masks_follow_the_reference(tag):
    import sparseforge_b200 as sf

    g = Golden("block_masks")
    spec = json.loads(str(g["cases_json"]))[tag]
    cfg = sf.SparseLinearConfig(**dict(json.loads(str(g["base_json"])), **spec["cfg"]))
    out_f, in_f = spec["shape"]
    layer = sf.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False).to(DEV)
    layer.initialize()
    layer.weight.data.copy_(g[f"{tag}_W"].to(DEV))
    layer.hessian_diag.data.copy_(g[f"{tag}_H"].to(DEV))
    layer.invalidate_masked_weight()
    x = g[f"{tag}_x"].to(DEV)
    for step in range(5):
        assert layer._temperature(step) == pytest.approx(g.scalar(f"{tag}_s{step}_T"), rel=1e-12)
        assert layer._effective_sparsity(step) == pytest.approx(g.scalar(f"{tag}_s{step}_sp"), rel=1e-12, abs=1e-15)
        assert rel_err(layer.compute_gate_target(step), g[f"{tag}_s{step}_G"]) <= 1e-5
        layer.update_mask(step, lambda_mid=0.25)
        assert rel_err(layer.mask.data, g[f"{tag}_s{step}_mask"]) <= 1e-5, (tag, step)
        assert layer.hardening_x == pytest.approx(g.scalar(f"{tag}_s{step}_hx"))
        assert int(layer.weight.flipped_mask) == g.scalar(f"{tag}_s{step}_flips"), (tag, step)
        assert torch.equal(layer._hard_mask_from_soft(layer.mask.data).cpu(), g[f"{tag}_s{step}_hard"])
        with torch.no_grad():
            assert rel_err(layer(x), g[f"{tag}_s{step}_y"]) <= 1e-5
    if cfg.hard_mask_type == "block16":
        return
    # the blockified tensor is block-constant and keeps the ragged tail
    t = torch.rand(out_f, in_f, device=DEV)
    b = layer._blockify_tensor(t)
    bs = 16 if cfg.hard_mask_type == "block_sparse16" else 32
    ob, ib = out_f // bs, in_f // bs
    want = t.clone()
    want[: ob * bs, : ib * bs] = t[: ob * bs, : ib * bs].reshape(ob, bs, ib, bs).mean(dim=(1, 3)) \
        .repeat_interleave(bs, 0).repeat_interleave(bs, 1)
    assert rel_err(b, want) <= 1e-6


def test_mask_stats_block_keys():
    """mask_stats of a block-sparse layer adds the lower / upper half block means (legacy/utils.py:2155-2188)."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    g = Golden("block_masks")
    spec = json.loads(str(g["cases_json"]))["bs16"]
    cfg = sf.SparseLinearConfig(**dict(json.loads(str(g["base_json"])), **spec["cfg"]))
    layer = sf.SparseLinear(160, 128, sparselinear_config=cfg, bias=False).to(DEV)
    mask = g["bs16_s3_mask"]
    layer.mask.data.copy_(mask.to(DEV))
    st = U.mask_stats(layer, sample_per_layer=256)
    means = torch.sort(mask.reshape(8, 16, 10, 16).mean(dim=(1, 3)).flatten()).values.double()
    assert st["blk_total_blocks"] == 80
    assert st["blk_lower_half_mean"] == pytest.approx(float(means[:40].mean()), rel=1e-6)
    assert st["blk_upper_half_mean"] == pytest.approx(float(means[40:].mean()), rel=1e-6)
    assert st["blk_separation"] == pytest.approx(float(means[40:].mean() - means[:40].mean()), rel=1e-5)


def test_tile16_projection_ties_and_random():
    """Per-tile top-k against a stable descending sort of each tile: random values, heavy ties and
    the all-equal tile (the initial all-ones mask)."""
    from oracle import sparselinear_oracle as O
    from sparseforge_b200 import ops

    torch.manual_seed(9)
    for keep_k in (1, 64, 128, 200, 255):
        for soft in (torch.rand(64, 96), torch.randint(0, 4, (64, 96)).float() / 4, torch.ones(32, 32),
                     torch.randn(48, 80)):
            want = O._tile16_topk(soft, keep_k)
            got = ops.project_tile16(soft.to(DEV), keep_k)
            assert torch.equal(got.cpu(), want), (keep_k, tuple(soft.shape))
    assert int(ops.project_tile16(torch.rand(16, 16, device=DEV), 0).sum()) == 0
    assert int(ops.project_tile16(torch.rand(16, 16, device=DEV), 256).sum()) == 256
