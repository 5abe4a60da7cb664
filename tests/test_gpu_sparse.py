"""GPU parity of the hard-2:4 compressed path and the block-sparse-16 path.

The reference has neither a compressed format nor a block-sparse backward; their semantics are the
dense masked products with the binary mask (legacy/main_llama.py:2552-2563,
legacy/sparse_modeling.py:72-132), which is what the oracle computes. Compressed values, metadata
and block-CSR indices are compared bit-exactly; GEMM outputs at 1e-2 (bf16) relative to the largest
reference magnitude.
"""
import pytest
import torch

from oracle import sparselinear_oracle as O
from tests.golden_io import Golden, rel_err

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from sparseforge_b200 import ops as _ops

    return _ops


def test_compress_round_trip_bit_exact(ops):
    torch.manual_seed(0)
    for shape in ((16, 64), (130, 256), (4096, 4096)):
        W = (torch.randn(shape) * 0.02).to(torch.bfloat16)
        vals, meta = ops.sparse24_compress(W.to(DEV), W.float().abs().to(DEV))
        ovals, ometa, ohard = O.sparse24_compress(W, W.float().abs())
        assert torch.equal(vals.cpu().view(torch.int16), ovals.view(torch.int16))
        assert torch.equal(meta.cpu(), ometa)
        dense = ops.sparse24_decompress(vals, meta)
        assert torch.equal(dense.cpu().float(), (W * ohard.to(torch.bfloat16)).float())  # +-0 compare equal


def test_compress_ties_lower_index(ops):
    W = torch.ones(8, 32).to(torch.bfloat16)
    vals, meta = ops.sparse24_compress(W.to(DEV), torch.ones(8, 32, device=DEV))
    assert bool((meta.cpu() == 0x44).all())  # columns 0 and 1 of every group: nibble 0 | 1 << 2


def test_pack_meta_is_the_documented_permutation(ops):
    torch.manual_seed(1)
    out, k = 256, 384
    meta = torch.randint(0, 256, (out, k // 8), dtype=torch.uint8)
    tc = ops.sparse24_pack_meta(meta.to(DEV), out, k).cpu()
    assert tc.numel() == (out // 128) * (k // 128) * 2048
    k_tiles = k // 128
    for (row, col) in [(0, 0), (7, 16), (8, 31), (137, 200), (255, 383), (128, 128), (100, 96)]:
        mt, m = divmod(row, 128)
        kt, kk = divmod(col, 128)
        m0, m1, m2 = m % 8, (m // 8) % 2, m // 16
        k0, k1, k2 = kk % 16, (kk // 16) % 2, kk // 32
        off = (mt * k_tiles + kt) * 2048 + 256 * m2 + 128 * k1 + 16 * m0 + 4 * k2 + 2 * m1 + (k0 >> 3)
        assert int(tc[off]) == int(meta[row, col // 8]), (row, col)


SPARSE_SHAPES = [
    (1, 128, 128), (16, 256, 128), (17, 384, 256), (128, 512, 384), (100, 272, 200), (1024, 1024, 512),
    (1, 4096, 4096), (16, 4096, 4096), (128, 4096, 11008), (1024, 11008, 4096), (8192, 4096, 4096),
    # one wave of 256 x 256 pair tiles (single accumulator): T = 1024 on 4096 rows, ragged variants
    (1024, 4096, 4096), (1000, 512, 1280), (520, 256, 4096),
    # two weight tiles per CTA: ragged token count, a weight-row count that half fills the last 512-row tile,
    # a row count that is not a multiple of 8 (scalar stores in the epilogue)
    (8000, 1024, 1280), (8192, 11008, 4096), (8192, 256, 4100),
]


@pytest.mark.parametrize("T,k,n", SPARSE_SHAPES)
def test_sparse24_gemm(ops, T, k, n):
    torch.manual_seed(T + k + n)
    W = (torch.randn(n, k, device=DEV) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    vals, meta = ops.sparse24_compress(W, W.float().abs())
    meta_tc = ops.sparse24_pack_meta(meta, n, k)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    y = ops.sparse24_gemm(x, vals, meta_tc, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, f"a device-side wait ran out, code {int(status[0])}"
    wd = ops.sparse24_decompress(vals, meta)
    ref = x.float() @ wd.float().t()
    assert rel_err(y, ref) <= BF16_TOL
    # and it agrees with the dense masked GEMM on the same pruned weight
    if T % 8 == 0 and n % 8 == 0:
        assert rel_err(y, ops.gemm_fwd(x, wd).float()) <= BF16_TOL


@pytest.mark.parametrize("T,k,n", [(8000, 1024, 1280), (8192, 4096, 4096), (8192, 512, 4104)])
def test_sparse24_gemm_one_tile_kernel_kept(ops, T, k, n, monkeypatch):
    """The one-tile pair kernel (the A/B switch) gives the same product as the default dispatch."""
    torch.manual_seed(T + k + n)
    W = (torch.randn(n, k, device=DEV) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    b = torch.randn(n, device=DEV).to(torch.bfloat16)
    vals, meta = ops.sparse24_compress(W, W.float().abs())
    meta_tc = ops.sparse24_pack_meta(meta, n, k)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    y2 = ops.sparse24_gemm(x, vals, meta_tc, bias=b, status=status)
    monkeypatch.setenv("SF_SPARSE24_ONE_TILE", "1")
    y1 = ops.sparse24_gemm(x, vals, meta_tc, bias=b, status=status)
    monkeypatch.delenv("SF_SPARSE24_ONE_TILE")
    assert int(status[0]) == 0
    assert torch.equal(y1, y2)  # same MMA order over K, same rounding
    ref = x.float() @ ops.sparse24_decompress(vals, meta).float().t() + b.float()
    assert rel_err(y2, ref) <= BF16_TOL


def test_sparse24_gemm_bias(ops):
    torch.manual_seed(5)
    T, k, n = 40, 256, 136
    W = (torch.randn(n, k, device=DEV) * 0.05).to(torch.bfloat16)
    x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    b = torch.randn(n, device=DEV).to(torch.bfloat16)
    vals, meta = ops.sparse24_compress(W, W.float().abs())
    y = ops.sparse24_gemm(x, vals, ops.sparse24_pack_meta(meta, n, k), bias=b)
    ref = x.float() @ ops.sparse24_decompress(vals, meta).float().t() + b.float()
    assert rel_err(y, ref) <= BF16_TOL


@pytest.mark.parametrize("T,k,n", [(1, 1024, 256), (16, 1152, 136), (100, 2048, 384), (128, 4096, 4096), (8, 11008, 4096)])
@pytest.mark.parametrize("splits", [0, 2, 3, 5, 8])
def test_sparse24_gemm_split_k(ops, T, k, n, splits):
    """K ranges of a weight tile computed by several CTAs and summed in the fp32 workspace give the
    unsplit result to fp32 rounding, with bias, and leave the workspace clean for the next call."""
    torch.manual_seed(T + k + n)
    W = (torch.randn(n, k, device=DEV) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    b = torch.randn(n, device=DEV).to(torch.bfloat16)
    vals, meta = ops.sparse24_compress(W, W.float().abs())
    meta_tc = ops.sparse24_pack_meta(meta, n, k)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    y1 = ops.sparse24_gemm(x, vals, meta_tc, bias=b, status=status, splits=1)
    ref = x.float() @ ops.sparse24_decompress(vals, meta).float().t() + b.float()
    for _ in range(3):  # the same workspace three times in a row
        ys = ops.sparse24_gemm(x, vals, meta_tc, bias=b, status=status, splits=splits)
        assert rel_err(ys, ref) <= BF16_TOL
        # one bf16 ulp at most against the unsplit kernel (fp32 sums in another order)
        assert float((ys.float() - y1.float()).abs().max()) <= 2.0 ** -7 * float(y1.float().abs().max())
        if _ == 0:
            first = ys.clone()
        assert torch.equal(ys, first)  # the partial sums are added in K order, whoever arrives last
    assert int(status[0]) == 0
    # the arrival tickets at the head of the workspace are back at zero
    ws = ops._SPLITK_WS[(torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)]
    assert int(ws[: 64 * 1024].count_nonzero()) == 0


# ---------------------------------------------------------------------------------------
# block-sparse-16
# ---------------------------------------------------------------------------------------
def test_bsr16_build_matches_reference_fixture(ops):
    g = Golden("block_sparse")
    blocks, row_ptr, col_idx = ops.bsr16_build(g["W"].to(DEV), g["mask"].to(DEV))
    assert torch.equal(row_ptr.cpu(), g["row_ptr"]) and torch.equal(col_idx.cpu(), g["col_idx"])
    assert torch.equal(blocks.cpu(), g["blocks"])
    y = ops.bsr16_fwd(g["X"].to(DEV), blocks, row_ptr, col_idx, g["W"].shape[0])
    assert rel_err(y, g["Y"]) <= 1e-5


@pytest.mark.parametrize("shape,T", [((64, 96), 24), ((256, 512), 200), ((11008, 4096), 2048)])
def test_bsr16_products(ops, shape, T):
    torch.manual_seed(shape[0])
    out, k = shape
    W = (torch.randn(out, k) * 0.02).to(torch.bfloat16)
    mask = O.block16_keep_mask(W.float(), 0.5).to(torch.bfloat16)
    blocks, row_ptr, col_idx = ops.bsr16_build(W.to(DEV), mask.to(DEV))
    ob, orp, oci = O.bsr16_convert(W, mask)
    assert torch.equal(row_ptr.cpu(), orp) and torch.equal(col_idx.cpu(), oci)
    assert torch.equal(blocks.cpu().float(), ob.float())
    assert int(row_ptr[-1]) == round(0.5 * (out // 16) * (k // 16))
    dense = ops.bsr16_to_dense(blocks, row_ptr, col_idx, out, k)
    assert torch.equal(dense.cpu().float(), (W * mask).float())
    x = torch.randn(T, k, device=DEV).to(torch.bfloat16)
    dy = torch.randn(T, out, device=DEV).to(torch.bfloat16)
    wd = dense.float()
    assert rel_err(ops.bsr16_fwd(x, blocks, row_ptr, col_idx, out), x.float() @ wd.t()) <= BF16_TOL
    assert rel_err(ops.bsr16_dgrad(dy, blocks, row_ptr, col_idx, k), dy.float() @ wd) <= BF16_TOL
    dblocks = ops.bsr16_wgrad(dy, x, row_ptr, col_idx)
    full = (dy.float().t() @ x.float())
    got_dense = ops.bsr16_to_dense(dblocks, row_ptr, col_idx, out, k).float()
    assert rel_err(got_dense, full * mask.to(DEV).float()) <= BF16_TOL


def test_block_sparse_linear_module(ops):
    from sparseforge_b200.block_sparse import BlockSparseLinear, get_sparsity_info

    torch.manual_seed(9)
    W = (torch.randn(128, 256, device=DEV) * 0.02).to(torch.bfloat16)
    mask = O.block16_keep_mask(W.float().cpu(), 0.5).to(DEV).to(torch.bfloat16)
    layer = BlockSparseLinear.from_dense(W, mask)
    info = get_sparsity_info(layer.block_row_indices, 256 // 16)
    assert info["block_sparsity"] == pytest.approx(0.5)
    x = torch.randn(2, 24, 256, device=DEV).to(torch.bfloat16).requires_grad_(True)
    layer.sparse_blocks.requires_grad_(True)
    y = layer(x)
    y.float().sum().backward()
    assert rel_err(y.reshape(48, 128), x.detach().float().reshape(48, 256) @ (W * mask).float().t()) <= BF16_TOL
    assert rel_err(x.grad.reshape(48, 256), torch.ones(48, 128, device=DEV) @ (W * mask).float()) <= BF16_TOL
    assert layer.sparse_blocks.grad.shape == layer.sparse_blocks.shape
    # the scattered weight is kept between calls: a second call reuses it, an in-place update of the blocks
    # (version counter) or an explicit invalidation rebuilds it
    with torch.no_grad():
        y2 = layer(x.detach())
        assert layer._workspace_key is not None and torch.equal(y2, y.detach())
        layer.sparse_blocks.mul_(2)
        assert rel_err(layer(x.detach()).float(), 2 * y.detach().float()) <= BF16_TOL
        layer.sparse_blocks.data.mul_(0.5)
        layer.invalidate_workspace()
        assert torch.equal(layer(x.detach()), y.detach())

