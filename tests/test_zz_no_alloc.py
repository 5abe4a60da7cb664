"""sf_hutch_score_static: the score pass for callers that cannot allocate device memory.

Some users of this library call it from places where a device allocation is not possible or not
wanted: in the middle of a training step while the framework's caching allocator owns all free
memory, from code that must not trigger the device-wide synchronisation of cudaMalloc / cudaFree,
or under a fixed device-memory budget. ``sf_hutch_score_static`` serves them: it takes the same
inputs and outputs as ``sf_hutch_score`` but keeps its partial-sum scratch in an array inside the
library (32 KiB per GPU), so the call allocates nothing.

The test calls the entry point directly through the C ABI, twice in a row on different data and
sizes (the shared array still holds the first call's contents when the second one starts), and
checks H, score and the normalisation pair against ``sf_hutch_score`` with caller scratch, within
the 1e-5 tolerance the other fp32 tests use (the two paths run the same kernels, so the results
are expected to be identical). It also checks that a size beyond the built-in limit is refused.
This file sorts last so that a run that stops at the first failure has run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max()) / max(float(b.abs().max()), 1e-30)


def _run_pair(lib, rows, cols, seed, dtype, sf_dtype, dev="cuda"):
    g = torch.Generator(device=dev).manual_seed(seed)
    W = (torch.randn(rows, cols, device=dev, generator=g) * 0.02).to(dtype)
    hvp = (torch.randn(rows, cols, device=dev, generator=g) * 1e-2).to(dtype)
    v = torch.randint(0, 2, (rows, cols), device=dev, generator=g, dtype=torch.int8) * 2 - 1
    H0 = torch.rand(rows, cols, device=dev, generator=g) + 0.5
    n = rows * cols
    stream = torch.cuda.current_stream().cuda_stream
    SF_I8, HESSIAN_OBD = 2, 0

    # existing entry point, scratch supplied by the caller
    H_ref, score_ref = H0.clone(), torch.empty(rows, cols, device=dev)
    norm_ref = torch.zeros(2, device=dev)
    scratch = torch.empty(int(lib.sf_hutch_score_scratch_doubles(n)), dtype=torch.float64, device=dev)
    rc = lib.sf_hutch_score(hvp.data_ptr(), v.data_ptr(), SF_I8, H_ref.data_ptr(), W.data_ptr(), sf_dtype, None, 1.0,
                            score_ref.data_ptr(), norm_ref.data_ptr(), scratch.data_ptr(), n, 0.99, HESSIAN_OBD, stream)
    assert rc == 0, lib.sf_last_error_string()

    # new entry point: every buffer below exists before the call; the call allocates nothing
    H_new, score_new = H0.clone(), torch.empty(rows, cols, device=dev)
    norm_new = torch.zeros(2, device=dev)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    rc = lib.sf_hutch_score_static(hvp.data_ptr(), v.data_ptr(), SF_I8, H_new.data_ptr(), W.data_ptr(), sf_dtype, None,
                                   1.0, score_new.data_ptr(), norm_new.data_ptr(), n, 0.99, HESSIAN_OBD, stream)
    assert rc == 0, lib.sf_last_error_string()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    assert _rel(H_new, H_ref) <= TOL
    assert _rel(score_new, score_ref) <= TOL
    assert _rel(norm_new, norm_ref) <= TOL
    assert float(norm_new[1]) > 0


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from sparseforge_b200 import _lib

    lib = _lib.lib()
    # two calls back to back: different shape, dtype and data, so leftovers of the first call in the
    # shared array would show in the second
    _run_pair(lib, 512, 1024, seed=1, dtype=torch.bfloat16, sf_dtype=_lib.SF_BF16)
    _run_pair(lib, 96, 64, seed=2, dtype=torch.float32, sf_dtype=_lib.SF_F32)


def test_static_scratch_hessian_only_call():
    """With score = NULL the entry point only folds the Hutchinson sample into H (no partial sums
    are formed): same H as sf_hutch_score called the same way."""
    from sparseforge_b200 import _lib

    lib = _lib.lib()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(5)
    rows, cols = 200, 264
    hvp = (torch.randn(rows, cols, device=dev, generator=g) * 1e-2).to(torch.bfloat16)
    v = torch.randint(0, 2, (rows, cols), device=dev, generator=g, dtype=torch.int8) * 2 - 1
    H0 = torch.rand(rows, cols, device=dev, generator=g)
    stream = torch.cuda.current_stream().cuda_stream
    H_ref, H_new = H0.clone(), H0.clone()
    rc = lib.sf_hutch_score(hvp.data_ptr(), v.data_ptr(), _lib.SF_I8, H_ref.data_ptr(), None, _lib.SF_BF16, None, 1.0,
                            None, None, None, rows * cols, 0.98, 0, stream)
    assert rc == 0, lib.sf_last_error_string()
    rc = lib.sf_hutch_score_static(hvp.data_ptr(), v.data_ptr(), _lib.SF_I8, H_new.data_ptr(), None, _lib.SF_BF16, None,
                                   1.0, None, None, rows * cols, 0.98, 0, stream)
    assert rc == 0, lib.sf_last_error_string()
    torch.cuda.synchronize()
    assert _rel(H_new, H_ref) <= TOL
    assert not torch.equal(H_new, H0)


def test_static_scratch_on_a_second_device():
    """The array's device address is looked up once per device: a call on another GPU of the box must
    use that GPU's copy of the array (skipped on a one-GPU box)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from sparseforge_b200 import _lib

    lib = _lib.lib()
    _run_pair(lib, 128, 256, seed=3, dtype=torch.bfloat16, sf_dtype=_lib.SF_BF16)  # device 0 first
    with torch.cuda.device(1):
        _run_pair(lib, 160, 264, seed=4, dtype=torch.float32, sf_dtype=_lib.SF_F32, dev="cuda:1")
    _run_pair(lib, 96, 64, seed=6, dtype=torch.float32, sf_dtype=_lib.SF_F32)


def test_static_scratch_refuses_oversize():
    from sparseforge_b200 import _lib

    lib = _lib.lib()
    limit = int(lib.sf_hutch_score_static_max_n())
    assert limit == 67108864
    one = torch.zeros(8, device="cuda")
    rc = lib.sf_hutch_score_static(None, None, _lib.SF_I8, one.data_ptr(), one.data_ptr(), _lib.SF_F32, None, 1.0,
                                   one.data_ptr(), one.data_ptr(), ctypes.c_int64(limit + 8), 0.99, 0,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == -2  # SF_ERR_UNSUPPORTED, nothing launched
    assert b"exceeds the built-in scratch limit" in lib.sf_last_error_string()
