"""ctypes binding of ``libsparseforge_b200.so`` (declared in ``include/sparseforge_b200.h``).

There is no CPU or eager fallback: if the shared library is missing, loading fails with an
error that says how to build it, and every op in this package fails with it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libsparseforge_b200.so")

SF_F32, SF_BF16, SF_I8 = 0, 1, 2
METRICS = {"hessian_obd": 0, "hessian_ratio": 1, "magnitude": 2, "hessian": 3, "movement": 4}
PENALTY_NONE, PENALTY_TOPN, PENALTY_MID = 0, 1, 2
MSTAT_FLIPS, MSTAT_SUM_M, MSTAT_SUM_M1M, MSTAT_SUM_TOP2, MSTAT_SUM_BOT2, MSTAT_COUNT_LT_HALF = range(6)
MSTAT_COUNT = 8

_P = c_void_p
_SIGNATURES = {
    "sf_version": (c_int, []),
    "sf_last_error_string": (c_char_p, []),
    "sf_hutch_score_scratch_doubles": (c_int64, [c_int64]),
    "sf_hutch_score": (c_int, [_P, _P, c_int, _P, _P, c_int, _P, c_double, _P, _P, _P, c_int64, c_double, c_int, _P]),
    "sf_score_norm_from_sums": (c_int, [_P, c_double, _P, _P]),
    "sf_grad_hessian_ema": (c_int, [_P, _P, c_int, _P, c_int64, c_double, _P]),
    "sf_hutch_score_static_max_n": (c_int64, []),
    "sf_hutch_score_static": (c_int, [_P, _P, c_int, _P, _P, c_int, _P, c_double, _P, _P, c_int64, c_double, c_int, _P]),
    "sf_mask_update_nm24": (c_int, [_P, _P, _P, _P, _P, c_int, _P, _P, _P, c_int64, c_int64, c_double, c_double, c_double,
                                    c_int, c_double, c_double, c_double, c_int, c_int, _P]),
    "sf_mask_update_nm24_joint": (c_int, [_P, _P, _P, _P, _P, _P, c_int, _P, _P, _P, c_int64, c_int64, c_double, c_double,
                                          c_double, c_int, c_double, c_double, c_double, c_int, c_int, _P]),
    "sf_mask_update_nm24_from_weight": (c_int, [_P, c_int, _P, c_int, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_double,
                                                c_double, c_double, c_int, c_double, c_double, c_double, c_int, _P]),
    "sf_score_sum": (c_int, [_P, _P, _P, _P, _P, c_int64, _P]),
    "sf_project_nm24": (c_int, [_P, c_int, c_int64, _P, c_int, c_int64, _P, c_int64, c_int64, _P]),
    "sf_effective_weight": (c_int, [_P, c_int, _P, _P, _P, c_int64, c_int64, c_double, c_int, c_double, _P]),
    "sf_adamw_masked": (c_int, [_P, _P, _P, _P, _P, c_int, c_int64, c_double, c_double, c_double, c_double, c_double,
                                c_double, c_double, c_double, c_double, _P, c_double, c_int64, _P]),
    "sf_adamw_masked_amsgrad": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int64, c_double, c_double, c_double, c_double,
                                        c_double, c_double, c_double, c_double, c_double, _P]),
    "sf_adamw_masked_score": (c_int, [_P, _P, _P, _P, _P, c_int, c_int64, c_double, c_double, c_double, c_double,
                                      c_double, c_double, c_double, c_double, c_double, _P, _P, c_int, c_double,
                                      _P, _P, _P, _P, c_int, _P]),
    "sf_mask_stats": (c_int, [_P, _P, c_int64, c_int64, _P]),
    "sf_mask_update_nm": (c_int, [_P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int64, c_int64, c_int, c_int, c_double, c_double,
                                  c_double, c_int, c_double, c_double, c_double, c_int, c_int, c_int, _P]),
    "sf_project_nm": (c_int, [_P, c_int, c_int64, _P, c_int, c_int64, c_int64, c_int64, c_int, c_int, _P]),
    "sf_effective_weight_nm": (c_int, [_P, c_int, _P, _P, c_int64, c_int64, c_int, c_int, c_double, c_int, c_int, _P]),
    "sf_mask_update_tile16": (c_int, [_P, _P, _P, _P, _P, c_int, _P, _P, c_int64, c_int64, c_int, c_double, c_double, c_double,
                                      c_int, c_double, c_double, _P]),
    "sf_project_tile16": (c_int, [_P, _P, _P, c_int, _P, c_int64, c_int64, c_int, c_double, _P]),
    "sf_block_sums": (c_int, [_P, c_int64, c_int64, c_int, _P, _P, _P, _P]),
    "sf_block_mask_update": (c_int, [_P, c_int64, c_int64, c_int, _P, _P, c_double, c_double, c_double, _P, _P]),
    "sf_block_mask_apply": (c_int, [_P, _P, c_int, _P, c_int64, c_int64, c_int, _P, _P, c_double, _P]),
    "sf_mask_summary": (c_int, [_P, c_int64, c_double, _P, _P]),
    "sf_mask_sample_hist": (c_int, [_P, _P, c_int64, c_int, _P, _P]),
    "sf_masked_gemm_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, c_float, c_int, _P, _P]),
    "sf_masked_gemm_fwd_lowrank": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int, _P, _P]),
    "sf_masked_gemm_dgrad": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, _P, _P]),
    "sf_masked_gemm_wgrad": (c_int, [_P, _P, _P, c_int64, c_int64, c_int64, c_int, _P, _P]),
    "sf_masked_gemm_configure_stream": (c_int, [_P, c_int]),
    "sf_bias_grad": (c_int, [_P, c_int, _P, c_int64, c_int64, _P]),
    "sf_kl_div_fwd": (c_int, [_P, _P, c_int, c_int64, c_int64, c_double, c_double, _P, _P, _P]),
    "sf_kl_div_bwd": (c_int, [_P, _P, c_int, _P, _P, c_int64, c_int64, c_double, c_double, _P, _P]),
    "sf_masked_gemm_fwd_allgather": (c_int, [_P, _P, _P, _P, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                             c_int, _P, _P]),
    "sf_mask_update_nm24_frozen": (c_int, [_P, _P, _P, _P, c_double, c_double, c_int, _P, _P, c_int, _P, _P, _P, c_int64,
                                           c_int64, c_double, c_double, c_double, c_int, c_double, c_double, c_double,
                                           c_int, c_int, _P]),
    "sf_wanda_scratch_floats": (c_int64, [c_int64]),
    "sf_wanda_add_batch": (c_int, [_P, c_int, c_int64, c_int64, _P, c_int, c_double, c_double, _P, _P]),
    "sf_wanda_score": (c_int, [_P, c_int, _P, c_int, c_int64, c_int64, c_double, _P, _P, _P, _P]),
    "sf_masked_gemm_fwd_multicast": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int64, c_float,
                                             c_int, _P, _P]),
    "sf_masked_gemm_dgrad_reducescatter": (c_int, [_P, _P, _P, c_int, c_int, c_int64, c_int64, c_int64, c_int, _P, _P]),
    "sf_multimem_reduce": (c_int, [_P, _P, c_int64, c_int, c_int, _P]),
    "sf_reduce_slots": (c_int, [_P, _P, c_int64, c_int64, c_int, _P]),
    "sf_selftest_bounded_wait": (c_int, [c_double, _P, _P]),
    "sf_selftest_mma_issue_rate": (c_int, [c_int, c_int, c_int, c_int, _P, _P, _P]),
    "sf_peer_handle_bytes": (c_int, []),
    "sf_peer_export": (c_int, [_P, _P, _P]),
    "sf_peer_open": (c_int, [_P, c_int64, _P, _P]),
    "sf_peer_close": (c_int, [_P]),
    "sf_sparse24_compress": (c_int, [_P, _P, _P, _P, c_int64, c_int64, _P]),
    "sf_sparse24_decompress": (c_int, [_P, _P, _P, c_int64, c_int64, _P]),
    "sf_sparse24_meta_tc_bytes": (c_int64, [c_int64, c_int64]),
    "sf_sparse24_pack_meta": (c_int, [_P, _P, c_int64, c_int64, _P]),
    "sf_sparse24_gemm": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int64, c_int64, _P, _P]),
    "sf_sparse24_splitk_workspace_bytes": (c_int64, [c_int64, c_int64]),
    "sf_sparse24_gemm_splitk": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int64, c_int64, _P, c_int64, c_int, _P, _P]),
    "sf_bsr16_build": (c_int, [_P, _P, c_int, c_int, _P, _P, _P, _P, c_int64, c_int64, _P]),
    "sf_bsr16_to_dense": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int, _P]),
    "sf_bsr16_fwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int, _P, _P]),
    "sf_bsr16_dgrad": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int, _P, _P]),
    "sf_bsr16_wgrad": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int64, c_int, _P, _P]),
}

_lib = None


def declared_symbols() -> list[str]:
    return list(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """The loaded shared library. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"sparseforge_b200: {LIB_PATH} is missing. Build it with "
                "`python -m sparseforge_b200.build` (needs nvcc). There is no fallback path."
            )
        h = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            try:
                fn = getattr(h, name)
            except AttributeError:
                continue  # reported by callers of missing(); ops using it fail on call
            fn.restype = res
            fn.argtypes = args
        _lib = h
    return _lib


def missing_symbols() -> list[str]:
    h = lib()
    return [n for n in _SIGNATURES if not hasattr(h, n)]


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().sf_last_error_string()
        raise RuntimeError(f"sparseforge_b200 {what} failed ({rc}): {msg.decode() if msg else ''}")


class PreparedCall:
    """One library call whose arguments were converted to ctypes once.

    A training step issues the same calls on the same buffers thousands of times; converting two dozen
    Python numbers per call costs more host time than the launch itself. ``prepare(name, *values)``
    wraps every value in the ctypes type of the symbol's signature. A value that is already a ctypes
    instance is kept as is: such a *cell* (``ctypes.c_double()``, ``ctypes.c_void_p()``, ...) can be
    given a new ``.value`` between calls (step count, temperature, an input pointer). Calling the
    object issues the call and raises ``RuntimeError`` with the library's message on a non-zero code.
    The caller keeps the tensors behind the pointers alive."""

    __slots__ = ("name", "fn", "args")

    def __init__(self, name, fn, args):
        self.name, self.fn, self.args = name, fn, args

    def __call__(self):
        rc = self.fn(*self.args)
        if rc != 0:
            check(rc, self.name)


def prepare(name: str, *values) -> PreparedCall:
    res, argtypes = _SIGNATURES[name]
    if len(values) != len(argtypes):
        raise TypeError(f"{name}: {len(argtypes)} arguments expected, got {len(values)}")
    args = []
    for v, t in zip(values, argtypes):
        if isinstance(v, ctypes._SimpleCData) or isinstance(v, ctypes.Array):
            args.append(v)
        elif v is None:
            args.append(t())  # a null pointer
        else:
            args.append(t(v))
    return PreparedCall(name, getattr(lib(), name), tuple(args))
