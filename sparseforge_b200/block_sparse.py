"""Block-sparse-16 linear layer on the B200 kernels.

Mirror of the reference's ``legacy/triton_block_sparse.py`` surface: ``convert_to_block_sparse``
(:46-103), ``get_sparsity_info`` (:106-120), ``BlockSparseLinear`` (:290-470) with ``from_dense`` /
``from_sparse_linear`` / ``forward``, and ``convert_model_to_block_sparse`` (:476-525). The block-CSR
layout is the reference's; it is built on the device. Unlike the reference (forward only, fp16
buffers), the layer keeps the weight dtype and is differentiable: dX and the gradient of the kept
blocks come from the dgrad / wgrad entry points.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import ops


def convert_to_block_sparse(weight: torch.Tensor, mask: torch.Tensor, block_size: int = 16
                            ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(sparse_blocks[nnz,16,16], block_row_indices[out/16+1] int32, block_col_indices[nnz] int32)."""
    if block_size != 16:
        raise NotImplementedError("only block_size=16 is implemented")
    out_f, in_f = weight.shape
    assert out_f % block_size == 0 and in_f % block_size == 0
    return ops.bsr16_build(weight.contiguous(), None if mask is None else mask.contiguous())


def get_sparsity_info(block_row_indices: torch.Tensor, num_block_cols: int) -> dict:
    rows = len(block_row_indices) - 1
    nnz = int(block_row_indices[-1].item())
    total = rows * num_block_cols
    sp = 1 - nnz / total
    return {"num_block_rows": rows, "num_block_cols": num_block_cols, "num_nonzero_blocks": nnz, "total_blocks": total,
            "block_sparsity": sp, "theoretical_speedup": 1 / (1 - sp) if sp < 1 else float("inf")}


class _BlockSparseFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, blocks, row_ptr, col_idx, bias, out_f, workspace, grad_workspace, dense_ready):
        ctx.save_for_backward(x2d, blocks, row_ptr, col_idx)
        ctx.workspace, ctx.grad_workspace, ctx.has_bias = workspace, grad_workspace, bias is not None
        return ops.bsr16_fwd(x2d, blocks, row_ptr, col_idx, out_f, bias=bias, workspace=workspace, dense_ready=dense_ready)

    @staticmethod
    def backward(ctx, gy):
        x2d, blocks, row_ptr, col_idx = ctx.saved_tensors
        gy = gy.contiguous()
        # the forward left the scattered weight in the workspace; the weight gradient has a workspace of its own
        gx = ops.bsr16_dgrad(gy, blocks, row_ptr, col_idx, x2d.shape[1], workspace=ctx.workspace, dense_ready=True) \
            if ctx.needs_input_grad[0] else None
        gb = ops.bsr16_wgrad(gy, x2d, row_ptr, col_idx, workspace=ctx.grad_workspace) if ctx.needs_input_grad[1] else None
        gbias = ops.bias_grad(gy).to(gy.dtype) if (ctx.has_bias and ctx.needs_input_grad[4]) else None
        return gx, gb, None, None, gbias, None, None, None, None


class BlockSparseLinear(nn.Module):
    def __init__(self, sparse_blocks, block_row_indices, block_col_indices, in_features, out_features,
                 bias: Optional[torch.Tensor] = None, block_size: int = 16):
        super().__init__()
        if block_size != 16:
            raise NotImplementedError("only block_size=16 is implemented")
        self.in_features, self.out_features, self.block_size = in_features, out_features, block_size
        self.sparse_blocks = nn.Parameter(sparse_blocks.contiguous(), requires_grad=False)
        self.register_buffer("block_row_indices", block_row_indices.contiguous())
        self.register_buffer("block_col_indices", block_col_indices.contiguous())
        if bias is not None:
            self.register_buffer("bias", bias.contiguous())
        else:
            self.bias = None
        self.sparsity_info = get_sparsity_info(block_row_indices, in_features // block_size)
        self._workspace = None
        self._workspace_key = None
        self._grad_workspace = None

    def invalidate_workspace(self):
        """Call after editing ``sparse_blocks`` through ``.data`` (an edit the version counter does not see)."""
        self._workspace_key = None

    @classmethod
    def from_dense(cls, weight, mask, bias=None, block_size: int = 16):
        blocks, rp, ci = convert_to_block_sparse(weight, mask, block_size)
        return cls(blocks, rp, ci, weight.shape[1], weight.shape[0], bias, block_size)

    @classmethod
    def from_sparse_linear(cls, sparse_linear_module, block_size: int = 16):
        w = sparse_linear_module.weight.data
        m = sparse_linear_module.hard_mask if hasattr(sparse_linear_module, "hard_mask") else sparse_linear_module.mask.data
        b = sparse_linear_module.bias.data if sparse_linear_module.bias is not None else None
        return cls.from_dense(w, m, b, block_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2d = x.reshape(-1, self.in_features).to(self.sparse_blocks.dtype).contiguous()
        if self._workspace is None or self._workspace.device != x2d.device or self._workspace.dtype != x2d.dtype:
            self._workspace = torch.empty((self.out_features, self.in_features), dtype=x2d.dtype, device=x2d.device)
            self._workspace_key = None
        # the scattered weight is kept between calls and rebuilt only when the blocks have changed
        key = (self.sparse_blocks.data_ptr(), self.sparse_blocks._version, self.block_col_indices.data_ptr())
        ready = self._workspace_key == key
        self._workspace_key = key
        grad_ws = None
        if torch.is_grad_enabled() and self.sparse_blocks.requires_grad:
            if self._grad_workspace is None or self._grad_workspace.device != x2d.device:
                self._grad_workspace = torch.empty_like(self._workspace)
            grad_ws = self._grad_workspace
        bias = None if self.bias is None else self.bias.to(x2d.dtype)
        y = _BlockSparseFn.apply(x2d, self.sparse_blocks, self.block_row_indices, self.block_col_indices, bias,
                                 self.out_features, self._workspace, grad_ws, ready)
        return y.view(*shape[:-1], self.out_features)

    def extra_repr(self) -> str:
        i = self.sparsity_info
        return (f"in_features={self.in_features}, out_features={self.out_features}, block_size={self.block_size}, "
                f"sparsity={i['block_sparsity']:.1%}, nnz_blocks={i['num_nonzero_blocks']}")


def convert_model_to_block_sparse(model: nn.Module, block_size: int = 16, target_modules: Optional[list] = None,
                                  verbose: bool = True) -> nn.Module:
    converted = 0
    for name, module in list(model.named_modules()):
        if hasattr(module, "hard_mask") or (hasattr(module, "mask") and hasattr(module, "weight")):
            if target_modules is not None and not any(t in name for t in target_modules):
                continue
            parent_name, _, attr = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, attr, BlockSparseLinear.from_sparse_linear(module, block_size))
            converted += 1
    if verbose:
        print(f"[convert] Total converted: {converted} layers")
    return model
