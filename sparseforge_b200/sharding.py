"""Row sharding of a SparseLinear layer over the GPUs of one box.

Rows of the weight (``out_features``) are split evenly over the ranks of a process group. 2:4 groups
run along ``in_features``, so the soft mask, hard projection, metadata, Hessian diagonal, Adam state
and the weight gradient of a shard are local to its rank. What crosses ranks:

* forward: the output columns of the shards are all-gathered;
* backward: the partial input gradients of the shards are summed (all-reduce);
* mask update: the score normalisation is layer-wide (legacy/sparse_modeling.py:1084-1088), so
  sum(score), sum(score^2) of the shards are all-reduced before mean / std are formed.

The reference shards the same layer through FSDP flat parameters and gathers every parameter for a
mask update (legacy/utils.py:246-251); here nothing but the three items above is exchanged.
``RowShardedLinear`` does the exchange with ``torch.distributed`` collectives (NCCL on GPUs; backend-agnostic,
exercised with gloo in the CPU tests, differentiable twice); ``PeerShardedLinear`` does it inside the GEMM
epilogues through peer memory (``PeerArena``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


def shard_bounds(out_features: int, world: int, rank: int, multiple: int = 16) -> Tuple[int, int]:
    """[start, stop) rows of ``rank``. Every shard has out_features / world rows, a multiple of
    ``multiple`` (16 keeps block-16 tiles and 16-byte rows whole)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    if out_features % world != 0 or (out_features // world) % multiple != 0:
        raise ValueError(f"out_features={out_features} cannot be split into {world} shards of a multiple of {multiple} rows")
    rows = out_features // world
    return rank * rows, (rank + 1) * rows


def combine_score_sums(sums: torch.Tensor, n_local: int, group=None) -> Tuple[torch.Tensor, int]:
    """All-reduce (sum s, sum s^2) of the shards of one layer; returns the layer-wide sums and count."""
    world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
    if world > 1:
        dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
    return sums, n_local * world


class _GatherColumns(torch.autograd.Function):
    """[T, rows] per rank -> [T, rows * world]; backward keeps the rank's own column block."""

    @staticmethod
    def forward(ctx, y_local, group):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ctx.rank, ctx.rows = rank, y_local.shape[-1]
        flat = torch.empty(world * y_local.numel(), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(flat, y_local.contiguous().view(-1), group=group)
        parts = flat.view((world,) + tuple(y_local.shape))
        # parts[r] holds the columns of rank r: move the rank axis next to the column axis
        return parts.movedim(0, -2).reshape(*y_local.shape[:-1], world * y_local.shape[-1])

    @staticmethod
    def backward(ctx, gy):
        r, n = ctx.rank, ctx.rows
        return gy[..., r * n:(r + 1) * n].contiguous(), None


class _SumInputGrad(torch.autograd.Function):
    """Identity in forward; backward sums the partial input gradients of the shards."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, gx):
        gx = gx.contiguous()
        dist.all_reduce(gx, op=dist.ReduceOp.SUM, group=ctx.group)
        return gx, None


def gather_columns(y_local: torch.Tensor, group=None) -> torch.Tensor:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return y_local
    return _GatherColumns.apply(y_local, group)


def sum_input_grad(x: torch.Tensor, group=None) -> torch.Tensor:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return x
    return _SumInputGrad.apply(x, group)


class RowShardedLinear(nn.Module):
    """Wraps the shard of a linear layer held by this rank (any module mapping [..., in] to
    [..., out / world], e.g. a ``SparseLinear`` built with ``out_features // world`` rows)."""

    def __init__(self, shard: nn.Module, group=None):
        super().__init__()
        self.shard = shard
        self.group = group
        if hasattr(shard, "_row_shard_group"):
            shard._row_shard_group = group
            shard._row_sharded = True

    def forward(self, x):
        return gather_columns(self.shard(sum_input_grad(x, self.group)), self.group)


def shard_sparse_linear(full_weight: torch.Tensor, config, bias: Optional[torch.Tensor] = None, group=None,
                        device=None, dtype=None) -> RowShardedLinear:
    """Builds this rank's ``SparseLinear`` shard from the full weight and wraps it."""
    from .sparse_modeling import SparseLinear

    world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
    rank = dist.get_rank(group) if world > 1 else 0
    out_f, in_f = full_weight.shape
    lo, hi = shard_bounds(out_f, world, rank)
    layer = SparseLinear(in_f, hi - lo, sparselinear_config=config, bias=bias is not None)
    layer = layer.to(device=device or full_weight.device, dtype=dtype or full_weight.dtype)
    layer.mask.data = layer.mask.data.float()
    layer.hessian_diag.data = layer.hessian_diag.data.float()
    with torch.no_grad():
        layer.weight.copy_(full_weight[lo:hi])
        if bias is not None:
            layer.bias.copy_(bias[lo:hi])
    layer.initialize()
    return RowShardedLinear(layer, group)


class _PeerShardedFn(torch.autograd.Function):
    """Forward and backward of ``PeerShardedLinear``: the exchange is done by the GEMM epilogues."""

    @staticmethod
    def forward(ctx, x, weight, bias, mod):
        from . import ops

        shard, arena = mod.shard, mod.arena
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        T = x2.shape[0]
        mod._check(x2)
        wm = shard.masked_weight()
        par = mod._next_parity()
        y_off, _ = mod._offsets(par)
        rows = shard.out_features
        b = None if bias is None else bias.to(x2.dtype).contiguous()
        if arena.mc_base:
            ops.gemm_fwd_multicast(x2, wm, arena.mc_ptr(y_off), mod.out_total, arena.rank * rows, bias=b)
        else:
            ops.gemm_fwd_allgather(x2, wm, arena.ptrs(y_off), mod.out_total, arena.rank * rows, bias=b)
        arena.barrier()  # every rank's columns have landed once the stream is past this
        y = arena.view(y_off, (T, mod.out_total), x2.dtype).clone()
        ctx.save_for_backward(x2, wm)
        ctx.mod, ctx.par, ctx.x_shape, ctx.has_bias = mod, par, x.shape, bias is not None
        return y.view(*x.shape[:-1], mod.out_total)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy):
        from . import ops

        x2, wm = ctx.saved_tensors
        mod = ctx.mod
        arena, rows = mod.arena, mod.shard.out_features
        world, rank = arena.world, arena.rank
        T, in_f = x2.shape
        dyl = gy.reshape(-1, gy.shape[-1])[:, rank * rows:(rank + 1) * rows].contiguous()
        grad_x = grad_w = grad_b = None
        if ctx.needs_input_grad[1]:
            grad_w = ops.gemm_wgrad(dyl, x2)  # no mask: straight-through (legacy/sparse_modeling.py:117-125)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = ops.bias_grad(dyl).to(dyl.dtype)
        if ctx.needs_input_grad[0]:
            rows_t = T // world
            _, s_off = mod._offsets(ctx.par)
            # rows of owner c of this shard's partial input gradient go into the slot owner c keeps for this rank
            ops.gemm_dgrad_reducescatter(dyl, wm, arena.ptrs(s_off + rank * rows_t * in_f * 2), rank)
            arena.barrier()
            mine = ops.reduce_slots(arena.view(s_off, (world, rows_t, in_f), dyl.dtype))
            full = torch.empty(T, in_f, dtype=dyl.dtype, device=dyl.device)
            dist.all_gather_into_tensor(full, mine, group=arena.group)  # x is replicated: every rank needs all rows
            grad_x = full.view(ctx.x_shape)
        return grad_x, grad_w, grad_b, None


class PeerShardedLinear(nn.Module):
    """``RowShardedLinear`` with the exchange inside the GEMM kernels: the forward epilogue stores this
    shard's output columns into every rank's buffer (one multicast store per piece where the arena has
    a multicast address), the input-gradient epilogue stores every owner's token rows into that owner's
    slot, and the owner adds its slots (``ops.gemm_fwd_multicast`` / ``gemm_fwd_allgather``,
    ``gemm_dgrad_reducescatter``, ``reduce_slots``). One rank barrier per forward and one per backward
    (a one-element all-reduce on the current stream); the landing buffers alternate between two copies,
    so a buffer is rewritten only after every rank has passed a later barrier.

    bf16, more than 128 tokens per call, tokens a multiple of 8 and of the world size, at most
    ``max_tokens``. The backward is not differentiable a second time (use ``RowShardedLinear`` under a
    Hessian-vector product). Every rank must take the same calls in the same order, and ask for the input
    gradient on all ranks or on none."""

    N_BUFFERS = 2

    def __init__(self, shard: nn.Module, out_total: int, max_tokens: int, group=None, multicast: bool = True, arena=None):
        super().__init__()
        self.shard = shard
        self.group = group
        self.out_total = int(out_total)
        self.max_tokens = int(max_tokens)
        dev = shard.weight.device
        self._y_bytes = self.max_tokens * self.out_total * 2
        self._s_bytes = self.max_tokens * shard.in_features * 2
        self.arena = arena if arena is not None else PeerArena(self.N_BUFFERS * (self._y_bytes + self._s_bytes), dev, group,
                                                                multicast=multicast)
        if self.arena.world * shard.out_features != self.out_total:
            raise ValueError(f"{self.arena.world} shards of {shard.out_features} rows do not make {self.out_total}")
        self._calls = 0
        if hasattr(shard, "_row_shard_group"):
            shard._row_shard_group = group
            shard._row_sharded = True

    def _next_parity(self) -> int:
        self._calls += 1
        return self._calls % self.N_BUFFERS

    def _offsets(self, par: int):
        base = par * (self._y_bytes + self._s_bytes)
        return base, base + self._y_bytes

    def _check(self, x2: torch.Tensor) -> None:
        T = x2.shape[0]
        if x2.dtype != torch.bfloat16 or self.shard.weight.dtype != torch.bfloat16:
            raise TypeError("PeerShardedLinear: bfloat16 activations and weights (the sharded epilogues are bf16 only)")
        if T <= 128 or T % 8 or T % self.arena.world or T > self.max_tokens:
            raise ValueError(f"PeerShardedLinear: {T} tokens; need more than 128, a multiple of 8 and of the world size "
                             f"({self.arena.world}), at most max_tokens={self.max_tokens}")

    def forward(self, x):
        return _PeerShardedFn.apply(x, self.shard.weight, self.shard.bias, self)

    def close(self):
        """Releases the arena (every rank, no kernel in flight)."""
        if self.arena is not None:
            self.arena.close()
            self.arena = None


class PeerArena:
    """One device buffer per rank that every other rank of the node can store into: the landing
    zone of the sharded GEMM epilogues (``ops.gemm_fwd_allgather`` / ``ops.gemm_fwd_multicast`` /
    ``ops.gemm_dgrad_reducescatter``).

    Each rank allocates ``nbytes``, exports it through CUDA IPC, and opens the buffers of the other
    ranks; ``ptrs(offset)`` then lists, rank by rank, the address of the same byte offset in every
    arena (its own memory for its own rank). One export per rank, so a process never opens an
    allocation twice. ``barrier()`` orders ranks: what a rank stored before its barrier is in the
    peers' memory once they have passed theirs."""

    def __init__(self, nbytes: int, device, group=None, multicast: bool = True):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.mc_base = 0
        self._bases, self._ptrs, self._symm = [], [], None
        if multicast and self._open_symmetric(int(nbytes), device):
            pass
        else:
            self._open_ipc(int(nbytes), device)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)

    def _open_symmetric(self, nbytes: int, device) -> bool:
        """Arena in torch symmetric memory: peer addresses plus one multicast address whose stores
        the NVSwitch replicates into every rank's arena. All ranks agree on the outcome; False
        (nothing kept) when any of them could not map it, and the IPC arena is used instead."""
        buf = handle = None
        try:
            import torch.distributed._symmetric_memory as symm

            buf = symm.empty(nbytes, dtype=torch.uint8, device=torch.device(device))
            handle = symm.rendezvous(buf, dist.group.WORLD if self.group is None else self.group)
            ok = int(handle.multicast_ptr) != 0 and len(handle.buffer_ptrs) == self.world
        except Exception:  # no symmetric-memory support in this build / on this node
            ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if not int(flag.item()):
            return False
        self.buf, self._symm = buf, handle
        self._ptrs = [int(p) for p in handle.buffer_ptrs]
        self.mc_base = int(handle.multicast_ptr)
        return True

    def _open_ipc(self, nbytes: int, device) -> None:
        from . import ops

        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        handle, off = ops.peer_export(self.buf)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (handle, off), group=self.group)
        for r, (h, o) in enumerate(gathered):
            if r == self.rank:
                self._ptrs.append(self.buf.data_ptr())
            else:
                base, ptr = ops.peer_open(h, o)
                self._bases.append(base)
                self._ptrs.append(ptr)

    def mc_ptr(self, offset: int = 0) -> int:
        """Multicast address of byte ``offset`` of every rank's arena; 0 without multicast."""
        if offset % 16:
            raise ValueError("PeerArena offsets must be multiples of 16 bytes")
        return self.mc_base + int(offset) if self.mc_base else 0

    def ptrs(self, offset: int = 0):
        if offset % 16:
            raise ValueError("PeerArena offsets must be multiples of 16 bytes")
        return [p + int(offset) for p in self._ptrs]

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = torch.empty((), dtype=dtype).element_size()
        for d in shape:
            n *= int(d)
        return self.buf[offset:offset + n].view(dtype).view(*shape)

    def barrier(self, async_op: bool = False):
        """A one-element all-reduce ordered after the work already queued on the current stream.
        With ``async_op`` the returned work's ``wait()`` makes the current stream wait for it, so
        kernels queued in between run beside the barrier."""
        return dist.all_reduce(self._flag, group=self.group, async_op=async_op)

    def close(self):
        """Unmaps the peers' buffers and drops this rank's own. Every rank must call it, with none of
        its kernels in flight; the buffers are released even if the synchronisation in here fails, so
        that a rank never exits while its memory is still bound to the multicast object."""
        from . import ops

        try:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        finally:
            bases, self._bases = self._bases, []
            self.mc_base, self._symm, self.buf = 0, None, None
            for b in bases:
                ops.peer_close(b)
            torch.cuda.synchronize()
