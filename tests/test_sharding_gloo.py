"""Row-sharding collectives on CPU ranks (gloo, world size 2): gathering output columns, summing
partial input gradients and combining the score sums must reproduce the unsharded layer."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sparseforge_b200.sharding import RowShardedLinear, combine_score_sums, shard_bounds

        torch.manual_seed(0)  # identical "full" tensors on every rank
        out_f, in_f, T = 64, 48, 10
        W = torch.randn(out_f, in_f, dtype=torch.float64)
        X = torch.randn(2, T // 2, in_f, dtype=torch.float64)
        dY = torch.randn(2, T // 2, out_f, dtype=torch.float64)
        lo, hi = shard_bounds(out_f, world, rank)
        shard = torch.nn.Linear(in_f, hi - lo, bias=False, dtype=torch.float64)  # stand-in for the local shard
        with torch.no_grad():
            shard.weight.copy_(W[lo:hi])
        layer = RowShardedLinear(shard)
        x = X.clone().requires_grad_(True)
        y = layer(x)
        y.backward(dY)
        ref_x = X.clone().requires_grad_(True)
        ref_y = ref_x @ W.t()
        ref_y.backward(dY)
        ok = torch.allclose(y, ref_y) and torch.allclose(x.grad, ref_x.grad)
        ok = ok and torch.allclose(shard.weight.grad, (dY.reshape(T, out_f).t() @ X.reshape(T, in_f))[lo:hi])
        # layer-wide score statistics from per-shard sums
        score = (W * W)[lo:hi]
        sums = torch.stack([score.sum(), (score * score).sum()])
        sums, n = combine_score_sums(sums, score.numel())
        mean = sums[0] / n
        std = (sums[1] / n - mean * mean).sqrt()
        full = W * W
        ok = ok and n == full.numel() and torch.allclose(mean, full.mean()) and torch.allclose(std, full.std(unbiased=False))
        out_q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_row_sharded_layer_matches_unsharded_on_two_gloo_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    results = dict(q.get(timeout=10) for _ in range(world))
    assert results == {0: True, 1: True}


def _guard_worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sparseforge_b200 import utils as U

        # step 0: every rank is fine; step 1: rank 1 sees a NaN loss; step 2: rank 0's step raises
        seen = []
        seen.append(U.loss_is_finite_on_all_ranks(torch.tensor(1.5)))
        seen.append(U.loss_is_finite_on_all_ranks(torch.tensor(float("nan") if rank == 1 else 2.0)))
        try:
            if rank == 0:
                raise RuntimeError("injected host-side failure")
            ok = True
        except RuntimeError:
            ok = False
        seen.append(U.all_ranks_ok(ok))
        seen.append(U.all_ranks_ok(True))  # the group is still usable afterwards
        out_q.put((rank, seen))
    finally:
        dist.destroy_process_group()


def test_one_failing_rank_makes_every_rank_skip_the_step():
    """Failure detection as the reference does it: on the host, through an all-reduced ok-flag."""
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_guard_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    results = dict(q.get(timeout=10) for _ in range(world))
    assert results == {0: [True, False, False, True], 1: [True, False, False, True]}


def _accum_worker(rank, world, port, out_q):
    """Gradient accumulation under DistributedDataParallel with the loop's guard (legacy/main_llama.py:
    1997-2108): micro-steps before the last exchange nothing, the last one averages the accumulated
    gradients over the ranks; a non-finite loss on ONE rank makes EVERY rank leave the micro-step loop
    before its backward, so no collective is left unmatched and the next step runs normally."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from torch.nn.parallel import DistributedDataParallel as DDP

        from sparseforge_b200 import utils as U

        torch.manual_seed(0)
        core = torch.nn.Linear(6, 4, bias=False, dtype=torch.float64)
        model = DDP(core)
        accum = 3
        g = torch.Generator().manual_seed(10 + rank)
        xs = [torch.randn(5, 6, dtype=torch.float64, generator=g) for _ in range(accum)]

        def run_step(poison_at=None):
            """One optimizer step's worth of micro-steps; returns (skipped, grads seen after each micro-step)."""
            model.zero_grad(set_to_none=True)
            seen, skipped = [], False
            for micro in range(accum):
                last = micro == accum - 1
                with U.grad_sync_context(model, last):
                    loss = model(xs[micro]).pow(2).sum() / accum
                    if poison_at is not None and micro == poison_at[0] and rank == poison_at[1]:
                        loss = loss * float("nan")
                    if not U.loss_is_finite_on_all_ranks(loss):
                        skipped = True
                        break
                    loss.backward()
                seen.append(core.weight.grad.clone())
            return skipped, seen

        skipped, seen = run_step()
        ok = not skipped and len(seen) == accum
        local = [2 * (x @ core.weight.detach().t()).t() @ x / accum for x in xs]  # d/dW of sum((x W^T)^2) / accum
        # before the last micro-step the gradient is this rank's own running sum
        ok = ok and torch.allclose(seen[0], local[0]) and torch.allclose(seen[1], local[0] + local[1])
        # after it: the average over the ranks of the accumulated gradients
        total = local[0] + local[1] + local[2]
        both = [torch.zeros_like(total) for _ in range(world)]
        dist.all_gather(both, total)
        ok = ok and torch.allclose(seen[2], sum(both) / world)
        ok = ok and not torch.allclose(both[0], both[1])  # the ranks really had different data
        # a NaN on rank 1 at micro-step 1: both ranks skip, nothing hangs, and the next step is normal again
        skipped2, seen2 = run_step(poison_at=(1, 1))
        ok = ok and skipped2 and len(seen2) == 1
        skipped3, seen3 = run_step()
        ok = ok and not skipped3 and torch.allclose(seen3[2], sum(both) / world)
        out_q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_gradient_accumulation_without_sync_and_the_finite_loss_guard():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_accum_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    results = dict(q.get(timeout=10) for _ in range(world))
    assert results == {0: True, 1: True}


def test_single_process_is_a_no_op():
    from sparseforge_b200.sharding import gather_columns, sum_input_grad

    x = torch.randn(3, 4)
    assert gather_columns(x) is x and sum_input_grad(x) is x
