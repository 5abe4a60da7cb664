"""Row-sharded SparseLinear on two GPUs (NCCL) against the same layer unsharded on one GPU.
Skipped on a box with a single GPU. A rank leaves only after its last collective has completed."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    import traceback

    # a short collective timeout: if one rank fails, the other one errors out instead of waiting
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        import sparseforge_b200 as sf
        from sparseforge_b200 import utils as U
        from sparseforge_b200.sharding import shard_bounds, shard_sparse_linear

        torch.manual_seed(0)
        out_f, in_f, T = 512, 256, 256
        bf = torch.bfloat16
        W = (torch.randn(out_f, in_f) * 0.02).to(bf).to(dev)
        X = torch.randn(2, T // 2, in_f).to(bf).to(dev)
        dY = torch.randn(2, T // 2, out_f).to(bf).to(dev)
        cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", mask_update_period=1,
                                    sparsity_warmup_steps=0, mask_lr=0.1, mask_hardening_start=0, mask_hardening_duration=4)
        full = sf.SparseLinear(in_f, out_f, sparselinear_config=cfg, bias=False).to(dev).to(bf)
        full.weight.data.copy_(W)
        full.initialize()
        sharded = shard_sparse_linear(W, cfg)
        lo, hi = shard_bounds(out_f, world, rank)

        def rel(a, b):
            return float((a.double() - b.double()).abs().max()) / max(float(b.double().abs().max()), 1e-30)

        ok = True
        for step in range(2):
            U.calculate_model_mask(full, step=step)
            U.calculate_model_mask(sharded, step=step)
            ok = ok and rel(sharded.shard.mask.data, full.mask.data[lo:hi]) <= 1e-5
            ok = ok and sharded.shard.hardening_x == full.hardening_x
            x1 = X.clone().requires_grad_(True)
            x2 = X.clone().requires_grad_(True)
            y1, y2 = full(x1), sharded(x2)
            y1.backward(dY)
            y2.backward(dY)
            ok = ok and rel(y2, y1) <= 1e-2 and rel(x2.grad, x1.grad) <= 1e-2
            ok = ok and rel(sharded.shard.weight.grad, full.weight.grad[lo:hi]) <= 1e-2
        # the same exchange done by the GEMM epilogues through peer memory instead of NCCL
        from sparseforge_b200 import ops
        from sparseforge_b200.sharding import PeerArena

        Tt, in2, out2 = 512, 256, 512
        ol = out2 // world
        xs = torch.randn(Tt, in2, generator=torch.Generator().manual_seed(5)).to(bf).to(dev)
        wfull = (torch.randn(out2, in2, generator=torch.Generator().manual_seed(6)) * 0.05).to(bf).to(dev)
        dyf = torch.randn(Tt, out2, generator=torch.Generator().manual_seed(7)).to(bf).to(dev)
        y_bytes, slot_bytes = Tt * out2 * 2, Tt * in2 * 2
        arena = PeerArena(y_bytes + slot_bytes, dev, multicast=False)
        try:
            wl = wfull[rank * ol:(rank + 1) * ol].contiguous()
            dyl = dyf[:, rank * ol:(rank + 1) * ol].contiguous()
            rows = Tt // world
            ops.gemm_fwd_allgather(xs, wl, arena.ptrs(0), out2, rank * ol)
            ops.gemm_dgrad_reducescatter(dyl, wl, arena.ptrs(y_bytes + rank * rows * in2 * 2), rank)
            arena.barrier()
            y_full = arena.view(0, (Tt, out2), bf)
            dx_mine = ops.reduce_slots(arena.view(y_bytes, (world, rows, in2), bf))
            ok = ok and rel(y_full, ops.gemm_fwd(xs, wfull)) <= 1e-2
            ok = ok and rel(dx_mine, ops.gemm_dgrad(dyf, wfull)[rank * rows:(rank + 1) * rows]) <= 1e-2
        finally:
            arena.close()
        # the module whose forward / backward run those epilogues: same output and gradients as the unsharded layer
        from sparseforge_b200.sharding import PeerShardedLinear

        peer = PeerShardedLinear(sharded.shard, out_f, max_tokens=T, multicast=False)
        try:
            for _ in range(3):  # the two landing buffers are both reused
                full.weight.grad = None
                sharded.shard.weight.grad = None
                x1 = X.clone().requires_grad_(True)
                x2 = X.clone().requires_grad_(True)
                y1, y2 = full(x1), peer(x2)
                y1.backward(dY)
                y2.backward(dY)
                ok = ok and rel(y2, y1) <= 1e-2 and rel(x2.grad, x1.grad) <= 1e-2
                ok = ok and rel(sharded.shard.weight.grad, full.weight.grad[lo:hi]) <= 1e-2
            with torch.no_grad():
                ok = ok and rel(peer(X), full(X)) <= 1e-2
        finally:
            peer.close()
        flips = torch.tensor([int(sharded.shard.weight.flipped_mask)], device=dev)
        dist.all_reduce(flips)
        ok = ok and abs(int(flips) - int(full.weight.flipped_mask)) <= 2
        torch.cuda.synchronize()
        dist.barrier()
        q.put((rank, bool(ok)))
    except Exception:
        import sys

        msg = traceback.format_exc()
        print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)
        q.put((rank, msg))
        q.close()
        q.join_thread()
        os._exit(1)  # leave without waiting on the peer
    finally:
        dist.destroy_process_group()


def _multicast_worker(rank, world, port, q):
    """The output all-gather through the NVSwitch multicast address of a symmetric-memory arena
    (``multimem.st`` in the forward epilogue), in a process of its own. Whatever happens, a rank first
    drops its symmetric buffer (``PeerArena.close`` releases it even when its own synchronisation
    fails) and then leaves through a normal return: no rank exits while its memory is still bound to
    the multicast object."""
    import datetime
    import traceback

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    result, mc = "not run", None
    try:
        from sparseforge_b200 import ops
        from sparseforge_b200.sharding import PeerArena

        bf = torch.bfloat16
        Tt, in2, out2 = 512, 256, 512
        ol = out2 // world
        xs = torch.randn(Tt, in2, generator=torch.Generator().manual_seed(5)).to(bf).to(dev)
        wfull = (torch.randn(out2, in2, generator=torch.Generator().manual_seed(6)) * 0.05).to(bf).to(dev)
        wl = wfull[rank * ol:(rank + 1) * ol].contiguous()
        mc = PeerArena(Tt * out2 * 2, dev)
        if not mc.mc_base:
            result = "no multicast"  # the node offers no multicast object: the IPC arena is tested elsewhere
        else:
            mc.buf.zero_()
            mc.barrier()
            ops.gemm_fwd_multicast(xs, wl, mc.mc_ptr(0), out2, rank * ol)
            mc.barrier()
            got, want = mc.view(0, (Tt, out2), bf), ops.gemm_fwd(xs, wfull)
            err = float((got.double() - want.double()).abs().max()) / float(want.double().abs().max())
            same = len(mc.ptrs(0)) == world and mc.ptrs(0)[rank] == mc.buf.data_ptr()
            result = True if (err <= 1e-2 and same) else f"multicast all-gather differs: {err}"
            del got
            # the owner-side sum of the ranks' partial input gradients through the same multicast address
            # (multimem.ld_reduce): every rank holds a whole [T, in] partial, an owner reads the sum of its rows
            mc.barrier()
            parts = [(torch.randn(Tt, in2, generator=torch.Generator().manual_seed(40 + r))).to(bf) for r in range(world)]
            mc.view(0, (Tt, in2), bf).copy_(parts[rank].to(dev))
            torch.cuda.synchronize()
            mc.barrier()
            rows = Tt // world
            mine = torch.empty(rows, in2, dtype=bf, device=dev)
            ops.multimem_reduce(mc.mc_ptr(rank * rows * in2 * 2), mine, max_ctas=8)
            torch.cuda.synchronize()
            mc.barrier()
            want_sum = sum(p.double() for p in parts)[rank * rows:(rank + 1) * rows]
            err2 = float((mine.cpu().double() - want_sum).abs().max()) / float(want_sum.abs().max())
            if result is True and not err2 <= 1e-2:
                result = f"multimem reduce differs: {err2}"
    except Exception:
        result = traceback.format_exc()
    finally:
        try:
            if mc is not None:
                mc.close()
        except Exception:
            result = f"close failed after: {result}"
    q.put((rank, result))
    q.close()
    q.join_thread()
    try:
        dist.destroy_process_group()
    except Exception:
        pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_multicast_allgather_on_two_gpus():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_multicast_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=200)  # beyond the 60 s collective timeout, so that a failing rank has released its arena
    for p in procs:
        if p.is_alive():  # bounded: stop exactly the children this test started
            p.kill()
    results = {}
    while not q.empty():
        r, v = q.get(timeout=10)
        results[r] = v
    assert results in ({0: True, 1: True}, {0: "no multicast", 1: "no multicast"}), results


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_layer_matches_unsharded_on_two_gpus():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=150)
    for p in procs:
        if p.is_alive():  # bounded: stop exactly the children this test started
            p.kill()
    results = {}
    while not q.empty():
        r, v = q.get(timeout=10)
        results[r] = v
    assert results == {0: True, 1: True}, results


def _ddp_worker(rank, world, port, q):
    """Three steps of the training loop under DistributedDataParallel (each rank its half of the
    batch) against the same steps computed in one process from both halves: gradients averaged,
    clamp(hvp * v) averaged before the Hessian EMA (legacy/utils.py:860-865), masks identical."""
    import datetime
    import json
    import sys
    import traceback

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        from torch.nn.parallel import DistributedDataParallel as DDP

        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        import sparseforge_b200 as sf
        from golden_io import Golden
        from sparseforge_b200 import utils as U

        g = Golden("train_loop")
        hp, cfgd = json.loads(str(g["hp_json"])), json.loads(str(g["cfg_json"]))

        class TinyMLP(torch.nn.Module):
            def __init__(self):
                super().__init__()
                cfg = sf.SparseLinearConfig(**cfgd)
                self.fc1 = sf.SparseLinear(64, 128, sparselinear_config=cfg, bias=True)
                self.fc2 = sf.SparseLinear(128, 64, sparselinear_config=cfg, bias=False)

            def forward(self, x):
                return self.fc2(torch.nn.functional.gelu(self.fc1(x)))

        def make():
            m = TinyMLP().to(dev)
            m.load_state_dict({str(k): g["init/" + str(k)].to(dev) for k in g["state_keys"]}, strict=True)
            U.initialize_model(m)
            o = sf.AdamW([m.fc1.weight, m.fc1.bias, m.fc2.weight], lr=hp["lr"], betas=tuple(hp["betas"]),
                         weight_decay=hp["weight_decay"], srste_decay=cfgd["srste_decay"])
            return m, o

        dist_model, dist_opt = make()
        ddp = DDP(dist_model, device_ids=[rank])
        one_model, one_opt = make()

        def rel(a, b):
            return float((a.double() - b.double()).abs().max()) / max(float(b.double().abs().max()), 1e-30)

        ok = True
        X, Yt = g["X"].to(dev), g["Yt"].to(dev)
        mse = torch.nn.functional.mse_loss
        for it in range(3):
            lam = 0.1
            probes = [g[f"s{it}_probe{j}"].to(dev).float() for j in range(2)]
            halves = [(X[it][2 * r:2 * r + 2], Yt[it][2 * r:2 * r + 2]) for r in range(world)]
            # distributed: this rank's half
            xb, yb = halves[rank]
            loss = mse(ddp(xb), yb) + U.mid_penalty(ddp, lam)
            queue = [p.clone() for p in probes]
            U._rademacher_like = lambda t, qq=queue: qq.pop(0)
            U.update_hessian_hutchinson(ddp, loss)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(ddp.parameters(), hp["grad_clip"])
            dist_opt.step(decay=1e-4)
            dist_opt.zero_grad(set_to_none=True)
            U.calculate_model_mask(ddp, it, lambda_mid=lam)
            # one process: both halves, averaged by hand (run identically on every rank)
            layers = (one_model.fc1, one_model.fc2)
            ds = [torch.zeros_like(m.weight.data) for m in layers]
            losses = []
            for xh, yh in halves:
                lh = mse(one_model(xh), yh) + U.mid_penalty(one_model, lam)
                gr = torch.autograd.grad(lh, [m.weight for m in layers], create_graph=True, retain_graph=True)
                hv = torch.autograd.grad(sum((a * v).sum() for a, v in zip(gr, probes)), [m.weight for m in layers],
                                         retain_graph=True)
                for d, h, v in zip(ds, hv, probes):
                    d += torch.clamp((h * v).detach(), min=0.0) / world
                losses.append(lh)
            for m, d in zip(layers, ds):
                m.accumulate_hutchinson(d, torch.ones_like(d))
            (sum(losses) / world).backward()
            torch.nn.utils.clip_grad_norm_(one_model.parameters(), hp["grad_clip"])
            one_opt.step(decay=1e-4)
            one_opt.zero_grad(set_to_none=True)
            for m in layers:
                m.update_mask(it, lambda_mid=lam)
            for a, b in zip((dist_model.fc1, dist_model.fc2), layers):
                ok = ok and rel(a.weight.data, b.weight.data) <= 1e-4
                ok = ok and rel(a.hessian_diag.data, b.hessian_diag.data) <= 1e-4
                ok = ok and rel(a.mask.data, b.mask.data) <= 1e-4
                ok = ok and abs(int(a.weight.flipped_mask) - int(b.weight.flipped_mask)) <= 2
            ok = ok and U.loss_is_finite_on_all_ranks(loss)
        torch.cuda.synchronize()
        dist.barrier()
        q.put((rank, bool(ok)))
    except Exception:
        msg = traceback.format_exc()
        print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)
        q.put((rank, msg))
        q.close()
        q.join_thread()
        os._exit(1)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_training_loop_under_ddp_matches_one_process():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ddp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=150)
    for p in procs:
        if p.is_alive():
            p.kill()
    results = {}
    while not q.empty():
        r, v = q.get(timeout=10)
        results[r] = v
    assert results == {0: True, 1: True}, results
