"""Benchmark of the SparseLinear hot path on the LLaMA-2-7B layer set.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("llama2-7b-layerset-tempering"): the seven linear shapes of one LLaMA-2-7B decoder
layer (q/k/v/o [4096,4096], gate/up [11008,4096], down [4096,11008]) in bf16 with fp32 mask,
Hessian diagonal and score; activations [4,2048,in] (T = 8192 tokens). One step is one full
soft-mask tempering step of every matrix: masked forward GEMM, dgrad and wgrad GEMMs, Hutchinson
accumulate + |W|^2 H score, mask-aware AdamW, and the 2:4 soft-mask update with hard projection,
metadata and masked-weight emit, at a temperature annealed 1.0 -> 0.05 over 10 steps. Inputs are
seeded synthetic tensors with the shapes and N(0,0.02) / N(0,1) distributions of that model; the
Hessian-vector product fed to the Hutchinson kernel is a resident synthetic tensor (the parity tests
run the real double backward through the same three GEMM kernels).

`value` = algorithmic fwd+bwd GEMM FLOPs of the layer set (6*T*in*out per matrix) divided by the
whole step time, so the score / mask / optimizer passes count against it. With N GPUs the weights
are row-sharded (out/N rows per rank); the forward output is all-gathered and the input gradient
reduce-scattered by the GEMM epilogues through peer memory; the total work is fixed (strong scaling).

The N = 1 line also carries two compact blocks measured after the headline: `sparse24` (hard-2:4
compressed inference GEMM against the dense masked GEMM, three shapes x five activation heights) and
`bsr16` (block-sparse-16 products at the MLP shapes, 50 % of the blocks kept, 16384 tokens).

`--impl reference` times the reference's own Python code (compiled into oracle/_ref) on the host
cores; where that is missing, the oracle's restatement of it.
"""
from __future__ import annotations

import argparse
import ctypes
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

SHAPES = [("q", 4096, 4096), ("k", 4096, 4096), ("v", 4096, 4096), ("o", 4096, 4096),
          ("gate", 11008, 4096), ("up", 11008, 4096), ("down", 4096, 11008)]
DISTINCT = [("q", 4096, 4096), ("gate", 11008, 4096), ("down", 4096, 11008)]
T_TOKENS = 8192
METRIC = "SparseLinear fwd+bwd TFLOP/s (LLaMA-2-7B layer set, full tempering step)"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# algorithmic bytes per weight element at these dtypes (bf16 W/g/m/v/hvp, int8 probe, fp32 mask/H/score)
# optimizer pass: W,m,v read+written (12), g (2), hvp (2), probe (1), mask (4), H read+written (8);
# mask update: H (4), mask read+written (8), W (2), masked weight (2), metadata (0.125)
BYTES_OPTIM, BYTES_MASK = 29.0, 16.125
# DRAM bytes (read + write) of one GEMM launch from the ncu capture of the q-shaped matrix
# (mean of forward, dgrad, wgrad: 259.2 MB for 274.88 GFLOP), scaled to a launch by its FLOPs
GEMM_TRAFFIC_PER_GFLOP = 259.2e6 / 274.88
N_PARITY = 3  # landing buffers of the exchange: a buffer is rewritten three steps later
PULL_DEFAULT_WORLDS = ()  # world sizes whose input gradients go through the owner-side multimem reduce by default


def layer_flops(T, rows, cols):
    return 6.0 * T * rows * cols


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def schedule(it):
    """Temperature annealed 1.0 -> 0.05 over ten steps; hardening factor 1 -> 0 over steps 1..10."""
    decay_t = 0.05 ** (1.0 / 9.0)
    temp = max(0.05, decay_t ** (it % 10))
    hx = max(0.0, min(1.0, 1.0 - ((it % 10) - 1) / 9.0)) if (it % 10) >= 1 else 1.0
    return temp, hx


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons of one GPU while the timed region runs:
    read-only NVML queries every 10 ms from a thread, or one `nvidia-smi` query per sample where the NVML
    binding is missing. Nothing is set."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None
        self._nvml = self._handle = None
        try:
            import pynvml

            pynvml.nvmlInit()
            try:
                props = torch.cuda.get_device_properties(index)
                bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
                self._handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus)
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._nvml = pynvml
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n, h = self._nvml, self._handle
        sm = float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM))
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = int(get(h))
        flags = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        return [str(sm), str(self._max), ""] + ["Active" if bits & flags[k] else "Not Active" for k in self.NAMES]

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self.rows.append(self._sample_nvml())
                else:
                    out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                                          str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                    if out:
                        self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.01 if self._nvml is not None else 0.05)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, c in zip(self.NAMES, r[3:7]) if c.lower().startswith("active")})
        mx = max((float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()), default=None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm),
                "source": "nvml" if self._nvml is not None else "nvidia-smi"}


# ---------------------------------------------------------------------------------------------
# the product arm
# ---------------------------------------------------------------------------------------------
class Matrix:
    """One row shard of one SparseLinear weight with all its state resident in HBM, and the library
    calls of its step prepared once (sparseforge_b200._lib.prepare): per step only the cells change."""

    def __init__(self, index, name, rows, cols, rows_total, seed, dev):
        from sparseforge_b200 import ops

        g = torch.Generator(device=dev).manual_seed(seed)
        bf = torch.bfloat16
        self.index, self.name, self.rows, self.cols, self.rows_total = index, name, rows, cols, rows_total
        self.W = (torch.randn(rows, cols, device=dev, generator=g) * 0.02).to(bf)
        self.mask = torch.ones(rows, cols, device=dev)
        self.H = torch.ones(rows, cols, device=dev)
        self.m = torch.zeros(rows, cols, device=dev, dtype=bf)
        self.v = torch.zeros(rows, cols, device=dev, dtype=bf)
        self.hvp = (torch.randn(rows, cols, device=dev, generator=g) * 1e-3).to(bf)
        self.probe = (torch.randint(0, 2, (rows, cols), device=dev, generator=g, dtype=torch.int8) * 2 - 1)
        self.norm = torch.zeros(2, device=dev)
        self.scratch = ops.hutch_score_scratch(dev)
        self.stats = torch.zeros(8, dtype=torch.float64, device=dev)
        self.wm = torch.empty_like(self.W)
        self.dw = torch.empty_like(self.W)
        self.meta = torch.zeros(rows, cols // 8, dtype=torch.uint8, device=dev)
        ops.effective_weight(self.W, self.mask, self.wm, meta=self.meta, hx=1.0)
        # cells that change between calls
        self.x_ptr, self.dy_ptr = ctypes.c_void_p(), ctypes.c_void_p()
        self.bc1, self.bc2 = ctypes.c_double(), ctypes.c_double()
        self.temp, self.hx = ctypes.c_double(), ctypes.c_double()
        self.fwd = self.dgrad = self.wgrad = self.optim = self.mask_update = None
        self.reduce = []  # one prepared slot sum per parity


class Timers:
    def __init__(self):
        self.pairs = {}

    def region(self, key):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.pairs.setdefault(key, []).append((s, e))
        return s, e

    def totals_ms(self):
        return {k: sum(s.elapsed_time(e) for s, e in v) for k, v in self.pairs.items()}


def run_ours(args):
    import torch.distributed as dist

    from sparseforge_b200 import _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()  # fail loudly if the CUDA library is missing
    prepare = _lib.prepare
    T = T_TOKENS
    bf = torch.bfloat16
    shapes = [s for s in SHAPES if (not args.only or s[0] in args.only.split(","))]
    mats = [Matrix(j, n, r // world, c, r, 100 + i, dev)
            for j, (i, (n, r, c)) in enumerate((i, s) for i, s in enumerate(SHAPES) if s in shapes)]
    # activations: the same on every rank (seeded), one buffer per distinct width
    gx = torch.Generator(device=dev).manual_seed(7)
    widths = sorted({c for _, _, c in shapes} | {r for _, r, _ in shapes})
    X = {w: torch.randn(T, w, device=dev, generator=gx).to(bf) for w in widths}
    dYfull = {w: torch.randn(T, w, device=dev, generator=gx).to(bf) for w in widths}
    # a rank's upstream gradient is the column block of its own rows (what a split layer receives)
    dYres = {}
    for mt in mats:
        dYres[mt.name] = (dYfull[mt.rows_total] if world == 1 else
                          dYfull[mt.rows_total][:, rank * mt.rows:(rank + 1) * mt.rows].contiguous())

    main = torch.cuda.Stream(device=dev)   # tensor-core products
    dgs = torch.cuda.Stream(device=dev)    # input-gradient products, when they have a stream of their own
    wgs = torch.cuda.Stream(device=dev)    # weight-gradient products, when they run beside the exchange kernels
    side = torch.cuda.Stream(device=dev)   # HBM-bound tail of a matrix (optimizer + score, mask update)
    xchg = torch.cuda.Stream(device=dev)   # rank barrier and slot sums of the exchange
    copy_stream = torch.cuda.Stream(device=dev)
    overlap = args.overlap == "on" or (args.overlap == "auto" and world > 1)
    tail_stream = side if overlap else main

    # N > 1: the output all-gather and the input-gradient reduce-scatter are done by the GEMM epilogues
    # through peer memory. Every matrix has its own landing buffers (gathered output [T, out] and slots
    # [N, T/N, in]) in N_PARITY copies, used round-robin by step, so nothing is rewritten within a step
    # and ONE rank barrier per step orders everything: a rank joins the barrier of step s after its
    # products of step s and its slot sums of step s-1; it stores into the buffers of step s+3 only
    # after that barrier has completed. --collective nccl keeps the library collectives instead.
    arena, collective = None, "none"
    y_off, s_off = {}, {}
    if world > 1:
        collective = args.collective
        if collective == "p2p":
            try:
                from sparseforge_b200.sharding import PeerArena

                off = 0
                for p in range(N_PARITY):
                    for mt in mats:
                        y_off[(p, mt.index)] = off
                        off += T * mt.rows_total * 2
                        s_off[(p, mt.index)] = off
                        off += T * mt.cols * 2
                arena = PeerArena(off, dev, multicast=not args.no_multicast)
            except Exception as e:  # no peer mapping on this box: say so and use the library collectives
                print(f"[bench] peer memory unavailable ({e}); using NCCL collectives", file=sys.stderr, flush=True)
                collective = "nccl"
        flags = torch.tensor([1 if collective == "p2p" else 0], device=dev)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        if int(flags) == 0 and collective == "p2p":
            if arena is not None:
                arena.close()
            arena, collective = None, "nccl"
    allgather = "none" if arena is None else "multimem" if arena.mc_base else "stores"
    # Input-gradient reduce-scatter. "scatter": the dgrad epilogue stores every owner's rows into that
    # owner's slot, the owner adds its slots. "pull": dgrad writes its whole partial into this rank's
    # symmetric buffer at local speed; after the step's rank barrier every owner reads the sum of ITS rows
    # through the multicast address (multimem.ld_reduce: the switch adds the copies), on the exchange
    # stream, beside the tail of this step and the forward products of the next.
    pull = (arena is not None and bool(arena.mc_base) and
            (args.dgrad_exchange == "pull" or (args.dgrad_exchange == "auto" and world in PULL_DEFAULT_WORLDS)))
    if args.dgrad_exchange == "pull" and arena is not None and not pull:
        print("[bench] no multicast object on this node: the input gradients go through the store-based scatter",
              file=sys.stderr, flush=True)
    # From four GPUs on, the forward and input-gradient kernels wait on NVLink while the tensor cores idle.
    # The three products of a matrix are independent of one another, so each can have its own stream and a
    # share of the SMs: --gemm-ctas f,d,w gives the thread blocks of forward, input gradient and weight
    # gradient; a product with 0 runs on the forward's stream. Default: one stream up to two GPUs.
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    shares = args.gemm_ctas or ({4: "100,0,48", 8: "116,0,32"}.get(world, "0,0,0") if arena is not None else "0,0,0")
    f_ctas, d_ctas, w_ctas = [max(0, int(v)) // 2 * 2 for v in shares.split(",")]
    if not overlap:
        d_ctas = w_ctas = 0
    ops.gemm_configure_stream(main, max_ctas=f_ctas)
    ops.gemm_configure_stream(dgs, max_ctas=d_ctas)
    ops.gemm_configure_stream(wgs, max_ctas=w_ctas)
    s_fwd, s_dgrad, s_wgrad = main, (dgs if d_ctas else main), (wgs if w_ctas else main)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    rows_t = T // world

    # ---- prepared calls -------------------------------------------------------------------------
    ms, ss = main.cuda_stream, tail_stream.cuda_stream
    ds, ws_ = s_dgrad.cuda_stream, s_wgrad.cuda_stream
    # N = 1: one output buffer per shape (stream order keeps its uses apart); with library collectives every
    # matrix has its own, because a collective may still read the buffer when the next product starts
    own = world > 1 and arena is None
    y_buf = {(mt.index if own else mt.rows): None for mt in mats}
    dx_buf = {(mt.index if own else mt.cols): None for mt in mats}
    for mt in mats:
        ky, kx = (mt.index, mt.index) if own else (mt.rows, mt.cols)
        if arena is None and y_buf[ky] is None:
            y_buf[ky] = torch.empty(T, mt.rows, dtype=bf, device=dev)
        if arena is None and dx_buf[kx] is None:
            dx_buf[kx] = torch.empty(T, mt.cols, dtype=bf, device=dev)
        mt.y, mt.dx = y_buf[ky], dx_buf[kx]
    dxs = {mt.index: torch.empty(rows_t, mt.cols, dtype=bf, device=dev) for mt in mats} if arena is not None else {}
    P = lambda t: t.data_ptr()  # noqa: E731
    BF = _lib.SF_BF16
    y_cells = {mt.index: ctypes.c_void_p() for mt in mats}      # destination of the output all-gather (per parity)
    slot_arrays = {}                                            # dgrad slot pointers, per (parity, matrix)
    for mt in mats:
        if arena is None:
            mt.fwd = prepare("sf_masked_gemm_fwd", mt.x_ptr, P(mt.wm), None, P(mt.y), T, mt.cols, mt.rows, 1.0, BF,
                             P(status), ms)
            mt.dgrad = prepare("sf_masked_gemm_dgrad", mt.dy_ptr, P(mt.wm), P(mt.dx), T, mt.cols, mt.rows, BF,
                               P(status), ds)
        else:
            if arena.mc_base:
                mt.fwd = prepare("sf_masked_gemm_fwd_multicast", mt.x_ptr, P(mt.wm), None, y_cells[mt.index], T, mt.cols,
                                 mt.rows, mt.rows_total, rank * mt.rows, 1.0, BF, P(status), ms)
            else:
                mt.fwd_arrays = [(ctypes.c_void_p * world)(*arena.ptrs(y_off[(p, mt.index)])) for p in range(N_PARITY)]
                mt.fwd = [prepare("sf_masked_gemm_fwd_allgather", mt.x_ptr, P(mt.wm), None, mt.fwd_arrays[p], world, T,
                                  mt.cols, mt.rows, mt.rows_total, rank * mt.rows, 1.0, BF, P(status), ms)
                          for p in range(N_PARITY)]
            if pull:
                mt.dgrad = [prepare("sf_masked_gemm_dgrad", mt.dy_ptr, P(mt.wm), arena.buf.data_ptr() + s_off[(p, mt.index)],
                                    T, mt.cols, mt.rows, BF, P(status), ds) for p in range(N_PARITY)]
                mt.reduce = [prepare("sf_multimem_reduce", arena.mc_ptr(s_off[(p, mt.index)] + rank * rows_t * mt.cols * 2),
                                     P(dxs[mt.index]), rows_t * mt.cols, BF, args.pull_ctas, xchg.cuda_stream)
                             for p in range(N_PARITY)]
            else:
                for p in range(N_PARITY):
                    slot_arrays[(p, mt.index)] = (ctypes.c_void_p * world)(
                        *arena.ptrs(s_off[(p, mt.index)] + rank * rows_t * mt.cols * 2))
                mt.dgrad = [prepare("sf_masked_gemm_dgrad_reducescatter", mt.dy_ptr, P(mt.wm), slot_arrays[(p, mt.index)],
                                    world, rank, T, mt.cols, mt.rows, BF, P(status), ds) for p in range(N_PARITY)]
                mt.reduce = [prepare("sf_reduce_slots", arena.buf.data_ptr() + s_off[(p, mt.index)], P(dxs[mt.index]), world,
                                     rows_t * mt.cols, BF, xchg.cuda_stream) for p in range(N_PARITY)]
        mt.wgrad = prepare("sf_masked_gemm_wgrad", mt.dy_ptr, mt.x_ptr, P(mt.dw), T, mt.cols, mt.rows, BF, P(status), ws_)
        # the reference's order: Hutchinson sample into H, optimizer step, score statistics of the NEW weight
        # (one pass over the matrix); the mask update forms the score again from W and H (it reads W anyway),
        # so the optimizer pass writes no score tensor
        mt.optim = prepare("sf_adamw_masked_score", P(mt.W), P(mt.dw), P(mt.mask), P(mt.m), P(mt.v), BF, mt.W.numel(), 1e-4,
                           0.9, 0.95, 1e-8, 0.1, 2e-4, mt.bc1, mt.bc2, 0.0, P(mt.hvp), P(mt.probe), _lib.SF_I8, 0.99,
                           P(mt.H), None, P(mt.norm), P(mt.scratch), _lib.METRICS["hessian_obd"], ss)
        mt.mask_update = prepare("sf_mask_update_nm24_from_weight", P(mt.W), BF, P(mt.H), _lib.METRICS["hessian_obd"],
                                 P(mt.norm), None, P(mt.mask), P(mt.wm), P(mt.meta), P(mt.stats), mt.rows, mt.cols, mt.temp,
                                 0.1, 0.0, _lib.PENALTY_NONE, 0.0, 0.0, mt.hx, 0, ss)
    launches = 0

    # end-to-end leg: two staging buffers per operand, filled from pinned host memory on a copy stream
    stage_free = [torch.cuda.Event(), torch.cuda.Event()]
    step_done = [torch.cuda.Event(), torch.cuda.Event()]
    stage_xw = stage_dy = host_X = host_dY = None
    x_group = None  # its own communicator, so that these all-gathers never queue behind a step's rank barrier
    first_use = {}
    for j_, mt_ in enumerate(mats):
        first_use.setdefault(mt_.cols, j_)

    def prefetch(j, it):
        """Queues the host->device copies of matrix j's inputs on the copy stream. The activation
        of a width is an input of the step, shared by the matrices of that width (q, k, v, o, gate,
        up read the same 4096-wide tensor): it is copied once per step, into the buffer of the
        step's parity; the upstream gradient is per matrix."""
        mt, b, p = mats[j], j % 2, it % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(stage_free[b])
            xs = stage_xw[mt.cols][p]
            if first_use[mt.cols] == j:
                copy_stream.wait_event(step_done[p])  # the step before last has finished with this buffer
                if x_group is None:
                    xs.copy_(host_X[mt.cols], non_blocking=True)
                else:
                    # every rank needs the whole activation: each copies its T/N rows from the host and the rows
                    # are all-gathered over NVLink, so the step's inputs cross the host links once, not N times
                    mine = xs[rank * rows_t:(rank + 1) * rows_t]
                    mine.copy_(host_X[mt.cols], non_blocking=True)
                    dist.all_gather_into_tensor(xs, mine, group=x_group)
            dys = stage_dy[b][: T * mt.rows].view(T, mt.rows)
            dys.copy_(host_dY[mt.name], non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(copy_stream)
        return xs, dys, ready

    # events reused every step
    prod_streams = list(dict.fromkeys([s_fwd, s_dgrad, s_wgrad]))
    done_f = [torch.cuda.Event() for _ in mats]
    done_d = [torch.cuda.Event() for _ in mats]
    done_w = [torch.cuda.Event() for _ in mats]
    tail_done = [torch.cuda.Event() for _ in mats]
    tail_recorded = [False] * len(mats)
    stores_done = [torch.cuda.Event() for _ in prod_streams]
    barrier_done = [torch.cuda.Event() for _ in range(N_PARITY)]
    nccl_work = []

    def step(it, timers=None, e2e=False):
        nonlocal launches
        par = it % N_PARITY
        temp, hx = schedule(it)
        bc1, bc2 = 1.0 - 0.9 ** (it + 1), 1.0 - 0.95 ** (it + 1)
        if arena is not None and it >= N_PARITY:
            # the landing buffers of this parity were last read by the slot sums of step it - 3; every
            # rank has finished those before it joined the barrier of step it - 2
            for st in prod_streams:
                st.wait_event(barrier_done[(it - 2) % N_PARITY])
        pending = prefetch(0, it) if e2e else None
        for i, mt in enumerate(mats):
            if e2e:
                # inputs of this matrix arrive from pinned host memory on the copy stream while the
                # previous matrix computes; the next matrix's copy is queued before this one's kernels
                x, dy, ready = pending
                pending = prefetch(i + 1, it) if i + 1 < len(mats) else None
                for st in prod_streams:
                    st.wait_event(ready)
            else:
                x, dy = X[mt.cols], dYres[mt.name]
            mt.x_ptr.value, mt.dy_ptr.value = x.data_ptr(), dy.data_ptr()
            mt.bc1.value, mt.bc2.value, mt.temp.value, mt.hx.value = bc1, bc2, temp, hx
            if overlap and tail_recorded[i]:
                # this step's products read the masked weight the last tail wrote, and overwrite the weight
                # gradient it read
                for st in prod_streams:
                    st.wait_event(tail_done[i])

            def timed(key, call, stream):
                nonlocal launches
                if timers is None:
                    call()
                else:
                    s, e = timers.region(key.split(":")[0])
                    if ":" in key:  # also listed under its own kind (rank 0's breakdown in `passes`)
                        timers.pairs.setdefault(key, []).append((s, e))
                    s.record(stream)
                    call()
                    e.record(stream)
                launches += 1

            # the weight gradient first: it has the fewest thread blocks and then holds its SMs from the start
            if s_wgrad is not main:
                timed("gemm:wgrad", mt.wgrad, s_wgrad)
            if arena is not None:
                if arena.mc_base:
                    y_cells[mt.index].value = arena.mc_ptr(y_off[(par, mt.index)])
                    timed("gemm:fwd", mt.fwd, s_fwd)
                else:
                    timed("gemm:fwd", mt.fwd[par], s_fwd)
                timed("gemm:dgrad", mt.dgrad[par], s_dgrad)
            else:
                timed("gemm:fwd", mt.fwd, s_fwd)
                if world > 1:  # library collectives on NCCL's own stream, beside the next products
                    with torch.cuda.stream(main):
                        yg = torch.empty(world, T, mt.rows, dtype=bf, device=dev)
                        nccl_work.append(dist.all_gather_into_tensor(yg, mt.y, async_op=True))
                timed("gemm:dgrad", mt.dgrad, s_dgrad)
                if world > 1:
                    with torch.cuda.stream(main):
                        dxo = torch.empty(rows_t, mt.cols, dtype=bf, device=dev)
                        nccl_work.append(dist.reduce_scatter_tensor(dxo, mt.dx, async_op=True))
            if s_wgrad is main:
                timed("gemm:wgrad", mt.wgrad, s_wgrad)
            if overlap:
                # the tail rewrites the masked weight (read by forward and input gradient) and reads the weight
                # gradient: it starts when all three products of the matrix are done
                done_f[i].record(s_fwd)
                done_d[i].record(s_dgrad)
                done_w[i].record(s_wgrad)
                for ev in (done_f[i], done_d[i], done_w[i]):
                    side.wait_event(ev)
            timed("optim", mt.optim, tail_stream)
            launches += 1  # the one-block statistics kernel behind the score
            timed("mask", mt.mask_update, tail_stream)
            if overlap:
                tail_done[i].record(side)
                tail_recorded[i] = True
            if e2e:
                for st in prod_streams:
                    if st is not main:
                        main.wait_stream(st)
                stage_free[i % 2].record(main)
        if arena is not None:
            for ev, st in zip(stores_done, prod_streams):
                ev.record(st)
                xchg.wait_event(ev)
            with torch.cuda.stream(xchg):
                arena.barrier(async_op=True).wait()  # the exchange stream waits; the host does not
                barrier_done[par].record(xchg)
                for mt in mats:
                    timed("reduce", mt.reduce[par], xchg)
        for wk in nccl_work:
            with torch.cuda.stream(main):
                wk.wait()
        nccl_work.clear()
        if e2e:
            join_streams()
            step_done[it % 2].record(main)
            with torch.cuda.stream(main):
                return torch.stack([mt.stats for mt in mats]).to("cpu", non_blocking=False)
        return None

    def join_streams():
        for st in (side, xchg, dgs, wgs):
            main.wait_stream(st)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    torch.cuda.synchronize()
    it_next = 0
    host_warm = []
    for _ in range(args.warmup):
        h0 = time.perf_counter()
        step(it_next)
        host_warm.append((time.perf_counter() - h0) * 1e3)
        it_next += 1
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # N = 1: every launch is bracketed by events inside the headline loop (the device is saturated, the
    # host runs ahead). N > 1: the headline loop carries no per-launch events; the kinds are timed in a
    # short separate pass below.
    timers = Timers() if world == 1 else None
    launches = 0
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # at N > 1 a step lasts 2-5 ms and the host is only a step or two ahead of the devices: a collector pause
    # on one rank would stall every rank, so the collector rests while the steps are being issued
    gc.collect()
    gc.disable()
    t0.record(main)
    host_t0 = time.perf_counter()
    for _ in range(args.steps):
        step(it_next, timers)
        it_next += 1
    host_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps  # time to ENQUEUE one step (no sync inside)
    join_streams()
    t1.record(main)
    barrier()
    gc.enable()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t0.elapsed_time(t1)
    launches_timed = launches
    kinds_steps = args.steps
    if world > 1:
        timers = Timers()
        kinds_steps = 3
        for _ in range(kinds_steps):
            step(it_next, timers)
            it_next += 1
        join_streams()
        barrier()
    part = timers.totals_ms()

    # the exchange, checked on every rank outside the timing: one q-shaped matrix, gathered output and
    # summed input gradient against the unsharded products of the same operands
    exchange_err = None
    if arena is not None:
        mt = mats[0]
        par = it_next % N_PARITY
        with torch.cuda.stream(main):
            x, dy = X[mt.cols], dYres[mt.name]
            mt.x_ptr.value, mt.dy_ptr.value = x.data_ptr(), dy.data_ptr()
            arena.view(y_off[(par, mt.index)], (T, mt.rows_total), bf).zero_()
            arena.view(s_off[(par, mt.index)], (world, rows_t, mt.cols), bf).zero_()
            torch.cuda.synchronize()
            dist.barrier()
            if arena.mc_base:
                y_cells[mt.index].value = arena.mc_ptr(y_off[(par, mt.index)])
                mt.fwd()
            else:
                mt.fwd[par]()
            mt.dgrad[par]()
            torch.cuda.synchronize()
            dist.barrier()
            if pull:
                dx_mine = torch.empty(rows_t, mt.cols, dtype=bf, device=dev)
                ops.multimem_reduce(arena.mc_ptr(s_off[(par, mt.index)] + rank * rows_t * mt.cols * 2), dx_mine)
                torch.cuda.synchronize()
                dist.barrier()  # nobody rewrites its partial while another rank still reads it
            else:
                dx_mine = ops.reduce_slots(arena.view(s_off[(par, mt.index)], (world, rows_t, mt.cols), bf))
            y_all = arena.view(y_off[(par, mt.index)], (T, mt.rows_total), bf)
            wm_full = torch.empty(world * mt.rows, mt.cols, dtype=bf, device=dev)
            dist.all_gather_into_tensor(wm_full, mt.wm)
            dy_parts = torch.empty(world, T, mt.rows, dtype=bf, device=dev)
            dist.all_gather_into_tensor(dy_parts, dy.contiguous())
            dy_full = dy_parts.permute(1, 0, 2).reshape(T, world * mt.rows).contiguous()
            y_ref = ops.gemm_fwd(x, wm_full)
            dx_ref = ops.gemm_dgrad(dy_full, wm_full)[rank * rows_t:(rank + 1) * rows_t]
            rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max())  # noqa: E731
            exchange_err = max(rel(y_all, y_ref), rel(dx_mine, dx_ref))
            del y_all
        errs = torch.tensor([exchange_err], dtype=torch.float64, device=dev)
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        exchange_err = float(errs)

    # end to end: the same step fed from pinned host buffers, stats read back every step
    h2d = sum(T // world * w * 2 for w in {c for _, _, c in shapes}) + sum(T * (r // world) * 2 for _, r, _ in shapes)
    d2h = len(shapes) * 8 * 8
    e2e_ms = float("nan")
    if not args.no_e2e:
        if world > 1:
            x_group = dist.new_group(list(range(world)), backend="nccl")
        host_X = {w: X[w][rank * rows_t:(rank + 1) * rows_t].cpu().pin_memory() for w in {c for _, _, c in shapes}}
        host_dY = {mt.name: dYres[mt.name].cpu().pin_memory() for mt in mats}
        wmax = max(mt.rows for mt in mats)
        stage_xw = {w: [torch.empty(T, w, dtype=bf, device=dev) for _ in range(2)] for w in host_X}
        stage_dy = [torch.empty(T * wmax, dtype=bf, device=dev) for _ in range(2)]
        for ev in stage_free + step_done:
            ev.record(main)
        for _ in range(2):
            step(it_next, e2e=True)
            it_next += 1
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        gc.collect()
        gc.disable()
        e0.record(main)
        for _ in range(args.steps):
            step(it_next, e2e=True)
            it_next += 1
        e1.record(main)
        barrier()
        gc.enable()
        e2e_ms = e0.elapsed_time(e1)

    # every rank learns of a device-side wait that ran out on ANY rank, releases the arena with the
    # others, and only then raises
    bad = torch.tensor([int(status[0].item())], dtype=torch.int32, device=dev)
    if world > 1:
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    times = torch.tensor([total_ms, e2e_ms, part.get("gemm", 0.0), part.get("optim", 0.0), part.get("mask", 0.0)],
                         dtype=torch.float64, device=dev)
    host_all = torch.tensor([host_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        gathered = [torch.zeros_like(host_all) for _ in range(world)]
        dist.all_gather(gathered, host_all)
        host_all = torch.cat(gathered)
    total_ms, e2e_ms, gemm_ms, optim_ms, mask_ms = [float(x) for x in times.cpu()]
    host_list = [round(float(x), 4) for x in host_all.cpu()]
    if arena is not None:
        arena.close()
    if int(bad) != 0:
        if world > 1:
            dist.destroy_process_group()
        raise RuntimeError(f"a device-side wait ran out inside a GEMM (code {int(bad)}); the numbers are void")
    if exchange_err is not None and not exchange_err <= 1e-2:
        if world > 1:
            dist.destroy_process_group()
        raise RuntimeError(f"the exchange through the GEMM epilogues differs from the unsharded products ({exchange_err})")
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_src = load_peaks()
    flops_step = sum(layer_flops(T, r, c) for _, r, c in shapes)
    elems_rank = sum(r * c for _, r, c in shapes) / world
    ms_per_step = total_ms / args.steps
    value = flops_step / (ms_per_step * 1e-3) / 1e12
    gemm_tflops = (flops_step / world) * kinds_steps / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    gbs = lambda b, ms_: (elems_rank * b * kinds_steps) / (ms_ * 1e-3) / 1e9 if ms_ > 0 else None  # noqa: E731
    kinds = {k.split(":")[-1]: round(v / kinds_steps, 4) for k, v in sorted(part.items()) if ":" in k or k == "reduce"}
    out = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "llama2-7b-layerset-tempering" + (f" (reduced to {args.only})" if args.only else ""),
                   "shapes": "q,k,v,o[4096,4096] gate,up[11008,4096] down[4096,11008]",
                   "tokens": T, "row_sharded_over": world, "collective": collective,
                   "allgather": allgather, "dgrad_exchange": "none" if arena is None else ("pull" if pull else "scatter"),
                   "overlap_hbm_passes": overlap, "gemm_ctas_fwd_dgrad_wgrad": [f_ctas, d_ctas, w_ctas],
                   "rank_barriers_per_step": 0 if world == 1 else (1 if arena is not None else 0),
                   "l2": "inputs larger than L2 (each matrix pass touches >100 MB)",
                   "e2e_inputs": ("activations [T, in] and upstream gradient [T, out] from pinned host memory" if world == 1 else
                                  "per rank: its T/N rows of the activations (all-gathered over NVLink afterwards) and its column "
                                  "block of the upstream gradient, from pinned host memory"),
                   "e2e_reads_back": "mask statistics (448 B); outputs and input gradients stay on the device"},
        "clocks": clocks,
        "e2e": None if args.no_e2e else {"value": round(flops_step / (e2e_ms / args.steps * 1e-3) / 1e12, 2),
                                         "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_timed,
        "roofline": {"bound": "tensor", "achieved": round(gemm_tflops, 1) if gemm_tflops else None,
                     "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(gemm_tflops / peaks["bf16_tflops_sustained"], 4) if gemm_tflops else None,
                     "frac_of_burst": round(gemm_tflops / peaks["bf16_tflops"], 4) if gemm_tflops else None,
                     "traffic": round(GEMM_TRAFFIC_PER_GFLOP * flops_step / world / (3 * len(shapes)) / 1e9),
                     "traffic_source": "ncu capture of the q-shaped launches, scaled by FLOPs per launch (bytes)",
                     "peak_source": peak_src + " (sustained bf16 GEMM; frac_of_burst uses the burst figure)",
                     "timed_in": "the headline loop" if world == 1 else f"{kinds_steps} separate instrumented steps",
                     "kernel": f"gemm_bf16_pair_kernel (fwd, dgrad, wgrad: {3 * len(shapes)} launches per step)"},
        "passes": {
            "optim_score_gbs": gbs(BYTES_OPTIM, optim_ms),
            "mask_update_gbs": gbs(BYTES_MASK, mask_ms), "hbm_peak_gbs": peaks["hbm_gbs"],
            "gemm_ms_per_step": gemm_ms / kinds_steps, "optim_score_ms_per_step": optim_ms / kinds_steps,
            "mask_ms_per_step": mask_ms / kinds_steps,
            "rank0_ms_per_step": kinds,
            "host_enqueue_ms_per_step": host_list,
            "host_enqueue_ms_per_step_without_events": round(min(host_warm[1:]), 4) if len(host_warm) > 1 else None,
        },
    }
    for k in ("optim_score_gbs", "mask_update_gbs"):
        if out["passes"][k]:
            out["passes"][k.replace("_gbs", "_frac")] = round(out["passes"][k] / peaks["hbm_gbs"], 4)
            out["passes"][k] = round(out["passes"][k], 1)
    if arena is not None:
        # bytes that land on one GPU per step: the other ranks' output columns, and either the other ranks'
        # partial rows of this owner (scatter) or only the sum of its rows (pull)
        recv = (world - 1) / world * sum(T * r * 2 for _, r, _ in shapes)
        recv += sum(T * c * 2 for _, _, c in shapes) * ((1.0 / world) if pull else (world - 1) / world)
        out["passes"]["exchange_sent_bytes_per_gpu_per_step"] = int(
            sum(T * r * 2 for _, r, _ in shapes) / world * (1 if allgather == "multimem" else world - 1)
            + sum(T * c * 2 for _, _, c in shapes) * (1.0 if pull else (world - 1) / world))
        xms = kinds.get("fwd", 0.0) + kinds.get("dgrad", 0.0)
        out["config"]["exchange_checked"] = True
        out["passes"]["exchange"] = {"received_bytes_per_gpu_per_step": int(recv),
                                     "gbs_over_fwd_plus_dgrad_kernels": round(recv / (xms * 1e-3) / 1e9, 1) if xms > 0 else None,
                                     "gbs_over_step": round(recv / (ms_per_step * 1e-3) / 1e9, 1),
                                     "max_rel_err_vs_unsharded": exchange_err}
    if world == 1 and not args.only:
        if not args.no_extras:
            torch.cuda.synchronize()
            out["passes"]["module_ms_per_step"] = round(module_path_ms(dev), 3)
            out["passes"]["module_path"] = ("SparseLinear x 7 + utils.update_hessian_hutchinson (real double backward) + "
                                            "AdamW.step(decay=) + utils.calculate_model_mask, 3 steps after 2 warm-up")
            out["sparse24"] = sparse24_cases(dev, rows_sweep=(1, 16, 128, 1024, 8192), iters=10, status=status)
            out["bsr16"] = bsr16_cases(dev, status=status)
        if not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_reference_sample(steps=2, warmup=1)
    print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# the module path: the same layer set driven through SparseLinear, the real Hutchinson step and AdamW
# ---------------------------------------------------------------------------------------------
def module_path_ms(dev, steps=3, warmup=2, shapes=SHAPES):
    """One tempering step of the layer set through the package's module interface, in the order of the
    reference's training loop (legacy/main_llama.py:1997-2211): forward of every SparseLinear, a loss with
    curvature (sum gelu(y) * dy / T per layer), utils.update_hessian_hutchinson (the real double backward:
    three more GEMM-shaped products per layer and a differentiable backward), loss.backward(),
    AdamW.step(decay=), utils.calculate_model_mask. Returns milliseconds per step (CUDA events)."""
    import sparseforge_b200 as sf
    from sparseforge_b200 import utils as U

    bf = torch.bfloat16
    T = T_TOKENS
    cfg = sf.SparseLinearConfig(mask_type="structured", mask_metric="hessian_obd", N=2, M=4, mask_update_period=1,
                                sparsity_warmup_steps=0, mask_lr=0.1, beta=0.99, temp_init=1.0, temp_min=0.05,
                                temp_decay=0.05 ** (1.0 / 9.0), mask_hardening_start=1, mask_hardening_duration=9)
    g = torch.Generator(device=dev).manual_seed(11)
    layers = torch.nn.ModuleList()
    for _, rows, cols in shapes:
        layer = sf.SparseLinear(cols, rows, sparselinear_config=cfg, bias=False).to(dev).to(bf)
        layer.weight.data.copy_((torch.randn(rows, cols, device=dev, generator=g) * 0.02).to(bf))
        layer.initialize()
        layers.append(layer)
    opt = sf.AdamW([m.weight for m in layers], lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    widths = sorted({c for _, _, c in shapes})
    X = {w: torch.randn(4, T // 4, w, device=dev, generator=g).to(bf) for w in widths}
    dY = [torch.randn(4, T // 4, r, device=dev, generator=g).to(bf) for _, r, _ in shapes]

    def one(it):
        loss = None
        for layer, dy in zip(layers, dY):
            y = layer(X[layer.in_features])
            term = (torch.nn.functional.gelu(y) * dy).float().sum() / T
            loss = term if loss is None else loss + term
        U.update_hessian_hutchinson(layers, loss)
        loss.backward()
        opt.step(decay=2e-4)
        opt.zero_grad(set_to_none=True)
        U.calculate_model_mask(layers, step=it % 10, lambda_mid=0.0)

    for it in range(warmup):
        one(it)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for it in range(steps):
        one(warmup + it)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / steps
    del layers, opt, X, dY
    torch.cuda.empty_cache()
    return ms


def run_module(args):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    shapes = [s for s in SHAPES if (not args.only or s[0] in args.only.split(","))]
    ms = module_path_ms(dev, steps=max(1, min(args.steps, 10)), warmup=2, shapes=shapes)
    flops = sum(layer_flops(T_TOKENS, r, c) for _, r, c in shapes)
    print(json.dumps({"metric": METRIC + ", module path with the real Hutchinson double backward", "unit": UNIT, "n_gpus": 1,
                      "value": round(flops / (ms * 1e-3) / 1e12, 2), "ms_per_step": round(ms, 3), "dtype": "bf16",
                      "data": "synthetic", "config": {"workload": "llama2-7b-layerset-tempering (module path)",
                                                      "note": "value counts the forward + backward FLOPs of the training "
                                                              "products only (6 T in out), as the headline does; the double "
                                                              "backward runs about as many again"}}), flush=True)


# ---------------------------------------------------------------------------------------------
# hard-2:4 compressed inference GEMM and block-sparse-16 products (compact blocks of the N = 1 line)
# ---------------------------------------------------------------------------------------------
def _graph_timer(warmup=3):
    def capture(fn, iters):
        """`iters` launches captured in one CUDA graph, so that the host launch path is outside the
        timed region."""
        for _ in range(warmup):
            fn(0)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for j in range(iters):
                fn(j)
        graph.replay()
        torch.cuda.synchronize()
        return graph

    def replay_ms(graph, iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    def time_pair(fn_a, fn_b, iters, rounds=3):
        """Device time per launch of two products, replayed alternately (the clock drifts under the
        power cap, so the two are taken in the same thermal state); the median round is kept."""
        ga, gb = capture(fn_a, iters), capture(fn_b, iters)
        ta, tb = [], []
        for _ in range(rounds):
            ta.append(replay_ms(ga, iters))
            tb.append(replay_ms(gb, iters))
        return sorted(ta)[rounds // 2], sorted(tb)[rounds // 2]

    return time_pair


def sparse24_cases(dev, rows_sweep, iters, status, only=""):
    """Hard-2:4 compressed inference GEMM against the dense masked GEMM on the same pruned weight: three
    distinct LLaMA-2-7B weight shapes x activation heights. Every launch of a replay reads another copy
    of the weight, enough copies to exceed the L2 (126 MB) between two uses of one copy, so the small
    heights are measured cold from HBM."""
    from sparseforge_b200 import ops

    bf = torch.bfloat16
    time_pair = _graph_timer()
    cases = []
    for i, (name, out_f, in_f) in enumerate(s for s in DISTINCT if (not only or s[0] in only.split(","))):
        g = torch.Generator(device=dev).manual_seed(100 + i)
        W = (torch.randn(out_f, in_f, device=dev, generator=g) * 0.02).to(bf)
        vals0, meta = ops.sparse24_compress(W, W.float().abs())
        mtc0 = ops.sparse24_pack_meta(meta, out_f, in_f)
        wd0 = ops.sparse24_decompress(vals0, meta)
        del W
        comp_bytes = vals0.numel() * 2 + mtc0.numel()
        copies = min(iters, max(2, -(-2 * 126_000_000 // comp_bytes)))
        vals, mtc, wd = [vals0], [mtc0], [wd0]
        for _ in range(copies - 1):
            vals.append(vals0.clone()); mtc.append(mtc0.clone()); wd.append(wd0.clone())
        for T in rows_sweep:
            x = torch.randn(T, in_f, device=dev, generator=g).to(bf)
            xd = x if T % 8 == 0 else torch.cat([x, torch.zeros(8 - T % 8, in_f, device=dev, dtype=bf)])
            ts, td = time_pair(lambda j: ops.sparse24_gemm(x, vals[j % copies], mtc[j % copies], status=status),
                               lambda j: ops.gemm_fwd(xd, wd[j % copies], status=status), iters)
            flops = 2.0 * T * in_f * out_f
            bytes_s = in_f * out_f + in_f * out_f / 8 + 2.0 * T * (in_f + out_f)
            c = {"shape": name, "rows": T, "sparse_us": round(ts * 1e3, 1), "dense_us": round(td * 1e3, 1),
                 "speedup_vs_dense": round(td / ts, 3)}
            if T <= 128:
                c["sparse_gbs_cold"] = round(bytes_s / ts / 1e6, 1)
            else:
                c["sparse_tflops"] = round(flops / ts / 1e9, 1)
            cases.append(c)
        del vals, mtc, wd
    big = [c for c in cases if c["rows"] >= 8192]
    return {"workload": "llama2-7b-sparse24-inference", "timing": f"CUDA graph of {iters} back-to-back launches rotating over "
            "weight copies (> 2 x L2 in total), sparse and dense replayed alternately, median of three rounds",
            "speedup_rows_8192": round(sum(c["speedup_vs_dense"] for c in big) / max(1, len(big)), 3) if big else None,
            "cases": cases}


def bsr16_cases(dev, status, T=16384, density=0.5, iters=4):
    """Block-sparse-16 products at the MLP shapes: 16 x 16 blocks kept at 50 % by block Frobenius norm
    (global top-k over the layer), forward, input gradient and weight gradient, against the dense masked
    GEMMs on the same block-masked weight. useful = 2 T in out density FLOPs per product."""
    from sparseforge_b200 import ops

    bf = torch.bfloat16
    time_pair = _graph_timer()
    cases = []
    for i, (name, out_f, in_f) in enumerate([("gate", 11008, 4096), ("down", 4096, 11008)]):
        g = torch.Generator(device=dev).manual_seed(300 + i)
        W = (torch.randn(out_f, in_f, device=dev, generator=g) * 0.02).to(bf)
        ob, ib = out_f // 16, in_f // 16
        norms = W.float().view(ob, 16, ib, 16).pow(2).sum(dim=(1, 3)).flatten()
        keep = torch.zeros(ob * ib, device=dev)
        keep[torch.sort(norms, descending=True, stable=True).indices[: int(round(density * ob * ib))]] = 1.0
        mask = keep.view(ob, 1, ib, 1).expand(ob, 16, ib, 16).reshape(out_f, in_f).contiguous()
        blocks, row_ptr, col_idx = ops.bsr16_build(W, mask)
        wd = (W.float() * mask).to(bf)
        x = torch.randn(T, in_f, device=dev, generator=g).to(bf)
        dy = torch.randn(T, out_f, device=dev, generator=g).to(bf)
        ws = torch.empty(out_f, in_f, dtype=bf, device=dev)
        useful = 2.0 * T * in_f * out_f * (col_idx.numel() / (ob * ib))
        row = {"shape": name, "tokens": T, "blocks_kept": int(col_idx.numel()), "density": round(col_idx.numel() / (ob * ib), 4)}
        gws = torch.empty_like(ws)
        ops.bsr16_fwd(x, blocks, row_ptr, col_idx, out_f, workspace=ws, status=status)  # leaves the scattered weight in ws
        for kind, fs, fd in (
                ("fwd", lambda j: ops.bsr16_fwd(x, blocks, row_ptr, col_idx, out_f, workspace=ws, status=status, dense_ready=True),
                 lambda j: ops.gemm_fwd(x, wd, status=status)),
                ("fwd_with_scatter", lambda j: ops.bsr16_fwd(x, blocks, row_ptr, col_idx, out_f, workspace=ws, status=status),
                 lambda j: ops.gemm_fwd(x, wd, status=status)),
                ("dgrad", lambda j: ops.bsr16_dgrad(dy, blocks, row_ptr, col_idx, in_f, workspace=ws, status=status, dense_ready=True),
                 lambda j: ops.gemm_dgrad(dy, wd, status=status)),
                ("wgrad", lambda j: ops.bsr16_wgrad(dy, x, row_ptr, col_idx, workspace=gws, status=status),
                 lambda j: ops.gemm_wgrad(dy, x, status=status))):
            ts, td = time_pair(fs, fd, iters)
            row[kind] = {"us": round(ts * 1e3, 1), "dense_us": round(td * 1e3, 1), "speedup_vs_dense": round(td / ts, 3),
                         "useful_tflops": round(useful / ts / 1e9, 1), "dense_equiv_tflops": round(2.0 * T * in_f * out_f / ts / 1e9, 1)}
        cases.append(row)
        del W, mask, wd, x, dy, ws, gws, blocks
    return {"workload": "llama2-7b-mlp-block-sparse-16", "timing": f"CUDA graph of {iters} launches, block-sparse and dense "
            "replayed alternately, median of three rounds; fwd / dgrad with the scattered weight kept from the call before "
            "(a layer whose blocks did not change), fwd_with_scatter rebuilds it", "cases": cases}


def run_sparse24(args):
    """`--workload sparse24`: the compressed-GEMM sweep alone, on more launches per replay."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    res = sparse24_cases(dev, [int(r) for r in args.rows.split(",")], max(2, args.steps), status, only=args.only)
    if int(status[0].item()) != 0:
        raise RuntimeError("a device-side wait ran out inside a GEMM; the numbers are void")
    big = [c for c in res["cases"] if c["rows"] >= 8192]
    print(json.dumps({"metric": "hard-2:4 compressed GEMM, dense-equivalent TFLOP/s and speed-up over the dense masked GEMM",
                      "unit": "TFLOP/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
                      "value": round(sum(c["sparse_tflops"] for c in big) / max(1, len(big)), 1) if big else None,
                      "config": {"workload": res["workload"], "timing": res["timing"]},
                      "speedup_rows_8192": res["speedup_rows_8192"], "cases": res["cases"]}), flush=True)


def run_bsr16(args):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    res = bsr16_cases(dev, status, iters=max(2, min(args.steps, 10)))
    print(json.dumps({"metric": "block-sparse-16 products, useful TFLOP/s and speed-up over the dense masked GEMM",
                      "unit": "TFLOP/s", "n_gpus": 1, "dtype": "bf16", "data": "synthetic", **res}), flush=True)


# ---------------------------------------------------------------------------------------------
# the CPU arm: the reference's own code on the host cores (oracle/_ref), else the oracle's port of it
# ---------------------------------------------------------------------------------------------
def cpu_port_step(W, mask, H, m, v, X, dY, hvp, probe, it):
    """One tempering step of one matrix with the oracle (torch CPU ops in the reference's order)."""
    from oracle import sparselinear_oracle as O

    temp, _ = schedule(it)
    eff = O.effective_mask(mask, 1.0)
    O.linear_forward(X, W, eff)
    _, dW, _ = O.linear_backward(X, W, eff, dY)
    H = O.hutchinson_accumulate(H, hvp, probe, 0.99)
    W, m, v = O.adamw_step(W, dW, m, v, step=it + 1, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                           mask=mask, decay=2e-4)
    G = O.gate_target_structured(O.normalize_scores(O.importance_score(W, "hessian_obd", H=H)), temp)
    new_mask = O.mask_update(mask, G, mask_lr=0.1)
    O.flip_count(mask, new_mask)
    return W, new_mask, H, m, v


def cpu_port_steps(shapes, steps, warmup, threads):
    """The oracle's restatement timed like the reference arm: `warmup` + `steps` sample steps over one
    matrix of each shape in `shapes`."""
    torch.set_num_threads(threads)
    bf = torch.bfloat16
    states = []
    for i, (_, rows, cols) in enumerate(shapes):
        torch.manual_seed(100 + i)
        states.append(dict(W=(torch.randn(rows, cols) * 0.02).to(bf), mask=torch.ones(rows, cols), H=torch.ones(rows, cols),
                           m=torch.zeros(rows, cols, dtype=bf), v=torch.zeros(rows, cols, dtype=bf),
                           X=torch.randn(T_TOKENS, cols).to(bf), dY=torch.randn(T_TOKENS, rows).to(bf),
                           hvp=(torch.randn(rows, cols) * 1e-3).to(bf),
                           probe=(torch.randint(0, 2, (rows, cols), dtype=torch.int8) * 2 - 1).to(bf)))
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for s in states:
            s["W"], s["mask"], s["H"], s["m"], s["v"] = cpu_port_step(s["W"], s["mask"], s["H"], s["m"], s["v"], s["X"],
                                                                      s["dY"], s["hvp"], s["probe"], it)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return times, sum(layer_flops(T_TOKENS, r, c) for _, r, c in shapes), torch.get_num_threads()


def host_threads():
    """Host threads this process may use: its CPU affinity, cut to the cgroup's CPU quota where one is set
    (`torch.distributed.run` exports OMP_NUM_THREADS=1, so the count is set explicitly from this)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    try:
        with open("/sys/fs/cgroup/cpu.max") as f:
            quota, period = f.read().split()[:2]
        if quota != "max":
            n = max(1, min(n, int(float(quota) / float(period) + 0.5)))
    except (OSError, ValueError):
        pass
    return n


def cpu_reference_steps(shapes, steps, warmup):
    """(seconds per sample step, FLOPs per sample step, threads, kind, note)."""
    threads = host_threads()
    try:
        from oracle import ref_runner

        if not ref_runner.available():
            raise RuntimeError("oracle/_ref holds no compiled reference modules (oracle/build_ref.py makes them)")
        times, flops, used = ref_runner.timed_steps(shapes, T_TOKENS, steps, warmup, threads)
        return times, flops, used, "reference", ("the reference's own SparseLinear forward / backward, AdamW.step(decay=) and "
                                                 "calculate_model_mask (bytecode in oracle/_ref, tie-stable topk); Hutchinson tail "
                                                 "from a synthetic Hessian-vector product, as on the GPU arm")
    except Exception as e:  # the port stands in, and says why
        print(f"[bench] reference modules unavailable ({e}); timing the oracle's port", file=sys.stderr, flush=True)
        times, flops, used = cpu_port_steps(shapes, steps, warmup, threads)
        return times, flops, used, "port", f"oracle port (reference modules unavailable: {e})"


def cpu_reference_sample(steps=2, warmup=1):
    times, flops, used, kind, note = cpu_reference_steps(DISTINCT, steps, warmup)
    best = min(times)
    return {"value": round(flops / best / 1e12, 4), "unit": UNIT, "cores": used, "kind": kind,
            "sample": f"one matrix of each distinct shape (q, gate, down) of the seven, all {T_TOKENS} tokens, full tempering "
                      f"step, best of {steps} after {warmup} warm-up; {note}",
            "seconds_per_sample_step": round(best, 3)}


def run_reference(args):
    """The reference arm: `warmup` + `steps` sample steps on the host cores, all of them run, on rank 0."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    # the whole layer set when the run then still ends within a few minutes, else one matrix of each shape
    shapes, sample = DISTINCT, "one matrix of each distinct shape (q, gate, down)"
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    t_probe, _, _, _, _ = cpu_reference_steps(DISTINCT, 1, 0)
    est_full = t_probe[0] * (sum(r * c for _, r, c in SHAPES) / sum(r * c for _, r, c in DISTINCT))
    if est_full * (steps + warmup) <= 150.0:
        shapes, sample = SHAPES, "the whole layer set (seven matrices)"
    times, flops, used, kind, note = cpu_reference_steps(shapes, steps, warmup)
    mean = sum(times) / len(times)
    value = round(flops / mean / 1e12, 4)
    res = {"value": value, "unit": UNIT, "cores": used, "kind": kind,
           "sample": f"{sample}, all {T_TOKENS} tokens, full tempering step, mean of {steps} steps after {warmup} warm-up; {note}",
           "seconds_per_sample_step": round(mean, 3)}
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
           "steps": steps, "warmup": warmup, "ms_per_step": round(mean * 1e3, 1),
           "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "llama2-7b-layerset-tempering",
                      "shapes": "q,k,v,o[4096,4096] gate,up[11008,4096] down[4096,11008]", "tokens": T_TOKENS,
                      "row_sharded_over": 1, "sample": res["sample"], "host_threads": used},
           "cpu_baseline": res, "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0,
                                        "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the sparse24 and bsr16 blocks of the N = 1 line")
    ap.add_argument("--collective", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: exchange through the GEMM epilogues and peer memory (p2p) or NCCL collectives")
    ap.add_argument("--dgrad-exchange", default="auto", choices=["auto", "scatter", "pull"],
                    help="N > 1: input-gradient reduce-scatter by stores from the dgrad epilogue (scatter) or by an "
                         "owner-side multimem.ld_reduce of the ranks' partials after the rank barrier (pull)")
    ap.add_argument("--pull-ctas", type=int, default=64, help="thread blocks of the owner-side multimem reduce")
    ap.add_argument("--no-multicast", action="store_true",
                    help="output all-gather by one store per destination instead of NVSwitch multicast stores")
    ap.add_argument("--overlap", default="auto", choices=["auto", "on", "off"],
                    help="run each matrix's optimizer / mask passes on a second stream beside the next "
                         "matrix's products; auto = when the layer set is sharded (the exchange kernels wait on "
                         "NVLink and leave HBM idle; on one GPU the chip is power-capped and the overlap gains "
                         "0-4 %% while every kernel slows down)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--gemm-ctas", default="",
                    help="f,d,w: thread blocks of the forward, input-gradient and weight-gradient products of a matrix; a "
                         "product with a non-zero d or w runs on a stream of its own beside the forward (default: one "
                         "stream up to two GPUs; 100,0,48 from four GPUs on, where the forward and input gradient wait "
                         "on NVLink)")
    ap.add_argument("--only", default="", help="comma-separated matrix names (q,k,v,o,gate,up,down): a reduced "
                                               "workload for profiler captures; the JSON line then names it")
    ap.add_argument("--workload", default="tempering", choices=["tempering", "sparse24", "bsr16", "module"],
                    help="tempering = the headline layer-set step; sparse24 = compressed inference GEMM sweep; "
                         "bsr16 = block-sparse-16 products")
    ap.add_argument("--rows", default="1,16,128,1024,8192", help="activation rows of the sparse24 sweep")
    args = ap.parse_args()
    if args.workload == "sparse24":
        return run_sparse24(args)
    if args.workload == "bsr16":
        return run_bsr16(args)
    if args.workload == "module":
        return run_module(args)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
