"""Benchmark of the bit-sliced GEMV path (and its CPU reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the shape and bitwidth sweep of the sliced GEMV — the four Llama-3-8B
linear shapes x batch M in {1,2,4,8,16} x inference bitwidth b in {2,3,4,6,8}, fp16, group 128,
weights sliced from seeded 8-bit master codes.  One STEP is one pass over the 100 cells, launched
back to back from a CUDA graph; the loop order (M, shape, b) puts 20 other weight sets (~400 MB,
more than L2) between two uses of the same weights.  `value` is algorithmic GB/s of the whole step
(bytes a call must move: planes + scales + activations + output).  With N > 1 the same sweep runs
tensor-parallel: k/v and gate/up split N, q/o and down split K and all-reduce their partial outputs.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from matgptq_b200 import synth  # noqa: E402

METRIC = "sliced_gemv_algorithmic_bandwidth"
UNIT = "GB/s"
BATCHES = (1, 2, 4, 8, 16)
BITS = synth.BITWIDTHS
GROUP = 128
ROW_PARALLEL = {"q_o": True, "k_v": False, "gate_up": False, "down": True}
# dram__bytes_read+write of mg::gemv_kernel divided by its algorithmic bytes, from an ncu capture of
# gate/up at 4 bits, one activation row (30.32 MB measured / 30.31 MB algorithmic)
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0002
# warm-up replays of the sweep graph when it holds collectives (the same on every rank, see ours_main)
MULTI_RANK_WARMUP_REPLAYS = 192


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, maxc = [], set(), None
        for s in self.samples:
            try:
                clocks.append(float(s[0]))
                maxc = float(s[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": maxc,
                "reasons": sorted(reasons), "samples": len(clocks)}


# --------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's dequantise-then-matmul on the host cores
# --------------------------------------------------------------------------------------
def cpu_sample_cells():
    """Bounded sample of the sweep for the CPU arm: every shape and every bitwidth at M = 1 (20 of the 100 cells)."""
    return [(name, k, n, 1, b) for name, (k, n) in synth.LLAMA3_8B_SHAPES.items() for b in BITS]


def run_cpu_arm(steps: int, warmup: int) -> dict:
    from oracle import matgptq_oracle as oracle
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cells = cpu_sample_cells()
    layers = {name: synth.make_layer(n, k, GROUP, seed=1 + i, sym=True, dtype=torch.float16)
              for i, (name, (k, n)) in enumerate(synth.LLAMA3_8B_SHAPES.items())}
    xs = {k: synth.make_activations(1, k, seed=1, dtype=torch.float16) for k in {k for _, k, _, _, _ in cells}}
    nbytes = sum(synth.algorithmic_bytes(n, k, m, b, GROUP) for _, k, n, m, b in cells)

    parts = [0.0, 0.0]  # seconds in dequantize() and in F.linear, over the timed steps

    def step(timed: bool = False):
        for name, k, n, m, b in cells:
            layer, x = layers[name], xs[k]
            # the two halves of oracle.fake_matryoshka_linear (FakeMatryoshkaLinear.forward), timed apart
            t0 = time.perf_counter()
            w = oracle.dequantize_weight(layer.qweight, layer.scales, layer.zeros, 8, b)
            t1 = time.perf_counter()
            torch.nn.functional.linear(x, w)
            t2 = time.perf_counter()
            if timed:
                parts[0] += t1 - t0
                parts[1] += t2 - t1

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step(True)
    dt = (time.perf_counter() - t0) / steps
    return {"value": nbytes / dt / 1e9, "ms_per_step": dt * 1e3, "cores": cores,
            "dequant_ms_per_step": parts[0] / steps * 1e3, "matmul_ms_per_step": parts[1] / steps * 1e3,
            "sample": "oracle dequantise-then-matmul (torch CPU, fp16), the four Llama-3-8B shapes x b in {2,3,4,6,8} "
                      "at M=1: 20 of the sweep's 100 cells per step"}


def reference_main(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = run_cpu_arm(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama3-8b linear shapes x M{1,2,4,8,16} x b{2,3,4,6,8}, g128, fp16 (bounded CPU sample)"},
        "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"],
                         "dequant_ms_per_step": round(r["dequant_ms_per_step"], 2),
                         "matmul_ms_per_step": round(r["matmul_ms_per_step"], 2)},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def shard_shape(name: str, world: int) -> tuple[int, int]:
    """(k_loc, n_loc) of one rank's shard: row-parallel layers split K, the others split N."""
    k, n = synth.LLAMA3_8B_SHAPES[name]
    if world > 1 and ROW_PARALLEL[name]:
        return k // world, n
    if world > 1:
        return k, n // world
    return k, n


def shard_layer(name: str, world: int, rank: int, dev: torch.device) -> synth.SynthLayer:
    """The seeded master codes and scales of one rank's shard (any rank can draw any rank's shard)."""
    si = list(synth.LLAMA3_8B_SHAPES).index(name)
    k_loc, n_loc = shard_shape(name, world)
    return synth.make_layer(n_loc, k_loc, GROUP, seed=100 * si + rank, sym=True, dtype=torch.float16, device=dev)


def build_cells(world: int, rank: int, dev: torch.device):
    """Pack this rank's shard of every (shape, b) and allocate activations/outputs for every M."""
    from matgptq_b200 import ops  # noqa: F401
    weights = {}
    for si, (name, (k, n)) in enumerate(synth.LLAMA3_8B_SHAPES.items()):
        k_loc, n_loc = shard_shape(name, world)
        layer = shard_layer(name, world, rank, dev)
        scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n_loc, k_loc, GROUP)
        for b in BITS:
            packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n_loc, k_loc, 8, b, GROUP, 1)
            weights[(name, b)] = (packed, scales_r, n_loc, k_loc)
        del layer
    cells = []
    for m in BATCHES:
        for name, (k, n) in synth.LLAMA3_8B_SHAPES.items():
            for b in BITS:
                packed, scales_r, n_loc, k_loc = weights[(name, b)]
                x = synth.make_activations(m, k_loc, seed=m, dtype=torch.float16, device=dev)
                y = torch.empty(m, n_loc, dtype=torch.float16, device=dev)
                cells.append({"name": name, "m": m, "b": b, "k": k, "n": n, "k_loc": k_loc, "n_loc": n_loc,
                              "packed": packed, "scales": scales_r, "x": x, "y": y,
                              "bytes": synth.algorithmic_bytes(n, k, m, b, GROUP)})
    return cells


_PHASE = ["start", time.monotonic()]  # current phase and when it began


def progress(msg: str) -> None:
    """Remember the phase and its start (the watchdog reports both) and, with MATGPTQ_BENCH_VERBOSE=1, print it
    on stderr."""
    _PHASE[0] = msg
    _PHASE[1] = time.monotonic()
    if os.environ.get("MATGPTQ_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def start_watchdog(stall_seconds: float, total_seconds: float) -> None:
    """A multi-rank run that stalls (a rank that never joins a collective, a communicator that never comes
    up) would otherwise sit until somebody kills it.  When one phase lasts longer than `stall_seconds`, or
    the whole run longer than `total_seconds`, print where it stands as one JSON line on stdout (a launcher's
    traceback on stderr cannot bury it) and leave with exit code 3."""
    t_start = time.monotonic()

    def bark():
        while True:
            time.sleep(1.0)
            now = time.monotonic()
            stalled = now - _PHASE[1] > stall_seconds
            if stalled or now - t_start > total_seconds:
                line = {"stalled": True, "rank": int(os.environ.get("RANK", "0")), "phase": _PHASE[0],
                        "seconds_in_phase": round(now - _PHASE[1], 1), "seconds_total": round(now - t_start, 1),
                        "why": "no progress" if stalled else "overall limit"}
                print(json.dumps(line), flush=True)
                print(f"[bench rank {line['rank']}] watchdog: {line['why']}, last phase: {_PHASE[0]}", file=sys.stderr, flush=True)
                os._exit(3)
    threading.Thread(target=bark, daemon=True).start()


def make_peer_allreduce(dev: torch.device):
    """The peer-memory all-reduce of this process group, checked once against NCCL on a small product; every
    rank takes the same decision (a rank that cannot set the buffers up, or sees a wrong or late result, makes
    all ranks fall back to NCCL, and the line says why).  Returns (PeerAllReduce or None, note)."""
    from matgptq_b200 import _native
    ok, note, peer = 1, None, None
    try:
        from matgptq_b200.tp_comm import PeerAllReduce
        peer = PeerAllReduce(device=dev, max_rows=32, max_cols=8192)
    except Exception as e:  # noqa: BLE001  (symmetric memory not available on this box, ...)
        ok, note = 0, f"peer buffers unavailable: {type(e).__name__}"
    flag = torch.tensor([ok], device=dev, dtype=torch.int32)
    torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
    if int(flag.item()) == 0:
        return None, note or "peer buffers unavailable on another rank"
    world = torch.distributed.get_world_size()
    n, k = 1024, 128 * 4 * world
    layer = synth.make_layer(n, k // world, GROUP, seed=7 + torch.distributed.get_rank(), dtype=torch.float16, device=dev)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n, k // world, 8, 4, GROUP, 1)
    scales = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n, k // world, GROUP)
    x = synth.make_activations(3, k // world, seed=1, dtype=torch.float16, device=dev)
    torch.cuda.synchronize()
    torch.distributed.barrier()
    fused = peer.matmul(x, packed, scales, n, k // world, 4, GROUP, 1)
    part = torch.ops.matgptq_cuda.matmul_matgptq(x, packed, scales, n, k // world, 4, GROUP, 1).float()
    torch.distributed.all_reduce(part)
    torch.cuda.synchronize()
    err = (fused.float() - part).abs().max().item() / max(part.abs().max().item(), 1e-6)
    good = _native.device_status() == 0 and err <= 5e-3
    flag = torch.tensor([1 if good else 0], device=dev, dtype=torch.int32)
    torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
    if int(flag.item()) == 0:
        return None, "self-test of the fused all-reduce against NCCL failed"
    return peer, None


def launch_cell(c, flags: int, world: int, peer=None):
    """One cell; with several ranks the row-parallel cells include the all-reduce of their output: fused into
    the product's epilogue over peer memory (`peer`, a tp_comm.PeerAllReduce), or NCCL behind the product."""
    from matgptq_b200 import ops
    if world > 1 and ROW_PARALLEL[c["name"]] and peer is not None:
        peer.matmul(c["x"], c["packed"], c["scales"], c["n_loc"], c["k_loc"], c["b"], GROUP, flags, out=c["y"])
        return
    ops.matmul_matgptq_raw(c["x"], c["packed"], c["scales"], c["n_loc"], c["k_loc"], c["b"], GROUP, flags, out=c["y"])
    if world > 1 and ROW_PARALLEL[c["name"]]:
        torch.distributed.all_reduce(c["y"])


PARITY_TOLERANCE = 1e-2   # max|y - y_ref| / max|y_ref| against an fp32 accumulation over the oracle's weights
PARITY_SAMPLE_ROWS = 256  # out-features checked per (shape, bitwidth): evenly spread over N


def check_cells(cells, world: int, dev: torch.device) -> dict:
    """Outside the timed region: compare what the sweep left in every cell's output with the oracle
    (dequantise-then-matmul, fp32 accumulation) on a sample of out-features.  With several ranks, rank 0
    checks the all-reduced outputs of the row-parallel cells against the sum over every rank's shard and
    its own shard of the column-parallel ones.  Returns the worst relative error and the cell count."""
    from oracle import matgptq_oracle as oracle
    worst, checked, failed = 0.0, 0, []
    ref_cache = {}
    for c in cells:
        key = (c["name"], c["b"])
        if key not in ref_cache:
            n_loc = c["n_loc"]
            rows = torch.linspace(0, n_loc - 1, min(PARITY_SAMPLE_ROWS, n_loc)).long().unique()
            ranks = range(world) if (world > 1 and ROW_PARALLEL[c["name"]]) else (0,)
            shards = []
            for r in ranks:
                layer = shard_layer(c["name"], world, r, dev)
                q, sc, z = layer.qweight[rows.to(dev)].cpu(), layer.scales[rows.to(dev)].cpu(), layer.zeros[rows.to(dev)].cpu()
                shards.append(oracle.dequantize_weight(q, sc, z, 8, c["b"]))
                del layer
            ref_cache[key] = (rows, shards)
        rows, shards = ref_cache[key]
        x = c["x"].cpu()
        y_ref = sum(oracle.linear_fp32_accumulate(x, w) for w in shards)
        err = oracle.rel_err(c["y"][:, rows.to(dev)].cpu(), y_ref)
        worst = max(worst, err)
        checked += 1
        if not err <= PARITY_TOLERANCE:
            failed.append({"shape": c["name"], "m": c["m"], "b": c["b"], "rel_err": err})
    return {"checked_cells": checked, "max_rel_err": round(worst, 6), "tolerance": PARITY_TOLERANCE,
            "sample_rows": PARITY_SAMPLE_ROWS, "failed": failed[:8]}


def per_cell_table(dev: torch.device, flags: int) -> dict:
    """Cold-L2 time of every cell on its own: a graph of launches cycling over enough copies of the
    cell's weights to exceed L2 several times over. Returns per-bitwidth and per-cell figures."""
    from matgptq_b200 import ops
    out_cells = []
    peak, _ = measured_peaks()
    for si, (name, (k, n)) in enumerate(synth.LLAMA3_8B_SHAPES.items()):
        layer = synth.make_layer(n, k, GROUP, seed=100 * si, sym=True, dtype=torch.float16, device=dev)
        scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n, k, GROUP)
        for b in BITS:
            progress(f"per-cell table: {name} b={b}")
            packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n, k, 8, b, GROUP, 1)
            wbytes = packed.numel() * 4
            copies = max(2, min(64, -(-512 * 1024 * 1024 // wbytes)))
            packs = [packed] + [packed.clone() for _ in range(copies - 1)]
            scs = [scales_r] + [scales_r.clone() for _ in range(copies - 1)]
            for m in BATCHES:
                x = synth.make_activations(m, k, seed=m, dtype=torch.float16, device=dev)
                y = torch.empty(m, n, dtype=torch.float16, device=dev)
                reps = copies * 2
                stream = torch.cuda.Stream(device=dev)
                with torch.cuda.stream(stream):
                    for i in range(copies):
                        ops.matmul_matgptq_raw(x, packs[i], scs[i], n, k, b, GROUP, flags, out=y)
                    stream.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        for i in range(reps):
                            ops.matmul_matgptq_raw(x, packs[i % copies], scs[i % copies], n, k, b, GROUP, flags, out=y)
                    graph.replay()
                    stream.synchronize()
                    times = []
                    for _ in range(5):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        graph.replay()
                        e1.record(stream)
                        stream.synchronize()
                        times.append(e0.elapsed_time(e1) * 1e3 / reps)
                us = statistics.median(times)
                # the same launches on ONE copy of the weights: warm L2 (every shape fits in the 126 MB)
                with torch.cuda.stream(stream):
                    warm = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(warm, stream=stream):
                        for i in range(20):
                            ops.matmul_matgptq_raw(x, packs[0], scs[0], n, k, b, GROUP, flags, out=y)
                    warm.replay()
                    stream.synchronize()
                    wt = []
                    for _ in range(5):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        warm.replay()
                        e1.record(stream)
                        stream.synchronize()
                        wt.append(e0.elapsed_time(e1) * 1e3 / 20)
                nbytes = synth.algorithmic_bytes(n, k, m, b, GROUP)
                out_cells.append({"shape": name, "k": k, "n": n, "m": m, "b": b, "us": round(us, 3),
                                  "gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / peak, 3),
                                  "warm_l2_us": round(statistics.median(wt), 3)})
                del graph, warm
            del packs, scs, packed
        del layer
    per_b = {}
    for b in BITS:
        sel = [c for c in out_cells if c["b"] == b]
        tot_us = sum(c["us"] for c in sel)
        tot_bytes = sum(synth.algorithmic_bytes(c["n"], c["k"], c["m"], b, GROUP) for c in sel)
        per_b[str(b)] = {"mean_us": round(tot_us / len(sel), 3), "gbs": round(tot_bytes / tot_us / 1e3, 1)}
    return {"per_bitwidth": per_b, "cells": out_cells}


def ours_main(args) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if args.watchdog > 0:
        start_watchdog(args.watchdog, args.watchdog_total)
    if world > 1:
        progress("bringing the process group up")
        torch.distributed.init_process_group("nccl", device_id=dev)
    from matgptq_b200 import _native, ops  # noqa: F401

    flags = _native.FLAG_ASYNC | (_native.FLAG_PDL if not args.no_pdl else 0)
    peer, peer_note = None, None
    if world > 1 and args.allreduce == "fused":
        progress("setting up the peer-memory buffers")
        peer, peer_note = make_peer_allreduce(dev)
    progress("process group up, building cells")
    cells = build_cells(world, rank, dev)
    progress("cells built")
    step_bytes = sum(c["bytes"] for c in cells)
    launches_per_step = len(cells)

    stream = torch.cuda.Stream(device=dev)
    if world > 1:
        # the fused all-reduce waits for its peers inside the kernel, with a bound of about a second: the ranks
        # have to enter each phase together
        torch.cuda.synchronize()
        torch.distributed.barrier()
    with torch.cuda.stream(stream):
        for c in cells:  # eager pass: loads kernels, NCCL channels
            launch_cell(c, flags, world, peer)
        stream.synchronize()
        progress("eager pass done")
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for c in cells:
                launch_cell(c, flags, world, peer)
        progress("graph captured")
        if world > 1:
            stream.synchronize()
            torch.distributed.barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        # warm-up: at least W replays and about 0.3 s under load, so that the clocks have ramped up and
        # nvidia-smi has samples taken under the same load as the timed steps.  With several ranks the graph
        # holds all-reduces, so EVERY rank must replay it the same number of times: a count that each rank
        # derives from its own clock lets one rank queue collectives that its peers never match.  The
        # count is therefore a constant for world > 1 and only timed for a single rank.
        n_warm = 0
        if world > 1:
            for n_warm in range(1, max(args.warmup, 3, MULTI_RANK_WARMUP_REPLAYS) + 1):
                graph.replay()
                if n_warm % 16 == 0:
                    stream.synchronize()
                    progress(f"warm-up: {n_warm} replays")
        else:
            t_warm = time.perf_counter()
            while n_warm < max(args.warmup, 3) or time.perf_counter() - t_warm < 0.3:
                graph.replay()
                n_warm += 1
                if n_warm % 16 == 0:
                    stream.synchronize()
        stream.synchronize()
        progress(f"warm-up done ({n_warm} replays)")
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        elapsed_ms = e0.elapsed_time(e1)
        progress(f"timed steps done: {elapsed_ms:.2f} ms")
        clocks = sampler.stop() if rank == 0 else None
        parity = None
        if rank == 0 and not args.no_check:
            progress("checking the outputs of the sweep against the oracle")
            parity = check_cells(cells, world, dev)
        # a live CUDA graph that holds NCCL kernels blocks the process group's shutdown
        graph.reset()
        del graph
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # end to end through the operator, host buffers in, host buffers out
    e2e = None
    if world == 1:
        e2e = run_e2e(cells, dev, flags, max(1, min(args.steps, 5)))

    extra = {}
    cpu = None
    if rank == 0 and world == 1:
        if not args.no_table:
            extra = per_cell_table(dev, flags)
            extra["tensor_core_cells"] = run_tensor_core_cells(dev)
        cpu = run_cpu_arm(steps=2, warmup=1)
    progress("sweep finished")
    if not args.no_decode:
        # mixed-precision decode, Llama-3.1-8B architecture, mean 3.0 bits, prompt 128, 128 new tokens
        dec = [run_decode(world, rank, dev, "8b", batch, 128, 128, 3.0, peer=peer) for batch in ((1, 8, 32) if world == 1 else (1,))]
        if world > 1:
            # tensor-parallel decode of the Llama-3.1-70B architecture: seeded 3.5-bit mixture, prompt 512, 256 new tokens
            dec += [run_decode(world, rank, dev, "70b", batch, 512, 256, 3.5, peer=peer) for batch in (1, 16)]
        extra["decode"] = dec

    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama3-8b linear shapes (q/o 4096x4096, k/v 4096x1024, gate/up 4096x14336, down 14336x4096) "
                               "x M{1,2,4,8,16} x b{2,3,4,6,8}, g128, fp16, sliced from 8-bit masters",
                   "cells_per_step": launches_per_step, "l2_policy": "inputs larger than L2: ~400 MB of other weights between reuses",
                   "parallelism": "tp%d" % world if world > 1 else "single", "pdl": not args.no_pdl,
                   "allreduce": ("fused into the row-parallel kernels over peer memory" if peer is not None
                                 else "nccl" + (f" ({peer_note})" if peer_note else "")) if world > 1 else None},
        "clocks": clocks,
        "parity_checked": bool(parity and parity["checked_cells"] == launches_per_step and not parity["failed"]),
        "parity": parity,
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(value / world, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(value / world / peak, 4),
                     "traffic": round(step_bytes / launches_per_step * DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE),
                     "peak_kind": peak_kind, "kernel": "mg::gemv_kernel (all instantiations of the step)",
                     "algorithmic_bytes_per_launch": round(step_bytes / launches_per_step),
                     "mean_launch_us": round(ms_per_step * 1e3 / launches_per_step, 3)},
    }
    if e2e is not None:
        line["e2e"] = e2e
    if cpu is not None:
        line["cpu_baseline"] = {"value": round(cpu["value"], 4), "unit": UNIT, "cores": cpu["cores"], "kind": "port",
                                "sample": cpu["sample"], "dequant_ms_per_step": round(cpu["dequant_ms_per_step"], 2),
                                "matmul_ms_per_step": round(cpu["matmul_ms_per_step"], 2)}
    line.update(extra)
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def run_decode(world: int, rank: int, dev: torch.device, model_name: str, batch: int, prompt_len: int, new_tokens: int,
               mean_bits: float, layers: int | None = None, uniform_bits: int = 0, peer=None) -> dict:
    """Greedy decode of a random-init Llama-architecture model over packed linears: random prompt ids,
    seeded per-layer bitwidths from {2,3,4,6,8} with the given parameter-weighted mean, one CUDA-graph
    replay per token; tok/s = generated tokens * batch / device time of the decode phase (max over ranks)."""
    from matgptq_b200 import decode
    shape = {"8b": decode.LLAMA31_8B, "70b": decode.LLAMA31_70B}[model_name]
    if layers:
        shape = decode.LlamaShape(shape.hidden, shape.intermediate, shape.n_heads, shape.n_kv_heads, layers, shape.vocab)
    names = decode.layer_names(shape)
    if uniform_bits:
        bits = {n: uniform_bits for n in names}
    else:
        bits = decode.mixed_bitwidths(shape, mean_bits, seed=0)
    achieved_bits = sum(bits[n] * names[n] for n in names) / sum(names.values())
    progress(f"decode: building {model_name} batch {batch}")
    model = decode.PackedLlama(shape, bits, dtype=torch.float16, tp_rank=rank, tp_size=world, seed=0, batch=batch,
                               max_seq=prompt_len + new_tokens, device=dev, peer_allreduce=peer)
    progress("decode: model built")
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, shape.vocab, (batch, prompt_len), generator=g).to(dev)
    r = model.generate(prompt, new_tokens, use_graph=True)
    progress("decode: generated")
    t = torch.tensor([r["decode_s"], r["prefill_s"]], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    decode_s, prefill_s = float(t[0]), float(t[1])
    wbytes = model.weight_bytes()
    out = {"model": f"llama-3.1-{model_name} architecture, random init" + (f", {layers} layers" if layers else ""),
           "tp": world, "batch": batch, "prompt_len": prompt_len, "new_tokens": new_tokens,
           "mean_bits": round(achieved_bits, 3), "tok_per_s": round(r["decode_steps"] * batch / decode_s, 1),
           "ms_per_token": round(decode_s / r["decode_steps"] * 1e3, 4), "prefill_ms": round(prefill_s * 1e3, 2),
           "packed_weight_gb_per_rank": round(wbytes / 1e9, 3),
           "weight_stream_gbs_per_rank": round(wbytes / (decode_s / r["decode_steps"]) / 1e9, 1)}
    del model
    torch.cuda.empty_cache()
    return out


def run_tensor_core_cells(dev: torch.device) -> list:
    """Tensor-core regime: bf16, M in {32,64,128,256}, b in {3,4,8}, next to torch's dense bf16 GEMM on the
    dequantised weights.  Cold L2: launches rotate over copies of the weights."""
    from matgptq_b200 import _native, ops
    from oracle import matgptq_oracle as oracle
    out = []
    # launched as the decode harness and the sweep above launch the operator: with programmatic dependent launch
    tc_flags = _native.FLAG_ASYNC | _native.FLAG_BF16 | _native.FLAG_PDL
    for si, (name, (k, n)) in enumerate(synth.LLAMA3_8B_SHAPES.items()):
        layer = synth.make_layer(n, k, GROUP, seed=300 + si, sym=True, dtype=torch.bfloat16, device=dev)
        rows_dev = torch.linspace(0, n - 1, min(PARITY_SAMPLE_ROWS, n)).long().unique().to(dev)
        scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n, k, GROUP)
        for b in (3, 4, 8):
            progress(f"tensor-core cells: {name} b={b}")
            packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n, k, 8, b, GROUP, 3)
            dense = torch.ops.matgptq_cuda.dequantize_matgptq(packed, scales_r, n, k, b, GROUP, 3)
            copies = max(2, min(16, -(-300 * 1024 * 1024 // (dense.numel() * 2))))
            packs = [packed] + [packed.clone() for _ in range(copies - 1)]
            denses = [dense] + [dense.clone() for _ in range(copies - 1)]
            for m in (32, 64, 128, 256):
                x = synth.make_activations(m, k, seed=m, dtype=torch.bfloat16, device=dev)
                y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
                need = ops._lib.matgptq_b200_matmul_workspace_bytes(n, k, m)
                ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)

                def ours(i):
                    ops.matmul_matgptq_raw(x, packs[i % copies], scales_r, n, k, b, GROUP, tc_flags, out=y, workspace=ws if need else None)

                def torch_dense(i):
                    torch.matmul(x, denses[i % copies].t(), out=y)

                times = {}
                reps = 2 * copies
                for label, fn in (("ours", ours), ("dense", torch_dense)):
                    stream = torch.cuda.Stream(device=dev)
                    with torch.cuda.stream(stream):
                        for i in range(copies):
                            fn(i)
                        stream.synchronize()
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph, stream=stream):
                            for i in range(reps):
                                fn(i)
                        graph.replay()
                        stream.synchronize()
                        ts = []
                        for _ in range(5):
                            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                            e0.record(stream)
                            graph.replay()
                            e1.record(stream)
                            stream.synchronize()
                            ts.append(e0.elapsed_time(e1) * 1e3 / reps)
                        times[label] = statistics.median(ts)
                        del graph
                flops = 2.0 * m * n * k
                # outside the timed region: this cell's output against the oracle on a sample of out-features
                y.zero_()
                ours(0)
                torch.cuda.synchronize()
                w_ref = oracle.dequantize_weight(layer.qweight[rows_dev].cpu(), layer.scales[rows_dev].cpu(),
                                                 layer.zeros[rows_dev].cpu(), 8, b)
                err = oracle.rel_err(y[:, rows_dev].cpu(), oracle.linear_fp32_accumulate(x.cpu(), w_ref))
                out.append({"shape": name, "m": m, "b": b, "us": round(times["ours"], 2), "dense_bf16_us": round(times["dense"], 2),
                            "tflops": round(flops / times["ours"] / 1e6, 1),
                            "gbs": round(synth.algorithmic_bytes(n, k, m, b, GROUP) / times["ours"] / 1e3, 1),
                            "rel_err": round(err, 6), "parity_ok": bool(err <= PARITY_TOLERANCE)})
            del packs, denses
        del layer
    return out


def run_e2e(cells, dev, flags, steps: int) -> dict:
    """The same step through torch.ops.matgptq_cuda.matmul_matgptq_out with pinned host activations in and pinned host
    outputs out: per step one H2D copy of all activations, the 100 operator calls, one D2H copy of all outputs,
    all inside the timed region.  Two
    figures: the calls captured once into a CUDA graph and replayed per step (how the reference's callers run
    the operator: `do_bench_cudagraph` in its kernel benchmark, `reduce-overhead` in its HF loop, CUDA graphs in
    vLLM), and the same calls issued eagerly from Python (bound by ~50 us of host work per call)."""
    # one pinned host buffer with every cell's activations, one with every cell's output: a step copies the first
    # to the device in one transfer, runs the 100 operator calls on views of it, each writing its slice of one
    # output buffer, and copies that buffer back in one transfer
    x_off, y_off, nx, ny = [], [], 0, 0
    for c in cells:
        x_off.append(nx)
        y_off.append(ny)
        nx += c["x"].numel()
        ny += c["m"] * c["n_loc"]
    h2d, d2h = nx * 2, ny * 2
    step_bytes = sum(c["bytes"] for c in cells)
    op = torch.ops.matgptq_cuda.matmul_matgptq_out  # the operator's out= form: each call writes its slice of the output buffer

    class Slot:
        """One set of buffers: a step in flight.  `first` rotates the order of the calls, so that two steps in flight
        are half a sweep apart and never read the same weights close in time (the L2 stays cold for both)."""
        def __init__(self, first: int):
            self.order = list(range(first, len(cells))) + list(range(first))
            self.host_x = torch.empty(nx, dtype=torch.float16).pin_memory()
            self.host_y = torch.empty(ny, dtype=torch.float16).pin_memory()
            for c, o in zip(cells, x_off):
                self.host_x[o:o + c["x"].numel()].copy_(c["x"].reshape(-1).cpu())
            self.dev_x = torch.empty(nx, dtype=torch.float16, device=dev)
            self.dev_y = torch.empty(ny, dtype=torch.float16, device=dev)
            self.x_views = [self.dev_x[xo:xo + c["x"].numel()].view(c["m"], c["k_loc"]) for c, xo in zip(cells, x_off)]
            self.y_views = [self.dev_y[yo:yo + c["m"] * c["n_loc"]].view(c["m"], c["n_loc"]) for c, yo in zip(cells, y_off)]
            self.host_y_views = [self.host_y[o:o + c["m"] * c["n_loc"]].view(c["m"], c["n_loc"]) for c, o in zip(cells, y_off)]

        def step(self):
            self.dev_x.copy_(self.host_x, non_blocking=True)
            for i in self.order:
                c = cells[i]
                op(self.x_views[i], c["packed"], c["scales"], c["n_loc"], c["k_loc"], c["b"], GROUP, flags, self.y_views[i])
            self.host_y.copy_(self.dev_y, non_blocking=True)

    slots = [Slot(0), Slot(len(cells) // 2)]

    def timed(fn) -> float:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for _ in range(2):
        slots[0].step()
    eager_ms = timed(slots[0].step)

    # captured: one graph per slot, each on its own stream
    streams = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]
    graphs = []
    for slot, stream in zip(slots, streams):
        with torch.cuda.stream(stream):
            slot.step()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                slot.step()
            for _ in range(3):
                graph.replay()
            stream.synchronize()
            graphs.append(graph)

    # one step at a time: copy in, 100 calls, copy out, then the next step
    with torch.cuda.stream(streams[0]):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(streams[0])
        for _ in range(steps):
            graphs[0].replay()
        e1.record(streams[0])
        streams[0].synchronize()
        serial_ms = e0.elapsed_time(e1) / steps

    # two steps in flight (double buffering, as a server feeding batches would): the copies of one step run while
    # the other computes; every step still copies all its inputs in and all its outputs out inside the timed region
    torch.cuda.synchronize()
    start, stops = torch.cuda.Event(enable_timing=True), []
    start.record(streams[0])
    streams[1].wait_event(start)
    for i in range(steps):
        with torch.cuda.stream(streams[i & 1]):
            graphs[i & 1].replay()
    for stream in streams:
        e = torch.cuda.Event(enable_timing=True)
        e.record(stream)
        stops.append(e)
    torch.cuda.synchronize()
    piped_ms = max(start.elapsed_time(e) for e in stops) / steps

    # the graphs' copies really moved the data: the host outputs of both slots hold the last replays' results
    ok = None
    if all("y" in c for c in cells):
        ok = all(torch.equal(hy, c["y"].cpu()) for slot in slots for c, hy in list(zip(cells, slot.host_y_views))[::7])
    del graphs
    return {"value": round(step_bytes / (piped_ms * 1e-3) / 1e9, 2), "unit": UNIT, "ms_per_step": round(piped_ms, 4),
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "mode": "per step one H2D copy of all activations from pinned memory, 100 calls of torch.ops.matgptq_cuda.matmul_matgptq_out "
                    "(each into its slice of one output buffer), one D2H copy of all outputs to pinned memory; a step is one replay of "
                    "a captured CUDA graph; two steps in flight on two streams with their own buffers (double buffering)",
            "serial_value": round(step_bytes / (serial_ms * 1e-3) / 1e9, 2), "serial_ms_per_step": round(serial_ms, 4),
            "eager_value": round(step_bytes / (eager_ms * 1e-3) / 1e9, 2), "eager_ms_per_step": round(eager_ms, 4),
            "host_outputs_match_device": ok}


def single_cell_main(args) -> None:
    """Launch one cell a few times, eagerly, over rotating weight copies (for profilers)."""
    from matgptq_b200 import _native, ops
    name, b, m = args.cell.split(":")
    b, m = int(b), int(m)
    k, n = synth.LLAMA3_8B_SHAPES[name]
    dev = torch.device("cuda", 0)
    dtype = torch.bfloat16 if args.bf16 else torch.float16
    layer = synth.make_layer(n, k, GROUP, seed=1, sym=True, dtype=dtype, device=dev)
    scales_r = torch.ops.matgptq_cuda.reorder_matgptq_scales(layer.scales, n, k, GROUP)
    packed = torch.ops.matgptq_cuda.slice_pack_matgptq_qweights(layer.qweight, n, k, 8, b, GROUP, 1)
    copies = max(2, min(32, -(-256 * 1024 * 1024 // (packed.numel() * 4))))
    packs = [packed] + [packed.clone() for _ in range(copies - 1)]
    x = synth.make_activations(m, k, seed=m, dtype=dtype, device=dev)
    y = torch.empty(m, n, dtype=dtype, device=dev)
    flags = _native.FLAG_ASYNC | (_native.FLAG_PDL if not args.no_pdl else 0) | (_native.FLAG_BF16 if args.bf16 else 0)
    need = ops._lib.matgptq_b200_matmul_workspace_bytes(n, k, m)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    for i in range(args.launches):
        ops.matmul_matgptq_raw(x, packs[i % copies], scales_r, n, k, b, GROUP, flags, out=y, workspace=ws if need else None)
    torch.cuda.synchronize()
    print(json.dumps({"cell": args.cell, "launches": args.launches, "copies": copies,
                      "algorithmic_bytes": synth.algorithmic_bytes(n, k, m, b, GROUP)}))


def decode_main(args) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if args.watchdog > 0:
        start_watchdog(args.watchdog, args.watchdog_total)
    if world > 1:
        progress("bringing the process group up")
        torch.distributed.init_process_group("nccl", device_id=dev)
    peer = None
    if world > 1 and args.allreduce == "fused":
        from matgptq_b200 import ops  # noqa: F401
        peer, _ = make_peer_allreduce(dev)
    parts = args.decode.split(":")
    uniform = int(parts[4][1:]) if parts[4].startswith("u") else 0  # "u4": every layer at 4 bits
    r = run_decode(world, rank, dev, parts[0], int(parts[1]), int(parts[2]), int(parts[3]),
                   0.0 if uniform else float(parts[4]), int(parts[5]) if len(parts) > 5 else None, uniform_bits=uniform, peer=peer)
    if rank == 0:
        print(json.dumps({"metric": "decode_tokens_per_s", "value": r["tok_per_s"], "unit": "tok/s", "n_gpus": world, **r}), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cell", type=str, default=None,
                    help="shape:b:m, e.g. q_o:4:1 - only launch this cell (--launches times) and exit")
    ap.add_argument("--launches", type=int, default=8)
    ap.add_argument("--bf16", action="store_true", help="with --cell: bfloat16 activations, scales and output")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--watchdog", type=float, default=150.0,
                    help="seconds one phase may last before the run reports where it stands and exits 3 (0 = off)")
    ap.add_argument("--watchdog-total", type=float, default=900.0, help="the same for the whole run")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch")
    ap.add_argument("--allreduce", choices=["fused", "nccl"], default="fused",
                    help="several ranks: all-reduce of the row-parallel layers fused into their kernels over peer memory, or NCCL")
    ap.add_argument("--no-table", action="store_true", help="skip the per-cell cold-L2 table")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of the sweep's outputs with the oracle")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode measurement")
    ap.add_argument("--decode", type=str, default=None,
                    help="model:batch:prompt:new:bits[:layers] - only run this decode and exit; bits is the mean of a seeded "
                         "per-layer mixture (70b:16:512:256:3.5) or uN for N bits everywhere (70b:1:512:256:u4)")
    args = ap.parse_args()
    if args.decode:
        decode_main(args)
    elif args.cell:
        single_cell_main(args)
    elif args.impl == "reference":
        reference_main(args)
    else:
        ours_main(args)


if __name__ == "__main__":
    main()
