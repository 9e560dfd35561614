#!/usr/bin/env python
"""Benchmark of the tail-biting trellis encoder: weights encoded per second (L=16, K=3).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one pass of the hot path over one batch: the tiles of one 4096 x 4096 matrix
(iid N(0, 0.02^2) with 1 % outliers x20, CPU generator seed 0) after randomized-Hadamard
incoherence processing with seed 0, i.e. 65 536 independent 256-weight tiles, encoded at
K = 3 with the 3INST codebook (packed codes, reconstruction and per-tile squared error out).
The matrix is synthetic: seeded random values with the shape and distribution the reference's
real weights would have; it is built on the host exactly as the configuration states it
(``trellis_b200.workloads.cfg2_tiles``), so the tiles, and ``mse_z``, are the same on every box.

With N > 1 (launched by torchrun, one rank per GPU) every rank encodes a matrix of that
shape (weak scaling: work shards by whole matrices, no exchange during compute) and the
packed codes are gathered over NCCL inside the timed step.  After the timed region two
further multi-GPU measurements are taken once each and added to the line:
  tile_split    ONE such matrix cut into contiguous tile ranges over the N ranks, packed
                codes all-gathered (strong scaling of a single plain matrix);
  model_encode  a fixed slice of the Qwen3-8B-shaped model (8 of 36 layers = 56 matrices,
                1.54 G weights, LDLQ with synthetic Hessians on the 24 MLP matrices), whole
                matrices placed longest-first on the ranks, three matrices in flight per GPU,
                packed codes gathered to rank 0 (strong scaling of the model-level encode).

Printed: ONE JSON line on rank 0 with
  value     whole-job weights/s with the tiles resident in HBM, timed with CUDA events
            over exactly K steps between barriers, max over ranks;
  e2e       the same through the public Python API with HOST tensors (pinned): each step
            copies the tiles host->device and the results device->host inside the timing;
  roofline  the Viterbi step kernel alone, timed live with CUDA events through the
            forward-only entry point, against the fp32/INT lane-issue ceiling;
  cpu_baseline  the CPU oracle (a C port of the reference's PyTorch dynamic programme)
            on a bounded sample of the same tiles, all host threads (N = 1 only);
  parity    64 tiles spread over the last timed step's output and 64 tiles of the launches the
            roofline leg times, checked bit for bit against the CPU oracle after the timing.

``--impl reference`` times the reference's own ``viterbi_tb`` (fp32 PyTorch DP, the staged copy under
``oracle/_ref``) on the host cores, rank 0 only, on tiles of the same workload, and prints the same kind of
line with the C port's rate beside it; without the staged copy it times the C port.
``--impl reference-triton`` (never the default; one GPU) times the reference's Triton encoder on the GPU.
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
for _p in (ROOT, os.path.join(ROOT, "trellis-everywhere_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

K_BITS = 3
CODEBOOK = "3inst"
MATRIX = (4096, 4096)
T_SEQ = 256
STATE_EVALS_PER_WEIGHT = 2 * 65536            # two passes x 2^16 add-compare-select per step
LANE_OPS_PER_EVAL = 4                         # fsub, fmul, fadd, compare-select: the algorithmic minimum
WORKLOAD = ("config 2: 4096x4096 fp32 matrix, N(0,0.02^2) + 1% outliers x20, incoherence-processed, "
            "65536 tiles of 256, K=3, L=16, 3INST")


# ------------------------------------------------------------------------------------ helpers
def measured_peaks() -> dict:
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi (read-only) while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = [int(r[0]) for r in self.rows]
        busy = [c for c in sm if c > 0.5 * max(sm)] or sm
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": int(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


def workload_tiles_host(lut_cpu):
    """The second benchmark configuration's tiles, built on the host as the configuration states: [65536, 256] fp32."""
    from trellis_b200 import workloads
    return workloads.cfg2_tiles(lut_cpu)


def host_threads() -> int:
    """Cores this process may run on.  Not the OpenMP default: torchrun exports OMP_NUM_THREADS=1 to every rank, which
    would make the CPU legs single-threaded whenever the benchmark is launched for more than one GPU."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_port_rate(tiles_np, seconds: float, threads: int):
    """Weights/s of the CPU oracle on a bounded sample of `tiles_np`, sized to take about `seconds`."""
    from oracle import oracle as O
    lut = O.codebook_lut(CODEBOOK)
    probe = min(len(tiles_np), max(threads, 8))
    t0 = time.perf_counter()
    O.viterbi_tb(tiles_np[:probe], K_BITS, lut, nthreads=threads)
    per_tile = (time.perf_counter() - t0) / probe
    n = int(max(probe, min(len(tiles_np), seconds / max(per_tile, 1e-9))))
    n = max(threads, n // threads * threads)
    t0 = time.perf_counter()
    O.viterbi_tb(tiles_np[:n], K_BITS, lut, nthreads=threads)
    dt = time.perf_counter() - t0
    return n * T_SEQ / dt, n, dt


# ------------------------------------------------------------------------------------ reference arms
def run_reference(args, rank: int, world: int) -> None:
    """The reference's CPU implementation of the path on the box's host cores, rank 0 only.

    With the staged reference (``oracle/_ref``): its own ``viterbi_tb(w, K, lut, dp_dtype=float32)``, all host threads,
    one batch of the workload's tiles per step at the batch size (16 / 64 / 256 tiles) that the warm-up found fastest
    and that keeps the run within a few minutes; the C port's rate on the same tiles is reported beside it.
    """
    if rank != 0:
        return
    import numpy as np
    import torch
    from oracle import make_ref
    from oracle import oracle as O
    O.build()
    threads = host_threads()
    torch.set_num_threads(threads)
    lut_np = O.codebook_lut(CODEBOOK)
    tiles = workload_tiles_host(torch.from_numpy(lut_np))
    port_rate, port_n, port_dt = cpu_port_rate(tiles[:4096].numpy(), min(args.cpu_seconds, 8.0), threads)
    port = {"value": port_rate, "unit": "weights/s", "cores": threads, "kind": "port",
            "sample": f"first {port_n} tiles of the same workload, {port_dt:.1f} s (C/OpenMP restatement of the same DP)"}
    if make_ref.staged() is not None:
        rq, _ = make_ref.import_reference()
        lut = rq.codebook_lut(CODEBOOK)
        assert np.array_equal(lut.numpy().view(np.uint32), lut_np.view(np.uint32))
        rates = {}
        for b in (16, 64, 256):                              # warm-up doubles as the batch-size probe
            t0 = time.perf_counter()
            rq.viterbi_tb(tiles[:b], K_BITS, lut, dp_dtype=torch.float32)
            rates[b] = (b * T_SEQ / (time.perf_counter() - t0), time.perf_counter() - t0)
        fits = {b: r for b, (r, dt) in rates.items() if dt * (args.steps + args.warmup) <= 150.0} or {16: rates[16][0]}
        batch = max(fits, key=fits.get)
        kind, what = "reference", "the reference's own viterbi_tb (fp32 PyTorch DP)"

        def step(i):
            lo = (i * batch) % (tiles.shape[0] - batch)
            rq.viterbi_tb(tiles[lo:lo + batch], K_BITS, lut, dp_dtype=torch.float32)
        probe = {str(b): r for b, (r, _) in rates.items()}
    else:
        batch = max(threads, (args.ref_tiles // threads) * threads)
        kind, what, probe = "port", "C/OpenMP restatement of the reference's DP (reference modules not staged)", None
        tiles_np = tiles.numpy()

        def step(i):
            lo = (i * batch) % (tiles_np.shape[0] - batch)
            O.viterbi_tb(tiles_np[lo:lo + batch], K_BITS, lut_np, nthreads=threads)
    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(args.warmup + i)
    dt = (time.perf_counter() - t0) / args.steps
    value = batch * T_SEQ / dt
    line = {
        "impl": "reference", "metric": f"weights encoded/sec (L=16, K={K_BITS})", "value": value, "unit": "weights/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "K": K_BITS, "codebook": CODEBOOK, "tiles_per_step": batch},
        "cpu_baseline": {"value": value, "unit": "weights/s", "cores": threads, "kind": kind,
                         "sample": f"{batch} tiles of the workload per step through {what}; the full 65536 would take "
                                   f"{65536 * T_SEQ / value / 60:.0f} min", "batch_probe_weights_per_s": probe, "port": port},
        "e2e": {"value": value, "unit": "weights/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_triton(args) -> None:
    """Side arm, one GPU: the reference's Triton encoder (``viterbi_tb_triton``, MCG only) as Triton JIT-compiles it for
    this GPU, at 2 048 and 16 384 tiles, K = 2 and 3, next to this library on the same tiles (rates, code agreement, MSE)."""
    import torch
    from oracle import make_ref
    if make_ref.staged() is None:
        print(json.dumps({"impl": "reference-triton", "unavailable": "reference modules not staged under oracle/_ref"}), flush=True)
        return
    rq, _ = make_ref.import_reference()
    try:
        from trellis.viterbi_triton import viterbi_tb_triton
    except Exception as e:                                   # triton missing or unusable on this box
        print(json.dumps({"impl": "reference-triton", "unavailable": f"cannot import the Triton encoder: {e}"[:200]}), flush=True)
        return
    from trellis_b200 import qtip
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    lut = rq.codebook_lut("mcg").to(dev)
    rows = []

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            out = fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps, out

    with ClockSampler(0) as clocks:
        for K in (2, 3):
            for n in (2048, 16384):
                g = torch.Generator(device=dev).manual_seed(K * 100000 + n)
                w = torch.randn(n, T_SEQ, generator=g, device=dev) * 1.2437
                ms_t, (bits_t, dq_t) = timed(lambda: viterbi_tb_triton(w, K, lut), max(1, args.steps // 2))
                ms_b, r = timed(lambda: qtip.encode(w, K, "mcg", want_bits=True), max(3, args.steps))
                _, dq_ref = rq.viterbi_tb(w[:64], K, lut, dp_dtype=torch.float32)       # its own fp32 DP, on the GPU
                rows.append({"K": K, "tiles": n, "triton_ms": ms_t, "triton_weights_per_s": n * T_SEQ / (ms_t * 1e-3),
                             "b200_ms": ms_b, "b200_weights_per_s": n * T_SEQ / (ms_b * 1e-3), "speedup": ms_t / ms_b,
                             "symbols_equal_frac": float((bits_t == r.bits).float().mean()),
                             "mse_triton": float(((w - dq_t) ** 2).mean()), "mse_b200": float(((w - r.dq) ** 2).mean()),
                             "b200_equals_reference_fp32_dp_on_64_tiles": bool(torch.equal(r.dq[:64], dq_ref)),
                             "triton_equals_reference_fp32_dp_on_64_tiles": bool(torch.equal(dq_t[:64], dq_ref))})
    head = rows[-1]
    print(json.dumps({"impl": "reference-triton", "metric": "weights encoded/sec (L=16, K=3)", "value": head["triton_weights_per_s"],
                      "unit": "weights/s", "n_gpus": 1, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "SIDE ARM: the reference's viterbi_tb_triton (MCG) vs this library on N(0, 1.2437^2) tiles"},
                      "cases": rows, "clocks": clocks.summary()}), flush=True)


# ------------------------------------------------------------------------------------ B200 arm
def check_parity(torch, qtip, lib, _lib, tiles, last, dev, cid) -> dict:
    """After the timing: the last timed step's output and the roofline leg's launches against the CPU oracle."""
    import numpy as np
    from oracle import oracle as O
    O.build()
    lut = O.codebook_lut(CODEBOOK)
    n = tiles.shape[0]
    idx = torch.linspace(0, n - 1, min(64, n), device=dev).round().long()
    w_np = tiles[idx].cpu().numpy()
    bits, dq, sse = O.viterbi_tb(w_np, K_BITS, lut, with_sse=True)
    ok_packed = np.array_equal(last.packed[idx].cpu().numpy().view(np.uint32), O.pack_bits(bits, K_BITS))
    ok_dq = np.array_equal(last.dq[idx].cpu().numpy().view(np.uint32), dq.view(np.uint32))
    ok_sse = np.array_equal(last.sse[idx].cpu().numpy().view(np.uint32), sse.view(np.uint32))
    # the launches the roofline leg times: one full chunk through the pass-level entry point (same launch code and
    # tile-group shape as tcq_forward_pass), states of 64 spread tiles against the oracle's passes
    chunk = min(n, 24 * torch.cuda.get_device_properties(dev).multi_processor_count)
    s1 = qtip.viterbi_pass_b200(tiles[:chunk], K_BITS, None, cid, roll=128)
    jdx = torch.linspace(0, chunk - 1, min(64, chunk), device=dev).round().long()
    w2 = tiles[:chunk][jdx].cpu().numpy()
    o1 = O.viterbi_pass(np.roll(w2, 128, axis=1), K_BITS, lut, None)
    ok_p1 = np.array_equal(s1[jdx].cpu().numpy(), o1)
    ov = (s1[:, 128] >> K_BITS).to(torch.int32)
    s2 = qtip.viterbi_pass_b200(tiles[:chunk], K_BITS, ov, cid)
    o2 = O.viterbi_pass(w2, K_BITS, lut, (o1[:, 128] >> K_BITS).astype(np.int32))
    ok_p2 = np.array_equal(s2[jdx].cpu().numpy(), o2)
    return {"tiles": int(idx.numel()), "bits_equal": bool(ok_packed), "dq_equal": bool(ok_dq), "sse_equal": bool(ok_sse),
            "pass_tiles": int(jdx.numel()), "pass1_states_equal": bool(ok_p1), "pass2_states_equal": bool(ok_p2),
            "against": "CPU oracle (oracle/tcq_oracle.c), bit for bit"}


def measure_tile_split(torch, dist, qtip, tdist, tiles, world: int, rank: int, dev, cid, fence, reps: int = 3) -> dict:
    """ONE matrix of the workload cut into contiguous tile ranges over the ranks; packed codes all-gathered."""
    n = tiles.shape[0]
    lo, hi = tdist.tile_range(n, rank, world)
    mine = tiles[lo:hi].contiguous()

    def once():
        r = qtip.encode(mine, K_BITS, cid, want_dq=True, want_sse=True)
        return tdist.gather_packed(r.packed, n) if world > 1 else r.packed

    once()
    fence()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        out = once()
    b.record()
    fence()
    t = torch.tensor([a.elapsed_time(b) / reps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    per_round = (sms // 2) * 6                                # tiles one round of 2-SM clusters advances at K = 3
    return {"what": "one 65536-tile matrix split by contiguous tile ranges, all-gather of packed codes (strong scaling)",
            "ms": ms, "weights_per_s": n * T_SEQ / (ms * 1e-3), "tiles_per_rank": hi - lo,
            "rounds_per_rank": (hi - lo) / per_round, "whole_rounds_per_rank": -(-(hi - lo) // per_round),
            "gathered_rows": int(out.shape[0])}


def measure_model_encode(torch, dist, args, world: int, rank: int, dev) -> dict:
    """A fixed slice of the Qwen3-8B-shaped model through ``model.encode_model`` (strong scaling over the ranks)."""
    from trellis_b200 import model
    shapes = model.qwen3_8b_shapes(layers=args.model_layers)
    # Warm-up, untimed: a two-matrix model of small shapes through the same code (one plain, one LDLQ matrix per rank and
    # the gather), so that one-time costs are not billed to the measurement: cuSOLVER / cuBLAS handles of the block-LDL
    # step, the library's kernel images, NCCL's point-to-point connections for the gather (about a second per rank
    # together, the same at every N, which would read as a scaling loss at N = 8 where the measurement takes six).
    warm = {f"model.layers.{i}.{m}": s for i in range(world) for m, s in (("self_attn.k_proj", (64, 256)), ("mlp.down_proj", (64, 256)))}
    model.encode_model(warm, K_BITS, "mcg", device=dev, streams=args.model_streams,
                       hessian_fn=lambda name, k, d: model.synthetic_hessian(name, k, d, rows=512))
    recs = []
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    results, own = model.encode_model(shapes, K_BITS, "mcg", device=dev, log=recs.append, streams=args.model_streams, gather=False)
    torch.cuda.synchronize(dev)
    busy = time.perf_counter() - t0                           # this rank's own matrices, before it waits for anyone
    ldlq_names = [n for n in shapes if model.is_mlp(n)]
    gathered = model.gather_model_codes(shapes, ldlq_names, own, K_BITS, world, rank, dev)
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t0
    ldlq_s = sum(r["seconds"] for r in recs if r["ldlq"])
    plain_s = sum(r["seconds"] for r in recs if not r["ldlq"])
    stats = torch.tensor([busy, ldlq_s, plain_s, float(len(recs))], dtype=torch.float64, device=dev)
    if world > 1:
        allst = [torch.empty_like(stats) for _ in range(world)]
        dist.all_gather(allst, stats)
        w_t = torch.tensor([wall], dtype=torch.float64, device=dev)
        dist.all_reduce(w_t, op=dist.ReduceOp.MAX)
        wall = float(w_t)
    else:
        allst = [stats]
    total = sum(a * b for a, b in shapes.values())
    busy_all = [float(x[0]) for x in allst]
    return {"what": f"{args.model_layers} of 36 Qwen3-8B-shaped layers ({len(shapes)} matrices, {total} weights), K={K_BITS} MCG, "
                    f"LDLQ (synthetic Hessians from 8192 rows) on the MLP matrices, {args.model_streams} matrices in flight per GPU, "
                    "whole matrices placed longest-first, packed codes gathered to rank 0; includes weight and Hessian synthesis",
            "seconds": wall, "weights_per_s": total / wall, "matrices": len(shapes), "weights": total,
            "rank_busy_seconds": busy_all, "imbalance_max_over_mean": max(busy_all) / (sum(busy_all) / len(busy_all)),
            "gather_and_wait_seconds": wall - max(busy_all),
            "matrix_seconds_ldlq": [float(x[1]) for x in allst], "matrix_seconds_plain": [float(x[2]) for x in allst],
            "matrices_per_rank": [int(x[3]) for x in allst],
            "gathered_matrices": len(gathered) if gathered is not None else 0,
            "note": "matrix_seconds_* add up the per-matrix times of overlapping matrices, so they exceed the busy time"}


def run_b200(args, rank: int, local_rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist
    from trellis_b200 import _lib, qtip
    from trellis_b200 import dist as tdist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 encoder has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.lib()
    cid = qtip.CODEBOOK_IDS[CODEBOOK]

    # torchrun exports OMP_NUM_THREADS=1; the host-side build of the workload is a few matmuls.  Every rank builds it at the
    # same time, so each takes its share of the cores (all ranks asking for all cores makes the OpenMP teams fight).
    torch.set_num_threads(max(1, host_threads() // max(world, 1)))
    host = workload_tiles_host(qtip.codebook_lut(CODEBOOK, "cpu")).pin_memory()
    if args.tiles:                                       # reduced case for profiler captures; not the benchmark
        host = host[:args.tiles].contiguous().pin_memory()
    tiles = host.to(dev)
    n = tiles.shape[0]
    nw = T_SEQ * K_BITS // 32
    gathered = torch.empty((world * n, nw), dtype=torch.int32, device=dev) if world > 1 else None

    def step():
        r = qtip.encode(tiles, K_BITS, cid, want_dq=True, want_sse=True)
        if world > 1:                                    # the one collective: packed codes to every rank's buffer
            dist.all_gather_into_tensor(gathered, r.packed)
        return r

    def fence():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 1)):
        step()
    ws_bytes = int(lib.tcq_workspace_bytes(n, K_BITS))
    launches_per_step = int(lib.tcq_encode_launches(n, K_BITS, ws_bytes))

    # ---- device-resident throughput ----
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for _ in range(args.steps):
            last = step()
        e1.record()
        fence()
    ms = e0.elapsed_time(e1)
    mse = float(last.sse.double().sum() / tiles.numel())
    qtip.workspace_status(n, K_BITS, dev)                 # raises if a bounded wait gave up or a weight was not finite

    # ---- end to end: host tensors through the public API ----
    h2d = host.numel() * 4
    d2h = n * nw * 4 + n * T_SEQ * 4 + n * 4
    host_out = qtip.Encoded(torch.empty((n, nw), dtype=torch.int32, pin_memory=True),
                            torch.empty((n, T_SEQ), dtype=torch.float32, pin_memory=True),
                            torch.empty((n,), dtype=torch.float32, pin_memory=True), None)
    qtip.encode(host, K_BITS, cid, out=host_out)          # warm the staging path
    fence()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        r_host = qtip.encode(host, K_BITS, cid, want_dq=True, want_sse=True, out=host_out)   # returns with results on the host
        if world > 1:
            dist.all_gather_into_tensor(gathered, r_host.packed.to(dev, non_blocking=True))
    fence()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    if not torch.equal(r_host.packed, last.packed.cpu()):
        raise SystemExit("end-to-end leg produced different codes than the device-resident leg")

    # ---- the step kernel alone (roofline), one chunk per launch exactly as encode uses it ----
    chunk = min(n, 24 * torch.cuda.get_device_properties(dev).multi_processor_count)
    ws = qtip._workspace(dev, chunk, K_BITS)
    ov = torch.randint(0, 1 << (16 - K_BITS), (chunk,), dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    kern_ms = []
    for overlap, roll, bp_steps in ((None, 128, 128), (ov, 0, 256)):       # pass 1 and pass 2 as the encoder runs them
        args_c = (tiles.data_ptr(), chunk, K_BITS, cid, overlap.data_ptr() if overlap is not None else None, roll,
                  bp_steps, ws.data_ptr(), ws.numel(), stream)
        _lib.check(lib.tcq_forward_pass(*args_c), "tcq_forward_pass")
        torch.cuda.synchronize(dev)
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        k0.record()
        for _ in range(reps):
            _lib.check(lib.tcq_forward_pass(*args_c), "tcq_forward_pass")
        k1.record()
        torch.cuda.synchronize(dev)
        kern_ms.append(k0.elapsed_time(k1) / reps)

    # ---- parity of what was timed (rank 0 checks its own output; every rank ran the same kernels) ----
    parity = check_parity(torch, qtip, lib, _lib, tiles, last, dev, cid) if rank == 0 and not args.no_parity else None
    if parity is not None and not all(v for k, v in parity.items() if k.endswith("_equal")):
        raise SystemExit(f"parity check against the CPU oracle FAILED: {parity}")

    # ---- the harder multi-GPU shapes, once each ----
    tile_split = model_enc = None
    if not args.tiles and not args.no_scaling_extras:
        tile_split = measure_tile_split(torch, dist, qtip, tdist, tiles, world, rank, dev, cid, fence)
        qtip.release_workspaces()
        model_enc = measure_model_encode(torch, dist, args, world, rank, dev)

    # ---- reduce over ranks ----
    times = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = (float(x) for x in times)
    total_weights = world * n * T_SEQ * args.steps

    line = None
    if rank == 0:
        peaks = measured_peaks()
        props = torch.cuda.get_device_properties(dev)
        sms = props.multi_processor_count
        sm_max_mhz = float(peaks.get("sm_max_mhz", 1965.0))
        peak_lane_ops = sms * 128 * sm_max_mhz * 1e6
        avg_kernel_ms = sum(kern_ms) / 2
        evals_per_launch = chunk * T_SEQ * 65536
        achieved = evals_per_launch * LANE_OPS_PER_EVAL / (avg_kernel_ms * 1e-3)
        bp_bytes = chunk * (128 + 256) / 2 * (1 << (16 - K_BITS)) * K_BITS / 8      # mean of the two passes
        ck = clocks.summary()
        roofline = {
            "bound": "alu", "kernel": f"Viterbi step kernel (tcq_forward_cluster_kernel, K={K_BITS}, {CODEBOOK}, 2 CTAs per cluster)",
            "achieved": achieved / 1e12, "peak": peak_lane_ops / 1e12, "unit": "Tlane-op/s", "frac": achieved / peak_lane_ops,
            "peak_source": f"{sms} SMs x 128 fp32/int lanes x {sm_max_mhz:.0f} MHz (max SM clock of MEASURED_PEAKS.json"
                           f"{'' if peaks else '; file absent, nominal clock used'}); the path does no tensor-core or "
                           "HBM-bound work, so the measured HBM/bf16 peaks do not bound it",
            "algorithmic": "4 lane-ops (fsub, fmul, fadd, compare-select) x 65536 state evaluations per tile-step",
            "launch_ms": {"pass1": kern_ms[0], "pass2": kern_ms[1]}, "tiles_per_launch": chunk,
            "frac_at_sampled_clock": (achieved / (sms * 128 * ck["sm_mhz"] * 1e6)) if ck.get("sm_mhz") else None,
            # ncu dram__bytes_read+write of an 888-tile launch pair = 0.89 of its algorithmic backpointer bytes
            # (profiles/step_kernel_k3_3inst_888tiles_ncu_full.md), scaled here by the tiles per launch
            "traffic": 0.89 * bp_bytes,
            "hbm": {"algorithmic_bytes_per_launch": bp_bytes, "achieved_GBps": bp_bytes / (avg_kernel_ms * 1e-3) / 1e9,
                    "peak_GBps": peaks.get("hbm_gbs"), "note": "packed backpointer stream, K bits per edge per step"},
        }
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as O
            O.build()
            threads = host_threads()
            rate, n_s, dt = cpu_port_rate(host[:4096].numpy(), args.cpu_seconds, threads)
            cpu = {"value": rate, "unit": "weights/s", "cores": threads, "kind": "port",
                   "sample": f"first {n_s} tiles of the same workload, {dt:.1f} s"}
        line = {
            "metric": f"weights encoded/sec (L=16, K={K_BITS})", "value": total_weights / (ms * 1e-3), "unit": "weights/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": (WORKLOAD if not args.tiles else f"REDUCED to {n} tiles (profiling case) of: " + WORKLOAD)
                       + ("" if (K_BITS, CODEBOOK) == (3, "3inst") else f" -- SIDE MEASUREMENT at K={K_BITS}, {CODEBOOK}"),
                       "K": K_BITS, "codebook": CODEBOOK, "tiles_per_gpu": n,
                       "parallelism": f"{world} x whole matrices, NCCL all-gather of packed codes" if world > 1 else "1 GPU",
                       "l2": "each step streams 2.7 GiB of backpointer scratch, far more than the 126 MB L2, so nothing "
                             "survives between steps; the 64 MiB of tiles are re-read from HBM"},
            "e2e": {"value": total_weights / (e2e_ms * 1e-3), "unit": "weights/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": ck, "roofline": roofline, "cpu_baseline": cpu, "mse_z": mse, "parity": parity,
            "tile_split": tile_split, "model_encode": model_enc,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def run_decode_matvec(args) -> None:
    """Side measurement of the consumer of the packed format: y = x Zq^T from packed codes (lm_head-shaped matrix).

    One step = one product of the [n_out, k_in] code matrix (K bits per weight, random code words: every bit pattern is a
    valid stream) with ``m`` right-hand sides.  The packed words (larger than L2) stay resident in HBM, as weights do when
    serving; ``e2e`` copies x from pinned host memory and y back inside the timing.
    """
    import numpy as np
    import torch
    from trellis_b200 import _lib, qtip
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n_out, k_in, m = args.n_out or 151936, args.k_in or 4096, args.m
    tiles = (n_out // 16) * (k_in // 16)
    g = torch.Generator(device=dev).manual_seed(0)
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (tiles, 8 * K_BITS), dtype=torch.int32, device=dev, generator=g)
    x = torch.randn(m, k_in, device=dev, generator=g)
    xh = x.cpu().pin_memory()
    yh = torch.empty((m, n_out), dtype=torch.float32, pin_memory=True)
    launches = (m + 3) // 4

    def step_device():
        return qtip.decode_matvec(packed, n_out, k_in, K_BITS, CODEBOOK, x)

    def step_host():
        yh.copy_(qtip.decode_matvec(packed, n_out, k_in, K_BITS, CODEBOOK, xh.to(dev, non_blocking=True)), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    with ClockSampler(0) as clocks:
        ms = timed(step_device)
        ms_host = timed(step_host)
        t_end = time.time() + 1.0                       # keep the GPU busy long enough for a few clock samples
        while time.time() < t_end:
            step_device()
        torch.cuda.synchronize()
    weights = n_out * k_in
    peaks = measured_peaks()
    hbm = peaks.get("hbm_gbs")
    packed_gbs = weights * K_BITS / 8 / (ms * 1e-3) / 1e9
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    ck = clocks.summary()
    line = {
        "metric": f"weights decoded and multiplied/sec (decode-matvec, L=16, K={K_BITS})", "value": weights / (ms * 1e-3),
        "unit": "weights/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"SIDE MEASUREMENT (consumer of the packed format): [{n_out}, {k_in}] code matrix, K={K_BITS}, "
                               f"{CODEBOOK}, {m} right-hand side(s); packed words {weights * K_BITS / 8 / 2 ** 20:.0f} MiB resident "
                               "in HBM (larger than L2, no flush needed)", "n_out": n_out, "k_in": k_in, "m": m},
        "e2e": {"value": weights / (ms_host * 1e-3), "unit": "weights/s", "h2d_bytes_per_step": m * k_in * 4,
                "d2h_bytes_per_step": m * n_out * 4},
        "gpu_launches": launches * args.steps,
        "roofline": {"bound": "hbm", "kernel": f"tcq_decode_matvec_kernel<K={K_BITS}, {CODEBOOK}>", "achieved": packed_gbs,
                     "peak": hbm if hbm else 6650.0, "unit": "GB/s", "frac": packed_gbs / (hbm if hbm else 6650.0),
                     "peak_source": "MEASURED_PEAKS.json hbm_gbs (of measured)" if hbm else "fallback 6.65 TB/s (of fallback)",
                     "traffic": None,
                     "note": "the kernel is bound by instruction issue, not HBM: see weights_per_clk_per_sm",
                     "weights_per_clk_per_sm": weights / (ms * 1e-3) / sms / ((ck["sm_mhz"] or 1965.0) * 1e6)},
        "clocks": ck,
    }
    if not args.no_cpu_baseline:
        from oracle import oracle as O
        O.build()
        rows = min(n_out, 2048)                              # bounded sample: the first tile rows of the same matrix
        pk = packed[: (rows // 16) * (k_in // 16)].cpu().numpy().view(np.uint32)
        xn = x.cpu().numpy()
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < min(args.cpu_seconds, 10.0):
            zq = O.decode_packed(pk, K_BITS, CODEBOOK).reshape(rows // 16, k_in // 16, 16, 16).transpose(0, 2, 1, 3).reshape(rows, k_in)
            _ = xn @ zq.T
            reps += 1
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": rows * k_in * reps / dt, "unit": "weights/s", "cores": O.max_threads(), "kind": "port",
                                "sample": f"first {rows} rows of the same matrix, window decode (C oracle) + numpy product, {reps} repeats"}
    print(json.dumps(line), flush=True)


def run_decode(args) -> None:
    """Side measurement of the packed decode kernel (codes -> reconstruction): 4 bytes written + K/8 read per weight.

    262 144 tiles of random code words (every bit pattern is a valid stream): 256 MiB of output, larger than L2, so
    back-to-back launches run at DRAM speed.  ``e2e`` copies the packed words from pinned host memory and the
    reconstruction back inside the timing."""
    import numpy as np
    import torch
    from trellis_b200 import _lib, qtip
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n = args.tiles or 262144
    nw = 8 * K_BITS
    g = torch.Generator(device=dev).manual_seed(0)
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, nw), dtype=torch.int32, device=dev, generator=g)
    dq = torch.empty((n, T_SEQ), dtype=torch.float32, device=dev)
    L = _lib.lib()
    cid = qtip.CODEBOOK_IDS[CODEBOOK]
    st = torch.cuda.current_stream().cuda_stream
    ph = packed.cpu().pin_memory()
    dh = torch.empty((n, T_SEQ), dtype=torch.float32, pin_memory=True)

    def step_device():
        _lib.check(L.tcq_decode_packed(packed.data_ptr(), n, K_BITS, cid, dq.data_ptr(), st), "tcq_decode_packed")

    def step_host():
        dh.copy_(qtip.decode_packed(ph.to(dev, non_blocking=True), K_BITS, cid), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, reps):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    with ClockSampler(0) as clocks:
        ms = timed(step_device, max(args.steps, 20))
        ms_host = timed(step_host, args.steps)
        t_end = time.time() + 1.0
        while time.time() < t_end:
            step_device()
        torch.cuda.synchronize()
    from oracle import oracle as O
    O.build()
    want = O.decode_packed(packed[:64].cpu().numpy().view(np.uint32), K_BITS, CODEBOOK)
    ok = bool(np.array_equal(dq[:64].cpu().numpy().view(np.uint32), want.view(np.uint32)))
    hbm = measured_peaks().get("hbm_gbs") or 6650.0
    byt = n * T_SEQ * 4 + n * nw * 4
    gbs = byt / (ms * 1e-3) / 1e9
    line = {"metric": f"weights decoded/sec (packed decode, L=16, K={K_BITS})", "value": n * T_SEQ / (ms * 1e-3), "unit": "weights/s",
            "n_gpus": 1, "steps": max(args.steps, 20), "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"SIDE MEASUREMENT: packed decode of {n} tiles, K={K_BITS}, {CODEBOOK}; {n * T_SEQ * 4 / 2 ** 20:.0f} MiB out "
                                   "(larger than L2, no flush needed)", "tiles": n},
            "e2e": {"value": n * T_SEQ / (ms_host * 1e-3), "unit": "weights/s", "h2d_bytes_per_step": n * nw * 4, "d2h_bytes_per_step": n * T_SEQ * 4},
            "gpu_launches": max(args.steps, 20),
            "roofline": {"bound": "hbm", "kernel": f"tcq_decode_packed_kernel<K={K_BITS}, {CODEBOOK}>", "achieved": gbs, "peak": hbm, "unit": "GB/s",
                         "frac": gbs / hbm, "traffic": None, "algorithmic": "4 B written + K/8 B read per weight"},
            "parity": {"tiles": 64, "dq_equal": ok, "against": "CPU oracle window decode, bit for bit"}, "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def run_ldlq(args) -> None:
    """Side measurement of the third benchmark configuration: LDLQ + TCQ of one 12288 -> 4096 (down_proj-shaped) matrix.

    ``workloads.cfg3_case``: weights N(0, 0.02^2), proxy Hessian from 8 192 activation rows with log-uniform channel scales;
    sigma_reg 0.025, 16-row blocks, 128-row spans (the reference's parameters), MCG, K bits.  One step = the whole matrix
    through ``model.encode_matrix`` (incoherence processing, block LDL, the recursion with its k_in/16 strictly serial encoder
    calls of n_out/16 tiles, restore); the recursion alone and one encoder call alone are timed beside it."""
    import torch
    from trellis_b200 import ldlq as L
    from trellis_b200 import model, qtip, workloads
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n_out, k_in = args.n_out or 4096, args.k_in or 12288
    w, H = workloads.cfg3_case(n_out, k_in, rows=8192, device=dev)
    lut = qtip.codebook_lut("mcg", dev)

    def whole(groups):
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        packed, w_hat, rel = model.encode_matrix(w, K_BITS, "mcg", 0, H, row_groups=groups)
        torch.cuda.synchronize(dev)
        return time.perf_counter() - t0, rel

    with ClockSampler(0) as clocks:
        whole(1)                                                      # warm-up: handles, kernel images, scratch
        t_whole = min(whole(1)[0] for _ in range(max(1, args.steps // 2)))
        t_groups, rel = whole(2)
        t_groups = min(t_groups, whole(2)[0])
        ip = qtip.IPContext(w, lut.square().mean().sqrt().item(), seed=0)
        Lm = L.block_ldl(L.regularize_H(L._transform_H(H, ip.su, block=128), 0.025), b=16)
        zt = ip.z.t().contiguous()
        L.ldlq_b200(zt, Lm, K_BITS, "mcg")
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        L.ldlq_b200(zt, Lm, K_BITS, "mcg")
        torch.cuda.synchronize(dev)
        t_rec = time.perf_counter() - t0
        rows, comp = zt[:16], torch.zeros_like(zt[:16])
        wq, err = torch.empty_like(rows), torch.empty_like(rows)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        qtip.encode_rows(rows, comp, K_BITS, "mcg", wq, err)
        a.record()
        for _ in range(50):
            qtip.encode_rows(rows, comp, K_BITS, "mcg", wq, err)
        b.record()
        torch.cuda.synchronize(dev)
        call_ms = a.elapsed_time(b) / 50
    weights = n_out * k_in
    calls = k_in // 16
    peaks = measured_peaks()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    peak_lane_ops = sms * 128 * float(peaks.get("sm_max_mhz", 1965.0)) * 1e6
    achieved = weights * STATE_EVALS_PER_WEIGHT * LANE_OPS_PER_EVAL / t_whole
    print(json.dumps({
        "metric": f"weights encoded/sec (LDLQ + TCQ, L=16, K={K_BITS})", "value": weights / t_whole, "unit": "weights/s", "n_gpus": 1,
        "steps": max(1, args.steps // 2), "warmup": 1, "ms_per_step": t_whole * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"SIDE MEASUREMENT, config 3: LDLQ + TCQ of one {k_in} -> {n_out} fp32 matrix N(0,0.02^2), Hessian from 8192 "
                               f"rows with log-uniform channel scales, sigma_reg 0.025, 16-row blocks, 128-row spans, MCG, K={K_BITS}",
                   "n_out": n_out, "k_in": k_in, "encoder_calls": calls, "tiles_per_call": n_out // 16},
        "recursion_only": {"seconds": t_rec, "weights_per_s": weights / t_rec},
        "two_column_groups": {"seconds": t_groups, "weights_per_s": weights / t_groups},
        "encoder_call": {"ms": call_ms, "calls_x_ms_seconds": calls * call_ms * 1e-3, "weights_per_s": (n_out // 16) * T_SEQ / (call_ms * 1e-3)},
        "rel_err": rel, "gpu_launches": 4 * calls,
        "roofline": {"bound": "alu", "kernel": "Viterbi step kernel at n_out/16 tiles per launch", "achieved": achieved / 1e12,
                     "peak": peak_lane_ops / 1e12, "unit": "Tlane-op/s", "frac": achieved / peak_lane_ops, "traffic": None,
                     "note": "whole matrix incl. LDL, GEMMs and restore; a 256-tile launch fills 64 of the 74 two-SM clusters"},
        "clocks": clocks.summary()}), flush=True)


def run_ip(args) -> None:
    """Side measurement of the incoherence-processing kernels (the producer of the encoder's tiles and the consumer of
    its reconstruction) through the C ABI with preallocated buffers: forward = 20 algorithmic bytes per weight (w read
    twice, one intermediate written and read, tiles written), restore = 16."""
    import torch
    from trellis_b200 import _lib, qtip
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n, k = args.n_out or 12288, args.k_in or 4096
    g = torch.Generator(device=dev).manual_seed(0)
    w = torch.randn(n, k, device=dev, generator=g) * 0.02
    ip = qtip.IPContext(w, 0.9, seed=0)
    L = _lib.lib()
    ws = torch.empty(int(L.tcq_ip_workspace_bytes(n, k)), dtype=torch.uint8, device=dev)
    tiles, out = torch.empty_like(ip.tiles), torch.empty_like(w)
    out_s, in_s, scale = torch.empty_like(ip.out_s), torch.empty_like(ip.in_s), torch.empty(1, device=dev)
    st = torch.cuda.current_stream().cuda_stream

    def fwd():
        _lib.check(L.tcq_ip_forward(w.data_ptr(), n, k, ip.sv.data_ptr(), ip.su.data_ptr(), 0.9, 1, tiles.data_ptr(), out_s.data_ptr(),
                                    in_s.data_ptr(), scale.data_ptr(), ws.data_ptr(), ws.numel(), st), "tcq_ip_forward")

    def inv():
        _lib.check(L.tcq_ip_restore(tiles.data_ptr(), 1, n, k, ip.sv.data_ptr(), ip.su.data_ptr(), out_s.data_ptr(), in_s.data_ptr(),
                                    scale.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), st), "tcq_ip_restore")

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    with ClockSampler(0) as clocks:
        ms_f, ms_i = timed(fwd), timed(inv)
        t_end = time.time() + 1.0
        while time.time() < t_end:
            fwd()
        torch.cuda.synchronize()
    err = float((out - w).norm() / w.norm())
    hbm = measured_peaks().get("hbm_gbs") or 6650.0
    gbs_f, gbs_i = n * k * 20 / (ms_f * 1e-3) / 1e9, n * k * 16 / (ms_i * 1e-3) / 1e9
    print(json.dumps({
        "metric": "weights incoherence-processed/sec (forward)", "value": n * k / (ms_f * 1e-3), "unit": "weights/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_f, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"SIDE MEASUREMENT: incoherence processing of a [{n}, {k}] fp32 matrix ({n * k * 4 / 2 ** 20:.0f} MiB, larger "
                               "than L2) through tcq_ip_forward / tcq_ip_restore, buffers preallocated", "n": n, "k": k},
        "restore": {"ms_per_step": ms_i, "weights_per_s": n * k / (ms_i * 1e-3), "round_trip_rel_err": err},
        "gpu_launches": 5 * args.steps,
        "roofline": {"bound": "hbm", "kernel": "ip_row_sumsq + ip_had_rows + ip_had_cols (forward, 5 launches)", "achieved": gbs_f,
                     "peak": hbm, "unit": "GB/s", "frac": gbs_f / hbm, "traffic": None,
                     "restore": {"achieved": gbs_i, "frac": gbs_i / hbm}},
        "clocks": clocks.summary()}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("b200", "reference", "reference-triton"), default="b200")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed kernels' output")
    ap.add_argument("--no-scaling-extras", action="store_true", help="skip the tile_split and model_encode measurements")
    ap.add_argument("--model-layers", type=int, default=8, help="layers of the Qwen3-8B shape in the model_encode measurement")
    ap.add_argument("--model-streams", type=int, default=3, help="matrices in flight per GPU in the model_encode measurement")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="CPU time budget of the cpu_baseline leg")
    ap.add_argument("--ref-tiles", type=int, default=256, help="tiles per step of the reference arm")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--K", type=int, default=3, choices=(2, 3, 4),
                    help="bits per weight; anything but the default 3 is a side measurement, not the benchmark")
    ap.add_argument("--codebook", default="3inst", choices=("1mad", "3inst", "mcg"),
                    help="codebook; anything but the default 3inst is a side measurement, not the benchmark")
    ap.add_argument("--path", choices=("encode", "decode", "decode_matvec", "ip", "ldlq"), default="encode",
                    help="encode = the benchmark; decode / decode_matvec / ip / ldlq = side measurements of the packed decode kernel, the "
                         "packed format's consumer kernel, the incoherence-processing kernels and the LDLQ matrix of configuration 3")
    ap.add_argument("--n-out", type=int, default=0, help="side measurements: output rows (defaults: decode_matvec 151936 = lm_head of "
                                                         "the model shape, ip 12288, ldlq 4096)")
    ap.add_argument("--k-in", type=int, default=0, help="side measurements: input columns (defaults: decode_matvec 4096, ip 4096, ldlq 12288)")
    ap.add_argument("--m", type=int, default=1, help="decode_matvec: right-hand sides")
    ap.add_argument("--tiles", type=int, default=0,
                    help="encode only the first N tiles of the workload (small cases for ncu captures; the printed line "
                         "is then not a benchmark result)")
    args = ap.parse_args()
    global K_BITS, CODEBOOK
    K_BITS, CODEBOOK = args.K, args.codebook
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.path != "encode":
        if args.impl != "b200" or args.gpus != 1:
            raise SystemExit(f"--path {args.path} is a one-GPU side measurement of this library")
        if rank == 0:
            {"decode_matvec": run_decode_matvec, "decode": run_decode, "ip": run_ip, "ldlq": run_ldlq}[args.path](args)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    elif args.impl == "reference-triton":
        if rank == 0:
            run_reference_triton(args)
    else:
        if world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
        run_b200(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
