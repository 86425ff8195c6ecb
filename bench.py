#!/usr/bin/env python
"""Benchmark of the SpMM hot path: effective TFLOP/s of the OPT-66B-shaped skinny SpMMs at N = 16, 80 % sparsity.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-cpu] [--workload layer|tp-chain]

One step = the four sparse matmuls of one OPT-66B decoder layer (QKV 27648x9216, out-proj 9216x9216,
FFN1 36864x9216, FFN2 9216x36864) on N = 16 tokens, fp16, weights 80 % unstructured-sparse in tiled-CSL.
With --gpus N > 1 (one process per GPU, launched by torch.distributed.run) the weight rows (output features) of
every matrix are partitioned evenly over the ranks; there is no data-path collective, the job-wide time is the
maximum over ranks.  Inputs are seeded synthetic matrices of those shapes (no checkpoint is read).

Cold HBM at every N: each matrix is held in several replicas (same words, different addresses) and successive steps
rotate through them, so that a GPU touches at least 512 MB of compressed weights before it sees an address again
(the L2 holds 126 MB).  The K timed steps are repeated until the timed region lasts about half a second; the
figures are medians over those repetitions (each repetition: barrier + synchronise, CUDA events around exactly K
steps, maximum over ranks).

The JSON line: `value` (whole-job effective TFLOP/s = 2*M*N*K over the four matmuls / device time, launch overlap on,
Split_K given as an upper bound and the launch plan deciding the cut), `e2e` (the same through the C ABI with HOST
activations and results: pinned H2D copies of B and D2H copies of C inside the timed region), `roofline` of the
dominant kernel (FFN1-shaped SpMM alone, rotating replicas, algorithmic bytes / CUDA-event time against the measured
HBM copy bandwidth), `dropin` (what a caller of the reference API gets without touching anything: launch overlap off,
Split_K = the reference's own table), `reference_gpu` (the unmodified reference CUDA kernel, compiled for sm_100a, on
the same device buffers with its own Split_K table; 1 GPU only), `encode_ms` (host and device tiled-CSL encoders on
the FFN1 matrix), `opt175b` (the same step on the OPT-175B shapes 36864x12288, 12288x12288, 49152x12288,
12288x49152, sharded the same way), `sweep` (FFN1 at other N and sparsities; 1 GPU only) and `cpu_baseline` (host
fp32 dense GEMM of the oracle on a bounded row sample, all host threads; 1 GPU only).

--workload tp-chain     the tensor-parallel layer chain instead (column-parallel QKV/FFN1, row-parallel
                        out-proj/FFN2, all-reduce after each row-parallel SpMM), parity against the host layer asserted.
--impl reference        the unmodified reference library (oracle/_ref, built from the reference's own sources) through
                        its own SpMM_SplitK_API on one GPU, same inputs, its own Split_K table; rank 0 only.  Where that
                        build or a GPU is missing: the CPU path below.
--impl reference-cpu    the reference's host side alone (host tiled-CSL encode + host fp32 dense GEMM), rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402,F401
import torch  # noqa: E402

# (name, M, K, Split_K of the reference's own table: kernel_benchmark/benchmark.sh:13-15).  This library is given
# OURS_SPLIT_K as an upper bound (it sizes the workspace) and cuts K only as far as filling the GPU takes.
OPT66B_LAYER = [("qkv", 27648, 9216, 2), ("out_proj", 9216, 9216, 6), ("ffn1", 36864, 9216, 3), ("ffn2", 9216, 36864, 6)]
OPT175B_LAYER = [("qkv", 36864, 12288, 3), ("out_proj", 12288, 12288, 9), ("ffn1", 49152, 12288, 9),
                 ("ffn2", 12288, 49152, 9)]
OURS_SPLIT_K = 64
N_TOKENS = 16
SPARSITY = 0.8
SEED = 0xF1A50000
FALLBACK_HBM_GBS = 6650.0
COLD_BYTES = 512e6          # compressed bytes a GPU streams before an address repeats
TIMED_REGION_S = 0.6        # the K timed steps are repeated until about this much device time has been measured
# DRAM bytes (read + write) per algorithmic byte of the SpMM kernel, from one ncu capture of a half-height FFN1 case
# (see profiles/); traffic grows with the rows, so a full launch is reported as this ratio times its algorithmic bytes.
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.018


def measured_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons for one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.window = index, [], None, (0.0, float("inf"))

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            deadline = time.time() + 5.0  # nvidia-smi needs a moment before its first line
            while not self.rows and time.time() < deadline:
                time.sleep(0.02)
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def mark(self, t0: float, t1: float):
        """Only samples taken between t0 and t1 (the timed region) count."""
        self.window = (t0, t1)

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            self.proc.wait()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        rows = [r for t, r in self.rows if self.window[0] <= t <= self.window[1]]
        sm = [int(r[0]) for r in rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v.strip()]
        if local_rank < len(ids) and ids[local_rank].strip().isdigit():
            return int(ids[local_rank])
    return local_rank


def _device_alloc(dev):
    return lambda n: (lambda t: (t, t.data_ptr()))(torch.zeros(n + 64, dtype=torch.int32, device=dev))


class Layer:
    """One rank's row shard of a decoder layer's four weight matrices, encoded on the device and held in enough
    replicas for cold-HBM timing, plus activations and outputs."""

    def __init__(self, fl, shapes, rank: int, world: int, dev, n_tokens: int = N_TOKENS, sparsity: float = SPARSITY,
                 seed: int = SEED, host_buffers: bool = True):
        self.fl, self.dev, self.items, self.n_tokens = fl, dev, [], n_tokens
        stream = torch.cuda.current_stream(dev).cuda_stream
        for idx, (name, M, K, split_ref) in enumerate(shapes):
            assert M % (128 * world) == 0, (name, M, world)
            rows = (rank * M // world, (rank + 1) * M // world)
            m = rows[1] - rows[0]
            A = fl.synthetic.sparse_uniform_matrix(M, K, sparsity, seed + idx, device=dev, rows=rows)
            comp, offs, num_offsets, words = fl.encode_on_device(stream, A.data_ptr(), m, K, _device_alloc(dev),
                                                                 _device_alloc(dev), lambda owner, i: owner[i].item())
            del A
            bytes_alg = 4 * words + 4 * num_offsets + 2 * K * n_tokens + 2 * m * n_tokens
            # enough replicas that looping this one matrix never finds its words in the L2 either
            replicas = max(1, math.ceil(COLD_BYTES / bytes_alg) + (1 if bytes_alg < COLD_BYTES else 0))
            copies = [(comp, offs)] + [(comp.clone(), offs.clone()) for _ in range(replicas - 1)]
            B = fl.synthetic.dense_uniform_matrix(n_tokens, K, (seed + idx) ^ 0xB, device=dev)
            self.items.append(dict(name=name, M_full=M, M=m, K=K, split_ref=split_ref, copies=copies, words=words, B=B,
                                   C=torch.empty((n_tokens, m), dtype=torch.float16, device=dev),
                                   ws=torch.empty((OURS_SPLIT_K, n_tokens, m), dtype=torch.float16, device=dev),
                                   bytes_alg=bytes_alg))
        self.bytes_alg = sum(it["bytes_alg"] for it in self.items)
        self.flops = sum(2.0 * M * n_tokens * K for _, M, K, _ in shapes)  # whole job, all ranks
        self.calls = 0
        if host_buffers:
            self._make_host_buffers()
        torch.cuda.synchronize(dev)

    def _make_host_buffers(self):
        # The step's activations and results each live in one device buffer and one pinned host buffer, so that the
        # end-to-end step moves them with one copy per direction (16-byte aligned sub-ranges per matrix).
        dev = self.dev

        def packed(sizes, device, pin=False):
            offs, total = [], 0
            for n in sizes:
                offs.append(total)
                total += (n + 7) // 8 * 8
            buf = torch.empty(total, dtype=torch.float16, device=device)
            return (buf.pin_memory() if pin else buf), offs
        b_sizes = [it["B"].numel() for it in self.items]
        c_sizes = [it["C"].numel() for it in self.items]
        self.B_all, b_off = packed(b_sizes, dev)
        self.C_all, c_off = packed(c_sizes, dev)
        self.B_all_host, _ = packed(b_sizes, "cpu", pin=True)
        self.C_all_host, _ = packed(c_sizes, "cpu", pin=True)
        for it, bo, co in zip(self.items, b_off, c_off):
            self.B_all_host[bo:bo + it["B"].numel()].copy_(it["B"].flatten().cpu())
            self.B_all[bo:bo + it["B"].numel()].copy_(it["B"].flatten())
            it["B"] = self.B_all[bo:bo + it["B"].numel()].view_as(it["B"])
            it["C"] = self.C_all[co:co + it["C"].numel()].view_as(it["C"])
        # End-to-end steps move the first matrix's activations and the last matrix's results on their own and the rest
        # in one copy each, on side streams, so that only those two small copies are not hidden behind the SpMMs.
        self.b_split, self.c_split = b_off[1], c_off[-1]
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]

    def spmm(self, it, stream, split_k: int | None = None, reference=None):
        comp, offs = it["copies"][self.calls % len(it["copies"])]
        self.calls += 1
        if reference is not None:  # the unmodified reference kernel on the same buffers
            rc = reference(stream, comp.data_ptr(), offs.data_ptr(), it["B"].data_ptr(), it["C"].data_ptr(), it["M"],
                           self.n_tokens, it["K"], it["ws"].data_ptr(), it["split_ref"])
            assert rc == 0, rc
            return
        self.fl.SpMM_SplitK_API(stream, None, comp.data_ptr(), offs.data_ptr(), it["B"].data_ptr(), it["C"].data_ptr(),
                                it["M"], self.n_tokens, it["K"], it["ws"].data_ptr(),
                                OURS_SPLIT_K if split_k is None else split_k)

    def step(self, stream, reference_splits: bool = False, reference=None):
        for it in self.items:
            self.spmm(it, stream, it["split_ref"] if reference_splits else None, reference)

    def step_e2e(self, stream, reference=None):
        """Host activations in, host results out.  Steps do not overlap one another: a step begins after the previous
        step's results have reached the host and ends when its own have."""
        cur = torch.cuda.current_stream(self.dev)
        bs, cs = self.b_split, self.c_split
        self.s_in.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            self.B_all[:bs].copy_(self.B_all_host[:bs], non_blocking=True)
            self.ev_in[0].record()
            self.B_all[bs:].copy_(self.B_all_host[bs:], non_blocking=True)
            self.ev_in[1].record()
        last = len(self.items) - 1
        for i, it in enumerate(self.items):
            if i < 2:
                cur.wait_event(self.ev_in[i])
            self.spmm(it, stream, None, reference)
            if i == last - 1:
                self.ev_out[0].record(cur)
        self.ev_out[1].record(cur)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_out[0])
            self.C_all_host[:cs].copy_(self.C_all[:cs], non_blocking=True)
            self.s_out.wait_event(self.ev_out[1])
            self.C_all_host[cs:].copy_(self.C_all[cs:], non_blocking=True)
        cur.wait_stream(self.s_out)

    def replicas(self) -> dict:
        return {it["name"]: len(it["copies"]) for it in self.items}


class Ranks:
    """Barrier and maximum over ranks (no-ops on one GPU)."""

    def __init__(self, world: int, dev):
        self.world, self.dev = world, dev
        if world > 1:
            import torch.distributed as dist
            self.dist = dist
            dist.init_process_group("nccl", device_id=dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def max(self, values):
        """Element-wise maximum over the ranks of a list of floats."""
        if self.world == 1:
            return list(values)
        t = torch.tensor(list(values), dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def time_loop(fn, steps: int, dev) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on the current stream, synchronised on both sides."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize(dev)
    return start.elapsed_time(stop)


def timed_repetitions(fn, steps: int, dev, ranks: Ranks, budget_s: float = TIMED_REGION_S, max_reps: int = 400):
    """Repeats [barrier + synchronise, exactly `steps` calls of fn between two CUDA events, synchronise] until about
    `budget_s` of device time has been measured.  Returns (median ms per repetition after the maximum over ranks,
    number of repetitions)."""
    ranks.barrier()
    pilot = ranks.max([time_loop(fn, steps, dev)])[0]
    reps = int(min(max_reps, max(3, math.ceil(budget_s * 1e3 / max(pilot, 1e-3)))))
    samples = []
    for _ in range(reps):
        ranks.barrier()
        samples.append(time_loop(fn, steps, dev))
    return statistics.median(ranks.max(samples)), reps


def cpu_baseline(sample_seconds: float = 12.0) -> dict:
    """Host fp32 dense GEMM (OpenMP, all host threads) on a row sample of the FFN1-shaped matrix."""
    import flash_llm_b200 as fl
    from oracle import cpu_oracle
    name, M, K, _ = OPT66B_LAYER[2]
    cores = os.cpu_count() or 1
    cpu_oracle.set_threads(cores)  # torch.distributed.run pins OMP_NUM_THREADS=1 in the ranks' environment
    rows = 1024
    A = fl.synthetic.sparse_uniform_matrix(M, K, SPARSITY, SEED + 2, rows=(0, rows)).numpy()
    B = fl.synthetic.dense_uniform_matrix(N_TOKENS, K, (SEED + 2) ^ 0xB).numpy()
    cpu_oracle.gemm_f32(A[:128], B, timed=True)  # warm the thread pool
    t0, reps = time.perf_counter(), 0
    while True:
        cpu_oracle.gemm_f32(A, B, timed=True)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > sample_seconds or reps >= 200:
            break
    tflops = 2.0 * rows * N_TOKENS * K * reps / dt / 1e12
    t0 = time.perf_counter()
    if cpu_oracle.reference_available():
        cpu_oracle.reference_encode(A, True)
        enc_kind = "reference"
    else:
        cpu_oracle.encode(A, True)
        enc_kind = "port"
    enc_s = time.perf_counter() - t0
    return {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{reps} x host fp32 dense GEMM of {rows} of the {M} rows of the {name} matrix ({M}x{K}, N={N_TOKENS}); "
                      f"single-thread {enc_kind} tiled-CSL encode of those rows took {enc_s:.2f} s "
                      f"(~{enc_s * M / rows:.0f} s for the matrix)"}


def config_dict(world: int, layer: Layer | None = None) -> dict:
    cfg = {"workload": "OPT-66B decoder-layer SpMMs (27648x9216, 9216x9216, 36864x9216, 9216x36864), N=16 tokens, "
                       "80% uniform-random sparsity, fp16, tiled-CSL; Split_K: this library is given 64 as an upper bound "
                       "and its launch plan decides, the reference uses its own table 2/6/3/6",
           "sharding": f"weight rows split evenly over {world} GPU(s), no collective",
           "tokens": N_TOKENS, "sparsity": SPARSITY,
           "launch": "programmatic stream serialisation between consecutive library kernels (weights resident)"}
    if layer is not None:
        per_step = layer.bytes_alg
        cfg["l2"] = (f"cold HBM: replicas of every matrix are rotated so that each GPU streams at least "
                     f"{COLD_BYTES / 1e6:.0f} MB of compressed weights before an address repeats (126 MB L2); this "
                     f"GPU's step is {per_step / 1e6:.0f} MB, replicas per matrix {layer.replicas()}")
    return cfg


def measure_layer(fl, layer: Layer, steps: int, dev, ranks: Ranks, stream, budget_s: float) -> dict:
    """Device-resident throughput of one layer object: median over repetitions of exactly `steps` steps."""
    ms, reps = timed_repetitions(lambda: layer.step(stream), steps, dev, ranks, budget_s)
    return {"value": layer.flops * steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms / steps,
            "hbm_gbs_per_gpu": layer.bytes_alg * steps / (ms * 1e-3) / 1e9, "repetitions": reps}


def per_shape_timings(fl, layer: Layer, dev, stream, reps: int, reference=None) -> dict:
    out = {}
    for it in layer.items:
        for _ in range(5):
            layer.spmm(it, stream, None, reference)
        t = time_loop(lambda it=it: layer.spmm(it, stream, None, reference), reps, dev) / reps
        rec = {"ms": t, "gbs": it["bytes_alg"] / (t * 1e-3) / 1e9,
               "tflops": 2.0 * it["M"] * layer.n_tokens * it["K"] / (t * 1e-3) / 1e12, "bytes_alg": it["bytes_alg"]}
        if reference is None:
            rec["plan"] = fl.get_plan(it["M"], layer.n_tokens, it["K"], OURS_SPLIT_K)
        out[it["name"]] = rec
    return out


def encode_timings(fl, dev) -> dict:
    """Host and device tiled-CSL encoders on the FFN1 matrix (36864x9216, 80 %), milliseconds."""
    name, M, K, _ = OPT66B_LAYER[2]
    stream = torch.cuda.current_stream(dev).cuda_stream
    A = fl.synthetic.sparse_uniform_matrix(M, K, SPARSITY, SEED + 2, device=dev)
    alloc = _device_alloc(dev)
    fl.encode_on_device(stream, A.data_ptr(), M, K, alloc, alloc, lambda o, i: o[i].item())  # warm-up
    t_dev = []
    for _ in range(3):
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        fl.encode_on_device(stream, A.data_ptr(), M, K, alloc, alloc, lambda o, i: o[i].item())
        torch.cuda.synchronize(dev)
        t_dev.append((time.perf_counter() - t0) * 1e3)
    A_h = A.cpu().numpy()
    del A
    t0 = time.perf_counter()
    fl.InitSparseMatrixA_API(A_h)
    t_host = (time.perf_counter() - t0) * 1e3
    return {"matrix": f"{name} {M}x{K}, {int(SPARSITY * 100)} % sparse", "device": min(t_dev), "host": t_host,
            "host_threads": os.cpu_count() or 1,
            "device_gbs_on_dense_bytes": 2.0 * M * K / (min(t_dev) * 1e-3) / 1e9,
            "note": "device = count + scan + pack kernels and the read-back of the word count (wall clock, synchronised); "
                    "host = this library's multi-threaded InitSparseMatrixA_API; the reference's single-thread encoder is "
                    "timed in cpu_baseline.sample"}


def sweep_ffn1(fl, dev, stream, peak: float) -> list:
    """The FFN1 matrix alone at other token counts and sparsities (one GPU), cold HBM."""
    name, M, K, split_ref = OPT66B_LAYER[2]
    out = []
    for sparsity, tokens in ((0.8, 8), (0.8, 32), (0.8, 64), (0.7, 16), (0.9, 16)):
        layer = Layer(fl, [(name, M, K, split_ref)], 0, 1, dev, n_tokens=tokens, sparsity=sparsity, seed=SEED + 2,
                      host_buffers=False)
        it = layer.items[0]
        for _ in range(5):
            layer.spmm(it, stream)
        t = time_loop(lambda: layer.spmm(it, stream), 60, dev) / 60
        gbs = it["bytes_alg"] / (t * 1e-3) / 1e9
        out.append({"M": M, "K": K, "N": tokens, "sparsity": sparsity, "ms": t, "gbs": gbs, "frac_of_peak": gbs / peak,
                    "tflops": 2.0 * M * tokens * K / (t * 1e-3) / 1e12})
        del layer
        torch.cuda.empty_cache()
    return out


def run_ours(args) -> None:
    import flash_llm_b200 as fl
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    ranks = Ranks(world, dev)
    fl.library()
    layer = Layer(fl, OPT66B_LAYER, rank, world, dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    steps, warmup = args.steps, max(args.warmup, 3)
    # The compressed weights are resident and final before the loop (inference): consecutive kernels may overlap.
    fl.set_launch_overlap(True)

    # ---- device-resident throughput
    for _ in range(warmup):
        layer.step(stream)
    ranks.barrier()
    before = fl.launch_count()
    layer.step(stream)
    launches_per_step = fl.launch_count() - before
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        t_begin = time.time()
        main = measure_layer(fl, layer, steps, dev, ranks, stream, TIMED_REGION_S)
        clocks.mark(t_begin, time.time())
        time.sleep(0.05)
    status = fl.consume_status()
    assert status == 0, f"kernel status {status:#x}"

    # ---- end to end: host activations in, host results out, every step
    for _ in range(3):
        layer.step_e2e(stream)
    ms_e2e, reps_e2e = timed_repetitions(lambda: layer.step_e2e(stream), steps, dev, ranks, TIMED_REGION_S / 2)
    h2d = layer.B_all_host.numel() * 2
    d2h = layer.C_all_host.numel() * 2

    # ---- every shape alone (rotating replicas), the dominant one for the roofline
    per_shape = per_shape_timings(fl, layer, dev, stream, max(60, steps))
    peak, peak_kind = measured_peak_gbs()
    dom = per_shape["ffn1"]
    plan = dom["plan"]
    roofline = {"bound": "hbm",
                "kernel": f"SpMM kernel of the FFN1 shard ({layer.items[2]['M']}x{layer.items[2]['K']}, N={N_TOKENS}; "
                          f"plan path {plan['path']}, {plan['scatter_warps']} scatter warps)",
                "achieved": dom["gbs"], "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                "frac": dom["gbs"] / peak, "frac_of_nominal_8000": dom["gbs"] / 8000.0,
                "traffic": DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * dom["bytes_alg"], "launch_ms": dom["ms"],
                "algorithmic_bytes": dom["bytes_alg"]}

    # ---- what an untouched caller of the reference API gets: no launch overlap, the reference's own Split_K table
    fl.set_launch_overlap(False)
    for _ in range(3):
        layer.step(stream, reference_splits=True)
    ms_drop, _ = timed_repetitions(lambda: layer.step(stream, reference_splits=True), steps, dev, ranks, TIMED_REGION_S / 3)
    dropin = {"value": layer.flops * steps / (ms_drop * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_drop / steps,
              "split_k": [s for _, _, _, s in OPT66B_LAYER], "launch_overlap": False,
              "plans": {it["name"]: {k: v for k, v in fl.get_plan(it["M"], N_TOKENS, it["K"], it["split_ref"]).items()
                                     if k in ("cluster_k", "workspace_k")} for it in layer.items}}
    fl.set_launch_overlap(True)

    # ---- the unmodified reference CUDA kernel on the same buffers (one GPU: its kernel needs M % 256 == 0)
    reference_gpu = None
    if world == 1:
        reference_gpu = reference_gpu_record(fl, layer, steps, dev, ranks, stream, with_e2e=False)

    # ---- the OPT-175B shapes, sharded the same way
    layer175 = Layer(fl, OPT175B_LAYER, rank, world, dev, seed=SEED + 0x175, host_buffers=False)
    for _ in range(3):
        layer175.step(stream)
    opt175b = measure_layer(fl, layer175, steps, dev, ranks, stream, TIMED_REGION_S / 2)
    opt175b["per_shape"] = per_shape_timings(fl, layer175, dev, stream, 30)
    opt175b["workload"] = ("OPT-175B decoder-layer SpMMs (36864x12288, 12288x12288, 49152x12288, 12288x49152), N=16, 80 % "
                           f"sparsity, weight rows split over {world} GPU(s); replicas {layer175.replicas()}")
    del layer175
    torch.cuda.empty_cache()
    status = fl.consume_status()
    assert status == 0, f"kernel status {status:#x}"

    line = {"metric": "spmm_effective_tflops", "value": main["value"], "unit": "TFLOP/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(config_dict(world, layer),
                           timing=f"median of {main['repetitions']} repetitions of exactly {steps} steps (barrier + "
                                  "synchronise, CUDA events, max over ranks per repetition)"),
            "hbm_gbs": main["hbm_gbs_per_gpu"] * world,
            "e2e": {"value": layer.flops * steps / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / steps, "repetitions": reps_e2e},
            "gpu_launches": launches_per_step * steps, "clocks": clocks.summary(), "roofline": roofline,
            "per_shape": per_shape, "dropin": dropin, "reference_gpu": reference_gpu, "opt175b": opt175b}
    if world == 1 and not args.quick:
        line["sweep"] = sweep_ffn1(fl, dev, stream, peak)
        line["encode_ms"] = encode_timings(fl, dev)
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
    if rank == 0:
        print(json.dumps(line), flush=True)
    ranks.close()


def reference_gpu_record(fl, layer: Layer, steps: int, dev, ranks: Ranks, stream, with_e2e: bool) -> dict | None:
    """The unmodified reference kernel (oracle/_ref, compiled from the reference's own sources for sm_100a) on the
    layer's device buffers, with its own Split_K table."""
    from oracle import cpu_oracle
    if not cpu_oracle.reference_available():
        return None
    ref = cpu_oracle.reference_spmm
    for _ in range(3):
        layer.step(stream, reference=ref)
    ms, reps = timed_repetitions(lambda: layer.step(stream, reference=ref), steps, dev, ranks, TIMED_REGION_S / 3)
    rec = {"value": layer.flops * steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms / steps,
           "split_k": [it["split_ref"] for it in layer.items], "repetitions": reps,
           "per_shape": {k: {"ms": v["ms"], "gbs": v["gbs"]}
                         for k, v in per_shape_timings(fl, layer, dev, stream, 30, reference=ref).items()}}
    if with_e2e:
        for _ in range(3):
            layer.step_e2e(stream, reference=ref)
        ms_e2e, _ = timed_repetitions(lambda: layer.step_e2e(stream, reference=ref), steps, dev, ranks, TIMED_REGION_S / 3)
        rec["e2e_ms_per_step"] = ms_e2e / steps
    return rec


def run_reference(args) -> None:
    """The reference arm: the unmodified reference library through its own SpMM_SplitK_API on one GPU (the whole,
    unsharded workload: its kernel has no row-shard form and needs M % 256 == 0), rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import cpu_oracle
    if not (cpu_oracle.reference_available() and torch.cuda.is_available()):
        run_reference_cpu(args)
        return
    import flash_llm_b200 as fl
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    ranks = Ranks(1, dev)
    layer = Layer(fl, OPT66B_LAYER, 0, 1, dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    steps, warmup = args.steps, max(args.warmup, 3)
    for _ in range(warmup):
        layer.step(stream, reference=cpu_oracle.reference_spmm)
    with ClockSampler(physical_gpu_index(dev.index)) as clocks:
        t_begin = time.time()
        rec = reference_gpu_record(fl, layer, steps, dev, ranks, stream, with_e2e=True)
        clocks.mark(t_begin, time.time())
        time.sleep(0.05)
    base = cpu_baseline(8.0) if not args.no_cpu_baseline else None
    line = {"impl": "reference", "metric": "spmm_effective_tflops", "value": rec["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": rec["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(config_dict(1, layer),
                           reference="unmodified reference CUDA library built from its own sources for sm_100a "
                                     "(oracle/_ref/libSpMM_API_ref.so), SpMM_SplitK_API with Split_K 2/6/3/6, one GPU, "
                                     "whole matrices"),
            "e2e": {"value": layer.flops / (rec["e2e_ms_per_step"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": layer.B_all_host.numel() * 2, "d2h_bytes_per_step": layer.C_all_host.numel() * 2,
                    "ms_per_step": rec["e2e_ms_per_step"]},
            "per_shape": rec["per_shape"], "clocks": clocks.summary()}
    if base is not None:
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)


def run_reference_cpu(args) -> None:
    """The reference's host side for this operation: host tiled-CSL encode + host fp32 dense GEMM."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps = max(args.steps, 1)
    # one step = a bounded row sample of the workload, sized for a few seconds of host time
    per_step = max(2.0, min(20.0, 90.0 / (steps + max(args.warmup, 0))))
    for _ in range(min(args.warmup, 1)):
        cpu_baseline(1.0)
    t0 = time.perf_counter()
    results = [cpu_baseline(per_step) for _ in range(steps)]
    wall = time.perf_counter() - t0
    value = statistics.mean(r["value"] for r in results)
    base = results[-1]
    base["value"] = value
    line = {"impl": "reference", "metric": "spmm_effective_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": wall * 1e3 / steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(args.gpus), "cpu_baseline": base,
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# Tolerance of the tensor-parallel chain against the unsharded host layer (the same the chain tests use): every rank
# rounds its partial sums to fp16 before they are added, and two more matmuls carry that along.
CHAIN_REL_TOL, CHAIN_ABS_TOL_OF_MAX = 5e-2, 2e-3


def run_tp_chain(args) -> None:
    """The tensor-parallel sparse layer chain at OPT-66B dimensions.  QKV and FFN1 are column-parallel, out-proj and
    FFN2 row-parallel over the ranks, with an NCCL all-reduce of [N][H] (fp32 sum of the ranks' fp16 partial matrices,
    one rounding) after each row-parallel SpMM; weights N(0, 0.02) magnitude-pruned to 80 % per matrix, activations
    N(0, 1), N = 16."""
    import flash_llm_b200 as fl
    from flash_llm_b200 import tp_chain
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    ranks = Ranks(world, dev)
    fl.library()
    H, F = 9216, 36864
    shape = tp_chain.ChainShape(hidden=H, ffn=F, tokens=N_TOKENS, world=world)
    seed = SEED + 0x50
    full = [fl.synthetic.magnitude_pruned_matrix(m, k, SPARSITY, 0.02, seed + i, device=dev)
            for i, (m, k) in enumerate(((3 * H, H), (H, H), (F, H), (H, F)))]
    shards = tp_chain.shard_weights(shape, rank, *full)
    chain = tp_chain.DeviceChain(fl, shape, shards, dev, split_k=64)
    x = fl.synthetic.normal_matrix(N_TOKENS, H, 1.0, seed + 9, device=dev).to(torch.float16)
    fl.set_launch_overlap(True)
    all_reduce = tp_chain.fp32_all_reduce(ranks.dist if world > 1 else None)
    # The row-parallel layers go through the library's fused SpMM + all-reduce (peer stores, no NCCL on the data path);
    # --nccl-chain keeps the plain SpMM followed by an NCCL all-reduce, which is also timed beside it as the baseline.
    group = tp_chain.PeerGroup(fl, ranks.dist, rank, world, N_TOKENS * H) if world > 1 else None
    fused = group is not None and not args.nccl_chain
    step_nccl = lambda: chain.step(x, all_reduce)  # noqa: E731
    step = (lambda: chain.step(x, comm=group.comm)) if fused else step_nccl

    # ---- parity of the sharded chain over the real collective against the unsharded layer on the host (rank 0)
    want = tp_chain.reference_chain(shape, x.cpu(), *[w.cpu() for w in full]) if rank == 0 else None
    del full

    def parity_of(run_step) -> list:
        ranks.barrier()  # the fused call waits for its partners for a bounded time only: start the ranks together
        out = run_step().clone()
        torch.cuda.synchronize(dev)
        status = fl.consume_status()
        assert status == 0, f"kernel status {status:#x}"
        figures = [0.0, 0.0]
        if rank == 0:
            got = out.cpu().float()
            rms = float(want.pow(2).mean().sqrt())
            figures = [float(((got - want).abs() / want.abs().clamp_min(0.05 * rms)).max()),
                       float((got - want).abs().max() / want.abs().max())]
        figures = ranks.max(figures)  # every rank learns rank 0's figures and fails together
        assert figures[0] <= CHAIN_REL_TOL and figures[1] <= CHAIN_ABS_TOL_OF_MAX, \
            f"chain output differs from the host layer: rel {figures[0]:.3e}, abs/peak {figures[1]:.3e}"
        return figures
    parity = parity_of(step)
    parity_nccl = parity_of(step_nccl) if fused else parity

    steps = args.steps
    for _ in range(max(args.warmup, 3)):
        step()
    ranks.barrier()
    before = fl.launch_count()
    step()
    launches_per_step = fl.launch_count() - before
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        t_begin = time.time()
        ms, reps = timed_repetitions(step, steps, dev, ranks)
        clocks.mark(t_begin, time.time())
        time.sleep(0.05)
    # the NCCL form of the chain, the same kernels without any collective (every rank on its own partial sums), and
    # the NCCL collective on its own
    ms_nccl = timed_repetitions(step_nccl, steps, dev, ranks, TIMED_REGION_S / 3)[0] if fused else ms
    ms_local, _ = timed_repetitions(lambda: chain.step(x, lambda t: t), steps, dev, ranks, TIMED_REGION_S / 3)
    buf = torch.zeros((N_TOKENS, H), dtype=torch.float16, device=dev)
    ms_coll = timed_repetitions(lambda: all_reduce(buf), steps, dev, ranks, TIMED_REGION_S / 3)[0] if world > 1 else 0.0
    status = fl.consume_status()
    assert status == 0, f"kernel status {status:#x}"
    if rank == 0:
        bytes_alg = sum(l["bytes_alg"] for l in chain.layers.values())
        print(json.dumps({
            "metric": "spmm_effective_tflops", "value": shape.flops() * steps / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "tensor-parallel sparse layer chain, OPT-66B dimensions (H=9216, F=36864), N=16, "
                                   "N(0,0.02) weights magnitude-pruned to 80 % per matrix, activations N(0,1): QKV -> "
                                   "out-proj -> all-reduce -> FFN1 -> ReLU -> FFN2 -> all-reduce",
                       "parallelism": f"tp{world}: QKV/FFN1 column-parallel, out-proj/FFN2 row-parallel; " +
                                      ("row-parallel SpMM with the all-reduce fused in: fp32 partial sums stored into "
                                       "every rank's receive buffer over NVLink, summed in rank order, one rounding"
                                       if fused else
                                       f"NCCL all-reduce of {N_TOKENS}x{H} (fp32 sum of fp16 partials) after each "
                                       "row-parallel SpMM"),
                       "shards": {k: list(v) for k, v in shape.shard_shapes().items()},
                       "timing": f"median of {reps} repetitions of exactly {steps} steps"},
            "ms_per_step_nccl_chain": ms_nccl / steps,
            "ms_per_step_without_collectives": ms_local / steps,
            "ms_per_nccl_all_reduce_alone": ms_coll / steps,
            "hbm_gbs_per_gpu": bytes_alg * steps / (ms * 1e-3) / 1e9,
            "parity_vs_host_layer": {"max_rel_err_floor_5pct_rms": parity[0], "max_abs_over_peak": parity[1],
                                     "nccl_chain": parity_nccl, "asserted": [CHAIN_REL_TOL, CHAIN_ABS_TOL_OF_MAX]},
            "gpu_launches": launches_per_step * steps, "clocks": clocks.summary()}), flush=True)
    if group is not None:
        ranks.barrier()  # nobody frees a buffer while a peer may still store into it
        group.close()
    ranks.close()


def main() -> None:
    global TIMED_REGION_S
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cpu"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true", help="skip the sweep, encoder and CPU-baseline sub-records")
    ap.add_argument("--nccl-chain", action="store_true",
                    help="tp-chain: plain SpMM + NCCL all-reduce for the row-parallel layers instead of the fused call")
    ap.add_argument("--workload", default="layer", choices=["layer", "tp-chain"],
                    help="layer: the four OPT-66B SpMMs, weight rows sharded, no collective (the headline metric); "
                         "tp-chain: the tensor-parallel layer chain with all-reduces")
    ap.add_argument("--timed-seconds", type=float, default=TIMED_REGION_S,
                    help="device time the repetitions of the K timed steps add up to (lower it for a profiler's launch "
                         "list; the default is what a reported number needs)")
    args = ap.parse_args()
    TIMED_REGION_S = args.timed_seconds
    if args.workload == "tp-chain" and args.impl == "ours":
        run_tp_chain(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-cpu":
        run_reference_cpu(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
