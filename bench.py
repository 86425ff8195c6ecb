#!/usr/bin/env python
"""Benchmark of the SpMM hot path: effective TFLOP/s of the OPT-66B-shaped skinny SpMMs at N = 16, 80 % sparsity.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-gpu]

One step = the four sparse matmuls of one OPT-66B decoder layer (QKV 27648x9216, out-proj 9216x9216,
FFN1 36864x9216, FFN2 9216x36864) on N = 16 tokens, fp16, weights 80 % unstructured-sparse in tiled-CSL.
With --gpus N > 1 (one process per GPU, launched by torch.distributed.run) the weight rows (output features) of
every matrix are partitioned evenly over the ranks; there is no data-path collective, the job-wide time is the
maximum over ranks.  Inputs are seeded synthetic matrices of those shapes (no checkpoint is read).

Prints one JSON line: metric/value/unit (whole-job effective TFLOP/s = 2*M*N*K summed over the four matmuls and
the steps, divided by the device time), `e2e` (the same through the C ABI with HOST activations and results:
pinned H2D copies of B and D2H copies of C inside the timed region, on side streams so that within a step all but the
first matrix's activations and the last matrix's results move while other matrices are being multiplied; steps do not
overlap one another), `roofline` of the dominant kernel (FFN1-shaped
SpMM, algorithmic bytes / CUDA-event time against the measured HBM copy bandwidth) and `cpu_baseline` (host fp32
dense GEMM of the oracle on a bounded row sample, all host threads).

--workload tp-chain     runs the tensor-parallel layer chain instead (column-parallel QKV/FFN1, row-parallel
                        out-proj/FFN2, NCCL all-reduce after each row-parallel SpMM), checked against the host layer.
--impl reference        times that CPU path alone (reference host encoder + host dense GEMM), rank 0 only.
--impl reference-gpu    times the unmodified reference CUDA kernel (built from its own sources) on the same inputs.
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
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

# (name, M, K, Split_K hint of this library's arm, the reference's hand-tuned Split_K: kernel_benchmark/benchmark.sh:13-15)
# (name, M, K, Split_K given to this library, Split_K of the reference's own table).  This library treats Split_K as an
# upper bound (it sizes the workspace) and cuts K only as far as filling the GPU takes, so one generous value serves
# every shard size; the reference cuts exactly Split_K ways (kernel_benchmark/benchmark.sh:13-15, tuned there).
OPT66B_LAYER = [("qkv", 27648, 9216, 64, 2), ("out_proj", 9216, 9216, 64, 6), ("ffn1", 36864, 9216, 64, 3),
                ("ffn2", 9216, 36864, 64, 6)]
N_TOKENS = 16
SPARSITY = 0.8
SEED = 0xF1A50000
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes (read + write) per algorithmic byte of the SpMM kernel, from one ncu capture of a half-height FFN1 case
# (18432x9216, N=16, 80 %: 136.52 MB read + 3.69 MB written for 136.98 MB algorithmic); traffic grows with the rows,
# so a full launch is reported as this ratio times its algorithmic bytes.
DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.024


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


class Layer:
    """One rank's row shard of the four weight matrices, encoded on the device, plus activations and outputs."""

    def __init__(self, fl, rank: int, world: int, dev, reference_splits: bool = False):
        self.fl, self.dev, self.items = fl, dev, []
        stream = torch.cuda.current_stream(dev).cuda_stream
        for idx, (name, M, K, split_ours, split_ref) in enumerate(OPT66B_LAYER):
            split_k = split_ref if reference_splits else split_ours
            assert M % (128 * world) == 0, (name, M, world)
            rows = (rank * M // world, (rank + 1) * M // world)
            m = rows[1] - rows[0]
            A = fl.synthetic.sparse_uniform_matrix(M, K, SPARSITY, SEED + idx, device=dev, rows=rows)
            comp, offs, num_offsets, words = fl.encode_on_device(
                stream, A.data_ptr(), m, K,
                lambda n: (lambda t: (t, t.data_ptr()))(torch.empty(n, dtype=torch.int32, device=dev)),
                lambda n: (lambda t: (t, t.data_ptr()))(torch.empty(n, dtype=torch.int32, device=dev)),
                lambda owner, i: owner[i].item())
            del A
            B = fl.synthetic.dense_uniform_matrix(N_TOKENS, K, (SEED + idx) ^ 0xB, device=dev)
            item = dict(name=name, M_full=M, M=m, K=K, split_k=split_k, comp=comp, offs=offs, words=words, B=B,
                        C=torch.empty((N_TOKENS, m), dtype=torch.float16, device=dev),
                        ws=torch.empty((split_k, N_TOKENS, m), dtype=torch.float16, device=dev),
                        bytes_alg=4 * words + 4 * num_offsets + 2 * K * N_TOKENS + 2 * m * N_TOKENS)
            self.items.append(item)
        # The step's activations and results each live in one device buffer and one pinned host buffer, so that the
        # end-to-end step moves them with one copy per direction (16-byte aligned sub-ranges per matrix).
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
        torch.cuda.synchronize(dev)

    def spmm(self, it, stream):
        self.fl.SpMM_SplitK_API(stream, None, it["comp"].data_ptr(), it["offs"].data_ptr(), it["B"].data_ptr(),
                                it["C"].data_ptr(), it["M"], N_TOKENS, it["K"], it["ws"].data_ptr(), it["split_k"])

    def step(self, stream):
        for it in self.items:
            self.spmm(it, stream)

    def step_e2e(self, stream):
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
            self.spmm(it, stream)
            if i == last - 1:
                self.ev_out[0].record(cur)
        self.ev_out[1].record(cur)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_out[0])
            self.C_all_host[:cs].copy_(self.C_all[:cs], non_blocking=True)
            self.s_out.wait_event(self.ev_out[1])
            self.C_all_host[cs:].copy_(self.C_all[cs:], non_blocking=True)
        cur.wait_stream(self.s_out)


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


def cpu_baseline(sample_seconds: float = 12.0) -> dict:
    """Host fp32 dense GEMM (OpenMP, all host threads) on a row sample of the FFN1-shaped matrix."""
    import flash_llm_b200 as fl
    from oracle import cpu_oracle
    name, M, K, _, _ = OPT66B_LAYER[2]
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


def config_dict(world: int) -> dict:
    return {"workload": "OPT-66B decoder-layer SpMMs (27648x9216, 9216x9216, 36864x9216, 9216x36864), N=16 tokens, "
                        "80% uniform-random sparsity, fp16, tiled-CSL, Split_K tuned per shape (ours: upper bound 64, the plan decides; reference 2/6/3/6)",
            "sharding": f"weight rows split evenly over {world} GPU(s), no collective",
            "l2": "inputs larger than L2: each step streams ~821 MB of compressed weights (126 MB L2)",
            "tokens": N_TOKENS, "sparsity": SPARSITY,
            "launch": "programmatic stream serialisation between consecutive library kernels (weights resident)"}



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
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    fl.library()
    layer = Layer(fl, rank, world, dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    # The compressed weights are resident and final before the loop (inference): consecutive kernels may overlap.
    fl.set_launch_overlap(True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput
    for _ in range(max(args.warmup, 3)):
        layer.step(stream)
    barrier()
    # The step's launches are captured once into a CUDA graph and replayed per step (a launch-bound inner loop when the
    # shards are small); the library is called through the same entry points during capture.  --no-graph, or a capture
    # that fails, leaves the eager loop.
    run_step, launch_mode, launches_per_step = (lambda: layer.step(stream)), "eager", None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            graph = torch.cuda.CUDAGraph()
            before = fl.launch_count()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    layer.step(side.cuda_stream)
            launches_per_step = fl.launch_count() - before
            torch.cuda.current_stream(dev).wait_stream(side)
            graph.replay()
            torch.cuda.synchronize(dev)
            # keep whichever is faster here: replay removes the launch gaps inside a step, eager launches let the last
            # kernel of a step overlap the first of the next (programmatic stream serialisation)
            pilot = min(100, max(10, args.steps))
            t_eager = max_over_ranks(time_loop(run_step, pilot, dev))
            t_graph = max_over_ranks(time_loop(graph.replay, pilot, dev))
            if t_graph < t_eager:
                run_step, launch_mode = graph.replay, "cuda graph replay"
            else:
                launches_per_step = None
        except Exception as e:  # noqa: BLE001 - any capture problem falls back to eager launches
            print(f"[bench] graph capture failed ({e!r}); using eager launches", file=sys.stderr)
            torch.cuda.synchronize(dev)
    for _ in range(3):
        run_step()
    barrier()
    launches_before = fl.launch_count()
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        t_begin = time.time()
        ms = time_loop(run_step, args.steps, dev)
        clocks.mark(t_begin, time.time())
        time.sleep(0.05)
    launches = (fl.launch_count() - launches_before) if launches_per_step is None else launches_per_step * args.steps
    barrier()
    ms = max_over_ranks(ms)
    status = fl.consume_status()
    assert status == 0, f"kernel status {status:#x}"
    flops_per_step = sum(2.0 * M * N_TOKENS * K for _, M, K, _, _ in OPT66B_LAYER)
    value = flops_per_step * args.steps / (ms * 1e-3) / 1e12

    # ---- end to end: host activations in, host results out, every step
    for _ in range(3):
        layer.step_e2e(stream)
    barrier()
    ms_e2e = max_over_ranks(time_loop(lambda: layer.step_e2e(stream), args.steps, dev))
    barrier()
    h2d = layer.B_all_host.numel() * 2
    d2h = layer.C_all_host.numel() * 2
    e2e_value = flops_per_step * args.steps / (ms_e2e * 1e-3) / 1e12

    # ---- per-kernel numbers (rank 0): every shape alone, dominant one for the roofline
    per_shape = {}
    for it in layer.items:
        for _ in range(5):
            layer.spmm(it, stream)
        reps = max(20, args.steps)
        t = time_loop(lambda it=it: layer.spmm(it, stream), reps, dev) / reps
        per_shape[it["name"]] = {"ms": t, "gbs": it["bytes_alg"] / (t * 1e-3) / 1e9,
                                 "tflops": 2.0 * it["M"] * N_TOKENS * it["K"] / (t * 1e-3) / 1e12,
                                 "bytes_alg": it["bytes_alg"],
                                 "plan": fl.get_plan(it["M"], N_TOKENS, it["K"], it["split_k"])}
    peak, peak_kind = measured_peak_gbs()
    dom = per_shape["ffn1"]
    roofline = {"bound": "hbm", "kernel": "spmm_tcgen05_direct_kernel<16,16,4,2> on the FFN1 shard", "achieved": dom["gbs"],
                "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": dom["gbs"] / peak,
                "frac_of_nominal_8000": dom["gbs"] / 8000.0,
                "traffic": DRAM_TRAFFIC_PER_ALGORITHMIC_BYTE * dom["bytes_alg"], "launch_ms": dom["ms"],
                "algorithmic_bytes": dom["bytes_alg"]}

    if rank == 0:
        line = {"metric": "spmm_effective_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic", "config": dict(config_dict(world), step_launch=launch_mode),
                "hbm_gbs": sum(it["bytes_alg"] for it in layer.items) * args.steps / (ms * 1e-3) / 1e9,
                "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": ms_e2e / args.steps},
                "gpu_launches": launches, "clocks": clocks.summary(), "roofline": roofline, "per_shape": per_shape}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_reference_cpu(args) -> None:
    """The reference's CPU path for this operation: host tiled-CSL encode + host fp32 dense GEMM."""
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


def run_reference_gpu(args) -> None:
    """The unmodified reference CUDA kernel (compiled for sm_100a from its own sources) on the same inputs."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import flash_llm_b200 as fl
    from oracle import cpu_oracle
    if not cpu_oracle.reference_available():
        print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref/libSpMM_API_ref.so has not been built"}))
        return
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    layer = Layer(fl, 0, 1, dev, reference_splits=True)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def step():
        for it in layer.items:
            rc = cpu_oracle.reference_spmm(stream, it["comp"].data_ptr(), it["offs"].data_ptr(), it["B"].data_ptr(),
                                           it["C"].data_ptr(), it["M"], N_TOKENS, it["K"], it["ws"].data_ptr(), it["split_k"])
            assert rc == 0, rc

    for _ in range(max(args.warmup, 3)):
        step()
    ms = time_loop(step, args.steps, dev)
    flops_per_step = sum(2.0 * M * N_TOKENS * K for _, M, K, _, _ in OPT66B_LAYER)
    per_shape = {}
    for it in layer.items:
        def one(it=it):
            cpu_oracle.reference_spmm(stream, it["comp"].data_ptr(), it["offs"].data_ptr(), it["B"].data_ptr(),
                                      it["C"].data_ptr(), it["M"], N_TOKENS, it["K"], it["ws"].data_ptr(), it["split_k"])
        t = time_loop(one, 20, dev) / 20
        per_shape[it["name"]] = {"ms": t, "gbs": it["bytes_alg"] / (t * 1e-3) / 1e9}
    print(json.dumps({"impl": "reference-gpu", "metric": "spmm_effective_tflops",
                      "value": flops_per_step * args.steps / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
                      "higher_is_better": True, "dtype": "f16", "data": "synthetic", "config": config_dict(1),
                      "per_shape": per_shape}), flush=True)


def run_tp_chain(args) -> None:
    """BASELINE config 5: the tensor-parallel sparse layer chain at OPT-66B dimensions.  QKV and FFN1 are
    column-parallel, out-proj and FFN2 row-parallel over the ranks, with an NCCL all-reduce of [N][H] fp16 after each
    row-parallel SpMM; weights N(0, 0.02) magnitude-pruned to 80 % per matrix, activations N(0, 1), N = 16."""
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
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
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

    def all_reduce(t):
        if world > 1:
            dist.all_reduce(t)
        return t

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- parity of the sharded chain over the real collective against the unsharded layer on the host (rank 0)
    out = chain.step(x, all_reduce).clone()
    torch.cuda.synchronize(dev)
    status = fl.consume_status()
    assert status == 0, f"kernel status {status:#x}"
    parity = None
    if rank == 0:
        want = tp_chain.reference_chain(shape, x.cpu(), *[w.cpu() for w in full])
        got = out.cpu().float()
        rms = float(want.pow(2).mean().sqrt())
        rel = float(((got - want).abs() / want.abs().clamp_min(0.05 * rms)).max())
        parity = {"max_rel_err_floor_5pct_rms": rel, "max_abs_over_peak": float((got - want).abs().max() / want.abs().max())}
    del full

    for _ in range(max(args.warmup, 3)):
        chain.step(x, all_reduce)
    barrier()
    launches_before = fl.launch_count()
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        t_begin = time.time()
        ms = time_loop(lambda: chain.step(x, all_reduce), args.steps, dev)
        clocks.mark(t_begin, time.time())
        time.sleep(0.05)
    launches = fl.launch_count() - launches_before
    barrier()
    ms = max_over_ranks(ms)
    # the same kernels without the collectives (every rank on its own partial sums), and the collective on its own
    ms_local = max_over_ranks(time_loop(lambda: chain.step(x, lambda t: t), args.steps, dev))
    buf = torch.zeros((N_TOKENS, H), dtype=torch.float16, device=dev)
    barrier()
    ms_coll = max_over_ranks(time_loop(lambda: all_reduce(buf), args.steps, dev)) if world > 1 else 0.0
    status = fl.consume_status()
    assert status == 0, f"kernel status {status:#x}"
    if rank == 0:
        bytes_alg = sum(l["bytes_alg"] for l in chain.layers.values())
        print(json.dumps({
            "metric": "spmm_effective_tflops", "value": shape.flops() * args.steps / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": "tensor-parallel sparse layer chain, OPT-66B dimensions (H=9216, F=36864), N=16, "
                                   "N(0,0.02) weights magnitude-pruned to 80 % per matrix, activations N(0,1): QKV -> "
                                   "out-proj -> all-reduce -> FFN1 -> ReLU -> FFN2 -> all-reduce",
                       "parallelism": f"tp{world}: QKV/FFN1 column-parallel, out-proj/FFN2 row-parallel, NCCL all-reduce "
                                      f"of {N_TOKENS}x{H} fp16 after each row-parallel SpMM",
                       "shards": {k: list(v) for k, v in shape.shard_shapes().items()}},
            "ms_per_step_without_collectives": ms_local / args.steps,
            "ms_per_all_reduce_alone": ms_coll / args.steps,
            "hbm_gbs_per_gpu": bytes_alg * args.steps / (ms * 1e-3) / 1e9,
            "parity_vs_host_layer": parity, "gpu_launches": launches, "clocks": clocks.summary()}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--workload", default="layer", choices=["layer", "tp-chain"],
                    help="layer: the four OPT-66B SpMMs, weight rows sharded, no collective (the headline metric); "
                         "tp-chain: the tensor-parallel layer chain with NCCL all-reduces")
    args = ap.parse_args()
    if args.workload == "tp-chain" and args.impl == "ours":
        run_tp_chain(args)
    elif args.impl == "reference":
        run_reference_cpu(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
