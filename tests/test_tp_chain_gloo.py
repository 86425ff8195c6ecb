"""The tensor-parallel layer chain (column-parallel QKV / FFN1, row-parallel out-proj / FFN2, an all-reduce after
each row-parallel matmul) with two gloo processes on CPU.

Every rank slices the full weights the way the GPU path does, encodes its shards with the product's host encoder,
multiplies with the CPU oracle's SpMM (the model of the kernel: fp32 accumulation, fp16 outputs) and all-reduces over
gloo; the result must agree with the unsharded layer computed on the host.  This is the host-side logic of
`bench.py --workload tp-chain`."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_weights(fl, H: int, F: int, seed: int):
    """Full matrices of the chain: N(0, 0.02) magnitude-pruned to 80 % per matrix."""
    mk = lambda m, k, s: fl.synthetic.magnitude_pruned_matrix(m, k, 0.8, 0.02, seed + s)  # noqa: E731
    return mk(3 * H, H, 0), mk(H, H, 1), mk(F, H, 2), mk(H, F, 3)


def _worker(rank: int, world: int, port: int, H: int, F: int, N: int, failures):
    sys.path.insert(0, ROOT)
    import flash_llm_b200 as fl
    from flash_llm_b200 import tp_chain
    from oracle import cpu_oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shape = tp_chain.ChainShape(hidden=H, ffn=F, tokens=N, world=world)
        full = make_weights(fl, H, F, seed=900)
        shards = tp_chain.shard_weights(shape, rank, *full)
        assert {k: tuple(v.shape) for k, v in shards.items()} == shape.shard_shapes()
        encoded = {}
        for name, w in shards.items():
            comp, offs, _ = fl.InitSparseMatrixA_API(w.numpy())
            encoded[name] = (comp, offs, w.shape[0], w.shape[1])
        x = fl.synthetic.normal_matrix(N, H, 1.0, 901).to(torch.float16)

        def matmul(name, act, relu=False):
            comp, offs, M, K = encoded[name]
            out = torch.from_numpy(cpu_oracle.spmm_splitk(comp, offs, act.contiguous().numpy(), M, N, K, 1).copy())
            return torch.relu(out) if relu else out

        got = tp_chain.run_chain(shape, x, matmul, tp_chain.fp32_all_reduce(dist))  # the collective bench.py uses
        if rank == 0:
            want = tp_chain.reference_chain(shape, x, *full)
            from helpers import error_metrics
            # Looser than one SpMM's 1e-2: every rank rounds its partial sums to fp16 before the all-reduce (the
            # unsharded layer rounds the full sum once), and two more matmuls carry that difference along.
            rel, ab = error_metrics(got.numpy(), want.numpy())
            if not (rel <= 5e-2 and ab <= 2e-3):
                failures.put(f"sharded chain differs from the unsharded layer: rel {rel:.3e}, abs/peak {ab:.3e}")
            if not torch.isfinite(got.float()).all() or float(got.float().abs().max()) == 0.0:
                failures.put("degenerate chain output")
    except Exception as e:  # surfaced by the parent
        failures.put(f"rank {rank}: {e!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_tensor_parallel_chain_two_ranks(lib, oracle, world):
    H, F, N = 512, 1024, 16
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, H, F, N, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    problems = []
    while not failures.empty():
        problems.append(failures.get())
    assert not problems, problems


def test_shard_shapes_of_the_opt66b_chain():
    sys.path.insert(0, ROOT)
    from flash_llm_b200 import tp_chain
    s = tp_chain.ChainShape(hidden=9216, ffn=36864, tokens=16, world=8)
    assert s.shard_shapes() == {"qkv": (3456, 9216), "out_proj": (9216, 1152), "ffn1": (4608, 9216), "ffn2": (9216, 4608)}
    with pytest.raises(ValueError):
        tp_chain.ChainShape(hidden=9216, ffn=36864, tokens=16, world=16)  # 9216/16 = 576 = 9 x 64 ok, 3*576 = 1728 rows no


def test_qkv_shard_takes_the_same_rows_of_q_k_and_v():
    sys.path.insert(0, ROOT)
    from flash_llm_b200 import tp_chain
    H, F, g = 256, 512, 2
    s = tp_chain.ChainShape(hidden=H, ffn=F, tokens=8, world=g)
    w_qkv = torch.arange(3 * H, dtype=torch.float32).view(-1, 1).expand(3 * H, H).contiguous()
    zeros = lambda m, k: torch.zeros((m, k))  # noqa: E731
    sh = tp_chain.shard_weights(s, 1, w_qkv, zeros(H, H), zeros(F, H), zeros(H, F))
    rows = sh["qkv"][:, 0].tolist()
    assert rows == list(range(128, 256)) + list(range(H + 128, H + 256)) + list(range(2 * H + 128, 2 * H + 256))
    assert sh["out_proj"].shape == (H, H // g) and sh["ffn2"].shape == (H, F // g)
