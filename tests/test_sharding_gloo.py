"""Row (output-feature) sharding over ranks, exercised with two gloo processes on CPU.

Each rank takes its slice of the weight rows, encodes it on its own with the product's host encoder, and runs the
CPU oracle's SpMM on its shard; nothing is exchanged on the data path.  The C slices are then gathered (only to
check them) and compared with the unsharded product.  This is the host-side logic `bench.py --gpus N` relies on."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, M: int, K: int, N: int, failures):
    sys.path.insert(0, ROOT)
    import flash_llm_b200 as fl
    from oracle import cpu_oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = (rank * M // world, (rank + 1) * M // world)
        A_shard = fl.synthetic.sparse_uniform_matrix(M, K, 0.8, seed=11, rows=rows).numpy()
        B = fl.synthetic.dense_uniform_matrix(N, K, seed=12).numpy()
        comp, offs, num_offsets = fl.InitSparseMatrixA_API(A_shard)
        assert num_offsets == ((rows[1] - rows[0]) // 128) * (K // 64) + 2
        C_shard = cpu_oracle.spmm_splitk(comp, offs, B, rows[1] - rows[0], N, K, 1)          # [N][m]
        gathered = [torch.empty((N, M // world), dtype=torch.float16) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(C_shard.copy()))
        C_all = torch.cat(gathered, dim=1).numpy()
        t = torch.tensor([float(comp.size)], dtype=torch.float64)
        dist.all_reduce(t)  # total compressed words over the ranks
        if rank == 0:
            A = fl.synthetic.sparse_uniform_matrix(M, K, 0.8, seed=11).numpy()
            comp_full, offs_full, _ = fl.InitSparseMatrixA_API(A)
            C_full = cpu_oracle.spmm_splitk(comp_full, offs_full, B, M, N, K, 1)
            if not np.array_equal(C_all, C_full):
                failures.put("sharded C differs from the unsharded product")
            if int(t.item()) != comp_full.size:
                failures.put(f"sharded encodings hold {int(t.item())} words, the full one {comp_full.size}")
    except Exception as e:  # surfaced by the parent
        failures.put(f"rank {rank}: {e!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_row_sharded_spmm_two_ranks(lib, oracle, world):
    M, K, N = 512, 384, 16
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, K, N, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    problems = []
    while not failures.empty():
        problems.append(failures.get())
    assert not problems, problems
