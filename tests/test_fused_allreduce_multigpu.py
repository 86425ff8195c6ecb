"""The tensor-parallel layer chain over real GPUs, one process per GPU, with the row-parallel layers going through the
fused SpMM + all-reduce (plain peer stores into every rank's receive buffer, bounded flag waits).  Needs at least two
GPUs; on a single-GPU box the emulated-rank tests of test_fused_allreduce_gpu.py cover the same kernels.  The ranks
exchange their 64-byte buffer handles over a gloo process group on 127.0.0.1 (host data only: no NCCL, no multicast)."""
import os
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, H, F, N, failures):
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import torch.distributed as dist
        import flash_llm_b200 as fl
        from flash_llm_b200 import tp_chain
        from test_tp_chain_gloo import make_weights
        from helpers import error_metrics
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        shape = tp_chain.ChainShape(hidden=H, ffn=F, tokens=N, world=world)
        full = make_weights(fl, H, F, seed=1300)
        chain = tp_chain.DeviceChain(fl, shape, tp_chain.shard_weights(shape, rank, *full), dev)
        x = fl.synthetic.normal_matrix(N, H, 1.0, 1301).to(torch.float16)
        group = tp_chain.PeerGroup(fl, dist, rank, world, N * H)
        try:
            outs = []
            for _ in range(4):  # successive layers alternate between the two halves of the receive buffers
                outs.append(chain.step(x.to(dev), comm=group.comm).clone())
            torch.cuda.synchronize(dev)
            status = fl.consume_status()
            if status != 0:
                failures.put(f"rank {rank}: kernel status {status:#x}")
            want = tp_chain.reference_chain(shape, x, *full)
            for i, out in enumerate(outs):
                rel, ab = error_metrics(out.cpu().numpy(), want.numpy())
                if not (rel <= 5e-2 and ab <= 2e-3):
                    failures.put(f"rank {rank} pass {i}: rel {rel:.3e}, abs/peak {ab:.3e}")
            gathered = [None] * world
            dist.all_gather_object(gathered, outs[-1].cpu())
            if rank == 0 and not all(torch.equal(g, gathered[0]) for g in gathered):
                failures.put("ranks hold different bits after the fused all-reduce")
            dist.barrier()  # nobody frees a buffer while a peer may still store into it
        finally:
            group.close()
        dist.destroy_process_group()
    except Exception as e:  # surfaced by the parent
        failures.put(f"rank {rank}: {e!r}")


@pytest.mark.parametrize("world", [2])
def test_chain_with_fused_allreduce_over_real_gpus(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, 1024, 4096, 16, failures)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    problems = []
    while not failures.empty():
        problems.append(failures.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            problems.append("a rank did not finish")
        elif p.exitcode != 0:
            problems.append(f"a rank exited with {p.exitcode}")
    assert not problems, problems
