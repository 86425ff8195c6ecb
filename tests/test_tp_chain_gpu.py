"""The tensor-parallel layer chain through the CUDA library on one GPU: the g ranks' shards are encoded and
multiplied one after another on the same device, and the all-reduce is a sum over the ranks' partial matrices, so
that the chain's shard shapes (K = H/g, M = 3H/g ...) and its data flow are checked against the host layer without
needing g GPUs.  Calls go through the C ABI of libSpMM_API.so."""
import sys

import numpy as np
import pytest
import torch

from helpers import error_metrics
from test_tp_chain_gloo import make_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("H,F,world", [(1024, 4096, 2), (1024, 4096, 8), (2048, 8192, 4)])
def test_chain_on_one_device_matches_the_host_layer(lib, oracle, H, F, world):
    from flash_llm_b200 import tp_chain
    N = 16
    dev = torch.device("cuda:0")
    shape = tp_chain.ChainShape(hidden=H, ffn=F, tokens=N, world=world)
    full = make_weights(lib, H, F, seed=700 + world)
    chains = [tp_chain.DeviceChain(lib, shape, tp_chain.shard_weights(shape, r, *full), dev) for r in range(world)]
    x = lib.synthetic.normal_matrix(N, H, 1.0, 701).to(torch.float16)
    x_d = x.to(dev)
    h = H // world

    def summed(name, inputs):
        parts = [c.matmul(name, inp).float().clone() for c, inp in zip(chains, inputs)]
        # what tp_chain.fp32_all_reduce does over the real ranks: fp32 sum of the fp16 partials, one rounding
        return torch.stack(parts).sum(0).to(torch.float16)

    v = [c.matmul("qkv", x_d)[:, 2 * h:3 * h].contiguous() for c in chains]
    attn = summed("out_proj", v)
    y1 = [c.matmul("ffn1", attn, relu=True).clone() for c in chains]
    got = summed("ffn2", y1)
    torch.cuda.synchronize()
    assert lib.consume_status() == 0
    want = tp_chain.reference_chain(shape, x, *full)
    rel, ab = error_metrics(got.cpu().numpy(), want.numpy())
    assert rel <= 5e-2 and ab <= 2e-3, f"H={H} F={F} g={world}: rel {rel:.3e}, abs/peak {ab:.3e}"


def test_run_chain_with_one_rank_is_the_plain_layer(lib, oracle):
    """world = 1: `run_chain` itself on the device, the all-reduce being the identity."""
    from flash_llm_b200 import tp_chain
    H, F, N = 1024, 2048, 16
    dev = torch.device("cuda:0")
    shape = tp_chain.ChainShape(hidden=H, ffn=F, tokens=N, world=1)
    full = make_weights(lib, H, F, seed=800)
    chain = tp_chain.DeviceChain(lib, shape, tp_chain.shard_weights(shape, 0, *full), dev)
    x = lib.synthetic.normal_matrix(N, H, 1.0, 801).to(torch.float16)
    got = chain.step(x.to(dev), lambda t: t)
    torch.cuda.synchronize()
    assert lib.consume_status() == 0
    want = tp_chain.reference_chain(shape, x, *full)
    rel, ab = error_metrics(got.cpu().numpy(), want.numpy())
    assert rel <= 2e-2 and ab <= 2e-3, f"rel {rel:.3e}, abs/peak {ab:.3e}"
