"""Tensor-parallel sparse decoder-layer chain: QKV SpMM -> out-proj SpMM -> all-reduce -> FFN1 SpMM -> ReLU ->
FFN2 SpMM -> all-reduce, the way the reference's FasterTransformer integration shards an OPT layer over g GPUs
(end2end_inference/ft_tools/huggingface_opt_convert_Phase1.py:82-91 for the Q/K/V row slices; column-parallel
QKV and FFN1, row-parallel out-proj and FFN2, one NCCL all-reduce of [N][H] after each row-parallel matmul,
ft.patch ParallelGpt decoder layers).

The chain has no attention, LayerNorm, bias or residual: the out-proj input is the V third of the QKV output, which
is what attention returns for a single-position context.  All four matmuls are `Y[N][M] = X[N][K] @ W[M][K]^T` with
W tiled-CSL encoded, i.e. SpMM_SplitK_API calls; everything else here is plumbing (slicing, the collective, ReLU).

The matmul and the collective are injected, so that the same chain runs
  * on a GPU through libSpMM_API.so and torch.distributed (NCCL), and
  * in the CPU tests through a host GEMM and the gloo backend.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class ChainShape:
    hidden: int  # H
    ffn: int     # F
    tokens: int  # N
    world: int   # g

    def __post_init__(self):
        g = self.world
        for what, m, k in (("QKV", 3 * self.hidden // g, self.hidden), ("out-proj", self.hidden, self.hidden // g),
                           ("FFN1", self.ffn // g, self.hidden), ("FFN2", self.hidden, self.ffn // g)):
            if self.hidden % g or self.ffn % g or m % 128 or k % 64:
                raise ValueError(f"{what} shard {m}x{k} of H={self.hidden}, F={self.ffn} over {g} ranks is not a whole "
                                 "number of 128x64 tiles")

    def shard_shapes(self) -> dict:
        """(M, K) of every rank's four weight shards."""
        g, H, F = self.world, self.hidden, self.ffn
        return {"qkv": (3 * H // g, H), "out_proj": (H, H // g), "ffn1": (F // g, H), "ffn2": (H, F // g)}

    def flops(self) -> float:
        """Dense-equivalent flops of the whole layer (all ranks together), 2*M*N*K per matmul."""
        H, F, N = self.hidden, self.ffn, self.tokens
        return 2.0 * N * (3 * H * H + H * H + F * H + H * F)


def shard_weights(shape: ChainShape, rank: int, w_qkv: torch.Tensor, w_out: torch.Tensor, w_ffn1: torch.Tensor,
                  w_ffn2: torch.Tensor) -> dict:
    """Rank `rank`'s slices of the full matrices W_qkv[3H][H] (Q rows, then K rows, then V rows), W_out[H][H],
    W_ffn1[F][H], W_ffn2[H][F].  Column-parallel layers keep whole rows (output features); row-parallel layers keep
    a slice of the contraction dimension, i.e. of the columns."""
    g, H, F = shape.world, shape.hidden, shape.ffn
    h, f = H // g, F // g
    q, k, v = w_qkv[0:H], w_qkv[H:2 * H], w_qkv[2 * H:3 * H]
    rows = slice(rank * h, (rank + 1) * h)
    return {"qkv": torch.cat([q[rows], k[rows], v[rows]], dim=0).contiguous(),
            "out_proj": w_out[:, rank * h:(rank + 1) * h].contiguous(),
            "ffn1": w_ffn1[rank * f:(rank + 1) * f].contiguous(),
            "ffn2": w_ffn2[:, rank * f:(rank + 1) * f].contiguous()}


def run_chain(shape: ChainShape, x: torch.Tensor, matmul: Callable[..., torch.Tensor],
              all_reduce: Callable[[torch.Tensor], torch.Tensor] | None = None,
              matmul_reduced: Callable[[str, torch.Tensor], torch.Tensor] | None = None) -> torch.Tensor:
    """One rank's pass over the layer.  `matmul(name, X[N][K], relu=False) -> Y[N][M]` multiplies by that rank's shard
    `name` (and applies ReLU to the result when asked: FFN1 is column-parallel, so its activation needs no partner).
    The two row-parallel layers need the sum over the ranks: either `all_reduce(t)` is applied to their outputs, or
    `matmul_reduced(name, X)` does the matmul and the sum in one step (the fused SpMM + all-reduce of the library).
    Returns the layer output [N][H] (same on every rank)."""
    if matmul_reduced is None:
        matmul_reduced = lambda name, t: all_reduce(matmul(name, t))  # noqa: E731
    h = shape.hidden // shape.world
    y_qkv = matmul("qkv", x)                               # [N][3H/g]: this rank's Q, K, V features
    v = y_qkv[:, 2 * h:3 * h].contiguous()                 # single-position attention returns V
    attn = matmul_reduced("out_proj", v)                   # [N][H], partial sums over the K slices added up
    y1 = matmul("ffn1", attn, relu=True)                   # [N][F/g]
    return matmul_reduced("ffn2", y1)                      # [N][H]


def fp32_all_reduce(dist=None) -> Callable[[torch.Tensor], torch.Tensor]:
    """The chain's collective: the ranks' fp16 partial matrices are widened, summed in fp32 (``dist.all_reduce``; NCCL
    on GPUs, gloo on CPU) and rounded to fp16 once.  Summing the fp16 partials in fp16, as a plain all-reduce of the
    SpMM outputs would, rounds after every addition: at eight ranks that alone put the layer output outside the
    tolerance the chain is checked with.  ``dist=None`` (one rank) returns the identity."""
    if dist is None:
        return lambda t: t

    def all_reduce(t: torch.Tensor) -> torch.Tensor:
        wide = t.float()
        dist.all_reduce(wide)
        return wide.to(torch.float16)
    return all_reduce


def reference_chain(shape: ChainShape, x: torch.Tensor, w_qkv: torch.Tensor, w_out: torch.Tensor,
                    w_ffn1: torch.Tensor, w_ffn2: torch.Tensor) -> torch.Tensor:
    """The unsharded layer on the host in fp32, rounding to fp16 where the kernels store fp16 (every matmul output)."""
    H = shape.hidden
    r16 = lambda t: t.to(torch.float16).float()  # noqa: E731
    y_qkv = r16(x.float() @ w_qkv.float().T)
    attn = r16(y_qkv[:, 2 * H:3 * H] @ w_out.float().T)
    y1 = torch.relu(r16(attn @ w_ffn1.float().T))
    return r16(y1 @ w_ffn2.float().T)


class DeviceChain:
    """One rank's shards encoded on its GPU plus the buffers of the chain; `step()` enqueues one pass."""

    def __init__(self, fl, shape: ChainShape, shards: dict, device, split_k: int = 64):
        self.fl, self.shape, self.dev, self.split_k = fl, shape, device, split_k
        self.layers = {}
        stream = torch.cuda.current_stream(device).cuda_stream
        N = shape.tokens
        for name, w in shards.items():
            M, K = w.shape
            w = w.to(device=device, dtype=torch.float16).contiguous()
            comp, offs, num_offsets, words = fl.encode_on_device(
                stream, w.data_ptr(), M, K,
                lambda n: (lambda t: (t, t.data_ptr()))(torch.empty(n, dtype=torch.int32, device=device)),
                lambda n: (lambda t: (t, t.data_ptr()))(torch.empty(n, dtype=torch.int32, device=device)),
                lambda owner, i: owner[i].item())
            self.layers[name] = dict(M=M, K=K, comp=comp, offs=offs,
                                     out=torch.empty((N, M), dtype=torch.float16, device=device),
                                     bytes_alg=4 * words + 4 * num_offsets + 2 * K * N + 2 * M * N)
        biggest = max(l["M"] for l in self.layers.values())
        self.ws = torch.empty((split_k, N, biggest), dtype=torch.float16, device=device)
        torch.cuda.synchronize(device)

    def matmul(self, name: str, x: torch.Tensor, relu: bool = False) -> torch.Tensor:
        layer = self.layers[name]
        assert x.is_contiguous() and x.dtype == torch.float16 and tuple(x.shape) == (self.shape.tokens, layer["K"])
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        self.fl.spmm_splitk_bias_act(stream, layer["comp"].data_ptr(), layer["offs"].data_ptr(), x.data_ptr(),
                                     layer["out"].data_ptr(), layer["M"], self.shape.tokens, layer["K"],
                                     self.ws.data_ptr(), self.split_k, None,
                                     self.fl.ACT_RELU if relu else self.fl.ACT_NONE)
        return layer["out"]

    def matmul_reduced(self, comm) -> Callable[[str, torch.Tensor], torch.Tensor]:
        """The row-parallel layers through the library's fused SpMM + all-reduce over the communicator `comm`."""
        def call(name: str, x: torch.Tensor) -> torch.Tensor:
            layer = self.layers[name]
            assert x.is_contiguous() and x.dtype == torch.float16 and tuple(x.shape) == (self.shape.tokens, layer["K"])
            stream = torch.cuda.current_stream(self.dev).cuda_stream
            self.fl.spmm_splitk_allreduce(comm, stream, layer["comp"].data_ptr(), layer["offs"].data_ptr(), x.data_ptr(),
                                          layer["out"].data_ptr(), layer["M"], self.shape.tokens, layer["K"])
            return layer["out"]
        return call

    def step(self, x: torch.Tensor, all_reduce: Callable[[torch.Tensor], torch.Tensor] | None = None,
             comm=None) -> torch.Tensor:
        """One pass; with `comm` (see PeerGroup) the row-parallel layers use the fused SpMM + all-reduce."""
        if comm is not None:
            return run_chain(self.shape, x, self.matmul, matmul_reduced=self.matmul_reduced(comm))
        return run_chain(self.shape, x, self.matmul, all_reduce)


class PeerGroup:
    """This rank's communicator for the fused SpMM + all-reduce: allocates the local receive buffer, exchanges the
    inter-process handles over `dist` (any torch.distributed backend: the handles are 64 bytes of host data), maps the
    peers' buffers and builds the communicator.  `max_elems` = the largest M*N of a fused call."""

    def __init__(self, fl, dist, rank: int, world: int, max_elems: int):
        self.fl, self.rank, self.world = fl, rank, world
        self.local, handle = fl.comm_alloc_buffer(world, max_elems)
        handles = [None] * world
        dist.all_gather_object(handles, handle)
        self.buffers = [self.local if w == rank else fl.comm_open_peer_buffer(handles[w]) for w in range(world)]
        self.comm = fl.comm_create(rank, world, max_elems, self.buffers)
        dist.barrier()  # every buffer is cleared and mapped before anybody's first store into it

    def close(self):
        self.fl.comm_destroy(self.comm)
        for w, ptr in enumerate(self.buffers):
            if w != self.rank:
                self.fl.comm_close_peer_buffer(ptr)
        self.fl.comm_free_buffer(self.local)


class LocalGroup:
    """`world` communicators on ONE device, for tests without several GPUs: the ranks' receive buffers all live on
    this device.  The fused call never waits inside its first kernel, so the ranks' calls can be enqueued one after
    another on one stream: every "rank"'s stores have landed by the time any summing kernel runs ... provided that all
    ranks' first kernels are enqueued before any rank's second one, which is what `calls()` arranges."""

    def __init__(self, fl, world: int, max_elems: int):
        self.fl, self.world = fl, world
        self.buffers = [fl.comm_alloc_buffer(world, max_elems)[0] for _ in range(world)]
        self.comms = [fl.comm_create(r, world, max_elems, self.buffers) for r in range(world)]

    def close(self):
        for c in self.comms:
            self.fl.comm_destroy(c)
        for b in self.buffers:
            self.fl.comm_free_buffer(b)
