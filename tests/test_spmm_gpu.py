"""Parity of the CUDA path with the CPU oracle, through the C ABI of libSpMM_API.so.  Ordered from the
smallest case up so that a first failure points at the simplest broken thing."""
import numpy as np
import pytest
import torch

from helpers import DeviceProblem, assert_close, random_problem

pytestmark = pytest.mark.gpu


def _run_case(lib, oracle, M, K, N, sparsity, split_k=1, seed=1, reorder=True, plan=None):
    A, B = random_problem(lib, M, K, N, sparsity, seed)
    comp, offs, _ = (lib.InitSparseMatrixA_API if reorder else lib.InitSparseMatrixA_API_NoReorder)(A)
    want = oracle.gemm_f32(A, B)
    lib.set_plan(**(plan or {}))
    try:
        got = DeviceProblem(lib, comp, offs, B, M, N, K, split_k).run()
    finally:
        lib.set_plan()
    assert_close(got, want, f"M={M} K={K} N={N} s={sparsity} Split_K={split_k} plan={plan}")
    return got


def test_library_is_the_cuda_one(lib):
    assert torch.cuda.is_available()
    before = lib.launch_count()
    _ = lib.get_plan(4096, 16, 4096, 1)
    assert lib.launch_count() == before


def test_single_nonzero_lands_in_the_right_cell(lib, oracle):
    """One weight at (r, c): C[n][r] must equal B[n][c] exactly, every other output row stays zero."""
    M, K, N = 128, 64, 16
    B = lib.synthetic.dense_uniform_matrix(N, K, 77).numpy()
    for r, c in ((0, 0), (1, 1), (5, 9), (8, 8), (31, 63), (77, 17), (127, 63), (64, 40)):
        A = np.zeros((M, K), np.float16)
        A[r, c] = 1.0
        comp, offs, _ = lib.InitSparseMatrixA_API(A)
        lib.set_plan(cluster_k=1)
        try:
            got = DeviceProblem(lib, comp, offs, B, M, N, K).run()
        finally:
            lib.set_plan()
        want = np.zeros((N, M), np.float16)
        want[:, r] = B[:, c]
        assert np.array_equal(got, want), f"(r={r}, c={c})"


@pytest.mark.parametrize("N", [16, 8, 32, 64, 128])
def test_one_tile(lib, oracle, N):
    _run_case(lib, oracle, 128, 64, N, 0.8, plan=dict(cluster_k=1))


@pytest.mark.parametrize("M,K", [(128, 256), (256, 64), (384, 512), (1024, 1024)])
@pytest.mark.parametrize("N", [16, 64])
def test_small_shapes_single_cta_per_row(lib, oracle, M, K, N):
    _run_case(lib, oracle, M, K, N, 0.8, plan=dict(cluster_k=1))


@pytest.mark.parametrize("cluster_k", [2, 3, 4, 8])
@pytest.mark.parametrize("N", [8, 16, 32, 64, 128])
def test_cluster_split_k(lib, oracle, cluster_k, N):
    _run_case(lib, oracle, 256, 1024, N, 0.8, plan=dict(cluster_k=cluster_k))


@pytest.mark.parametrize("split_k,workspace_k,cluster_k", [(4, 2, 1), (8, 4, 2), (16, 8, 1), (6, 3, 3), (8, 2, 4), (2, 1, 2), (3, 1, 1)])
def test_workspace_split_k(lib, oracle, split_k, workspace_k, cluster_k):
    _run_case(lib, oracle, 256, 2048, 16, 0.9, split_k=split_k, plan=dict(cluster_k=cluster_k, workspace_k=workspace_k))


@pytest.mark.parametrize("plan", [dict(a_stages=4, b_stages=1, b_batch=1), dict(a_stages=5, b_stages=8, b_batch=3),
                                  dict(a_stages=8, b_stages=2, b_batch=8, scatter_warps=8),
                                  dict(scatter_warps=6, a_stages=7), dict(scatter_warps=10, a_stages=10, chunk_vectors=256, ring_slots=9),
                                  dict(scatter_warps=5, a_stages=5),
                                  dict(producers=1, ring_slots=9), dict(producers=4, chunk_vectors=128, ring_slots=32),
                                  dict(chunk_vectors=128, ring_slots=18, producers=3),
                                  dict(chunk_vectors=512, ring_slots=6, producers=2),
                                  dict(chunk_vectors=1024, ring_slots=3, a_stages=4)])
def test_pipeline_shapes(lib, oracle, plan):
    """Pipeline depths, ring geometries and producer counts of the ring form of the kernel."""
    _run_case(lib, oracle, 256, 1536, 16, 0.7, plan=dict(path=1, cluster_k=2, **plan))


@pytest.mark.parametrize("sparsity", [0.0, 0.3, 0.5, 0.95, 0.999, 1.0])
def test_density_extremes(lib, oracle, sparsity):
    """Fully dense tiles (2048 vectors each, four ring chunks per tile) down to empty tiles."""
    _run_case(lib, oracle, 256, 512, 16, sparsity)


def test_scan_order_encoding_is_accepted(lib, oracle):
    _run_case(lib, oracle, 512, 1024, 32, 0.8, reorder=False)


@pytest.mark.parametrize("N", [8, 16, 32, 64])
def test_config_single_spmm_4096(lib, oracle, N):
    """The 4096 x 4096, 80 % sparse single-SpMM configuration with the automatic plan."""
    _run_case(lib, oracle, 4096, 4096, N, 0.8, seed=0xF1A50001)


@pytest.mark.parametrize("split_k", [1, 2, 4, 8])
def test_split_k_stress_shapes_scaled(lib, oracle, split_k):
    """The split-K stress configuration's aspect ratio (K = 4 M, N = 8, 90 %) at a size the oracle does in seconds."""
    _run_case(lib, oracle, 1536, 6144, 8, 0.9, split_k=split_k, seed=split_k)


def test_split_k_not_dividing_k_tiles(lib, oracle):
    # 22 K tiles over 3 cluster parts x 3 workspace parts = 9 uneven parts (reference tuned Split_K = 9 for K = 12288)
    _run_case(lib, oracle, 256, 1408, 16, 0.8, split_k=9, plan=dict(cluster_k=3, workspace_k=3))


def test_small_m_large_k(lib, oracle):
    _run_case(lib, oracle, 256, 8192, 16, 0.7, split_k=4)


def test_special_values(lib, oracle):
    """-0.0 and NaN weights are dropped by the encoder; infinities and subnormals are kept."""
    M, K, N = 256, 256, 16
    A, B = random_problem(lib, M, K, N, 0.8, 21)
    bits = A.view(np.uint16).copy()
    rng = np.random.default_rng(3)
    idx = rng.choice(bits.size, 90, replace=False)
    flat = bits.reshape(-1)
    flat[idx[:30]] = 0x8000
    flat[idx[30:60]] = 0x7E00
    flat[idx[60:88]] = 0x0001
    flat[idx[88:]] = 0x7C00
    comp, offs, _ = lib.InitSparseMatrixA_API(bits)
    dense = oracle.decode(comp, offs, M, K)
    want = oracle.gemm_f32(dense, B)
    got = DeviceProblem(lib, comp, offs, B, M, N, K).run()
    assert_close(got, want, "special values")


def test_matches_oracle_split_k_model(lib, oracle):
    """Against the CPU model of the reference kernel's own split-K rounding (fp16 partials)."""
    M, K, N, split_k = 512, 3072, 16, 6
    A, B = random_problem(lib, M, K, N, 0.8, 31)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    want = oracle.spmm_splitk(comp, offs, B, M, N, K, split_k)
    got = DeviceProblem(lib, comp, offs, B, M, N, K, split_k).run()
    assert_close(got, want.astype(np.float32), "oracle split-K model", fp16_partials=split_k)


def test_matches_reference_kernel_on_device(lib, oracle):
    """The unmodified reference kernel (compiled for sm_100a) and this library on the same device buffers, fed
    with each other's encodings."""
    if not oracle.reference_available():
        pytest.skip("reference build (oracle/_ref) not present")
    for (M, K, N, sparsity, split_k) in ((256, 512, 16, 0.8, 1), (1024, 2048, 8, 0.8, 2), (2048, 1024, 32, 0.7, 1),
                                         (512, 4096, 64, 0.9, 4), (4096, 4096, 16, 0.8, 1)):
        A, B = random_problem(lib, M, K, N, sparsity, 41 + N)
        comp, offs, _ = lib.InitSparseMatrixA_API(A)
        comp_ref, offs_ref = oracle.reference_encode(A, True)
        assert np.array_equal(comp, comp_ref) and np.array_equal(offs, offs_ref)
        prob = DeviceProblem(lib, comp, offs, B, M, N, K, split_k)
        mine = prob.run()
        prob.C.fill_(float("nan"))
        rc = oracle.reference_spmm(torch.cuda.current_stream().cuda_stream, prob.comp.data_ptr(), prob.offs.data_ptr(),
                                   prob.B.data_ptr(), prob.C.data_ptr(), M, N, K, prob.ws.data_ptr(), split_k)
        torch.cuda.synchronize()
        assert rc == 0
        theirs = prob.C.cpu().numpy()
        assert_close(mine, theirs.astype(np.float32), f"vs reference kernel M={M} K={K} N={N}",
                     fp16_partials=split_k if split_k > 1 else 0)
        assert_close(theirs, oracle.gemm_f32(A, B), "reference kernel vs host GEMM", fp16_partials=split_k if split_k > 1 else 0)


def test_splitk_reduction_entry_point(lib):
    M, N, parts = 256, 16, 5
    ws = torch.randn((parts, N, M), device="cuda").to(torch.float16)
    out = torch.empty((N, M), dtype=torch.float16, device="cuda")
    lib.splitk_reduction(torch.cuda.current_stream().cuda_stream, out.data_ptr(), ws.data_ptr(), M, N, parts)
    torch.cuda.synchronize()
    want = ws.float().sum(0).to(torch.float16)
    assert torch.equal(out, want)


def test_repeated_calls_and_streams(lib, oracle):
    M, K, N = 1024, 1024, 16
    A, B = random_problem(lib, M, K, N, 0.8, 51)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    want = oracle.gemm_f32(A, B)
    prob = DeviceProblem(lib, comp, offs, B, M, N, K)
    side = torch.cuda.Stream()
    for i in range(20):
        with torch.cuda.stream(side if i % 2 else torch.cuda.current_stream()):
            got = prob.run()
        assert_close(got, want, f"call {i}")


def test_launch_overlap_keeps_stream_order(lib, oracle):
    """With launch overlap on, a kernel may start before its predecessor has finished, but must not read B or write C
    early: a two-layer chain (the second SpMM's B is the first one's C), enqueued many times back to back."""
    N, K1, M1, M2 = 16, 1024, 2048, 1024
    A1 = lib.synthetic.sparse_uniform_matrix(M1, K1, 0.8, 61).numpy()
    A2 = (lib.synthetic.sparse_uniform_matrix(M2, M1, 0.8, 62) * 0.05).to(torch.float16).numpy()
    B_versions = [lib.synthetic.dense_uniform_matrix(N, K1, 70 + i).numpy() for i in range(4)]
    c1, o1, _ = lib.InitSparseMatrixA_API(A1)
    c2, o2, _ = lib.InitSparseMatrixA_API(A2)
    dev = torch.device("cuda:0")
    to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    c1_d, o1_d, c2_d, o2_d = to_dev(c1.view(np.int32)), to_dev(o1), to_dev(c2.view(np.int32)), to_dev(o2)
    Bs = [to_dev(b) for b in B_versions]
    X = torch.empty((N, K1), dtype=torch.float16, device=dev)
    H = torch.empty((N, M1), dtype=torch.float16, device=dev)
    ws = torch.empty((8, N, M1), dtype=torch.float16, device=dev)
    outs = [torch.empty((N, M2), dtype=torch.float16, device=dev) for _ in range(12)]
    stream = torch.cuda.current_stream().cuda_stream
    want = []
    for b in B_versions:
        h = oracle.gemm_f32(A1, b).astype(np.float16)
        want.append(oracle.gemm_f32(A2, h))
    lib.set_launch_overlap(True)
    try:
        for i, out in enumerate(outs):
            X.copy_(Bs[i % 4], non_blocking=True)
            lib.SpMM_SplitK_API(stream, None, c1_d.data_ptr(), o1_d.data_ptr(), X.data_ptr(), H.data_ptr(), M1, N, K1,
                                ws.data_ptr(), 8)
            lib.SpMM_SplitK_API(stream, None, c2_d.data_ptr(), o2_d.data_ptr(), H.data_ptr(), out.data_ptr(), M2, N, M1,
                                ws.data_ptr(), 8)
        torch.cuda.synchronize()
    finally:
        lib.set_launch_overlap(False)
    assert lib.consume_status() == 0
    for i, out in enumerate(outs):
        assert_close(out.cpu().numpy(), want[i % 4], f"chained call {i}")
