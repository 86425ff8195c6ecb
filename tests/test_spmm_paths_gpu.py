"""Every form of the SpMM kernel against the CPU oracle, whichever of them the automatic plan prefers: the ring form
(bulk copies of the compressed stream into shared memory) and the register-streaming form (global loads of a whole tile
into the scatter warps' registers) in its three shapes: 8 stages with one CTA per SM, 4 stages with two CTAs per SM,
and 4 stages with two warps sharing every tile.  Calls go through the C ABI of libSpMM_API.so."""
import numpy as np
import pytest
import torch

from helpers import DeviceProblem, assert_close, random_problem

pytestmark = pytest.mark.gpu

FORMS = [dict(path=1), dict(path=2, scatter_warps=8), dict(path=2, scatter_warps=4),
         dict(path=2, scatter_warps=4, producers=2)]
FORM_IDS = ["ring", "direct8", "direct4", "direct4x2"]


def _check(lib, oracle, A, B, N, split_k, plan, note):
    M, K = A.shape
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    want = oracle.gemm_f32(A, B)
    lib.set_plan(**plan)
    try:
        got = DeviceProblem(lib, comp, offs, B, M, N, K, split_k).run()
        used = lib.get_plan(M, N, K, split_k)
    finally:
        lib.set_plan()
    assert used["path"] == plan["path"]
    assert_close(got, want, f"{note} plan={plan}")
    return got


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
@pytest.mark.parametrize("N", [8, 16, 32, 64, 128])
def test_every_n_tile(lib, oracle, form, N):
    A, B = random_problem(lib, 384, 1024, N, 0.8, 100 + N)
    _check(lib, oracle, A, B, N, 1, dict(cluster_k=1, **form), f"N={N}")


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
@pytest.mark.parametrize("sparsity", [0.0, 0.3, 0.6, 0.7, 0.75, 0.95, 0.999, 1.0])
def test_densities(lib, oracle, form, sparsity):
    """From fully dense tiles (2048 vectors, far beyond what the register-streaming form keeps in registers) through
    the densities around its register budget (512 and 768 vectors per tile) down to empty tiles."""
    A, B = random_problem(lib, 256, 1536, 16, sparsity, 7)
    _check(lib, oracle, A, B, 16, 1, dict(cluster_k=1, **form), f"s={sparsity}")


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
def test_dense_and_sparse_tiles_alternate_in_a_stage(lib, oracle, form):
    """Successive tiles of one stage switch between tiles above the register budget of the register-streaming form,
    tiles within it and empty tiles, in every order."""
    M, K, N = 256, 64 * 48, 16
    rng = np.random.default_rng(11)
    A = np.zeros((M, K), np.float16)
    density = rng.choice([0.0, 0.02, 0.2, 0.3, 0.45, 1.0], size=(M // 128, K // 64))
    for r in range(M // 128):
        for c in range(K // 64):
            tile = rng.uniform(-1, 1, (128, 64)).astype(np.float16)
            tile[tile == 0] = np.float16(0.5)
            tile[rng.random((128, 64)) >= density[r, c]] = 0
            A[r * 128:(r + 1) * 128, c * 64:(c + 1) * 64] = tile
    B = lib.synthetic.dense_uniform_matrix(N, K, 12).numpy()
    _check(lib, oracle, A, B, N, 1, dict(cluster_k=1, **form), "alternating densities")


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
@pytest.mark.parametrize("reduce", [1, 2], ids=["second-kernel", "last-cta"])
@pytest.mark.parametrize("cluster_k,workspace_k,split_k", [(2, 1, 1), (4, 1, 1), (1, 3, 6), (2, 2, 4), (8, 1, 1), (3, 1, 1),
                                                           (5, 2, 4), (6, 1, 1), (7, 1, 1), (1, 32, 64), (1, 2, 5)])
def test_k_splits(lib, oracle, form, reduce, cluster_k, workspace_k, split_k):
    """Every way of cutting K: parts summed inside clusters of any size up to 8, workspace parts summed by the last
    CTA of an output tile to finish or by the second kernel, and both at once."""
    if workspace_k == 1 and reduce == 1:
        pytest.skip("no workspace parts: the reduce mode does not matter")
    A, B = random_problem(lib, 256, 2048, 16, 0.8, 13)
    _check(lib, oracle, A, B, 16, split_k,
           dict(cluster_k=cluster_k, workspace_k=workspace_k, reduce=reduce, **form), "K split")


@pytest.mark.parametrize("N", [16, 64, 256])
def test_sum_by_last_cta_is_deterministic_and_leaves_its_counters_clean(lib, oracle, N):
    """The order in which the CTAs of an output tile finish changes from launch to launch; the sum must not.  Repeated
    launches on one stream reuse the same counters, which therefore have to be back at zero every time; a second
    stream gets counters of its own."""
    M, K, split_k = 1152, 4096, 16
    A, B = random_problem(lib, M, K, N, 0.8, 77 + N)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    want = oracle.gemm_f32(A, B)
    lib.set_plan(cluster_k=1, workspace_k=8, reduce=2)
    try:
        prob = DeviceProblem(lib, comp, offs, B, M, N, K, split_k)
        first = prob.run().copy()
        assert_close(first, want, f"N={N}")
        for _ in range(20):
            assert np.array_equal(prob.run(), first)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            assert np.array_equal(prob.run(), first)
        second_kernel = None
        lib.set_plan(cluster_k=1, workspace_k=8, reduce=1)
        second_kernel = prob.run().copy()
    finally:
        lib.set_plan()
    assert np.array_equal(second_kernel, first)  # both add the parts in part order from the same fp32 partial sums


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
def test_fewer_tiles_than_scatter_warps(lib, oracle, form):
    for k_tiles in (1, 2, 3, 5, 9):
        A, B = random_problem(lib, 128, 64 * k_tiles, 16, 0.8, 20 + k_tiles)
        _check(lib, oracle, A, B, 16, 1, dict(cluster_k=1, **form), f"{k_tiles} K tiles")


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
def test_forms_agree(lib, oracle, form):
    """The forms differ in how words reach the stage and in how many accumulators the tiles are dealt to (the
    register-streaming form keeps one per MMA-issuing thread and adds them at the end), so results agree to fp32
    summation order."""
    M, K, N = 1024, 4096, 32
    A, B = random_problem(lib, M, K, N, 0.8, 31)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    prob = DeviceProblem(lib, comp, offs, B, M, N, K, 1)
    results = []
    for plan in (dict(path=1, cluster_k=2), dict(cluster_k=2, **form)):
        lib.set_plan(**plan)
        try:
            results.append(prob.run().copy())
        finally:
            lib.set_plan()
    assert_close(results[1], results[0].astype(np.float32), f"{form} against the ring form")


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
def test_malformed_offsets_are_reported_not_followed(lib, oracle, form):
    """A TileOffsets entry that runs backwards makes the kernel give up with status bit 2 instead of reading there."""
    M, K, N = 256, 1024, 16
    A, B = random_problem(lib, M, K, N, 0.8, 41)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    offs = offs.copy()
    offs[5] = offs[4] - 3
    lib.set_plan(cluster_k=1, **form)
    try:
        DeviceProblem(lib, comp, offs, B, M, N, K, 1).run(check_status=False)
        # A caller of the reference interface never reads the status word: the next call, made without clearing it,
        # must compute as if nothing had happened (a give-up belongs to the launch it happened in).
        comp, offs, _ = lib.InitSparseMatrixA_API(A)
        got = DeviceProblem(lib, comp, offs, B, M, N, K, 1).run(check_status=False)
        status = lib.consume_status()
    finally:
        lib.set_plan()
    assert status & 2
    assert_close(got, oracle.gemm_f32(A, B), "call after a malformed one")
    assert lib.consume_status() == 0


@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
@pytest.mark.parametrize("N", [256, 384])
def test_n_beyond_one_mma_tile(lib, oracle, form, N):
    """N a multiple of 128 (the reference's large-N dispatch, csrc/SpMM_API.cu:97-112): several N tiles per tile row."""
    A, B = random_problem(lib, 256, 1024, N, 0.8, 500 + N)
    _check(lib, oracle, A, B, N, 4, dict(**form), f"N={N}")


def test_more_streams_than_counter_sets_fall_back_to_the_second_kernel(lib, oracle):
    """The in-kernel split-K sum binds a set of arrival counters to each stream it is used on (32 sets per device);
    calls on further streams must still be right (they are summed by the second kernel)."""
    M, K, N, split_k = 512, 2048, 16, 8
    A, B = random_problem(lib, M, K, N, 0.8, 91)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    want = oracle.gemm_f32(A, B)
    prob = DeviceProblem(lib, comp, offs, B, M, N, K, split_k)
    lib.set_plan(cluster_k=1, workspace_k=4, reduce=2)
    try:
        first = prob.run().copy()
        assert_close(first, want, "default stream")
        streams = [torch.cuda.Stream() for _ in range(40)]
        for s_ in streams:
            with torch.cuda.stream(s_):
                assert np.array_equal(prob.run(), first)
    finally:
        lib.set_plan()


@pytest.mark.parametrize("plan", [dict(cluster_k=1), dict(cluster_k=2), dict(cluster_k=1, workspace_k=4),
                                  dict(cluster_k=1, workspace_k=4, reduce=2)], ids=["plain", "cluster", "parts", "parts-last-cta"])
@pytest.mark.parametrize("offset_halves", [1, 2, 3])
def test_output_that_is_only_two_byte_aligned(lib, oracle, plan, offset_halves):
    """The reference interface asks nothing of C's alignment beyond that of a half; the wide stores of the cluster sum
    and of the sums over workspace parts must give way to narrow ones (or to an uncut launch) for such a C."""
    M, K, N, split_k = 256, 2048, 16, 8
    A, B = random_problem(lib, M, K, N, 0.8, 97)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    want = oracle.gemm_f32(A, B)
    dev = torch.device("cuda:0")
    comp_d = torch.from_numpy(np.ascontiguousarray(comp.view(np.int32))).to(dev)
    offs_d, B_d = torch.from_numpy(offs).to(dev), torch.from_numpy(B).to(dev)
    backing = torch.full((N * M + 8,), float("nan"), dtype=torch.float16, device=dev)
    C = backing[offset_halves:offset_halves + N * M]
    ws = torch.empty((split_k, N, M), dtype=torch.float16, device=dev)
    lib.set_plan(**plan)
    try:
        lib.SpMM_SplitK_API(torch.cuda.current_stream().cuda_stream, None, comp_d.data_ptr(), offs_d.data_ptr(),
                            B_d.data_ptr(), C.data_ptr(), M, N, K, ws.data_ptr(), split_k)
        torch.cuda.synchronize()
    finally:
        lib.set_plan()
    assert lib.consume_status() == 0
    assert_close(C.view(N, M).cpu().numpy(), want, f"C at +{2 * offset_halves} bytes, plan {plan}")
    assert torch.isnan(backing[:offset_halves]).all() and torch.isnan(backing[offset_halves + N * M:]).all()
