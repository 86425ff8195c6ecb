"""flash-llm_b200 — B200-native Load-as-Sparse / Compute-as-Dense SpMM behind Flash-LLM's SpMM_API interface.

The product is ``build/libSpMM_API.so`` (sources under ``csrc/``).  This package is its thin Python host
side: it loads the library through its C ABI and mirrors the reference's operator names.  There is no
fallback: if the library is missing or cannot be loaded, importing :mod:`api` members raises.
"""
from .api import (  # noqa: F401
    ACT_NONE,
    ACT_RELU,
    LIBRARY_PATH,
    FlashLLMError,
    GenSparseMatrixBinFile,
    InitSparseMatrixA_API,
    InitSparseMatrixA_API_NoReorder,
    SpMM_SplitK_API,
    build_library,
    comm_alloc_buffer,
    comm_close_peer_buffer,
    comm_create,
    comm_destroy,
    comm_free_buffer,
    comm_open_peer_buffer,
    comm_set_wait_limit,
    consume_status,
    encode_on_device,
    gen_sparse_matrix_bin_file_device,
    get_plan,
    launch_count,
    library,
    load_sparse_matrix_bin_files,
    read_output_sizes,
    read_rank_lists,
    read_sparse_matrix_bin_files,
    set_launch_overlap,
    set_plan,
    splitk_reduction,
    spmm_splitk_bias_act,
    spmm_splitk_epilogue,
    spmm_splitk_allreduce,
    spmm_splitk_no_alloc,
    write_rank_lists,
)
from . import synthetic  # noqa: F401
