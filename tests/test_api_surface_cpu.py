"""Every entry point of the reference's binding layer is registered, under the
CUDA names and under the names of the MUSA checkout (reference:
src/pybind.cpp:114-150), plus this library's fused entry points.  Runs without
a GPU: the classes can be constructed, only their methods need a device."""
import torch

import flashoverlap_b200  # noqa: F401  (loads the native library)

BASELINE = ["nccl_init", "cublas_init", "cublas_gemm", "nccl_allreduce", "nccl_reducescatter", "nccl_all2all",
            "mccl_init", "mublas_init", "mublas_gemm", "mccl_allreduce", "mccl_reducescatter", "mccl_all2all",
            "gemm_allreduce", "gemm_reducescatter", "gemm_all2all"]
OVERLAP_REFERENCE = ["cutlass_init", "nccl_init", "overlap_init", "cutlass_gemm", "mutlass_init", "mccl_init", "mutlass_gemm",
                     "gemm_allreduce_overlap", "gemm_reducescatter_overlap", "gemm_allreduce", "gemm_reducescatter",
                     "gemm_all2all", "nccl_allreduce", "nccl_reducescatter", "nccl_all2all", "mccl_allreduce",
                     "mccl_reducescatter", "mccl_all2all", "seg_allreduce"]
OVERLAP_OWN = ["gemm_allreduce_fused", "gemm_reducescatter_fused", "allgather_gemm", "a2a_dispatch_gemm", "a2a_padded_rows",
               "gemm_rmsnorm", "gemm_allreduce_twostream", "gemm_reducescatter_twostream", "set_timeout_ms", "set_sm_count",
               "set_raster_group", "set_raster_taper", "set_l2_hints", "set_use_nvls", "allreduce_uses_nvls",
               "set_allgather_multicast", "set_phase_trace", "set_row_trace", "status", "status_string", "check_status",
               "reset", "transport", "num_algos", "algo_tile", "p2p_push", "p2p_push_bulk", "multimem_bench",
               "detach_symmetric"]
OPS = ["generate_nccl_id", "generate_mccl_id", "reorder_rmsnorm", "reorder_rmsnorm_eps", "rmsnorm", "tile_walk"]


def test_baseline_class_has_the_reference_methods():
    obj = torch.classes.flashoverlap_class.BaselineImpl()
    missing = [m for m in BASELINE if not hasattr(obj, m)]
    assert not missing, missing


def test_overlap_class_has_the_reference_and_the_fused_methods():
    obj = torch.classes.flashoverlap_class.OverlapImpl()
    missing = [m for m in OVERLAP_REFERENCE + OVERLAP_OWN if not hasattr(obj, m)]
    assert not missing, missing


def test_ops_are_registered():
    missing = [o for o in OPS if not hasattr(torch.ops.flashoverlap_op, o)]
    assert not missing, missing
    ident = torch.ops.flashoverlap_op.generate_nccl_id()
    assert len(ident) == 16          # the reference's 128-byte id as 16 int64 (src/mccl_utils.cpp:7-14)


def test_tile_table_matches_the_python_copy():
    from flashoverlap_b200.utils.config import ALGO_TILES

    obj = torch.classes.flashoverlap_class.OverlapImpl()
    assert obj.num_algos() == len(ALGO_TILES)
    for i, tile in enumerate(ALGO_TILES):
        assert tuple(obj.algo_tile(i))[:3] == tuple(tile)
