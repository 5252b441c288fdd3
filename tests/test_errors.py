"""Host-side error reporting of the native library (CPU).

Messages with several parts must come through as Python RuntimeErrors: the extension builds
them without iostreams because libc10's own weak stream symbols interpose on extensions built
with the system compiler and crash (see csrc/common/fo_check.h).
"""
import pytest
import torch


def test_multi_part_messages_raise_cleanly(lib):
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    with pytest.raises(RuntimeError, match="unknown option 'bogus'"):
        impl.set_option("bogus", 1)
    with pytest.raises(RuntimeError, match="world size must be in"):
        impl.nccl_init(0, 64, [0] * 16)
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        impl.cutlass_gemm(torch.randn(128, 64), torch.randn(256, 64), torch.empty(128, 256), 0)
    with pytest.raises(RuntimeError, match="X must be a contiguous CUDA tensor"):
        torch.ops.flashoverlap_op.rmsnorm(torch.randn(4, 8), torch.randn(4, 8), torch.randn(8), 1e-5)
    with pytest.raises(RuntimeError, match="16 int64"):
        base = torch.classes.flashoverlap_class.BaselineImpl()
        base.nccl_init(0, 2, [1, 2, 3])


def test_symmetric_output_helper_single_rank(lib):
    """With one rank there is nothing to share: the helper must not touch torch.distributed."""
    from flashoverlap_b200.parallel import symm

    class OneRank:
        def get_option(self, name):
            assert name == "world"
            return 1

    if not torch.cuda.is_available():
        pytest.skip("allocates a CUDA tensor")
    t, mc = symm.alloc_allreduce_output(OneRank(), (4, 8), torch.bfloat16)
    assert t.shape == (4, 8) and mc is False


def test_option_and_argument_checks_of_the_additions(lib):
    """Argument validation that runs before anything touches a GPU."""
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    with pytest.raises(RuntimeError, match="epi_bufs must be 2 or 4"):
        impl.set_option("epi_bufs", 3)
    with pytest.raises(RuntimeError, match="diag is a bit mask"):
        impl.set_option("diag", 9)
    with pytest.raises(RuntimeError, match="push_lag must be"):
        impl.set_option("push_lag", 7)
    impl.set_option("epi_bufs", 4)
    impl.set_option("stage_local", 1)
    assert impl.get_option("epi_bufs") == 4 and impl.get_option("stage_local") == 1
    with pytest.raises(RuntimeError, match="int64 CUDA tensor"):
        impl.set_trace(torch.zeros(16, dtype=torch.int32))
    impl.set_trace(torch.zeros(0, dtype=torch.int64))          # an empty tensor switches recording off
    with pytest.raises(RuntimeError, match="call nccl_init first"):
        impl.use_stage(torch.zeros(4))
    with pytest.raises(RuntimeError, match="call nccl_init first"):
        impl.gemm_all2all_fused(torch.zeros(1), torch.zeros(1), torch.zeros(1), 0, torch.zeros(1, 1, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="square int32 host tensor"):
        torch.ops.flashoverlap_op.all2all_plan(torch.zeros(9, 9, dtype=torch.int32), 0)
