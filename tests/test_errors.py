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
