"""The allocation-free C entry point, called through its exported symbol.

Some callers of this library cannot allocate device memory: code running inside another
allocator's callback, a process whose device memory belongs entirely to a serving runtime's
pool, or a plain C host without PyTorch.  ``fo_fused_loopback_noalloc`` gives them the fused
GEMM+collective emulation with its scratch (staging buffers, arrival counters, status words) in
a fixed array inside the library.  This test calls it twice in a row via ctypes and compares
each result with the regular entry point (``torch.ops.flashoverlap_op.fused_loopback``), which
takes its scratch from cudaMalloc.  The file sorts last so that a run stopping at the first
failure has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry(lib_path):
    lib = ctypes.CDLL(str(lib_path))
    fn = lib.fo_fused_loopback_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                   ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _call(fn, comm_op, A, B, out, M, N, K, algo, strided):
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(comm_op, len(A), _ptrs(A), _ptrs(B), _ptrs(out), M, N, K, 1, algo, int(strided),
            ctypes.c_void_p(stream), err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("comm_op,ranks", [("all_reduce", 2), ("reduce_scatter", 4)])
def test_noalloc_entry_matches_regular_entry(cuda, lib, comm_op, ranks):
    from flashoverlap_b200 import ops
    fn = _entry(lib)
    M, N, K, algo = 512, 1024, 256, 0
    rows = M if comm_op == "all_reduce" else M // ranks
    for call in range(2):                      # two calls in a row share the built-in scratch
        g = torch.Generator(device=cuda).manual_seed(100 + call)
        A = [(torch.randn(M, K, device=cuda, generator=g) * 0.5).to(torch.bfloat16) for _ in range(ranks)]
        B = [(torch.randn(N, K, device=cuda, generator=g) * 0.5).to(torch.bfloat16) for _ in range(ranks)]
        expect = [torch.empty(rows, N, device=cuda, dtype=torch.bfloat16) for _ in range(ranks)]
        st = ops.fused_loopback(comm_op, A, B, expect, algo=algo, strided_rows=True, natural_out=True)
        assert all(s[0] == 0 for s in st)
        got = [torch.full((rows, N), float("nan"), device=cuda, dtype=torch.bfloat16) for _ in range(ranks)]
        torch.cuda.synchronize()
        rc, msg = _call(fn, 0 if comm_op == "all_reduce" else 1, A, B, got, M, N, K, algo, True)
        assert rc == 0, msg
        ref = sum(a.float() @ b.float().t() for a, b in zip(A, B))
        tol = 0.02 * ref.abs().max().item() + 1e-3
        for r in range(ranks):
            assert (got[r].float() - expect[r].float()).abs().max().item() <= tol, (call, r)


def test_noalloc_entry_rejects_oversize(cuda, lib):
    fn = _entry(lib)
    A = [torch.zeros(128, 64, device=cuda, dtype=torch.bfloat16) for _ in range(2)]
    B = [torch.zeros(256, 64, device=cuda, dtype=torch.bfloat16) for _ in range(2)]
    out = [torch.zeros(128, 256, device=cuda, dtype=torch.bfloat16) for _ in range(2)]
    # 2 ranks x 4096 x 4096 x 2 B = 64 MiB of staging: beyond the 16 MiB built in
    rc, msg = _call(fn, 0, A, B, out, 4096, 4096, 64, 0, True)
    assert rc == -2 and "exceeds" in msg
    rc, msg = _call(fn, 0, A, B, out, 128, 256, 64, 1, True)       # CTA-pair Algos are refused
    assert rc == -1 and "Algo" in msg
    rc, msg = _call(fn, 0, A, B, out, 128, 256, 64, 3, True)
    assert rc == -1 and "Algo" in msg
    for bad in ((-128, -256, 64), (0, 256, 64), (128, 256, 0)):   # non-positive sizes never reach the size arithmetic
        rc, msg = _call(fn, 0, A, B, out, *bad, 0, True)
        assert rc == -1 and "positive" in msg, (bad, rc, msg)
