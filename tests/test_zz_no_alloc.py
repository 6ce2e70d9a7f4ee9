"""The matrix product that allocates nothing (rmx_gemm_tcgen05_static, declared in
rust-mlx_b200/csrc/kernels/rmx_no_alloc.h), called through its exported C symbol.

Some users of these kernels cannot call cudaMalloc where they need a product: they run inside
another program's memory pool, or in a loop that must not wait for the allocator.  For them
the library keeps the split-K scratch in its own device memory.  This test calls that entry
point with raw pointers, as such a caller would, twice in a row (the second call finds the
scratch as the first left it), and compares with the ordinary entry point, which is given
scratch by its caller.  Both run the same kernel, so equal bits are expected; the check allows
the tolerance of the other product tests.  The file is collected last, so a run that stops at
the first failure has already run everything else; it also passes alone in a fresh process.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def library():
    from rust_mlx_b200.kernels.library import kernels_library
    return kernels_library()


def call_static(lib, a, w, out, splits):
    m, k = a.shape
    n = w.shape[0]
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.rmx_gemm_tcgen05_static(c_void_p(a.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(m),
                                     c_int(n), c_int(k), c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)),
                                     c_int(1 if out.dtype == torch.float32 else 0), c_int(splits), stream)
    return rc


@pytest.mark.parametrize("m, n, k, splits", [(8, 4096, 4096, 4), (1, 6144, 4096, 0), (33, 1000, 1032, 2), (64, 512, 4096, 1)])
def test_static_scratch_product_matches_the_ordinary_entry_point(m, n, k, splits):
    from rust_mlx_b200.kernels import ops
    lib = library()
    torch.manual_seed(m + n)
    a = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.05).to(torch.bfloat16)
    want = a.double() @ w.double().t()
    for odt in (torch.bfloat16, torch.float32):
        ordinary = torch.empty(m, n, dtype=odt, device=DEV)
        ops.gemm_tcgen05(a, w, ordinary, splits=splits or None)
        tol = 1e-2 if odt == torch.bfloat16 else 1e-4
        for call in range(2):                      # two calls in a row share the library's scratch
            out = torch.full((m, n), float("nan"), dtype=odt, device=DEV)
            assert call_static(lib, a, w, out, splits) == 0, lib.rmx_last_error().decode()
            assert lib.rmx_gemm_tcgen05_static_status(c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
            assert ((out.double() - ordinary.double()).abs() <= tol * (1 + ordinary.double().abs())).all()
            assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()
            if splits:
                assert torch.equal(out, ordinary)   # the same kernel with the same slices: the same bits


def test_sizes_beyond_the_scratch_are_refused_with_a_clear_error():
    lib = library()
    a = torch.zeros(64, 4096, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8192, 4096, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(64, 8192, dtype=torch.bfloat16, device=DEV)
    assert call_static(lib, a, w, out, 8) != 0      # 8 * 64 * 8192 floats = 4 Mi floats > 2 Mi
    msg = lib.rmx_last_error().decode()
    assert "scratch" in msg and "fewer splits" in msg
    assert call_static(lib, a, w, out, 0) == 0      # the library's own choice fits
    torch.cuda.synchronize()
    a65 = torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV)
    assert call_static(lib, a65, w[:, :64].contiguous(), torch.zeros(65, 8192, dtype=torch.bfloat16, device=DEV), 1) != 0
    assert "1..64 rows" in lib.rmx_last_error().decode()
