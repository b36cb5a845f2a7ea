"""The allocation-free LayerNorm backward, called through its exported C symbol.

Some users of this library cannot allocate device memory around a call: think of a serving
process whose own memory manager already owns the whole GPU, or a plug-in living inside a
framework that forbids allocations outside its pool. For them the library exports
``b200_layernorm_bwd_noalloc``, which keeps its scratch in an array built into the library.
This test calls that symbol with raw pointers, twice in a row with different inputs (the
built-in scratch still holds the first call's partial sums during the second), and checks both
results against the regular entry point, which takes its scratch from the caller.

The file name sorts last so that a run stopping at the first failure has already run every
other test; the test also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _lib():
    from jax_gpt_b200 import _ext
    _ext.load()
    lib = ctypes.CDLL(_ext.LIB_PATH)
    fn = lib.b200_layernorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.b200_noalloc_strerror.restype = ctypes.c_char_p
    lib.b200_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _case(dev, M, D, seed, with_res):
    from jax_gpt_b200.ops import norm as N
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(M, D, device=dev, generator=g).to(torch.bfloat16)
    dy = torch.randn(M, D, device=dev, generator=g).to(torch.bfloat16)
    gamma = (torch.randn(D, device=dev, generator=g) * 0.3 + 1).to(torch.bfloat16)
    beta = torch.randn(D, device=dev, generator=g).to(torch.bfloat16)
    dres = torch.randn(M, D, device=dev, generator=g).to(torch.bfloat16) if with_res else None
    _, mean, rstd = N.norm_fwd(N.LAYERNORM, x, gamma, beta, 1e-5)
    # the gradients are accumulated, so start both paths from the same non-zero values
    dgamma0 = torch.randn(D, device=dev, generator=g)
    dbeta0 = torch.randn(D, device=dev, generator=g)
    return x, dy, gamma, mean, rstd, dres, dgamma0, dbeta0


@pytest.mark.parametrize("with_res", [False, True])
def test_noalloc_matches_regular_entry_point_twice(cuda_device, with_res):
    from jax_gpt_b200.ops import norm as N
    lib = _lib()
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    # calls back to back: different sizes and data, each re-uses the built-in scratch of the one before; the
    # small ones leave most warps of the partial-sum kernel without a row (they must write zero partials)
    for call, (M, D) in enumerate([(1500, 768), (333, 1024), (1, 256), (5, 64)]):
        x, dy, gamma, mean, rstd, dres, dgamma0, dbeta0 = _case(cuda_device, M, D, 100 + call, with_res)
        ref_dg, ref_db = dgamma0.clone(), dbeta0.clone()
        ref_dx = N.norm_bwd(N.LAYERNORM, dy, x, gamma, mean, rstd, ref_dg, ref_db, dres=dres)
        dx = torch.empty_like(x)
        dg, db = dgamma0.clone(), dbeta0.clone()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(cuda_device)
        # cudaMemGetInfo also sees allocations that bypass the caching allocator (a raw cudaMalloc in the
        # library); the first call of the process may create the context's own structures, so it is not compared
        free_before = torch.cuda.mem_get_info(cuda_device)[0]
        rc = lib.b200_layernorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                            rstd.data_ptr(), dres.data_ptr() if dres is not None else None,
                                            dx.data_ptr(), dg.data_ptr(), db.data_ptr(), M, D, stream)
        assert rc == 0, lib.b200_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(cuda_device) == before
        if call > 0:
            assert torch.cuda.mem_get_info(cuda_device)[0] == free_before
        assert _rel(dx, ref_dx) < 1e-2, (call, _rel(dx, ref_dx))
        assert _rel(dg, ref_dg) < 1e-3 and _rel(db, ref_db) < 1e-3, (call, _rel(dg, ref_dg), _rel(db, ref_db))


def test_noalloc_rejects_rows_beyond_the_builtin_scratch(cuda_device):
    lib = _lib()
    t = torch.zeros(64, device=cuda_device)
    p = t.data_ptr()
    rc = lib.b200_layernorm_bwd_noalloc(p, p, p, p, p, None, p, p, p, 4, 2048, None)
    assert rc == -1 and b"1024" in lib.b200_noalloc_strerror(rc)
    assert lib.b200_layernorm_bwd_noalloc(p, p, p, p, p, None, p, p, p, 4, 100, None) == -2
    assert lib.b200_layernorm_bwd_noalloc(None, p, p, p, p, None, p, p, p, 4, 64, None) == -3
