"""
The allocation-free LayerNorm backward entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at call time (no allocator of their own, a memory pool
that already owns the whole GPU, or a loop that must not hit the synchronisation inside cudaMalloc). For them
``rb200_layer_norm_bwd_noalloc`` keeps its scratch in a fixed array inside the library. This test checks it against the
regular entry point (which gets its scratch from the caller) on two calls in a row, the second with other sizes, so that
stale contents of the shared array from the first call would show.
"""

import ctypes
import pytest
import torch

gpu = pytest.mark.gpu


def _entry_points():
    from returnn_b200.ops import _lib

    lib = _lib.get_lib(required=True)
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    fwd = lib.rb200_layer_norm_fwd
    fwd.argtypes = [vp, vp, vp, vp, vp, vp, i64, i32, f32, i32, i32, i32, vp]
    fwd.restype = i32
    bwd = lib.rb200_layer_norm_bwd
    bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, vp]
    bwd.restype = i32
    noalloc = lib.rb200_layer_norm_bwd_noalloc
    noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, vp]
    noalloc.restype = i32
    lib.rb200_layer_norm_bwd_noalloc_max_n.restype = i32
    lib.rb200_layer_norm_bwd_noalloc_parts.restype = i32
    lib.rb200_last_error.restype = ctypes.c_char_p
    return lib, fwd, bwd, noalloc


def _one_call(rows, n, dtype, rms, seed):
    lib, fwd, bwd, noalloc = _entry_points()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    x = (torch.randn(rows, n, device="cuda", generator=g) * 1.5 + 0.3).to(dtype)
    dy = torch.randn(rows, n, device="cuda", generator=g).to(dtype)
    gamma = torch.rand(n, device="cuda", generator=g) + 0.5
    is_bf16 = 1 if dtype == torch.bfloat16 else 0
    y = torch.empty_like(x)
    mean = torch.empty(rows, device="cuda")
    rstd = torch.empty(rows, device="cuda")
    assert fwd(x.data_ptr(), gamma.data_ptr(), None, y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, n, 1e-6, is_bf16, 0, rms, stream) == 0
    parts = lib.rb200_layer_norm_bwd_noalloc_parts()
    # regular entry point: scratch from the caller
    dx_ref = torch.empty_like(x)
    scratch = torch.empty(2 * parts * n, device="cuda")
    dg_ref = torch.empty(n, device="cuda")
    db_ref = torch.empty(n, device="cuda")
    assert bwd(x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx_ref.data_ptr(), scratch.data_ptr(),
               dg_ref.data_ptr(), db_ref.data_ptr(), rows, n, parts, is_bf16, 0, rms, stream) == 0
    # allocation-free entry point: outputs only
    dx = torch.empty_like(x)
    dg = torch.empty(n, device="cuda")
    db = torch.empty(n, device="cuda")
    torch.cuda.synchronize()
    mem_before = torch.cuda.memory_allocated()
    st = noalloc(x.data_ptr(), dy.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dg.data_ptr(), db.data_ptr(),
                 rows, n, is_bf16, 0, rms, stream)
    assert st == 0, lib.rb200_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == mem_before
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(dx.float(), dx_ref.float(), atol=tol, rtol=tol)
    torch.testing.assert_close(dg, dg_ref, atol=tol, rtol=tol)
    torch.testing.assert_close(db, db_ref, atol=tol, rtol=tol)
    # and against plain torch in fp32
    x32 = x.float().requires_grad_(True)
    g32 = gamma.clone().requires_grad_(True)
    if rms:
        yr = x32 * torch.rsqrt(x32.square().mean(-1, keepdim=True) + 1e-6) * g32
    else:
        yr = torch.nn.functional.layer_norm(x32, (n,), g32, None, 1e-6)
    yr.backward(dy.float())
    tol2 = 8e-2 if dtype == torch.bfloat16 else 1e-3
    torch.testing.assert_close(dx.float(), x32.grad, atol=tol2, rtol=tol2)
    torch.testing.assert_close(dg, g32.grad, atol=tol2 * max(1.0, rows ** 0.5), rtol=tol2)


@gpu
def test_no_alloc_layer_norm_bwd_two_calls_in_a_row():
    _one_call(rows=777, n=512, dtype=torch.bfloat16, rms=0, seed=11)
    _one_call(rows=64, n=2048, dtype=torch.float32, rms=0, seed=12)
    _one_call(rows=3, n=8, dtype=torch.bfloat16, rms=1, seed=13)


@gpu
def test_no_alloc_rejects_sizes_beyond_the_maximum():
    lib, fwd, bwd, noalloc = _entry_points()
    max_n = lib.rb200_layer_norm_bwd_noalloc_max_n()
    x = torch.zeros(2, max_n + 8, device="cuda")
    st = noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                 2, max_n + 8, 0, 0, 0, torch.cuda.current_stream().cuda_stream)
    assert st != 0
    assert b"not supported" in lib.rb200_last_error()
