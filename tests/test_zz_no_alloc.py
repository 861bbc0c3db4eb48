"""The allocation-free RMSNorm backward, called the way a framework-less host would call it.

Some users of the kernel library own nothing but the input and output buffers they were handed
and cannot obtain more device memory while they run: for example a worker that has already given
every free byte of HBM to the rollout KV cache, or a small C program with a fixed memory budget.
``msrl_rmsnorm_bwd_noalloc`` serves them by keeping the partial weight-gradient sums in a scratch
array inside the library.  This test loads the shared library directly, calls the exported C
symbol with raw device pointers -- twice in a row, with different shapes, so that the second call
finds the scratch array full of the first call's leftovers -- and checks both results against the
regular entry point (``ops.rmsnorm_bwd``, caller-provided scratch) within the tolerance the other
RMSNorm tests use.  An oversized hidden dimension must be refused without launching anything.
"""
import ctypes

import pytest
import torch

from mindspeed_rl_b200 import ops
from mindspeed_rl_b200.ops import _lib

pytestmark = pytest.mark.gpu

CUDA_ERROR_INVALID_VALUE = 1


def _entry():
    lib = ctypes.CDLL(str(_lib.lib_path()))
    fn = lib.msrl_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
    return fn


def _run_case(fn, rows, h, with_residual, seed):
    torch.manual_seed(seed)
    dev = "cuda"
    x = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(h, device=dev)).bfloat16()
    dy = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    dres = torch.randn(rows, h, device=dev, dtype=torch.bfloat16) if with_residual else None
    _, rstd, _ = ops.rmsnorm_fwd(x, w, 1e-6)
    # regular entry point (scratch supplied by the Python front-end)
    dw_ref = torch.full((h,), 0.5, device=dev, dtype=torch.float32)
    dx_ref = ops.rmsnorm_bwd(dy, x, w, rstd, dw_ref, dres=dres)
    # allocation-free entry point through its C symbol; outputs are pre-allocated by the caller
    dx = torch.empty_like(x)
    dw = torch.full((h,), 0.5, device=dev, dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
            dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(), None, 1, rows, h,
            stream)
    assert rc == 0, f"msrl_rmsnorm_bwd_noalloc returned CUDA error {rc}"
    torch.cuda.synchronize()
    err_dx = (dx.float() - dx_ref.float()).abs()
    assert bool((err_dx <= 3e-2 + 3e-2 * dx_ref.float().abs()).all()), err_dx.max()
    err_dw = (dw - dw_ref).abs()
    assert bool((err_dw <= 5e-2 * rows ** 0.5 + 2e-2 * dw_ref.abs()).all()), err_dw.max()
    # the same outputs from the textbook fp32 formulation (not only from the sibling kernel)
    dx32, dw32 = _fp32_rmsnorm_bwd(dy, x, w, rstd, dres)
    err = (dx.float() - dx32).abs()
    assert bool((err <= 3e-2 + 3e-2 * dx32.abs()).all()), err.max()
    err = (dw - (0.5 + dw32)).abs()
    assert bool((err <= 5e-2 * rows ** 0.5 + 2e-2 * dw32.abs()).all()), err.max()
    # accumulate = 0 overwrites whatever the output held, and the bf16 gradient output works alone
    dw_over = torch.full((h,), 123.0, device=dev, dtype=torch.float32)
    dw16 = torch.full((h,), 7.0, device=dev, dtype=torch.bfloat16)
    dx2 = torch.empty_like(x)
    assert fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr() if dres is not None else None,
              dx2.data_ptr(), dw_over.data_ptr(), None, 0, rows, h, stream) == 0
    assert fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr() if dres is not None else None,
              dx2.data_ptr(), None, dw16.data_ptr(), 0, rows, h, stream) == 0
    torch.cuda.synchronize()
    tol = 5e-2 * rows ** 0.5 + 2e-2 * dw32.abs()
    assert bool(((dw_over - dw32).abs() <= tol).all())
    assert bool(((dw16.float() - dw32).abs() <= tol + 1e-2 * dw32.abs()).all())
    assert torch.equal(dx2, dx)


def _fp32_rmsnorm_bwd(dy, x, w, rstd, dres):
    """y = x * rstd * w  ->  dx = rstd * (g - x_hat * mean(g * x_hat)) (+ dres), dw = sum_rows dy * x_hat."""
    xf, g = x.float(), dy.float() * w.float()
    x_hat = xf * rstd.float().unsqueeze(-1)
    dx = rstd.float().unsqueeze(-1) * (g - x_hat * (g * x_hat).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    return dx, (dy.float() * x_hat).sum(0)


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    fn = _entry()
    # first call: wide rows, many of them (fills the scratch); second call: a different, smaller
    # problem that must not be disturbed by what the first call left behind
    _run_case(fn, rows=700, h=3584, with_residual=True, seed=0)
    _run_case(fn, rows=33, h=1024, with_residual=False, seed=1)


def test_noalloc_rmsnorm_bwd_rejects_oversized_rows():
    fn = _entry()
    h = 8192 + 8
    t = torch.zeros(2, h, device="cuda", dtype=torch.bfloat16)
    r = torch.ones(2, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), t[0].data_ptr(), r.data_ptr(), None, t.data_ptr(), None, None, 0, 2, h,
            torch.cuda.current_stream().cuda_stream)
    assert rc == CUDA_ERROR_INVALID_VALUE


def test_noalloc_rmsnorm_bwd_rejects_bad_pointers_without_launching():
    """A null or misaligned buffer is answered with an error code on the host; nothing runs on the GPU."""
    fn = _entry()
    h = 1024
    t = torch.zeros(4, h + 8, device="cuda", dtype=torch.bfloat16)
    good, odd = t[:, :h], t.view(-1)[1:1 + 2 * h].view(2, h)       # `odd` starts 2 bytes past a 16-byte boundary
    r = torch.ones(4, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(h, device="cuda")
    args = lambda dy, x, dx: (dy, x, w.data_ptr(), r.data_ptr(), None, dx, dw.data_ptr(), None, 0, 2, h, st)
    p = good.data_ptr()
    assert fn(*args(None, p, p)) == CUDA_ERROR_INVALID_VALUE
    assert fn(*args(p, None, p)) == CUDA_ERROR_INVALID_VALUE
    assert fn(*args(p, p, None)) == CUDA_ERROR_INVALID_VALUE
    assert fn(*args(odd.data_ptr(), p, p)) == CUDA_ERROR_INVALID_VALUE
    assert fn(p, p, w.data_ptr(), None, None, p, dw.data_ptr(), None, 0, 2, h, st) == CUDA_ERROR_INVALID_VALUE
    torch.cuda.synchronize()
