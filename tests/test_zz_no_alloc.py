"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some users of this library run where device allocation is off limits while work is in flight (a serving process
with a frozen memory pool, a plugin whose host owns the device heap).  For them the library exports
``uttt_rms_norm_bwd_noalloc``: same result as the regular backward, with its scratch in a fixed array inside the
library.  This test loads the shared object with ctypes, calls the symbol twice in a row on caller-owned buffers
and checks both results against the regular (allocating) entry point and against the fp32 PyTorch statement of the
backward.  This file sorts last on purpose.
"""
import ctypes
import gc
import glob
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import uttt_b200.ops as ops_pkg
    from uttt_b200.ops._ext import load
    load(required=True)                                  # torch's libraries are resident before dlopen
    path = sorted(glob.glob(os.path.join(os.path.dirname(ops_pkg.__file__), "_C*.so")))[-1]
    lib = ctypes.CDLL(path)
    fn = lib.uttt_rms_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    return fn


def _fp32_backward(dy, x, w, eps=1e-6):
    """dx, dw of y = x * rsqrt(mean(x^2) + eps) * w in fp32 autograd."""
    xf = x.detach().float().requires_grad_(True)
    wf = None if w is None else w.detach().float().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if wf is not None:
        y = y * wf
    grads = torch.autograd.grad(y, [xf] + ([wf] if wf is not None else []), dy.float())
    return grads[0], (grads[1] if wf is not None else None)


def _rel_fro(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 0), (torch.float32, 1)])
def test_no_alloc_rms_norm_backward_matches_regular_entry_point(dtype, code):
    from uttt_b200.ops._ext import load
    ext = load(required=True)
    fn = _lib()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    stream = torch.cuda.current_stream(dev)
    # calls in a row share the scratch; the shapes cover one block (rows < 4), the widest vector path (d > 2048),
    # a width that is a multiple of 8 but not of 64, and a parameter-free norm (w = NULL)
    cases = [(1000, 1536, True), (333, 384, True), (3, 4096, True), (37, 2056, True), (1, 512, True), (64, 768, False)]
    for call, (rows, d, affine) in enumerate(cases):
        x = torch.randn(rows, d, device=dev, dtype=dtype)
        dy = torch.randn(rows, d, device=dev, dtype=dtype)
        w = (torch.randn(d, device=dev) * 0.1 + 1).to(dtype) if affine else None
        _, rstd = ext.rms_norm_fwd(x, w, 1e-6)
        want_dx, want_dw = ext.rms_norm_bwd(dy, x, w, rstd)
        ref_dx, ref_dw = _fp32_backward(dy, x, w)
        ref_dx_cpu = ref_dx.cpu()
        dx = torch.empty_like(x)                         # caller-owned outputs
        dw = torch.full((d,), float("nan"), device=dev, dtype=torch.float32)
        del ref_dx                                       # the fp32 oracle's graph is gone before the measurement
        gc.collect()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        rc = fn(dy.data_ptr(), x.data_ptr(), None if w is None else w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                dw.data_ptr() if affine else None, rows, d, code, stream.cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0, (call, rc)
        assert torch.cuda.memory_allocated(dev) == before
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        torch.testing.assert_close(dx.float(), want_dx.float(), atol=tol, rtol=tol)
        assert _rel_fro(dx.cpu(), ref_dx_cpu) < (6e-3 if dtype == torch.bfloat16 else 1e-5), (call, rows, d)
        if affine:
            # both entry points accumulate the weight gradient in fp32: they agree far inside bf16 rounding of dy
            torch.testing.assert_close(dw, want_dw.float(), atol=1e-2, rtol=1e-3)
            assert _rel_fro(dw, ref_dw) < (1e-2 if dtype == torch.bfloat16 else 1e-5), (call, _rel_fro(dw, ref_dw))
        else:
            assert bool(torch.isnan(dw).all())           # not written for a parameter-free norm


def test_no_alloc_entry_point_rejects_oversize_and_bad_arguments():
    fn = _lib()
    t = torch.zeros(8, 8192, device="cuda")
    r = torch.zeros(8, device="cuda")
    assert fn(t.data_ptr(), t.data_ptr(), None, r.data_ptr(), t.data_ptr(), None, 8, 8192, 1, None) == 2
    assert fn(t.data_ptr(), t.data_ptr(), None, r.data_ptr(), t.data_ptr(), None, 8, 4100, 1, None) == 1
    assert fn(None, t.data_ptr(), None, r.data_ptr(), t.data_ptr(), None, 8, 4096, 1, None) == 1
