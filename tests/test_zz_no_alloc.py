"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory at the point where they need a kernel: a latency-critical
loop that may not touch the allocator, code running under another framework's memory pool, or a process with a fixed
device-memory budget.
``vlmt_rmsnorm_bwd_static`` serves them by keeping its scratch (per-block partial weight gradients) in a fixed
4.6 MiB array inside the library instead of a scratch tensor.  Here it is called twice in a row (the array is
shared between calls and keeps the previous call's contents) and both results are compared with the regular entry
point, which takes an allocated scratch tensor.  The file is named so that pytest collects it after every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from vlm_training_b200.ops import build

    lib = ctypes.CDLL(build.ext_path())
    fn = lib.vlmt_rmsnorm_bwd_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    return fn


def _case(rows, D, offset, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, D, device="cuda", generator=g).bfloat16()
    dy = torch.randn(rows, D, device="cuda", generator=g).bfloat16()
    w = (torch.randn(D, device="cuda", generator=g) * 0.3).bfloat16()
    dres = torch.randn(rows, D, device="cuda", generator=g).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    return x, dy, w, dres, rstd


def test_static_scratch_entry_matches_regular_entry_twice():
    from vlm_training_b200.ops import cuda as cu

    fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, D, offset) in enumerate([(777, 4096, 0), (300, 1152, 1)]):  # second call reuses the dirty scratch
        x, dy, w, dres, rstd = _case(rows, D, offset, seed=call)
        dx = torch.empty_like(x)
        dw = torch.full((D,), float("nan"), device="cuda")  # an output: the entry point must overwrite all of it
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), 0, rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                rows, D, offset, stream)
        assert rc == 0, f"vlmt_rmsnorm_bwd_static returned {rc}"
        dx_ref, dw_ref = cu._C.rmsnorm_bwd(dy, x, w, rstd, dres, bool(offset))
        torch.cuda.synchronize()
        torch.testing.assert_close(dx.float(), dx_ref.float(), atol=0.03, rtol=2e-2)
        torch.testing.assert_close(dw, dw_ref.float(), atol=0.5, rtol=2e-2)


@pytest.mark.parametrize("rows,D,w_fp32,with_dres", [(513, 8192, False, True), (260, 2048, True, True), (129, 4096, False, False),
                                                      (64, 1024, True, False)])
def test_static_scratch_entry_weight_types_widest_rows_and_no_residual(rows, D, w_fp32, with_dres):
    """fp32 norm weights, the widest supported row (D = 8192, the largest shared-memory request) and a call without the
    residual gradient, each against the regular entry point."""
    from vlm_training_b200.ops import cuda as cu

    fn = _lib()
    x, dy, w, dres, rstd = _case(rows, D, 0, seed=rows)
    w_arg = w.float() if w_fp32 else w
    dx = torch.empty_like(x)
    dw = torch.full((D,), float("nan"), device="cuda")
    rc = fn(dy.data_ptr(), x.data_ptr(), w_arg.data_ptr(), int(w_fp32), rstd.data_ptr(), dres.data_ptr() if with_dres else None,
            dx.data_ptr(), dw.data_ptr(), rows, D, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"vlmt_rmsnorm_bwd_static returned {rc}"
    dx_ref, dw_ref = cu._C.rmsnorm_bwd(dy, x, w_arg, rstd, dres if with_dres else None, False)
    torch.cuda.synchronize()
    torch.testing.assert_close(dx.float(), dx_ref.float(), atol=0.03, rtol=2e-2)
    torch.testing.assert_close(dw, dw_ref.float(), atol=0.5, rtol=2e-2)


def test_static_scratch_entry_without_rows_clears_dw():
    fn = _lib()
    D = 1024
    x = torch.zeros(1, D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(1, device="cuda")
    dw = torch.full((D,), float("nan"), device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x[0].data_ptr(), 0, rstd.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 0, D, 0,
            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and float(dw.abs().sum()) == 0.0


def test_static_scratch_entry_refuses_oversized_rows():
    fn = _lib()
    D = 8192 + 8
    x = torch.zeros(4, D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dw = torch.zeros(D, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x[0].data_ptr(), 0, rstd.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 4, D, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -1
