"""The allocation-free C entry point (csrc/kernels/dq_noalloc.h), called through its exported
symbol the way a non-PyTorch host would, against the regular operator.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  Two calls in a row check that the shared scratch array needs no clearing between
calls."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from dynamiq_sigcomm_artifact_b200.ops import build

    lib = ctypes.CDLL(str(build.lib_path()))
    lib.dq_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    lib.dq_rmsnorm_bwd_noalloc.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 3 + [ctypes.c_void_p]
    lib.dq_noalloc_strerror.restype = ctypes.c_char_p
    lib.dq_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_rmsnorm_backward_matches_operator(dtype):
    from dynamiq_sigcomm_artifact_b200 import ops

    dq = ops.require()
    lib = _lib()
    torch.manual_seed(0)
    side = torch.cuda.Stream()
    # every chunk-count branch of the dispatcher (hidden / 256 rounded up: 8, 1, 2, 3, 5 -> 6, 7 -> 8, 4); each
    # call after the first reuses the scratch the previous one left dirty; one call runs on a side stream
    for rows, hidden in [(4096, 2048), (77, 136), (33, 512), (50, 768), (19, 1280), (41, 1792), (600, 1024)]:
        x = torch.randn(rows, hidden, device="cuda").to(dtype)
        dy = torch.randn(rows, hidden, device="cuda").to(dtype)
        w = torch.randn(hidden, device="cuda")
        _, _, rstd = dq.norm_fwd(x, w, None, 1e-5, True)
        dx_ref, dw_ref, _ = dq.norm_bwd(dy, x, w, torch.empty(0, device="cuda"), rstd, True)
        dx = torch.empty_like(x)
        dw = torch.empty(hidden, device="cuda")
        torch.cuda.synchronize()
        stream = side.cuda_stream if hidden == 768 else torch.cuda.current_stream().cuda_stream
        rc = lib.dq_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                        dw.data_ptr(), rows, hidden, int(dtype == torch.bfloat16), stream)
        assert rc == 0, lib.dq_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)  # same kernel, same arithmetic
        tol = 2e-3
        assert torch.allclose(dw, dw_ref, atol=tol * max(1.0, float(dw_ref.abs().max())), rtol=tol)
        # and against plain PyTorch in fp32, so that this test stands without the other operator
        xf, dyf = x.float().requires_grad_(True), dy.float()
        wf = w.clone().requires_grad_(True)
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        y.backward(dyf)
        t16 = 3e-2 if dtype == torch.bfloat16 else 2e-4
        assert torch.allclose(dx.float(), xf.grad, atol=t16 * float(xf.grad.abs().max()), rtol=t16)
        assert torch.allclose(dw, wf.grad, atol=t16 * max(1.0, float(wf.grad.abs().max())), rtol=t16)


def test_noalloc_rejects_oversize_and_bad_arguments():
    lib = _lib()
    x = torch.zeros(8, 4096, device="cuda")
    w = torch.zeros(4096, device="cuda")
    r = torch.zeros(8, device="cuda")
    rc = lib.dq_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), r.data_ptr(), x.data_ptr(), w.data_ptr(),
                                    8, 4096, 0, None)
    assert rc == -1 and b"2048" in lib.dq_noalloc_strerror(rc)
    assert lib.dq_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), r.data_ptr(), x.data_ptr(),
                                      w.data_ptr(), 0, 2048, 0, None) == -2
    assert lib.dq_rmsnorm_bwd_noalloc(None, x.data_ptr(), w.data_ptr(), r.data_ptr(), x.data_ptr(), w.data_ptr(),
                                      8, 2048, 0, None) == -3
