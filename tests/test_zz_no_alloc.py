"""The allocation-free forward scan (qpam_scan_fwd_static) against the regular entry point.

Hosts that may not allocate device memory (all of it already belongs to a server's pool, or a
latency-critical loop forbids cudaMalloc) call the variant whose workspace is a fixed array inside
the library.  Both entry points run the same kernels, so outputs must agree bit for bit -- on two
calls in a row with different inputs, since the shared array keeps the previous call's contents.
This file sorts last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes as C

import pytest
import torch

from qllm2_b200 import _lib, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _args(q, k, v, gamma, y, s_final, ws):
    B, H, T, d = q.shape[:4]
    a = _lib.ScanArgs()
    a.q, a.k, a.v, a.gamma = q.data_ptr(), k.data_ptr(), v.data_ptr(), gamma.data_ptr()
    a.y, a.s_final = y.data_ptr(), s_final.data_ptr()
    a.B, a.H, a.T, a.d, a.K, a.S = B, H, T, d, 1, B
    a.chunk, a.io_dtype = 64, _lib.dtype_code(q.dtype)
    a.q_scale, a.gamma_eps = d ** -0.5, 1e-6
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


def _both(lib, seed, shape, dtype):
    B, H, T, d = shape
    inp = synthetic.scan_inputs(B, H, T, d, seed=seed, dtype=dtype)
    q, k, v = inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV)
    gamma = inp.gamma.to(DEV).unsqueeze(0).contiguous()
    outs = []
    for static in (False, True):
        y = torch.full_like(q, float("nan"))
        s_final = torch.full((1, B, H, d, d, 2), float("nan"), device=DEV)
        if static:
            a = _args(q, k, v, gamma, y, s_final, None)
            rc = lib.qpam_scan_fwd_static(C.byref(a), _lib.stream_ptr())
        else:
            a = _args(q, k, v, gamma, y, s_final, None)
            ws = torch.empty(lib.qpam_scan_workspace_bytes(C.byref(a), 0), dtype=torch.uint8, device=DEV)
            a = _args(q, k, v, gamma, y, s_final, ws)
            rc = lib.qpam_scan_fwd(C.byref(a), _lib.stream_ptr())
        _lib.check(rc, "scan forward")
        torch.cuda.synchronize()
        outs.append((y, s_final))
    return outs


def test_static_scratch_matches_regular_entry_point_twice():
    lib = _lib.lib()
    for seed, shape, dtype in ((0, (2, 4, 512, 32), torch.float32), (1, (1, 3, 200, 64), torch.bfloat16)):
        (y0, s0), (y1, s1) = _both(lib, seed, shape, dtype)
        assert not torch.isnan(y1.float()).any() and not torch.isnan(s1).any()
        assert torch.equal(y0, y1), "y differs between qpam_scan_fwd and qpam_scan_fwd_static"
        assert torch.equal(s0, s1), "s_final differs between qpam_scan_fwd and qpam_scan_fwd_static"


def test_static_scratch_rejects_oversized_shapes():
    lib = _lib.lib()
    B, H, T, d = 64, 16, 4096, 64      # needs ~2 GB of workspace, far above the built-in array
    a = _lib.ScanArgs()
    dummy = torch.zeros(8, device=DEV)
    a.q = a.k = a.v = a.gamma = a.y = dummy.data_ptr()
    a.B, a.H, a.T, a.d, a.K, a.S = B, H, T, d, 1, B
    a.io_dtype, a.q_scale, a.gamma_eps = 1, 0.125, 1e-6
    assert lib.qpam_scan_fwd_static(C.byref(a), _lib.stream_ptr()) == 2
    assert b"built-in scratch" in lib.qpam_last_error()
