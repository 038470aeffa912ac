"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from qllm2_b200 import _lib, build
    build.build()
    return _lib.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "qllm2_pam.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qpam_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    from qllm2_b200 import _lib
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/qllm2_pam.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)
    assert b"sm_100a" in lib.qpam_version()


def test_argument_errors_do_not_touch_the_gpu(lib):
    from qllm2_b200 import _lib
    a = _lib.ScanArgs()
    a.d, a.K, a.B, a.H, a.T, a.S = 48, 1, 1, 1, 8, 1
    assert lib.qpam_scan_fwd(C.byref(a), None) == 1
    assert b"head dim" in lib.qpam_last_error()
    a.d, a.K = 64, 9
    assert lib.qpam_scan_fwd(C.byref(a), None) == 1
    assert b"K=9" in lib.qpam_last_error()
    ce = _lib.CEArgs()
    assert lib.qpam_ce_partial(C.byref(ce), None, None, None, None, None) == 1
    assert lib.qpam_decode_step(None, 0, 1, 1, 0, None, None, None, None, None, None, None, 1, 1, 64, 1, 0, None) == 1


def test_tensor_core_only_entry_points_refuse_other_inputs_without_a_launch(lib):
    """qpam_scan_fwd_states / qpam_scan_bwd_state / qpam_scan_bwd_accumulate / qpam_head_logits exist on the tensor-core
    path only: anything else is refused with QPAM_EUNSUPPORTED (4) or QPAM_EINVAL (1) and a message, before any CUDA
    call (the pointers below are fake and never dereferenced)."""
    from qllm2_b200 import _lib
    fake = 1 << 20                     # non-null, 256-byte aligned
    a = _lib.ScanArgs()
    a.q = a.k = a.v = a.gamma = a.workspace = fake
    a.workspace_bytes = 1 << 30
    a.B, a.H, a.T, a.d, a.K, a.S = 1, 2, 256, 64, 3, 1
    a.io_dtype, a.q_scale, a.gamma_eps = _lib.QPAM_F32, 0.125, 1e-6
    assert lib.qpam_scan_fwd_states(C.byref(a), fake, None) == 4           # fp32 tokens
    assert b"tensor-core path" in lib.qpam_last_error()
    assert lib.qpam_scan_fwd_states(C.byref(a), None, None) == 1           # no output buffer
    a.io_dtype, a.K = _lib.QPAM_BF16, 1
    assert lib.qpam_scan_fwd_states(C.byref(a), fake, None) == 4           # one state: use qpam_scan_fwd
    a.K = 3
    assert lib.qpam_scan_bwd_state(C.byref(a), 3, fake, fake, fake, fake, fake, None, None, 0, None) == 1
    assert b"state 3" in lib.qpam_last_error()
    a.d = 32
    assert lib.qpam_scan_bwd_state(C.byref(a), 0, fake, fake, fake, fake, fake, None, None, 0, None) == 4
    a.K = 1
    assert lib.qpam_scan_bwd_accumulate(C.byref(a), fake, fake, fake, fake, fake, None, None, 1, None) == 4
    ce = _lib.CEArgs()
    ce.h = ce.w = fake
    ce.N, ce.V, ce.F, ce.io_dtype = 256, 50261, 1536, _lib.QPAM_F32
    assert lib.qpam_head_logits(C.byref(ce), fake, 50264, None) == 4        # fp32: the library GEMM's job
    ce.io_dtype = _lib.QPAM_BF16
    assert lib.qpam_head_logits(C.byref(ce), fake, 50261, None) == 1        # ld not a multiple of 8
    assert lib.qpam_head_logits(C.byref(ce), None, 50264, None) == 1


def test_workspace_sizes(lib):
    from qllm2_b200 import _lib
    a = _lib.ScanArgs()
    a.B, a.H, a.T, a.d, a.K, a.S = 2, 4, 512, 32, 1, 2
    fwd = lib.qpam_scan_workspace_bytes(C.byref(a), 0)
    bwd = lib.qpam_scan_workspace_bytes(C.byref(a), 1)
    slots = 2 * (512 // 64 + 1)
    assert fwd >= 4 * slots * 32 * 32 * 8
    assert bwd >= 2 * 4 * slots * 32 * 32 * 8 and bwd > fwd
    ce = _lib.CEArgs()
    ce.N, ce.V, ce.F, ce.io_dtype = 8192, 50261, 768, 1
    assert lib.qpam_ce_workspace_bytes(C.byref(ce), 1) > lib.qpam_ce_workspace_bytes(C.byref(ce), 0) > 0


def test_ops_fail_loudly_without_cuda():
    import torch
    from qllm2_b200 import _lib, ops
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    q = torch.zeros(1, 1, 8, 16, 2)
    with pytest.raises(_lib.QPamError):
        ops.pam_scan(q, q, q, torch.ones(1, 1, 8))


def test_wrappers_reject_inconsistent_tensors_before_any_launch():
    """Shape / dtype mismatches are caught in Python: the C ABI reads k and v through q's dtype, so a
    mismatch would otherwise read past the end of a buffer on the device."""
    import torch
    from qllm2_b200 import _lib, ops
    q = torch.zeros(1, 2, 8, 16, 2)
    with pytest.raises(_lib.QPamError):
        ops.pam_scan(q, q[:, :1], q, torch.ones(1, 2, 8))
    with pytest.raises(_lib.QPamError):
        ops.pam_scan(q, q, q, torch.ones(1, 2, 9))
    with pytest.raises(_lib.QPamError):
        ops.pam_scan(q, q, q, torch.ones(1, 2, 8), coef=torch.ones(1, 1, 2, 8))
