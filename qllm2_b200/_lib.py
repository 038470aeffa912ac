"""ctypes binding of libqllm2_pam_b200.so (the C ABI declared in include/qllm2_pam.h).

There is no CPU fallback: if the library is missing or an entry point reports an error the
caller gets a Python exception.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libqllm2_pam_b200.so")

QPAM_F32, QPAM_BF16 = 0, 1
MAX_STATES = 4

c_void_p, c_int32, c_int64, c_size_t, c_float = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float


class ScanArgs(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p),
        ("gamma", c_void_p), ("coef", c_void_p), ("s0", c_void_p), ("cu_seqlens", c_void_p),
        ("y", c_void_p), ("s_final", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("B", c_int32), ("H", c_int32), ("T", c_int32), ("d", c_int32), ("K", c_int32), ("S", c_int32),
        ("chunk", c_int32), ("io_dtype", c_int32),
        ("q_scale", c_float), ("gamma_eps", c_float),
    ]


class CEArgs(C.Structure):
    _fields_ = [
        ("h", c_void_p), ("w", c_void_p), ("targets", c_void_p), ("mask", c_void_p),
        ("N", c_int64), ("V", c_int64), ("v_offset", c_int64),
        ("F", c_int32), ("io_dtype", c_int32),
        ("ignore_index", c_int64),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


# name -> (restype, argtypes); every symbol declared in include/qllm2_pam.h
class FrontArgs(C.Structure):
    _fields_ = [
        ("qkv", c_void_p), ("dt", c_void_p), ("pg", c_void_p), ("phase", c_void_p), ("score", c_void_p),
        ("ld_qkv", c_int64), ("ld_dt", c_int64), ("ld_pg", c_int64), ("ld_phase", c_int64), ("ld_score", c_int64),
        ("dt_bias", c_void_p), ("state_dt_offset", c_void_p), ("rope", c_void_p), ("positions", c_void_p),
        ("rope_len", c_int64), ("offset", c_int64),
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("gamma", c_void_p), ("coef", c_void_p),
        ("gamma_floor", c_float), ("q_scale", c_float),
        ("B", c_int32), ("T", c_int32), ("H", c_int32), ("d", c_int32), ("K", c_int32), ("io_dtype", c_int32),
    ]


SIGNATURES = {
    "qpam_scan_workspace_bytes": (c_size_t, [C.POINTER(ScanArgs), c_int32]),
    "qpam_scan_fwd": (c_int32, [C.POINTER(ScanArgs), c_void_p]),
    "qpam_scan_fwd_tokens": (c_int32, [C.POINTER(ScanArgs), c_void_p]),
    "qpam_scan_fwd_static": (c_int32, [C.POINTER(ScanArgs), c_void_p]),
    "qpam_scan_bwd": (c_int32, [C.POINTER(ScanArgs), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_int32, c_void_p]),
    "qpam_scan_bwd_accumulate": (c_int32, [C.POINTER(ScanArgs), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int32, c_void_p]),
    "qpam_scan_fwd_states": (c_int32, [C.POINTER(ScanArgs), c_void_p, c_void_p]),
    "qpam_scan_bwd_state": (c_int32, [C.POINTER(ScanArgs), c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int32, c_void_p]),
    "qpam_decode_step": (c_int32, [c_void_p, c_int32, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                   c_int32, c_void_p]),
    "qpam_pool_store": (c_int32, [c_void_p, c_int32, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_int32,
                                  c_int32, c_int32, c_int32, c_void_p]),
    "qpam_ce_workspace_bytes": (c_size_t, [C.POINTER(CEArgs), c_int32]),
    "qpam_ce_partial": (c_int32, [C.POINTER(CEArgs), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "qpam_ce_finalize": (c_int32, [C.POINTER(CEArgs), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "qpam_ce_bwd": (c_int32, [C.POINTER(CEArgs), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "qpam_ce_bwd_overlap": (c_int32, [C.POINTER(CEArgs), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p]),
    "qpam_head_argmax": (c_int32, [C.POINTER(CEArgs), c_void_p, c_void_p, c_void_p]),
    "qpam_head_logits": (c_int32, [C.POINTER(CEArgs), c_void_p, c_int64, c_void_p]),
    "qpam_sample_workspace_bytes": (c_size_t, [c_int32, c_int32]),
    "qpam_sample_logits": (c_int32, [c_void_p, c_int32, c_int32, c_int32, c_int64, C.c_float, c_int32, C.c_float,
                                     C.c_float, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_void_p, c_int32,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "qpam_cnorm_fwd": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_int64, c_int32, C.c_float, c_void_p]),
    "qpam_cnorm_bwd": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_int64,
                                 c_int32, C.c_float, c_void_p]),
    "qpam_modact_fwd": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "qpam_modact_bwd": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int32, c_int64, c_int32, c_void_p]),
    "qpam_cgu_gate_fwd": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_void_p, c_int64, c_int32, c_void_p]),
    "qpam_cgu_gate_bwd": (c_int32, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int32, c_void_p, c_int64,
                                    c_void_p, c_int64, c_int64, c_int32, c_void_p]),
    "qpam_pam_prep_fwd": (c_int32, [c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "qpam_pam_prep_bwd": (c_int32, [c_void_p, c_int32, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "qpam_state_combine_fwd": (c_int32, [C.POINTER(c_void_p), c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int32, c_void_p]),
    "qpam_state_combine_tokens_fwd": (c_int32, [C.POINTER(c_void_p), c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                                c_int32, c_int32, c_void_p]),
    "qpam_state_combine_tokens_bwd": (c_int32, [C.POINTER(c_void_p), c_void_p, c_void_p, C.POINTER(c_void_p), c_void_p, c_int32,
                                                c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p]),
    "qpam_state_combine_bwd": (c_int32, [C.POINTER(c_void_p), c_void_p, c_void_p, C.POINTER(c_void_p), c_void_p, c_int32,
                                         c_int32, c_int64, c_int32, c_void_p]),
    "qpam_act_gate_packed_fwd": (c_int32, [c_void_p, c_int64, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "qpam_residual_cnorm_fwd": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64,
                                          c_int32, C.c_float, c_void_p]),
    "qpam_pam_front_fwd": (c_int32, [C.POINTER(FrontArgs), c_void_p]),
    "qpam_scaled_residual_fwd": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, c_void_p, c_void_p, c_int64, c_void_p]),
    "qpam_scaled_residual_bwd": (c_int32, [c_void_p, c_int32, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32,
                                           c_int64, c_void_p]),
    "qpam_block_weight_fwd": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_int32, c_int32, c_int32, c_void_p]),
    "qpam_block_weight_bwd": (c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p]),
    "qpam_pam_gates_fwd": (c_int32, [c_void_p] * 6 + [C.c_float] + [c_void_p] * 3 + [c_int32] * 4 + [c_void_p]),
    "qpam_pam_gates_bwd": (c_int32, [c_void_p] * 6 + [C.c_float] + [c_void_p] * 8 + [c_int32] * 5 + [c_void_p]),
    "qpam_cmagnitude_fwd": (c_int32, [c_void_p, c_int32, c_void_p, c_int64, c_void_p]),
    "qpam_cmagnitude_bwd": (c_int32, [c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p]),
    "qpam_launch_count": (C.c_longlong, []),
    "qpam_profile_begin": (c_int32, [c_void_p]),
    "qpam_profile_end": (c_int32, [C.c_char_p, c_size_t]),
    "qpam_device_status": (c_int32, [C.POINTER(c_int32), c_int32]),
    "qpam_selftest_wait_expiry": (c_int32, [c_int64, c_void_p]),
    "qpam_last_error": (C.c_char_p, []),
    "qpam_version": (C.c_char_p, []),
}

_lib = None


class QPamError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise QPamError(
                f"{LIB_PATH} is missing: build it with `python -m qllm2_b200.build` "
                "(there is no CPU or PyTorch fallback for the PAM kernels)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().qpam_last_error().decode("utf-8", "replace")
        raise QPamError(f"{what} failed with code {rc}: {msg}")


def dtype_code(dtype) -> int:
    import torch
    if dtype == torch.float32:
        return QPAM_F32
    if dtype == torch.bfloat16:
        return QPAM_BF16
    raise QPamError(f"unsupported dtype {dtype}: the PAM kernels take float32 or bfloat16")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def launch_count() -> int:
    return int(lib().qpam_launch_count())


def profile_begin() -> None:
    check(lib().qpam_profile_begin(stream_ptr()), "qpam_profile_begin")


def profile_end() -> dict:
    """{kernel name: (launches, total_ms)} since profile_begin()."""
    buf = C.create_string_buffer(1 << 16)
    check(lib().qpam_profile_end(buf, len(buf)), "qpam_profile_end")
    out = {}
    for line in buf.value.decode().splitlines():
        name, cnt, ms = line.rsplit(" ", 2)
        out[name] = (int(cnt), float(ms))
    return out


def device_status(clear: bool = True) -> int:
    """0 when every kernel so far completed its on-device handshakes and accepted its descriptors
    (2xx: a bounded wait gave up; 301: bad cu_seqlens).  Synchronises the device."""
    v = c_int32(0)
    check(lib().qpam_device_status(C.byref(v), 1 if clear else 0), "qpam_device_status")
    return int(v.value)


def raise_on_device_error(where: str = "") -> None:
    """Read (and clear) the device status word; raise QPamError when a kernel reported a failure.  Meant for
    points where the caller synchronises anyway: after an optimizer step, after a decode step's host read."""
    code = device_status(clear=True)
    if code != 0:
        what = "a packed scan was given an invalid cu_seqlens descriptor" if code == 301 else \
            "a bounded on-device wait gave up: the results of that launch are invalid"
        raise QPamError(f"device status {code}{' in ' + where if where else ''}: {what}")
