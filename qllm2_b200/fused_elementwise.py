"""Fused element-wise complex operators (forward and backward in one kernel pass each).

Same names, arguments and arithmetic as the reference's `v11/triton_kernels.py`
(`fused_complex_norm` :546, `fused_mod_swish` :552, `fused_mod_relu` :558, `fused_cgu_gate` :564; the
plain arithmetic they must match is `_pt_*` :489-519), on tensors laid out [..., C, 2].  `pam_prep`
covers the head split + rotary rotation + protect-gate scaling of the PAM layer's input stage
(`v11/model.py:271-350`).  CUDA tensors only: there is no PyTorch fallback in these functions.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import check, dtype_code, ptr, stream_ptr


def _autocast_dtype(t: torch.Tensor) -> torch.dtype:
    if t.is_cuda and torch.is_autocast_enabled("cuda"):
        return torch.get_autocast_dtype("cuda")
    return t.dtype


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.QPamError("the fused complex operators run on CUDA tensors only")


def _rows(t: torch.Tensor):
    """(tensor, N, C, row stride in scalars) of a [..., C, 2] tensor; copies only if rows are not uniform."""
    if t.dim() < 2 or t.shape[-1] != 2:
        raise _lib.QPamError(f"expected a [..., C, 2] tensor, got {tuple(t.shape)}")
    C = t.shape[-2]
    if C % 4:
        raise _lib.QPamError(f"the channel count must be a multiple of 4 (got {C})")
    if t.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.QPamError(f"unsupported dtype {t.dtype}")
    ok = t.stride(-1) == 1 and t.stride(-2) == 2 and t.data_ptr() % 16 == 0
    if ok and t.dim() > 2:
        ld = t.stride(-3)
        ok = ld >= 2 * C and ld % (16 // t.element_size()) == 0
        for i in range(t.dim() - 4, -1, -1):
            ok = ok and (t.shape[i] == 1 or t.stride(i) == t.stride(i + 1) * t.shape[i + 1])
    elif ok:
        ld = 2 * C
    if not ok:
        t = t.contiguous()
        ld = 2 * C
    N = t.numel() // (2 * C)
    return t, N, C, ld


def _param(p: torch.Tensor, C: int, name: str) -> torch.Tensor:
    if p.numel() != C:
        raise _lib.QPamError(f"{name} must have {C} entries, got {p.numel()}")
    return p.detach().float().contiguous()


# ------------------------------------------------------------------------------------ norm
class _ComplexNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, scale, eps, out_dtype):
        z = z.contiguous()
        D = z.shape[-2]
        N = z.numel() // (2 * D)
        sc = _param(scale, D, "scale")
        out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
        check(_lib.lib().qpam_cnorm_fwd(ptr(z), dtype_code(z.dtype), ptr(sc), ptr(out), dtype_code(out_dtype),
                                        N, D, float(eps), stream_ptr()), "qpam_cnorm_fwd")
        ctx.save_for_backward(z, scale)
        ctx.eps, ctx.out_dtype = eps, out_dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        z, scale = ctx.saved_tensors
        D = z.shape[-2]
        N = z.numel() // (2 * D)
        dout = dout.to(ctx.out_dtype).contiguous()
        P = max(4, min((N + 3) // 4 * 4, 148 * 16))
        part = torch.empty(P, D, dtype=torch.float32, device=z.device)
        dz = torch.empty_like(z)
        check(_lib.lib().qpam_cnorm_bwd(ptr(z), dtype_code(z.dtype), ptr(_param(scale, D, "scale")), ptr(dout),
                                        dtype_code(ctx.out_dtype), ptr(dz), ptr(part), P, N, D, float(ctx.eps),
                                        stream_ptr()), "qpam_cnorm_bwd")
        return dz, part.sum(0).to(scale.dtype).view_as(scale), None, None


def fused_complex_norm(z: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """z / (|z|+1e-8) * (|z| / rms) * scale over the channel axis of [..., D, 2]
    (v11/triton_kernels.py:489-494).  Under bf16 autocast the result is bf16 (the next operator is a
    projection that would cast it anyway); otherwise it has z's dtype."""
    _require_cuda(z, scale)
    if z.dim() < 2 or z.shape[-1] != 2 or z.shape[-2] % 4 or z.shape[-2] > 3072:
        raise _lib.QPamError(f"fused_complex_norm: expected [..., D, 2] with D a multiple of 4 up to 3072, got {tuple(z.shape)}")
    if z.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.QPamError(f"unsupported dtype {z.dtype}")
    out_dtype = _autocast_dtype(z)
    if out_dtype not in (torch.float32, torch.bfloat16) or (z.dtype == torch.bfloat16 and out_dtype == torch.float32):
        out_dtype = z.dtype
    return _ComplexNormFn.apply(z, scale, eps, out_dtype)


# ------------------------------------------------------------------------------------ activations
class _ModActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, bias, beta):
        z = z.contiguous()
        C = z.shape[-2]
        N = z.numel() // (2 * C)
        out = torch.empty_like(z)
        b = _param(bias, C, "bias")
        be = None if beta is None else _param(beta, C, "beta")
        check(_lib.lib().qpam_modact_fwd(ptr(z), dtype_code(z.dtype), ptr(b), ptr(be), ptr(out), N, C, stream_ptr()),
              "qpam_modact_fwd")
        ctx.save_for_backward(z, bias, beta)
        return out

    @staticmethod
    def backward(ctx, dout):
        z, bias, beta = ctx.saved_tensors
        C = z.shape[-2]
        N = z.numel() // (2 * C)
        dout = dout.to(z.dtype).contiguous()
        P = max(1, min(N, 1024))        # rows of partial parameter gradients = row partitions of the launch
        pb = torch.empty(P, C, dtype=torch.float32, device=z.device)
        pe = None if beta is None else torch.empty(P, C, dtype=torch.float32, device=z.device)
        dz = torch.empty_like(z)
        check(_lib.lib().qpam_modact_bwd(ptr(z), dtype_code(z.dtype), ptr(_param(bias, C, "bias")),
                                         None if beta is None else ptr(_param(beta, C, "beta")), ptr(dout), ptr(dz),
                                         ptr(pb), ptr(pe), P, N, C, stream_ptr()), "qpam_modact_bwd")
        dbias = pb.sum(0).to(bias.dtype).view_as(bias)
        dbeta = None if beta is None else pe.sum(0).to(beta.dtype).view_as(beta)
        return dz, dbias, dbeta


def _check_act_input(z, name):
    _require_cuda(z)
    if z.dim() < 2 or z.shape[-1] != 2 or z.shape[-2] % 4:
        raise _lib.QPamError(f"{name}: expected [..., C, 2] with C a multiple of 4, got {tuple(z.shape)}")
    if z.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.QPamError(f"unsupported dtype {z.dtype}")


def fused_mod_swish(z: torch.Tensor, bias: torch.Tensor, beta: torch.Tensor) -> torch.Tensor:
    """z/(|z|+1e-8) * |z| sigmoid(beta |z| + bias)   (v11/triton_kernels.py:497-501)."""
    _check_act_input(z, "fused_mod_swish")
    _require_cuda(bias, beta)
    return _ModActFn.apply(z, bias, beta)


def fused_mod_relu(z: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """z/(|z|+1e-8) * relu(|z| + bias)   (v11/triton_kernels.py:504-508)."""
    _check_act_input(z, "fused_mod_relu")
    _require_cuda(bias)
    return _ModActFn.apply(z, bias, None)


# ------------------------------------------------------------------------------------ gated unit
class _CguGateFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        gate, N, C, ldg = _rows(gate)
        up, Nu, Cu, ldu = _rows(up)
        out = torch.empty(*gate.shape[:-2], C, 2, dtype=gate.dtype, device=gate.device)
        check(_lib.lib().qpam_cgu_gate_fwd(ptr(gate), ldg, ptr(up), ldu, dtype_code(gate.dtype), ptr(out), N, C,
                                           stream_ptr()), "qpam_cgu_gate_fwd")
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, dout):
        gate, up = ctx.saved_tensors
        gate, N, C, ldg = _rows(gate)
        up, _, _, ldu = _rows(up)
        dout = dout.to(gate.dtype).contiguous()
        # two dense tensors: the consumers (the activation's backward, the projections' GEMMs) take them as they
        # are; halves of one buffer would be copied by the first consumer that needs dense rows
        dgate = torch.empty(*gate.shape[:-2], C, 2, dtype=gate.dtype, device=gate.device)
        dup = torch.empty_like(dgate)
        check(_lib.lib().qpam_cgu_gate_bwd(ptr(gate), ldg, ptr(up), ldu, ptr(dout), dtype_code(gate.dtype),
                                           ptr(dgate), 2 * C, ptr(dup), 2 * C, N, C, stream_ptr()),
              "qpam_cgu_gate_bwd")
        return dgate, dup


class _CguGatePackedFn(torch.autograd.Function):
    """gate and up as the two channel halves of one [..., 2C, 2] tensor; the gradient comes back packed."""

    @staticmethod
    def forward(ctx, gu):
        gu = gu.contiguous()
        C = gu.shape[-2] // 2
        N = gu.numel() // (4 * C)
        out = torch.empty(*gu.shape[:-2], C, 2, dtype=gu.dtype, device=gu.device)
        base = gu.data_ptr()
        check(_lib.lib().qpam_cgu_gate_fwd(base, 4 * C, base + 2 * C * gu.element_size(), 4 * C, dtype_code(gu.dtype),
                                           ptr(out), N, C, stream_ptr()), "qpam_cgu_gate_fwd")
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        C = gu.shape[-2] // 2
        N = gu.numel() // (4 * C)
        dout = dout.to(gu.dtype).contiguous()
        dgu = torch.empty_like(gu)
        base, dbase, off = gu.data_ptr(), dgu.data_ptr(), 2 * C * gu.element_size()
        check(_lib.lib().qpam_cgu_gate_bwd(base, 4 * C, base + off, 4 * C, ptr(dout), dtype_code(gu.dtype), dbase, 4 * C,
                                           dbase + off, 4 * C, N, C, stream_ptr()), "qpam_cgu_gate_bwd")
        return dgu


def fused_cgu_gate(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """gate/(|gate|+1e-8) * up * sigmoid(|gate|), complex product   (v11/triton_kernels.py:511-519)."""
    _require_cuda(gate, up)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise _lib.QPamError(f"fused_cgu_gate: gate {tuple(gate.shape)} {gate.dtype} and up {tuple(up.shape)} {up.dtype} differ")
    _check_act_input(gate, "fused_cgu_gate")
    return _CguGateFn.apply(gate, up)


def fused_cgu_gate_packed(gate_up: torch.Tensor) -> torch.Tensor:
    """`fused_cgu_gate(gate_up[..., :C, :], gate_up[..., C:, :])` for one projection output [..., 2C, 2]."""
    _check_act_input(gate_up, "fused_cgu_gate_packed")
    if gate_up.shape[-2] % 8:
        raise _lib.QPamError("fused_cgu_gate_packed: the packed channel count must be a multiple of 8")
    return _CguGatePackedFn.apply(gate_up)


# ------------------------------------------------------------------------------------ PAM input stage
class _PamPrepFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, rope, omp, positions, offset, H, d):
        qkv = qkv.contiguous()
        B, T = qkv.shape[0], qkv.shape[1]
        q, k, v = (torch.empty(B, H, T, d, 2, dtype=qkv.dtype, device=qkv.device) for _ in range(3))
        ompf = None if omp is None else omp.detach().float().contiguous()
        check(_lib.lib().qpam_pam_prep_fwd(ptr(qkv), dtype_code(qkv.dtype), ptr(rope), 0 if rope is None else rope.shape[0],
                                           ptr(positions), int(offset), ptr(ompf), ptr(q), ptr(k), ptr(v), B, T, H, d,
                                           stream_ptr()), "qpam_pam_prep_fwd")
        ctx.save_for_backward(qkv, rope, ompf, positions)
        ctx.meta = (offset, H, d, None if omp is None else omp.dtype)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, rope, ompf, positions = ctx.saved_tensors
        offset, H, d, omp_dtype = ctx.meta
        B, T = qkv.shape[0], qkv.shape[1]
        dq, dk, dv = (g.to(qkv.dtype).contiguous() for g in (dq, dk, dv))
        dqkv = torch.empty_like(qkv)
        domp = None if ompf is None else torch.empty(B, T, H, dtype=torch.float32, device=qkv.device)
        check(_lib.lib().qpam_pam_prep_bwd(ptr(qkv), dtype_code(qkv.dtype), ptr(rope), 0 if rope is None else rope.shape[0],
                                           ptr(positions), int(offset), ptr(ompf), ptr(dq), ptr(dk), ptr(dv), ptr(dqkv),
                                           ptr(domp), B, T, H, d, stream_ptr()), "qpam_pam_prep_bwd")
        return dqkv, None, None if domp is None else domp.to(omp_dtype), None, None, None, None


def pam_prep(qkv: torch.Tensor, rope: Optional[torch.Tensor], omp: Optional[torch.Tensor], *, n_heads: int,
             head_dim: int, positions: Optional[torch.Tensor] = None, offset: int = 0):
    """Split a fused projection `qkv` [B, T, 3*H*d, 2] into q, k, v' [B, H, T, d, 2]: q and k rotated by
    `rope[pos]` ([P, d, 2] = (cos, sin), float32; None = no rotation), v' = omp * v with omp [B, T, H]
    (the complement of the protect gate; None = 1).  pos = positions[b, t] (int64) or offset + t.
    One pass instead of the reference's view/transpose/contiguous, two complex products and the gate
    product (v11/model.py:279-306, 340-349)."""
    _require_cuda(qkv, rope, omp, positions)
    B, T = qkv.shape[0], qkv.shape[1]
    H, d = n_heads, head_dim
    if qkv.numel() != B * T * 3 * H * d * 2 or qkv.shape[-1] != 2:
        raise _lib.QPamError(f"pam_prep: qkv {tuple(qkv.shape)} is not [B, T, 3*{H}*{d}, 2]")
    if qkv.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.QPamError(f"unsupported dtype {qkv.dtype}")
    if d < 4 or d > 128 or d & (d - 1):
        raise _lib.QPamError(f"pam_prep: head_dim must be a power of two in [4, 128], got {d}")
    if rope is not None:
        if rope.dim() != 3 or rope.shape[1:] != (d, 2):
            raise _lib.QPamError(f"pam_prep: rope must be [P, {d}, 2], got {tuple(rope.shape)}")
        rope = rope.detach().float().contiguous()
        if positions is None and offset + T > rope.shape[0]:
            raise _lib.QPamError("pam_prep: the rotary table is shorter than offset + T")
    if omp is not None and tuple(omp.shape) != (B, T, H):
        raise _lib.QPamError(f"pam_prep: omp must be [B, T, H] = {(B, T, H)}, got {tuple(omp.shape)}")
    if positions is not None:
        if positions.numel() != B * T:
            raise _lib.QPamError("pam_prep: positions must have one entry per token")
        positions = positions.to(torch.int64).contiguous()
    return _PamPrepFn.apply(qkv, rope, omp, positions, offset, H, d)


# ------------------------------------------------------------------------------------ K-state read-out
class _StateCombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, coef, token_major, *yks):
        K = len(yks)
        yks = tuple(t.contiguous() for t in yks)
        d = yks[0].shape[-2]
        R = yks[0].numel() // (2 * d)
        cf = coef.detach().float().contiguous()
        arr = (_lib.c_void_p * K)(*[t.data_ptr() for t in yks])
        if token_major:
            B, H, T = yks[0].shape[:3]
            y = torch.empty(B, T, H * d, 2, dtype=yks[0].dtype, device=yks[0].device)
            check(_lib.lib().qpam_state_combine_tokens_fwd(arr, ptr(cf), ptr(y), dtype_code(y.dtype), K, B, H, T, d,
                                                           stream_ptr()), "qpam_state_combine_tokens_fwd")
        else:
            y = torch.empty_like(yks[0])
            check(_lib.lib().qpam_state_combine_fwd(arr, ptr(cf), ptr(y), dtype_code(y.dtype), K, R, d, stream_ptr()),
                  "qpam_state_combine_fwd")
        ctx.save_for_backward(cf, *yks)
        ctx.meta = (coef.dtype, token_major)
        return y

    @staticmethod
    def backward(ctx, dy):
        cf, *yks = ctx.saved_tensors
        coef_dtype, token_major = ctx.meta
        K = len(yks)
        d = yks[0].shape[-2]
        R = yks[0].numel() // (2 * d)
        dy = dy.to(yks[0].dtype).contiguous()
        dyks = [torch.empty_like(t) for t in yks]
        dcoef = torch.empty_like(cf)
        arr = (_lib.c_void_p * K)(*[t.data_ptr() for t in yks])
        darr = (_lib.c_void_p * K)(*[t.data_ptr() for t in dyks])
        if token_major:
            B, H, T = yks[0].shape[:3]
            check(_lib.lib().qpam_state_combine_tokens_bwd(arr, ptr(cf), ptr(dy), darr, ptr(dcoef), dtype_code(dy.dtype), K,
                                                           B, H, T, d, stream_ptr()), "qpam_state_combine_tokens_bwd")
        else:
            check(_lib.lib().qpam_state_combine_bwd(arr, ptr(cf), ptr(dy), darr, ptr(dcoef), dtype_code(dy.dtype), K, R, d,
                                                    stream_ptr()), "qpam_state_combine_bwd")
        return (dcoef.to(coef_dtype), None, *dyks)


class _StateCombineStackedFn(torch.autograd.Function):
    """`_StateCombineFn` for state outputs held in ONE tensor [K, ..., d, 2]: the gradient comes back as one tensor of
    the same shape, so a producer that made all K outputs at once gets it without a stacking copy."""

    @staticmethod
    def forward(ctx, coef, token_major, ys):
        ys = ys.contiguous()
        K = ys.shape[0]
        d = ys.shape[-2]
        R = ys[0].numel() // (2 * d)
        cf = coef.detach().float().contiguous()
        arr = (_lib.c_void_p * K)(*[ys[k_].data_ptr() for k_ in range(K)])
        if token_major:
            B, H, T = ys.shape[1:4]
            y = torch.empty(B, T, H * d, 2, dtype=ys.dtype, device=ys.device)
            check(_lib.lib().qpam_state_combine_tokens_fwd(arr, ptr(cf), ptr(y), dtype_code(y.dtype), K, B, H, T, d,
                                                           stream_ptr()), "qpam_state_combine_tokens_fwd")
        else:
            y = torch.empty_like(ys[0])
            check(_lib.lib().qpam_state_combine_fwd(arr, ptr(cf), ptr(y), dtype_code(y.dtype), K, R, d, stream_ptr()),
                  "qpam_state_combine_fwd")
        ctx.save_for_backward(cf, ys)
        ctx.meta = (coef.dtype, token_major)
        return y

    @staticmethod
    def backward(ctx, dy):
        cf, ys = ctx.saved_tensors
        coef_dtype, token_major = ctx.meta
        K = ys.shape[0]
        d = ys.shape[-2]
        R = ys[0].numel() // (2 * d)
        dy = dy.to(ys.dtype).contiguous()
        dys = torch.empty_like(ys)
        dcoef = torch.empty_like(cf)
        arr = (_lib.c_void_p * K)(*[ys[k_].data_ptr() for k_ in range(K)])
        darr = (_lib.c_void_p * K)(*[dys[k_].data_ptr() for k_ in range(K)])
        if token_major:
            B, H, T = ys.shape[1:4]
            check(_lib.lib().qpam_state_combine_tokens_bwd(arr, ptr(cf), ptr(dy), darr, ptr(dcoef), dtype_code(dy.dtype), K,
                                                           B, H, T, d, stream_ptr()), "qpam_state_combine_tokens_bwd")
        else:
            check(_lib.lib().qpam_state_combine_bwd(arr, ptr(cf), ptr(dy), darr, ptr(dcoef), dtype_code(dy.dtype), K, R, d,
                                                    stream_ptr()), "qpam_state_combine_bwd")
        return dcoef.to(coef_dtype), None, dys


def state_combine_stacked(coef: torch.Tensor, ys: torch.Tensor, token_major: bool = False) -> torch.Tensor:
    """`state_combine` for the K state outputs as one tensor ys [K, ..., d, 2] (same checks, same kernels)."""
    _require_cuda(coef, ys)
    K, shape, dt = ys.shape[0], ys.shape[1:], ys.dtype
    d = shape[-2]
    if not 1 <= K <= 4 or shape[-1] != 2:
        raise _lib.QPamError(f"state_combine: 1..4 states of shape [..., d, 2]; got {tuple(ys.shape)}")
    if dt not in (torch.float32, torch.bfloat16) or d < 4 or d > 128 or d & (d - 1):
        raise _lib.QPamError(f"state_combine: bf16/f32 and d a power of two in [4,128]; got {dt}, d={d}")
    if tuple(coef.shape) != (K, *shape[:-2], 2):
        raise _lib.QPamError(f"state_combine: coef must be {(K, *shape[:-2], 2)}, got {tuple(coef.shape)}")
    if token_major and len(shape) != 5:
        raise _lib.QPamError("state_combine: token_major needs [B,H,T,d,2] state outputs")
    return _StateCombineStackedFn.apply(coef, token_major, ys)


@torch.no_grad()
def state_combine_tokens(coef: torch.Tensor, yks) -> torch.Tensor:
    """Inference form of `state_combine` for yks[k] [B, H, T, d, 2]: the result is written token-major,
    [B, T, H*d, 2], which is the layout the output projection reads (no transpose copy)."""
    yks = [t.contiguous() for t in yks]
    _require_cuda(coef, *yks)
    K = len(yks)
    B, H, T, d, two = yks[0].shape
    if not 1 <= K <= 4 or two != 2 or any(t.shape != yks[0].shape or t.dtype != yks[0].dtype for t in yks):
        raise _lib.QPamError("state_combine_tokens: 1..4 state outputs of one [B,H,T,d,2] shape and dtype")
    if yks[0].dtype not in (torch.float32, torch.bfloat16) or d < 4 or d > 128 or d & (d - 1):
        raise _lib.QPamError(f"state_combine_tokens: bf16/f32 and d a power of two in [4,128]; got {yks[0].dtype}, d={d}")
    if tuple(coef.shape) != (K, B, H, T, 2):
        raise _lib.QPamError(f"state_combine_tokens: coef must be {(K, B, H, T, 2)}, got {tuple(coef.shape)}")
    cf = coef.float().contiguous()
    y = torch.empty(B, T, H * d, 2, dtype=yks[0].dtype, device=yks[0].device)
    arr = (_lib.c_void_p * K)(*[t.data_ptr() for t in yks])
    check(_lib.lib().qpam_state_combine_tokens_fwd(arr, ptr(cf), ptr(y), dtype_code(y.dtype), K, B, H, T, d, stream_ptr()),
          "qpam_state_combine_tokens_fwd")
    return y


def state_combine(coef: torch.Tensor, yks, token_major: bool = False) -> torch.Tensor:
    """y = sum_k coef[k] * yks[k] (complex): coef [K, ..., 2] over the leading axes of yks[k] [..., d, 2]
    (the K-state read-out of v11/model.py:766-781), forward and backward in one pass each.  token_major=True
    (yks[k] [B,H,T,d,2]) returns y as [B, T, H*d, 2], the layout the output projection reads."""
    yks = list(yks)
    _require_cuda(coef, *yks)
    K = len(yks)
    if not 1 <= K <= 4:
        raise _lib.QPamError(f"state_combine: 1..4 states, got {K}")
    shape, dt = yks[0].shape, yks[0].dtype
    d = shape[-2]
    if any(t.shape != shape or t.dtype != dt for t in yks) or shape[-1] != 2:
        raise _lib.QPamError("state_combine: the state outputs must share one [..., d, 2] shape and dtype")
    if dt not in (torch.float32, torch.bfloat16) or d < 4 or d > 128 or d & (d - 1):
        raise _lib.QPamError(f"state_combine: bf16/f32 and d a power of two in [4,128]; got {dt}, d={d}")
    if tuple(coef.shape) != (K, *shape[:-2], 2):
        raise _lib.QPamError(f"state_combine: coef must be {(K, *shape[:-2], 2)}, got {tuple(coef.shape)}")
    if token_major and len(shape) != 5:
        raise _lib.QPamError("state_combine: token_major needs [B,H,T,d,2] state outputs")
    return _StateCombineFn.apply(coef, token_major, *yks)


# ------------------------------------------------------------------------------------ residual, block weight
class _ScaledResidualFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, scale):
        x, delta = x.contiguous(), delta.contiguous()
        sc = scale.detach().float().reshape(1)
        out = torch.empty_like(x)
        check(_lib.lib().qpam_scaled_residual_fwd(ptr(x), dtype_code(x.dtype), ptr(delta), dtype_code(delta.dtype), ptr(sc),
                                                  ptr(out), x.numel(), stream_ptr()), "qpam_scaled_residual_fwd")
        ctx.save_for_backward(delta, sc)
        ctx.meta = (scale.dtype, scale.shape, x.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        delta, sc = ctx.saved_tensors
        s_dtype, s_shape, x_dtype = ctx.meta
        dout = dout.to(x_dtype).contiguous()
        P = max(1, min(148 * 8, delta.numel() // 4096 + 1))
        part = torch.empty(P, dtype=torch.float32, device=delta.device)
        ddelta = torch.empty_like(delta)
        check(_lib.lib().qpam_scaled_residual_bwd(ptr(dout), dtype_code(x_dtype), ptr(delta), dtype_code(delta.dtype), ptr(sc),
                                                  ptr(ddelta), ptr(part), P, delta.numel(), stream_ptr()),
              "qpam_scaled_residual_bwd")
        return dout, ddelta, part.sum().to(s_dtype).reshape(s_shape)


def scaled_residual(x: torch.Tensor, delta: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x + scale * delta with a learnable scalar `scale` (the two residual adds of V11Block.forward); the
    result has x's dtype, delta may be bf16 beside an fp32 residual stream."""
    _require_cuda(x, delta, scale)
    if x.shape != delta.shape or scale.numel() != 1 or x.numel() % 4:
        raise _lib.QPamError(f"scaled_residual: x {tuple(x.shape)} / delta {tuple(delta.shape)} must match (size a multiple "
                             f"of 4) and scale must be a scalar")
    for t in (x, delta):
        if t.dtype not in (torch.float32, torch.bfloat16):
            raise _lib.QPamError(f"unsupported dtype {t.dtype}")
    return _ScaledResidualFn.apply(x, delta, scale)


class _BlockWeightFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, wr, wi, out_dtype):
        wr, wi = wr.contiguous(), wi.contiguous()
        out_dim, in_dim = wr.shape
        w = torch.empty(2 * out_dim, 2 * in_dim, dtype=out_dtype, device=wr.device)
        check(_lib.lib().qpam_block_weight_fwd(ptr(wr), ptr(wi), dtype_code(wr.dtype), ptr(w), dtype_code(out_dtype), out_dim,
                                               in_dim, stream_ptr()), "qpam_block_weight_fwd")
        ctx.meta = (wr.dtype, out_dtype, out_dim, in_dim)
        return w

    @staticmethod
    def backward(ctx, dw):
        w_dtype, out_dtype, out_dim, in_dim = ctx.meta
        dw = dw.to(out_dtype).contiguous()
        dwr = torch.empty(out_dim, in_dim, dtype=w_dtype, device=dw.device)
        dwi = torch.empty_like(dwr)
        check(_lib.lib().qpam_block_weight_bwd(ptr(dw), dtype_code(out_dtype), ptr(dwr), ptr(dwi), dtype_code(w_dtype), out_dim,
                                               in_dim, stream_ptr()), "qpam_block_weight_bwd")
        return dwr, dwi, None


def block_weight(weight_real: torch.Tensor, weight_imag: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """[2*out, 2*in] real matrix with rows (o,re) = (Wr, -Wi), (o,im) = (Wi, Wr) over interleaved (re, im)
    columns: `F.linear(x.view(..., 2*in), block_weight(Wr, Wi))` is the complex projection of
    `ComplexLinear` (v11/complex_ops.py) with an interleaved result."""
    _require_cuda(weight_real, weight_imag)
    if weight_real.shape != weight_imag.shape or weight_real.dim() != 2 or weight_real.dtype != weight_imag.dtype:
        raise _lib.QPamError("block_weight: Wr and Wi must be two [out, in] matrices of one dtype")
    if weight_real.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.QPamError(f"unsupported dtype {weight_real.dtype}")
    out_dtype = out_dtype or weight_real.dtype
    return _BlockWeightFn.apply(weight_real, weight_imag, out_dtype)


# ------------------------------------------------------------------------------------ PAM gate arithmetic
class _PamGatesFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dt, pg, phase, score, dt_bias, dt_off, gamma_floor, K, want_coef):
        B, T, H = dt.shape
        f = lambda t: None if t is None else t.detach().float().contiguous()
        dtf, pgf, phf, scf, bf, of = f(dt), f(pg), f(phase), f(score), f(dt_bias), f(dt_off)
        dev = dt.device
        gamma = torch.empty(K, B, H, T, dtype=torch.float32, device=dev)
        omp = None if pg is None else torch.empty(B, T, H, dtype=torch.float32, device=dev)
        coef = torch.empty(K, B, H, T, 2, dtype=torch.float32, device=dev) if want_coef else None
        check(_lib.lib().qpam_pam_gates_fwd(ptr(dtf), ptr(pgf), ptr(phf), ptr(scf), ptr(bf), ptr(of), float(gamma_floor),
                                            ptr(gamma), ptr(omp), ptr(coef), B, T, H, K, stream_ptr()), "qpam_pam_gates_fwd")
        ctx.save_for_backward(dtf, pgf, phf, scf, bf, of)
        ctx.meta = (gamma_floor, K, tuple(None if t is None else t.dtype for t in (dt, pg, phase, score, dt_bias, dt_off)))
        outs = (gamma, omp if omp is not None else gamma.new_empty(0), coef if coef is not None else gamma.new_empty(0))
        return outs

    @staticmethod
    def backward(ctx, dgamma, domp, dcoef):
        dtf, pgf, phf, scf, bf, of = ctx.saved_tensors
        gamma_floor, K, dtypes = ctx.meta
        B, T, H = dtf.shape
        dev = dtf.device
        g = lambda t, ok: None if (t is None or not ok or t.numel() == 0) else t.float().contiguous()
        dgamma = torch.zeros(K, B, H, T, dtype=torch.float32, device=dev) if dgamma is None else dgamma.float().contiguous()
        domp, dcoef = g(domp, pgf is not None), g(dcoef, True)
        ddt = torch.empty_like(dtf)
        dpg = None if pgf is None else torch.empty_like(pgf)
        dph = None if phf is None else torch.empty_like(phf)
        dsc = None if scf is None else torch.empty_like(scf)
        P = max(1, min(148 * 4, (dtf.numel() + 255) // 256))
        part = torch.empty(P, H, K, dtype=torch.float32, device=dev)
        check(_lib.lib().qpam_pam_gates_bwd(ptr(dtf), ptr(pgf), ptr(phf), ptr(scf), ptr(bf), ptr(of), float(gamma_floor),
                                            ptr(dgamma), ptr(domp), ptr(dcoef), ptr(ddt), ptr(dpg), ptr(dph), ptr(dsc),
                                            ptr(part), P, B, T, H, K, stream_ptr()), "qpam_pam_gates_bwd")
        hk = part.sum(0)                                                   # [H,K]
        cast = lambda t, i: None if t is None else t.to(dtypes[i])
        return (cast(ddt, 0), cast(dpg, 1), cast(dph, 2), cast(dsc, 3), cast(hk.sum(1), 4),
                None if of is None else cast(hk.sum(0), 5), None, None, None)


def pam_gates(dt, pg, phase, score, dt_bias, state_dt_offset, gamma_floor: float, n_states: int):
    """Decay, protect gate and phase-routing read-out weights of the PAM layer from the outputs of its small
    Linears (v11/model.py:308-350, 630-655, 685-720), forward and backward in one kernel each:
    dt, pg [B,T,H]; phase, score [B,T,H,K] (pg / phase / score / state_dt_offset may be None).
    Returns gamma [K,B,H,T], omp = 1 - p [B,T,H] (None without pg), coef [K,B,H,T,2] (None without phase)."""
    _require_cuda(dt, pg, phase, score, dt_bias, state_dt_offset)
    B, T, H = dt.shape
    K = n_states
    if not 1 <= K <= 4:
        raise _lib.QPamError(f"pam_gates: 1..4 states, got {K}")
    if pg is not None and pg.shape != dt.shape:
        raise _lib.QPamError("pam_gates: pg must have dt's shape [B,T,H]")
    for t, name in ((phase, "phase"), (score, "score")):
        if t is not None and tuple(t.shape) != (B, T, H, K):
            raise _lib.QPamError(f"pam_gates: {name} must be [B,T,H,K] = {(B, T, H, K)}, got {tuple(t.shape)}")
    if dt_bias.numel() != H or (state_dt_offset is not None and state_dt_offset.numel() != K):
        raise _lib.QPamError("pam_gates: dt_bias must have H entries and state_dt_offset K")
    if score is not None and (K == 1 or phase is None):
        raise _lib.QPamError("pam_gates: routing scores need K > 1 and phases")
    gamma, omp, coef = _PamGatesFn.apply(dt, pg, phase, score, dt_bias, state_dt_offset, gamma_floor, K, phase is not None)
    return gamma, (omp if pg is not None else None), (coef if phase is not None else None)


# ------------------------------------------------------------------------------------ magnitude
class _MagnitudeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z):
        z = z.contiguous()
        out = torch.empty(z.shape[:-1], dtype=z.dtype, device=z.device)
        check(_lib.lib().qpam_cmagnitude_fwd(ptr(z), dtype_code(z.dtype), ptr(out), out.numel(), stream_ptr()), "qpam_cmagnitude_fwd")
        ctx.save_for_backward(z)
        return out

    @staticmethod
    def backward(ctx, dm):
        (z,) = ctx.saved_tensors
        dm = dm.to(z.dtype).contiguous()
        dz = torch.empty_like(z)
        check(_lib.lib().qpam_cmagnitude_bwd(ptr(z), ptr(dm), dtype_code(z.dtype), ptr(dz), dm.numel(), stream_ptr()),
              "qpam_cmagnitude_bwd")
        return dz


def complex_magnitude(z: torch.Tensor) -> torch.Tensor:
    """sqrt(re^2 + im^2 + 1e-8) over the last axis of [..., 2] (the `_magnitude` of v11/complex_ops.py)."""
    _require_cuda(z)
    if z.shape[-1] != 2 or (z.numel() // 2) % 4 or z.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.QPamError(f"complex_magnitude: expected a float32/bfloat16 [..., 2] tensor with a multiple of 4 values, got "
                             f"{tuple(z.shape)} {z.dtype}")
    return _MagnitudeFn.apply(z)
