"""torch-facing wrappers of the C ABI: autograd functions over raw device pointers.

torch is used here for what it is good at on this path -- owning device memory, the current
stream and autograd bookkeeping.  All arithmetic happens in libqllm2_pam_b200.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import CEArgs, ScanArgs, check, dtype_code, ptr, stream_ptr

GAMMA_EPS = 1e-6


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.QPamError("PAM kernels need CUDA tensors (there is no CPU path in this package)")


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


# --------------------------------------------------------------------------------------- scan
def _scan_args(q, k, v, gamma, coef, s0, cu_seqlens, y, s_final, q_scale, eps, chunk):
    B, H, T, d = q.shape[0], q.shape[1], q.shape[2], q.shape[3]
    K = gamma.shape[0]
    S = B if cu_seqlens is None else cu_seqlens.numel() - 1
    a = ScanArgs()
    a.q, a.k, a.v = ptr(q), ptr(k), ptr(v)
    a.gamma, a.coef, a.s0, a.cu_seqlens = ptr(gamma), ptr(coef), ptr(s0), ptr(cu_seqlens)
    a.y, a.s_final = ptr(y), ptr(s_final)
    a.B, a.H, a.T, a.d, a.K, a.S = B, H, T, d, K, S
    a.chunk, a.io_dtype = int(chunk), dtype_code(q.dtype)
    a.q_scale, a.gamma_eps = float(q_scale), float(eps)
    return a


class _PamScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, gamma, coef, s0, cu_seqlens, q_scale, eps, chunk, save_states):
        L = _lib.lib()
        _require_cuda(q, k, v, gamma)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        gamma = gamma.float().contiguous()
        coef = None if coef is None else coef.float().contiguous()
        s0 = None if s0 is None else s0.float().contiguous()
        B, H, T, d = q.shape[:4]
        K = gamma.shape[0]
        S = B if cu_seqlens is None else cu_seqlens.numel() - 1
        y = torch.empty_like(q)
        s_final = torch.empty(K, S, H, d, d, 2, dtype=torch.float32, device=q.device)
        need_bwd = any(t is not None and t.requires_grad for t in (q, k, v, gamma, coef, s0))
        a = _scan_args(q, k, v, gamma, coef, s0, cu_seqlens, y, s_final, q_scale, eps, chunk)
        nbytes = L.qpam_scan_workspace_bytes(C.byref(a), 1 if (need_bwd and save_states) else 0)
        ws = _workspace(nbytes, q.device)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        check(L.qpam_scan_fwd(C.byref(a), stream_ptr()), "qpam_scan_fwd")
        ctx.save_for_backward(q, k, v, gamma, coef, s0, cu_seqlens, ws if (need_bwd and save_states) else None)
        ctx.cfg = (q_scale, eps, chunk)
        ctx.set_materialize_grads(False)
        return y, s_final

    @staticmethod
    def backward(ctx, dy, ds_final):
        L = _lib.lib()
        q, k, v, gamma, coef, s0, cu_seqlens, ws = ctx.saved_tensors
        q_scale, eps, chunk = ctx.cfg
        dy = torch.zeros_like(q) if dy is None else dy.contiguous().to(q.dtype)
        if dy.shape != q.shape:
            raise _lib.QPamError(f"dy shape {tuple(dy.shape)} != y shape {tuple(q.shape)}")
        if ds_final is not None and ds_final.numel() != gamma.shape[0] * (q.shape[0] if cu_seqlens is None else cu_seqlens.numel() - 1) * q.shape[1] * q.shape[3] ** 2 * 2:
            raise _lib.QPamError("ds_final has the wrong number of elements")
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dgamma = torch.empty_like(gamma)
        dcoef = torch.empty_like(coef) if coef is not None else None
        ds0 = torch.empty_like(s0) if (s0 is not None and ctx.needs_input_grad[5]) else None
        if ds_final is not None:
            ds_final = ds_final.float().contiguous()
        a = _scan_args(q, k, v, gamma, coef, s0, cu_seqlens, None, None, q_scale, eps, chunk)
        states_valid = 1
        if ws is None:
            ws = _workspace(L.qpam_scan_workspace_bytes(C.byref(a), 1), q.device)
            states_valid = 0
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        check(L.qpam_scan_bwd(C.byref(a), ptr(dy), ptr(dq), ptr(dk), ptr(dv), ptr(dgamma), ptr(dcoef),
                              ptr(ds_final), ptr(ds0), states_valid, stream_ptr()), "qpam_scan_bwd")
        return dq, dk, dv, dgamma, dcoef, ds0, None, None, None, None, None


class _PamScanStatesFn(torch.autograd.Function):
    """K single-state scans over the same q, k, v (bf16, d = 64: the tensor-core kernels), one per decay row of
    `gamma` [K,B,H,T]: returns the per-state outputs ys [K,B,H,T,d,2] and final states [K,S,H,d,d,2].  The
    backward runs the K backward scans into ONE set of dq, dk, dv buffers: the first writes, the others add
    (qpam_scan_bwd_accumulate), so the sum over the states costs no extra pass."""

    @staticmethod
    def forward(ctx, q, k, v, gamma, s0, cu_seqlens, q_scale, eps, chunk):
        L = _lib.lib()
        _require_cuda(q, k, v, gamma)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        gamma = gamma.float().contiguous()
        s0 = None if s0 is None else s0.float().contiguous()
        B, H, T, d = q.shape[:4]
        K = gamma.shape[0]
        S = B if cu_seqlens is None else cu_seqlens.numel() - 1
        ys = torch.empty((K,) + tuple(q.shape), dtype=q.dtype, device=q.device)
        s_final = torch.empty(K, S, H, d, d, 2, dtype=torch.float32, device=q.device)
        need_bwd = any(t is not None and t.requires_grad for t in (q, k, v, gamma, s0))
        if 2 <= K <= 4 and T > 0:
            # one call: the chunk sums of all states from one pass over k and v, one carry launch, then the output
            # kernel per state; the workspace keeps every state's chunk states for the per-state backward calls
            a = _scan_args(q, k, v, gamma, None, s0, cu_seqlens, None, s_final, q_scale, eps, chunk)
            ws = _workspace(L.qpam_scan_workspace_bytes(C.byref(a), 1 if need_bwd else 0), q.device)
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            check(L.qpam_scan_fwd_states(C.byref(a), ptr(ys), stream_ptr()), "qpam_scan_fwd_states")
            ctx.save_for_backward(q, k, v, gamma, s0, cu_seqlens, *([ws] if need_bwd else []))
            ctx.cfg = (q_scale, eps, chunk, need_bwd)
            ctx.shared = True
            ctx.set_materialize_grads(False)
            return ys, s_final
        ctx.shared = False
        wss = []
        for kk in range(K):
            a = _scan_args(q, k, v, gamma[kk:kk + 1], None, None if s0 is None else s0[kk:kk + 1], cu_seqlens, ys[kk],
                           s_final[kk:kk + 1], q_scale, eps, chunk)
            ws = _workspace(L.qpam_scan_workspace_bytes(C.byref(a), 1 if need_bwd else 0), q.device)
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            check(L.qpam_scan_fwd(C.byref(a), stream_ptr()), "qpam_scan_fwd")
            wss.append(ws if need_bwd else None)
        ctx.save_for_backward(q, k, v, gamma, s0, cu_seqlens, *[w_ for w_ in wss if w_ is not None])
        ctx.cfg = (q_scale, eps, chunk, need_bwd)
        ctx.set_materialize_grads(False)
        return ys, s_final

    @staticmethod
    def backward(ctx, dys, ds_final):
        L = _lib.lib()
        q, k, v, gamma, s0, cu_seqlens, *wss = ctx.saved_tensors
        q_scale, eps, chunk, _ = ctx.cfg
        K = gamma.shape[0]
        dys = torch.zeros((K,) + tuple(q.shape), dtype=q.dtype, device=q.device) if dys is None else dys.contiguous().to(q.dtype)
        if dys.shape != (K,) + tuple(q.shape):
            raise _lib.QPamError(f"dys shape {tuple(dys.shape)} != ys shape {(K,) + tuple(q.shape)}")
        if ds_final is not None:
            ds_final = ds_final.float().contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dgamma = torch.empty_like(gamma)
        ds0 = torch.empty_like(s0) if (s0 is not None and ctx.needs_input_grad[4]) else None
        if ctx.shared:
            a = _scan_args(q, k, v, gamma, None, s0, cu_seqlens, None, None, q_scale, eps, chunk)
            a.workspace, a.workspace_bytes = wss[0].data_ptr(), wss[0].numel()
            for kk in range(K):
                dsf = None if ds_final is None else ds_final[kk:kk + 1]
                d0 = None if ds0 is None else ds0[kk:kk + 1]
                check(L.qpam_scan_bwd_state(C.byref(a), kk, ptr(dys[kk]), ptr(dq), ptr(dk), ptr(dv), ptr(dgamma[kk:kk + 1]),
                                            ptr(dsf), ptr(d0), 1 if kk > 0 else 0, stream_ptr()), "qpam_scan_bwd_state")
            return dq, dk, dv, dgamma, ds0, None, None, None, None
        for kk in range(K):
            a = _scan_args(q, k, v, gamma[kk:kk + 1], None, None if s0 is None else s0[kk:kk + 1], cu_seqlens, None, None,
                           q_scale, eps, chunk)
            ws = wss[kk]
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            dsf = None if ds_final is None else ds_final[kk:kk + 1]
            d0 = None if ds0 is None else ds0[kk:kk + 1]
            if kk == 0:
                check(L.qpam_scan_bwd(C.byref(a), ptr(dys[kk]), ptr(dq), ptr(dk), ptr(dv), ptr(dgamma[kk:kk + 1]), None,
                                      ptr(dsf), ptr(d0), 1, stream_ptr()), "qpam_scan_bwd")
            else:
                check(L.qpam_scan_bwd_accumulate(C.byref(a), ptr(dys[kk]), ptr(dq), ptr(dk), ptr(dv), ptr(dgamma[kk:kk + 1]),
                                                 ptr(dsf), ptr(d0), 1, stream_ptr()), "qpam_scan_bwd_accumulate")
        return dq, dk, dv, dgamma, ds0, None, None, None, None


def pam_scan(q, k, v, gamma, *, coef=None, s0=None, cu_seqlens=None, head_dim: Optional[int] = None,
             eps: float = GAMMA_EPS, chunk: int = 64, save_states: bool = True, token_major: bool = False):
    """Chunked dual-form PAM scan on the GPU.  (token_major=True returns y as [B, T, H*d, 2], the head merge
    of v11/model.py:835-836, straight from the last kernel where that kernel can write it.)

    q, k, v  [B,H,T,d,2] (float32 or bfloat16; q unscaled -- it is multiplied by head_dim**-0.5
             inside, as V11PAMLayer._forward_chunked_head does, v11/model.py:381-382)
    gamma    [B,H,T] or [K,B,H,T] decay in (0,1];  coef optional [K,B,H,T,2] read-out weights
    s0       optional [K,S,H,d,d,2] initial state;  cu_seqlens optional int32 [S+1] (then B == 1)
    Returns (y [B,H,T,d,2] in q's dtype, s_final float32 [K,S,H,d,d,2]).
    """
    # one dtype for the token tensors: under bf16 autocast the reference's matmuls round their inputs to
    # bf16 anyway, so mixed fp32/bf16 operands (RoPE promotes q and k to fp32) are taken as bf16;
    # otherwise they are promoted to the widest dtype present.  The C ABI reads all three through
    # q's dtype, so they must agree before the pointers are handed over.
    if torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16:
        io = torch.bfloat16
    else:
        io = torch.promote_types(torch.promote_types(q.dtype, k.dtype), v.dtype)
    q, k, v = q.to(io), k.to(io), v.to(io)
    if not (q.shape == k.shape == v.shape and q.dim() == 5 and q.shape[-1] == 2):
        raise _lib.QPamError(f"q, k, v must share one shape [B,H,T,d,2]; got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    B_, H_, T_ = q.shape[:3]
    gamma = gamma.float()
    if gamma.dim() == 3:
        gamma = gamma.unsqueeze(0)
    if gamma.shape[1:] != (B_, H_, T_):
        raise _lib.QPamError(f"gamma shape {tuple(gamma.shape)} does not match q {tuple(q.shape)}")
    if coef is not None:
        coef = coef.float()
        if coef.dim() == 4:
            coef = coef.unsqueeze(0)
    if coef is not None and coef.shape != gamma.shape + (2,):
        raise _lib.QPamError(f"coef shape {tuple(coef.shape)} != gamma shape + (2,)")
    n_seq = B_ if cu_seqlens is None else cu_seqlens.numel() - 1
    if s0 is not None:
        s0 = s0.float()
        if s0.shape != (gamma.shape[0], n_seq, H_, q.shape[3], q.shape[3], 2):
            raise _lib.QPamError(f"s0 shape {tuple(s0.shape)} != [K,S,H,d,d,2]")
    if cu_seqlens is not None and B_ != 1:
        raise _lib.QPamError("packed mode (cu_seqlens) needs B == 1")
    d = q.shape[3]
    head_dim = d if head_dim is None else head_dim
    if cu_seqlens is not None:
        if not cu_seqlens.is_cuda:
            # a host descriptor is checked here (the kernels check a device descriptor themselves and report
            # through the status word, see _lib.device_status)
            c = cu_seqlens.to(torch.int64)
            if c.numel() < 2 or int(c[0]) != 0 or bool((c[1:] < c[:-1]).any()) or int(c[-1]) > T_:
                raise _lib.QPamError(f"cu_seqlens must start at 0, never decrease and end at or before T={T_}; got {c.tolist()[:8]}...")
        cu_seqlens = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
    K = gamma.shape[0]
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, gamma, coef, s0))
    if K > 1 and q.dtype == torch.bfloat16 and d == 64 and needs_grad:
        # Phase-routed K-state scan on the tensor-core kernels: y = sum_k c_k y^(k), where y^(k) is the
        # single-state scan with decay gamma^(k) on the same q, k, v (the fused K-state form of the
        # reference, v11/model.py:657-781, is algebraically this sum).  autograd composes the backward:
        # K single-state backward scans with upstream conj(c_k) dy, and dc_k = <dy, y^(k)>.  With the chunk states kept
        # for the backward (save_states) the K scans share one autograd node whose backward accumulates dq, dk, dv in
        # place (qpam_scan_bwd_accumulate) instead of leaving K partial gradients for autograd to add.
        if save_states:
            ys_all, finals = _PamScanStatesFn.apply(q, k, v, gamma, s0, cu_seqlens, head_dim ** -0.5, eps, chunk)
            if coef is not None:
                from .fused_elementwise import state_combine_stacked
                return state_combine_stacked(coef, ys_all, token_major=token_major), finals
            y = ys_all.sum(dim=0)
            return (_merge_heads(y) if token_major else y), finals
        ys, finals = [], []
        for kk in range(K):        # states recomputed in the backward: one scan per state, autograd sums the gradients
            yk, sk = _PamScanFn.apply(q, k, v, gamma[kk:kk + 1], None, None if s0 is None else s0[kk:kk + 1],
                                      cu_seqlens, head_dim ** -0.5, eps, chunk, save_states)
            ys.append(yk)
            finals.append(sk)
        if coef is None:
            y = ys[0]
            for yk in ys[1:]:
                y = y + yk
        else:
            from .fused_elementwise import state_combine
            return state_combine(coef, ys, token_major=token_major), torch.cat(finals, dim=0)
        return (_merge_heads(y) if token_major else y), torch.cat(finals, dim=0)
    if token_major and not needs_grad:
        return pam_scan_tokens(q, k, v, gamma, coef=coef, s0=s0, cu_seqlens=cu_seqlens, head_dim=head_dim, eps=eps, chunk=chunk)
    y, s = _PamScanFn.apply(q, k, v, gamma, coef, s0, cu_seqlens, head_dim ** -0.5, eps, chunk, save_states)
    return (_merge_heads(y) if token_major else y), s


def _merge_heads(y):
    B, H, T, d = y.shape[:4]
    return y.transpose(1, 2).reshape(B, T, H * d, 2)


@torch.no_grad()
def pam_scan_states(k, v, gamma, s0=None, cu_seqlens=None, *, eps: float = GAMMA_EPS, chunk: int = 64):
    """Final state(s) of the scan only -- S after the last token, float32 [K,S,H,d,d,2] -- without forming Y:
    the chunk-local sums and the inter-chunk carry run, the output kernel does not (about a third of a forward
    scan).  k, v [B,H,T,d,2]; gamma [B,H,T] or [K,B,H,T]; s0 / cu_seqlens as in `pam_scan`."""
    L = _lib.lib()
    _require_cuda(k, v, gamma)
    if gamma.dim() == 3:
        gamma = gamma.unsqueeze(0)
    if k.dtype != v.dtype:
        dt = torch.promote_types(k.dtype, v.dtype)
        k, v = k.to(dt), v.to(dt)
    k, v = k.contiguous(), v.contiguous()
    gamma = gamma.float().contiguous()
    B, H, T, d = k.shape[:4]
    K = gamma.shape[0]
    if k.shape != v.shape or k.dim() != 5 or k.shape[-1] != 2 or tuple(gamma.shape) != (K, B, H, T):
        raise _lib.QPamError(f"pam_scan_states: k/v must be one [B,H,T,d,2] shape and gamma [K,B,H,T]; got {tuple(k.shape)}, "
                             f"{tuple(v.shape)}, {tuple(gamma.shape)}")
    if cu_seqlens is not None:
        if B != 1:
            raise _lib.QPamError("packed mode (cu_seqlens) needs B == 1")
        cu_seqlens = cu_seqlens.to(device=k.device, dtype=torch.int32).contiguous()
    S = B if cu_seqlens is None else cu_seqlens.numel() - 1
    if s0 is not None:
        if s0.numel() != K * S * H * d * d * 2:
            raise _lib.QPamError(f"s0 must be [K,S,H,d,d,2] = {(K, S, H, d, d, 2)}, got {tuple(s0.shape)}")
        s0 = s0.float().contiguous()
    s_final = torch.empty(K, S, H, d, d, 2, dtype=torch.float32, device=k.device)
    a = _scan_args(k, k, v, gamma, None, s0, cu_seqlens, None, s_final, d ** -0.5, eps, chunk)   # q is not read
    ws = _workspace(L.qpam_scan_workspace_bytes(C.byref(a), 0), k.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    check(L.qpam_scan_fwd(C.byref(a), stream_ptr()), "qpam_scan_fwd")
    return s_final


@torch.no_grad()
def pam_scan_tokens(q, k, v, gamma, coef=None, s0=None, cu_seqlens=None, *, head_dim=None, eps: float = 1e-6,
                    chunk: int = 64):
    """Inference form of `pam_scan`: same arguments, but Y comes back token-major, [B, T, H*d, 2] -- the layout
    the output projection reads (the head merge of v11/model.py:835-836) -- and nothing is kept for a backward
    pass (K phase-routed states in bf16 at d = 64 then run the fused K-state output kernel)."""
    B, H, T, d = q.shape[:4]
    gamma4 = gamma if gamma.dim() == 4 else gamma.unsqueeze(0)
    K = gamma4.shape[0]
    direct = (q.is_cuda and d == 64 and q.dtype == k.dtype == v.dtype == torch.bfloat16 and T > 0
              and (K > 1 or coef is None) and tuple(gamma4.shape) == (K, B, H, T)
              and q.shape == k.shape == v.shape and (cu_seqlens is None or B == 1))
    if not direct:
        y, s = pam_scan(q, k, v, gamma, coef=coef, s0=s0, cu_seqlens=cu_seqlens, head_dim=head_dim, eps=eps, chunk=chunk)
        return y.transpose(1, 2).reshape(B, T, H * d, 2), s
    # tensor-core path: the output kernel writes [B,T,H,d,2] itself
    L = _lib.lib()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    gamma4 = gamma4.float().contiguous()
    if coef is not None:
        if tuple(coef.shape) != (K, B, H, T, 2):
            raise _lib.QPamError(f"coef must be [K,B,H,T,2] = {(K, B, H, T, 2)}, got {tuple(coef.shape)}")
        coef = coef.float().contiguous()
    if cu_seqlens is not None:
        cu_seqlens = cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()
    S = B if cu_seqlens is None else cu_seqlens.numel() - 1
    if s0 is not None:
        if s0.numel() != K * S * H * d * d * 2:
            raise _lib.QPamError(f"s0 must be [K,S,H,d,d,2] = {(K, S, H, d, d, 2)}, got {tuple(s0.shape)}")
        s0 = s0.float().contiguous()
    y = torch.empty(B, T, H * d, 2, dtype=q.dtype, device=q.device)
    s_final = torch.empty(K, S, H, d, d, 2, dtype=torch.float32, device=q.device)
    a = _scan_args(q, k, v, gamma4, coef, s0, cu_seqlens, y, s_final, (d if head_dim is None else head_dim) ** -0.5, eps, chunk)
    ws = _workspace(L.qpam_scan_workspace_bytes(C.byref(a), 0), q.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    check(L.qpam_scan_fwd_tokens(C.byref(a), stream_ptr()), "qpam_scan_fwd_tokens")
    return y, s_final


# --------------------------------------------------------------------------------------- decode
def pam_decode_step(state_pool, slot_ids, q_scaled, k, v, gamma, coef=None, *, layer: int = 0):
    """One recurrent step, in place on ``state_pool`` [n_slots, L, K, H, d, d, 2].

    q_scaled, k, v [n,H,d,2]; gamma [K,n,H] (or [n,H]); coef optional [K,n,H,2];
    slot_ids int32 [n].  Returns y [n,H,d,2].  (v11/model.py:927-965)
    """
    L = _lib.lib()
    _require_cuda(state_pool, q_scaled)
    n_slots, n_layers, K, H, d = state_pool.shape[:5]
    if gamma.dim() == 2:
        gamma = gamma.unsqueeze(0)
    if coef is not None and coef.dim() == 3:
        coef = coef.unsqueeze(0)
    gamma = gamma.float().contiguous()
    coef = None if coef is None else coef.float().contiguous()
    k, v = k.to(q_scaled.dtype), v.to(q_scaled.dtype)
    q_scaled, k, v = q_scaled.contiguous(), k.contiguous(), v.contiguous()
    slot_ids = slot_ids.to(device=state_pool.device, dtype=torch.int32).contiguous()
    n = q_scaled.shape[0]
    if not (q_scaled.shape == k.shape == v.shape == (n, H, d, 2)):
        raise _lib.QPamError(f"q, k, v must be [n,H,d,2] = {(n, H, d, 2)}; got {tuple(q_scaled.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if slot_ids.numel() != n:
        raise _lib.QPamError("slot_ids must have one entry per sequence")
    if coef is not None and coef.shape != (K, n, H, 2):
        raise _lib.QPamError(f"coef shape {tuple(coef.shape)} != {(K, n, H, 2)}")
    if gamma.shape != (K, n, H):
        raise _lib.QPamError(f"gamma shape {tuple(gamma.shape)} != {(K, n, H)}")
    if not state_pool.is_contiguous():
        raise _lib.QPamError("state_pool must be contiguous")
    y = torch.empty_like(q_scaled)
    check(L.qpam_decode_step(state_pool.data_ptr(), dtype_code(state_pool.dtype), n_slots, n_layers, layer,
                             ptr(slot_ids), ptr(q_scaled), ptr(k), ptr(v), ptr(gamma), ptr(coef), ptr(y),
                             n, H, d, K, dtype_code(q_scaled.dtype), stream_ptr()), "qpam_decode_step")
    return y


def pam_pool_store(state_pool, slot_ids, states, *, layer: int = 0):
    """Write prefill states [K,S,H,d,d,2] (float32) into pool slots ``slot_ids`` [S]."""
    L = _lib.lib()
    n_slots, n_layers, K, H, d = state_pool.shape[:5]
    states = states.float().contiguous()
    S = states.shape[1]
    if states.shape != (K, S, H, d, d, 2) or slot_ids.numel() != S:
        raise _lib.QPamError(f"states must be [K,S,H,d,d,2] with one slot id per sequence; got {tuple(states.shape)}")
    slot_ids = slot_ids.to(device=state_pool.device, dtype=torch.int32).contiguous()
    check(L.qpam_pool_store(state_pool.data_ptr(), dtype_code(state_pool.dtype), n_slots, n_layers, layer,
                            ptr(slot_ids), ptr(states), S, H, d, K, stream_ptr()), "qpam_pool_store")


# --------------------------------------------------------------------------------------- CE
def _ce_args(h, w, targets, mask, ignore_index, v_offset=0):
    a = CEArgs()
    a.h, a.w, a.targets, a.mask = ptr(h), ptr(w), ptr(targets), ptr(mask)
    a.N, a.V, a.v_offset = h.shape[0], w.shape[0], int(v_offset)
    a.F, a.io_dtype = h.shape[1], dtype_code(h.dtype)
    a.ignore_index = int(ignore_index)
    return a


def ce_row_stats(h, w, targets, *, ignore_index=-100, v_offset=0):
    """Per-row shard statistics (max, sumexp, target logit, argmax) without forming logits."""
    L = _lib.lib()
    _require_cuda(h, w)
    h, w = h.contiguous(), w.contiguous()
    if h.dtype != w.dtype:
        w = w.to(h.dtype)
    if h.dim() != 2 or w.dim() != 2 or h.shape[1] != w.shape[1]:
        raise _lib.QPamError(f"h [N,F] and w [V,F] expected; got {tuple(h.shape)}, {tuple(w.shape)}")
    if targets is not None and (targets.dtype != torch.int64 or targets.numel() != h.shape[0]):
        raise _lib.QPamError("targets must be int64 with one entry per row of h")
    N = h.shape[0]
    f32 = dict(dtype=torch.float32, device=h.device)
    row_max, row_sum, row_tgt = torch.empty(N, **f32), torch.empty(N, **f32), torch.empty(N, **f32)
    row_arg = torch.empty(N, dtype=torch.int64, device=h.device)
    a = _ce_args(h, w, targets, None, ignore_index, v_offset)
    ws = _workspace(L.qpam_ce_workspace_bytes(C.byref(a), 0), h.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    check(L.qpam_ce_partial(C.byref(a), ptr(row_max), ptr(row_sum), ptr(row_tgt if targets is not None else None),
                            ptr(row_arg), stream_ptr()), "qpam_ce_partial")
    return row_max, row_sum, row_tgt, row_arg


def ce_finalize(h, w, targets, mask, stats, *, ignore_index=-100):
    """Combined stats -> dict(lse, per_token, loss_sum, denom, correct, tokens) (device tensors)."""
    L = _lib.lib()
    row_max, row_sum, row_tgt, row_arg = stats
    N = h.shape[0]
    f32 = dict(dtype=torch.float32, device=h.device)
    out = dict(lse=torch.empty(N, **f32), per_token=torch.empty(N, **f32), loss_sum=torch.zeros(1, **f32),
               denom=torch.ones(1, **f32), correct=torch.zeros(1, **f32), tokens=torch.zeros(1, **f32))
    a = _ce_args(h, w, targets, mask, ignore_index)
    ws = _workspace(256, h.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    check(L.qpam_ce_finalize(C.byref(a), ptr(row_max), ptr(row_sum), ptr(row_tgt), ptr(row_arg), ptr(out["lse"]),
                             ptr(out["per_token"]), ptr(out["loss_sum"]), ptr(out["denom"]), ptr(out["correct"]),
                             ptr(out["tokens"]), stream_ptr()), "qpam_ce_finalize")
    return out


def ce_backward(h, w, targets, mask, lse, grad_scale, denom, *, ignore_index=-100, v_offset=0, dh_ready_stream=None):
    """dH [N,F], dW [V,F] (dtype of h / w) for  grad_scale * loss_sum / denom.  `dh_ready_stream` (a
    torch.cuda.Stream) is made to wait until dH is complete while dW is still being formed on the current stream."""
    L = _lib.lib()
    dh = torch.empty_like(h)
    dw = torch.empty_like(w)
    a = _ce_args(h, w, targets, mask, ignore_index, v_offset)
    ws = _workspace(L.qpam_ce_workspace_bytes(C.byref(a), 1), h.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    side = None if dh_ready_stream is None else dh_ready_stream.cuda_stream
    check(L.qpam_ce_bwd_overlap(C.byref(a), ptr(lse), ptr(grad_scale), ptr(denom), ptr(dh), ptr(dw), stream_ptr(), side),
          "qpam_ce_bwd")
    return dh, dw


def head_logits(h, w):
    """Sampling decode head: bf16 logits [N, V] = h @ w^T (a view of rows padded to a multiple of 8 columns) on the
    tensor-core GEMM of the cross-entropy; h [N,F] and w [V,F] bfloat16 with 16-byte aligned rows
    (v11/model.py:1218-1221 forms the same product before its sampling block)."""
    L = _lib.lib()
    _require_cuda(h, w)
    h, w = h.contiguous(), w.contiguous()
    if h.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or h.dim() != 2 or w.dim() != 2 or h.shape[1] != w.shape[1]:
        raise _lib.QPamError(f"head_logits: bfloat16 h [N,F] and w [V,F] expected; got {tuple(h.shape)} {h.dtype}, {tuple(w.shape)} {w.dtype}")
    N, V = h.shape[0], w.shape[0]
    ld = (V + 7) // 8 * 8
    out = torch.empty(N, ld, dtype=torch.bfloat16, device=h.device)
    a = _ce_args(h, w, None, None, -100, 0)
    check(L.qpam_head_logits(C.byref(a), ptr(out), ld, stream_ptr()), "qpam_head_logits")
    return out[:, :V]


def head_argmax(h, w):
    """Greedy decode head: (ids int64 [N], best logit float32 [N]) of argmax_v (h @ w^T)."""
    row_max, _, _, row_arg = ce_row_stats(h, w, None)
    return row_arg, row_max


def sample_logits(logits, uniforms=None, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0,
                  repetition_penalty: float = 1.0, history=None, hist_len=None, slot_ids=None, append: bool = False,
                  return_stats: bool = False):
    """Draw one token per row of `logits` [n, V] on the device (one kernel; v11/model.py:1221-1244): temperature,
    repetition penalty over `history` (int64 [rows, cols] token ids; `hist_len` int32 [rows] valid entries per
    row, `slot_ids` int32 [n] maps logits rows to history rows), top-k, top-p, then the inverse-CDF draw of
    `uniforms` [n] (default: torch.rand on the logits' device, i.e. torch's generator).  `append=True` also writes
    the drawn id behind the row's history and advances `hist_len`.  Returns ids int64 [n] (and, with
    `return_stats`, float32 [n,4] = (max, kept mass, kept count, mass after top-k))."""
    L = _lib.lib()
    _require_cuda(logits)
    if logits.dim() != 2 or logits.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.QPamError(f"sample_logits: logits must be [n, V] float32 or bfloat16, got {tuple(logits.shape)} {logits.dtype}")
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    n, V = logits.shape
    dev = logits.device
    if uniforms is None:
        uniforms = torch.rand(n, device=dev, dtype=torch.float32)
    if uniforms.dtype != torch.float32 or uniforms.numel() != n or not uniforms.is_cuda:
        raise _lib.QPamError("sample_logits: uniforms must be a float32 CUDA tensor with one entry per row")
    rows = cols = ld = 0
    if history is not None:
        if history.dim() != 2 or history.dtype != torch.int64 or not history.is_cuda or history.stride(1) != 1:
            raise _lib.QPamError("sample_logits: history must be a 2-D int64 CUDA tensor with unit column stride")
        rows, cols, ld = history.shape[0], history.shape[1], history.stride(0)
        if slot_ids is None and rows < n:
            raise _lib.QPamError(f"sample_logits: history has {rows} rows for {n} rows of logits")
    if hist_len is not None and (history is None or hist_len.dtype != torch.int32 or hist_len.numel() != rows or not hist_len.is_cuda):
        raise _lib.QPamError("sample_logits: hist_len must be int32 [history rows] on the device")
    if slot_ids is not None and (slot_ids.dtype != torch.int32 or slot_ids.numel() != n or not slot_ids.is_cuda):
        raise _lib.QPamError("sample_logits: slot_ids must be int32 [n] on the device")
    if append and (history is None or hist_len is None):
        raise _lib.QPamError("sample_logits: append needs history and hist_len")
    ids = torch.empty(n, dtype=torch.int64, device=dev)
    stats = torch.empty(n, 4, dtype=torch.float32, device=dev) if return_stats else None
    need = L.qpam_sample_workspace_bytes(n, V)
    ws = _workspace(need, dev) if need else None
    check(L.qpam_sample_logits(logits.data_ptr(), dtype_code(logits.dtype), n, V, logits.stride(0), float(temperature), int(top_k),
                               float(top_p), float(repetition_penalty), ptr(slot_ids), ptr(history), rows, cols, ld,
                               ptr(hist_len), int(bool(append)), uniforms.data_ptr(), ids.data_ptr(), ptr(stats),
                               ptr(ws), need, stream_ptr()), "qpam_sample_logits")
    return (ids, stats) if return_stats else ids
