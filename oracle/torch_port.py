"""Multi-threaded CPU port of the reference's chunked PAM scan and row-chunked linear+CE.

TEST / BASELINE INFRASTRUCTURE ONLY.  Where no checkout of the reference (a Python/PyTorch project) is
importable, this file restates its CPU code path with the same operator mix -- batched
matmuls per chunk inside a Python chunk loop, autograd for the backward -- so that timing it on
the host cores is a fair stand-in for timing the reference itself
(v11/model.py:354-417 ``_dual_form_block`` + ``_forward_chunked_head``;
v11/fused_ce.py:26-82 ``_FusedLinearCE``).  It is checked against the numpy oracle in
tests/test_oracle_golden.py.  Complex numbers are torch.complex tensors here (one complex
matmul replaces the reference's four real ones; same flops).
"""
from __future__ import annotations

import torch


def to_c(x: torch.Tensor) -> torch.Tensor:
    return torch.view_as_complex(x.contiguous())


def chunked_scan(q, k, v, gamma, chunk: int = 64, eps: float = 1e-6):
    """q,k,v complex [B,H,T,d]; gamma real [B,H,T].  Returns (Y complex, S complex [B,H,d,d])."""
    B, H, T, d = q.shape
    qs = q * (d ** -0.5)
    S = torch.zeros(B, H, d, d, dtype=q.dtype)
    outs = []
    for c0 in range(0, T, chunk):
        c1 = min(c0 + chunk, T)
        qc, kc, vc = qs[:, :, c0:c1], k[:, :, c0:c1], v[:, :, c0:c1]
        a = torch.log(gamma[:, :, c0:c1] + eps)
        cum = torch.cumsum(a, dim=-1)
        diff = cum.unsqueeze(-1) - cum.unsqueeze(-2)
        L = c1 - c0
        tril = torch.tril(torch.ones(L, L, dtype=torch.bool))
        D = torch.where(tril, torch.exp(diff.clamp(max=0.0)), torch.zeros((), dtype=diff.dtype))
        W = qc @ kc.conj().transpose(-1, -2)
        y = (W * D) @ vc
        ecum = torch.exp(cum)
        if c0 > 0:
            y = y + ecum.unsqueeze(-1) * (qc @ S.transpose(-1, -2))
        outs.append(y)
        wv = vc * D[:, :, -1, :].unsqueeze(-1)
        S = S * ecum[:, :, -1, None, None] + wv.transpose(-1, -2) @ kc.conj()
    return torch.cat(outs, dim=2), S


def scan_fwd_bwd(q, k, v, g, dy, chunk: int = 64):
    """Split-real inputs [B,H,T,d,2] (float32), g pre-sigmoid logits; returns (Y, dq, dk, dv, dg)."""
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    g = g.detach().clone().requires_grad_(True)
    y, _ = chunked_scan(to_c(q), to_c(k), to_c(v), torch.sigmoid(g), chunk)
    yr = torch.view_as_real(y)
    grads = torch.autograd.grad(yr, [q, k, v, g], dy)
    return (yr.detach(), *grads)


def linear_ce_fwd_bwd(h, w, targets, chunk: int = 4096, ignore_index: int = -100):
    """Row-chunked CE with recompute in backward, fp32 math (v11/fused_ce.py:26-82)."""
    N, V = h.shape[0], w.shape[0]
    valid = targets != ignore_index
    denom = valid.sum().clamp_min(1).float()
    wf = w.float()
    loss_sum = torch.zeros(())
    for a in range(0, N, chunk):
        b = min(a + chunk, N)
        logits = h[a:b].float() @ wf.T
        loss_sum = loss_sum + torch.nn.functional.cross_entropy(
            logits, targets[a:b], ignore_index=ignore_index, reduction="sum")
    loss = loss_sum / denom
    dh = torch.zeros_like(h)
    dw = torch.zeros_like(w)
    for a in range(0, N, chunk):
        b = min(a + chunk, N)
        hc = h[a:b].float()
        p = torch.softmax(hc @ wf.T, dim=-1)
        t = torch.where(valid[a:b], targets[a:b], torch.zeros_like(targets[a:b]))
        p[torch.arange(b - a), t] -= 1.0
        p = p * (valid[a:b].float() / denom).unsqueeze(1)
        dh[a:b] = (p @ wf).to(dh.dtype)
        dw += (p.T @ hc).to(dw.dtype)
    return loss, dh, dw
