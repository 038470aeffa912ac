"""CPU oracle for the fused tied complex LM head + cross-entropy.

TEST INFRASTRUCTURE ONLY (see oracle/pam_oracle.py).  Restates in numpy float64 the
row-chunked linear + cross-entropy of the reference, v11/fused_ce.py:26-141, and the
tied complex head of v11/model.py:1136-1139,1175-1190:

    logits = lm_r @ E_r^T + lm_i @ E_i^T = [lm_r | lm_i] @ [E_r | E_i]^T = H @ W^T

loss      = sum_rows(mask_r * (lse_r - logit_r[target_r])) / denom
denom     = count(target != ignore_index).clamp_min(1)     (no mask)
          = mask.sum().clamp_min(1.0)                      (mask given)
rows whose target == ignore_index contribute 0 loss and 0 gradient
grad_H    = ((softmax - onehot) * scale_r) @ W,  grad_W = (...)^T @ H
scale_r   = grad_output / denom * mask_r
"""
from __future__ import annotations

import numpy as np


def tied_head_matrices(lm, embed_real, embed_imag):
    """lm [..., D, 2] -> H [N, 2D];  (E_r, E_i) [V, D] -> W [V, 2D]  (v11/model.py:1184-1185)."""
    lm = np.asarray(lm, dtype=np.float64)
    H = np.concatenate([lm[..., 0], lm[..., 1]], axis=-1).reshape(-1, 2 * lm.shape[-2])
    W = np.concatenate([np.asarray(embed_real, np.float64), np.asarray(embed_imag, np.float64)], axis=-1)
    return H, W


def _row_stats(H, W, targets, ignore_index, rows=1024):
    N = H.shape[0]
    lse = np.empty(N)
    tgt = np.zeros(N)
    amax = np.empty(N, dtype=np.int64)
    for a in range(0, N, rows):
        b = min(a + rows, N)
        z = H[a:b] @ W.T
        m = z.max(axis=1)
        lse[a:b] = m + np.log(np.exp(z - m[:, None]).sum(axis=1))
        amax[a:b] = z.argmax(axis=1)
        t = targets[a:b]
        ok = t != ignore_index
        tgt[a:b][ok] = z[np.arange(b - a)[ok], t[ok]]
    return lse, tgt, amax


def linear_ce(H, W, targets, mask=None, ignore_index=-100, grad_output=1.0, want_grads=True,
              rows=1024):
    """Returns dict(loss, denom, lse[N], per_token[N], dH, dW).  v11/fused_ce.py:26-82."""
    H = np.asarray(H, dtype=np.float64)
    W = np.asarray(W, dtype=np.float64)
    targets = np.asarray(targets, dtype=np.int64)
    N = H.shape[0]
    valid = targets != ignore_index
    if mask is not None:
        mask = np.asarray(mask, dtype=np.float64)
        denom = max(mask.sum(), 1.0)
    else:
        denom = float(max(valid.sum(), 1))
    lse, tgt, amax = _row_stats(H, W, targets, ignore_index, rows)
    per_token = np.where(valid, lse - tgt, 0.0)
    weighted = per_token * (mask if mask is not None else 1.0)
    out = dict(loss=weighted.sum() / denom, denom=denom, lse=lse, per_token=per_token,
               argmax=amax)
    if not want_grads:
        return out
    scale = np.full(N, grad_output / denom)
    if mask is not None:
        scale = scale * mask
    scale = scale * valid
    dH = np.zeros_like(H)
    dW = np.zeros_like(W)
    safe_t = np.where(valid, targets, 0)
    for a in range(0, N, rows):
        b = min(a + rows, N)
        p = np.exp(H[a:b] @ W.T - lse[a:b, None])
        p[np.arange(b - a), safe_t[a:b]] -= 1.0
        p *= scale[a:b, None]
        dH[a:b] = p @ W
        dW += p.T @ H[a:b]
    out.update(dH=dH, dW=dW)
    return out


def linear_ce_per_token(H, W, targets, ignore_index=-100):
    """Per-row CE [N], 0 at ignored rows.  v11/fused_ce.py:97-115."""
    return linear_ce(H, W, targets, ignore_index=ignore_index, want_grads=False)['per_token']


def linear_ce_stats(H, W, targets, mask=None, ignore_index=-100):
    """(loss_sum, correct, tokens).  v11/fused_ce.py:118-141."""
    r = linear_ce(H, W, targets, ignore_index=ignore_index, want_grads=False)
    targets = np.asarray(targets)
    tm = np.asarray(mask, np.float64) if mask is not None else (targets != ignore_index).astype(np.float64)
    correct = (r['argmax'] == targets).astype(np.float64)
    return float((r['per_token'] * tm).sum()), float((correct * tm).sum()), float(tm.sum())


def head_logits(H, W):
    """Full logits (decode head), v11/model.py:1136-1139."""
    return np.asarray(H, np.float64) @ np.asarray(W, np.float64).T
