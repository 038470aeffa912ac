"""Fused tied-head linear + cross-entropy: drop-in for the reference's v11/fused_ce.py.

Same names, argument meaning and return types as the reference functions
(``fused_linear_cross_entropy`` v11/fused_ce.py:85-94, ``linear_ce_per_token`` :97-115,
``linear_ce_stats`` :118-141), backed by the CUDA kernels of libqllm2_pam_b200.so.  ``chunk`` is
accepted and ignored: the kernels tile the vocabulary themselves and never hold [rows, V] logits.

An optional ``group`` (a torch.distributed process group) turns on the vocabulary-parallel form:
every rank passes its own row-shard ``weight_matrix`` [V/world, F] with ``vocab_start``; the
per-row (max, sum-exp, target-logit, arg-max) statistics cross the group in ONE all-gather (NCCL over
NVLink), ``grad_H`` is all-reduced on a side stream under the ``grad_W`` products, and ``grad_W`` stays
local to the shard.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def _combine_stats(stats, group):
    """Shard statistics -> global ones with ONE exchange: every rank contributes [4, N] floats (max, sum-exp,
    target logit, arg-max column) to an all-gather, and each rank folds the world's rows itself:
    M = max_r m_r,  S = sum_r s_r e^{m_r - M},  target logit = sum_r (only the owner's is non-zero),
    arg-max = lowest column among the ranks that attain M.  (Columns are carried as fp32: exact below 2^24.)"""
    import torch.distributed as dist
    row_max, row_sum, row_tgt, row_arg = stats
    world = dist.get_world_size(group)
    mine = torch.stack([row_max, row_sum, row_tgt, row_arg.to(row_max.dtype)])        # [4, N]
    everyone = torch.empty((world,) + tuple(mine.shape), dtype=mine.dtype, device=mine.device)
    dist.all_gather(list(everyone.unbind(0)), mine, group=group)       # one collective (NCCL and gloo alike)
    m, s_, t, a = everyone[:, 0], everyone[:, 1], everyone[:, 2], everyone[:, 3]
    gmax = m.max(dim=0).values
    gsum = (s_ * torch.exp(m - gmax)).sum(dim=0)
    gtgt = t.sum(dim=0)
    cand = torch.where(m == gmax, a, torch.full_like(a, float(1 << 24)))
    return gmax, gsum, gtgt, cand.min(dim=0).values.to(torch.int64)


_COMM_STREAMS = {}


def _comm_stream(device):
    """One side stream per device for the gradient all-reduce of the vocabulary-parallel form."""
    key = (device.type, device.index)
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = torch.cuda.Stream(device=device)
    return _COMM_STREAMS[key]


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_rows, weight_matrix, targets, mask, ignore_index, group, vocab_start):
        h = hidden_rows.contiguous()
        w = weight_matrix.contiguous()
        if w.dtype != h.dtype:
            w = w.to(h.dtype)
        targets = targets.contiguous()
        maskf = None if mask is None else mask.float().contiguous()
        if maskf is not None and maskf.numel() != h.shape[0]:
            raise ValueError("mask must have one entry per row of hidden_rows")
        ctx.empty = h.shape[0] == 0
        if ctx.empty:   # nothing to launch; the reference returns 0 / clamp_min(1) = 0
            ctx.save_for_backward(h, w)
            return torch.zeros((), dtype=torch.float32, device=h.device)
        stats = ops.ce_row_stats(h, w, targets, ignore_index=ignore_index, v_offset=vocab_start)
        if group is not None:
            stats = _combine_stats(stats, group)
        fin = ops.ce_finalize(h, w, targets, maskf, stats, ignore_index=ignore_index)
        loss = (fin["loss_sum"] / fin["denom"]).reshape(())
        ctx.save_for_backward(h, w, targets, maskf, fin["lse"], fin["denom"])
        ctx.cfg = (ignore_index, group, vocab_start, hidden_rows.dtype, weight_matrix.dtype)
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.empty:
            h, w = ctx.saved_tensors
            return torch.zeros_like(h), torch.zeros_like(w), None, None, None, None, None
        h, w, targets, maskf, lse, denom = ctx.saved_tensors
        ignore_index, group, vocab_start, h_dtype, w_dtype = ctx.cfg
        gs = grad_output.detach().float().reshape(1).contiguous()
        if group is None:
            dh, dw = ops.ce_backward(h, w, targets, maskf, lse, gs, denom, ignore_index=ignore_index, v_offset=vocab_start)
        else:
            # dH of the shards is summed over the group on a side stream that the library releases as soon as dH
            # is complete: the exchange runs under the dW products, which stay local to the shard
            import torch.distributed as dist
            cur, comm = torch.cuda.current_stream(h.device), _comm_stream(h.device)
            dh, dw = ops.ce_backward(h, w, targets, maskf, lse, gs, denom, ignore_index=ignore_index, v_offset=vocab_start,
                                     dh_ready_stream=comm)
            with torch.cuda.stream(comm):
                dist.all_reduce(dh, op=dist.ReduceOp.SUM, group=group)
            dh.record_stream(comm)
            cur.wait_stream(comm)
        return dh.to(h_dtype), dw.to(w_dtype), None, None, None, None, None


def fused_linear_cross_entropy(
    hidden_rows: torch.Tensor,
    weight_matrix: torch.Tensor,
    targets: torch.Tensor,
    mask: Optional[torch.Tensor] = None,
    chunk: int = 4096,
    ignore_index: int = -100,
    group=None,
    vocab_start: int = 0,
) -> torch.Tensor:
    """Mean cross-entropy of (hidden_rows @ weight_matrix.T) vs targets (fp32 0-dim tensor)."""
    del chunk
    return _FusedLinearCE.apply(hidden_rows, weight_matrix, targets, mask, ignore_index, group, vocab_start)


@torch.no_grad()
def linear_ce_per_token(hidden_rows, weight_matrix, targets, chunk: int = 4096, ignore_index: int = -100):
    """Detached per-row cross-entropy [N]; rows whose target is ignore_index give 0.0."""
    del chunk
    h, w = hidden_rows.contiguous(), weight_matrix.contiguous().to(hidden_rows.dtype)
    stats = ops.ce_row_stats(h, w, targets.contiguous(), ignore_index=ignore_index)
    fin = ops.ce_finalize(h, w, targets.contiguous(), None, stats, ignore_index=ignore_index)
    return fin["per_token"].to(hidden_rows.dtype)


@torch.no_grad()
def linear_ce_stats(hidden_rows, weight_matrix, targets, mask=None, chunk: int = 4096, ignore_index: int = -100):
    """(loss_sum, correct, tokens) as Python floats, without materialising logits."""
    del chunk
    h, w = hidden_rows.contiguous(), weight_matrix.contiguous().to(hidden_rows.dtype)
    targets = targets.contiguous()
    maskf = None if mask is None else mask.float().contiguous()
    stats = ops.ce_row_stats(h, w, targets, ignore_index=ignore_index)
    fin = ops.ce_finalize(h, w, targets, maskf, stats, ignore_index=ignore_index)
    vals = torch.cat([fin["loss_sum"], fin["correct"], fin["tokens"]]).tolist()
    return vals[0], vals[1], vals[2]
