"""Fused tied-head linear + cross-entropy: drop-in for the reference's v11/fused_ce.py.

Same names, argument meaning and return types as the reference functions
(``fused_linear_cross_entropy`` v11/fused_ce.py:85-94, ``linear_ce_per_token`` :97-115,
``linear_ce_stats`` :118-141), backed by the CUDA kernels of libqllm2_pam_b200.so.  ``chunk`` is
accepted and ignored: the kernels tile the vocabulary themselves and never hold [rows, V] logits.

An optional ``group`` (a torch.distributed process group) turns on the vocabulary-parallel form:
every rank passes its own row-shard ``weight_matrix`` [V/world, F] with ``vocab_start``; the
per-row (max, sum-exp, target-logit) statistics are all-reduced (NCCL over NVLink), ``grad_H``
is all-reduced and ``grad_W`` stays local to the shard.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def _combine_stats(stats, group):
    """All-reduce shard statistics into global ones: max, rescaled sum-exp, summed target logit."""
    import torch.distributed as dist
    row_max, row_sum, row_tgt, row_arg = stats
    gmax = row_max.clone()
    dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    packed = torch.stack([row_sum * torch.exp(row_max - gmax), row_tgt])
    dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
    # arg-max: the rank holding the global max wins; ties go to the lowest column index
    cand = torch.where(row_max == gmax, row_arg, torch.full_like(row_arg, torch.iinfo(torch.int64).max))
    dist.all_reduce(cand, op=dist.ReduceOp.MIN, group=group)
    return gmax, packed[0].contiguous(), packed[1].contiguous(), cand


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
        dh, dw = ops.ce_backward(h, w, targets, maskf, lse, gs, denom, ignore_index=ignore_index,
                                 v_offset=vocab_start)
        if group is not None:
            import torch.distributed as dist
            dist.all_reduce(dh, op=dist.ReduceOp.SUM, group=group)
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
