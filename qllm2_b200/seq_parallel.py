"""Sequence-parallel prefill: one long sequence split into contiguous segments over the ranks.

The scan is a linear recurrence, so the state after a segment is  D * S_in + U  with  D = prod(gamma + eps)
over the segment (per state, batch row and head) and U the segment's own contribution from a zero state.
Each rank therefore (1) computes U and D for its segment without forming outputs, (2) all-gathers the pairs
(D, U) -- K*B*H*(d*d*2 + 1) floats per rank, the only exchange -- and folds those of the ranks before it into
the state entering its segment, (3) runs the ordinary forward scan from that state.  The reference has no
multi-device prefill; its chunk loop (v11/model.py:378-417) carries the state the same way inside one device.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

GAMMA_EPS = 1e-6


def fold_segment_states(states: torch.Tensor, decays: torch.Tensor, rank: int, s0: Optional[torch.Tensor] = None):
    """State entering segment `rank`, from every segment's zero-state contribution `states` [W, K, S, H, d, d, 2]
    and total decay `decays` [W, K, S, H]:  S_in(0) = s0 (or 0),  S_in(r+1) = decays[r] * S_in(r) + states[r]."""
    acc = torch.zeros_like(states[0]) if s0 is None else s0.to(states.dtype).reshape(states[0].shape).clone()
    for j in range(rank):
        acc = acc * decays[j][..., None, None, None] + states[j]
    return acc


def segment_decay(gamma: torch.Tensor, eps: float = GAMMA_EPS) -> torch.Tensor:
    """prod_t (gamma_t + eps) over the last axis, accumulated in float64 (gamma [K,B,H,T] -> [K,B,H])."""
    return torch.exp(torch.log(gamma.double() + eps).sum(-1)).float()


@torch.no_grad()
def pam_scan_sequence_parallel(q, k, v, gamma, coef=None, s0=None, *, group=None, head_dim=None, eps: float = GAMMA_EPS,
                               chunk: int = 64, scan: Optional[Callable] = None, scan_states: Optional[Callable] = None):
    """Forward scan of this rank's segment of a sequence that is split over `group` in rank order.

    q, k, v [B,H,T_local,d,2]; gamma [B,H,T_local] or [K,B,H,T_local]; coef optional [K,B,H,T_local,2]; s0 the
    state before the WHOLE sequence (read on every rank, used by the first).  Returns (y of the segment, state
    after the segment); the last rank's state is the state after the whole sequence.  `scan` / `scan_states`
    default to `ops.pam_scan` / `ops.pam_scan_states` (they are parameters so that the exchange can be tested
    without a GPU)."""
    if scan is None or scan_states is None:
        from . import ops
        scan = scan or ops.pam_scan
        scan_states = scan_states or ops.pam_scan_states
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    gamma4 = gamma if gamma.dim() == 4 else gamma.unsqueeze(0)
    if world == 1:
        return scan(q, k, v, gamma4, coef=coef, s0=s0, head_dim=head_dim, eps=eps, chunk=chunk)
    local = scan_states(k, v, gamma4, eps=eps, chunk=chunk).float().contiguous()        # [K,B,H,d,d,2] from a zero state
    decay = segment_decay(gamma4, eps).to(local.device).contiguous()                    # [K,B,H]
    states = [torch.empty_like(local) for _ in range(world)]
    decays = [torch.empty_like(decay) for _ in range(world)]
    dist.all_gather(states, local, group=group)
    dist.all_gather(decays, decay, group=group)
    s_in = fold_segment_states(torch.stack(states), torch.stack(decays), rank, s0)
    return scan(q, k, v, gamma4, coef=coef, s0=s_in, head_dim=head_dim, eps=eps, chunk=chunk)
