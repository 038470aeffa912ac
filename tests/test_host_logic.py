"""Host-side logic that needs no GPU: the slot scheduler of the continuous batcher and the
vocabulary-parallel combination of cross-entropy statistics (2 gloo ranks on CPU)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ce_oracle
from qllm2_b200.serving import SlotScheduler


def test_scheduler_join_leave_without_reallocation():
    s = SlotScheduler(n_slots=3, max_prefill_tokens=100)
    for i in range(5):
        s.submit([1] * (10 + i), max_new_tokens=2 + (i % 2))
    first = s.admit()
    assert [r.rid for r in first] == [0, 1, 2] and sorted(r.slot for r in first) == [0, 1, 2]
    assert s.admit() == []                       # pool exhausted: the rest waits
    for r in first:
        r.generated.append(7)
    assert s.retire_finished() == []
    first[0].generated.append(7)                 # rid 0 reaches max_new_tokens == 2
    done = s.retire_finished()
    assert [r.rid for r in done] == [0]
    nxt = s.admit()
    assert [r.rid for r in nxt] == [3] and nxt[0].slot == done[0].slot   # the freed slot is reused
    assert first[1].position == len(first[1].prompt) + 1 - 1
    with pytest.raises(ValueError):
        s.submit([], 1)
    with pytest.raises(ValueError):
        SlotScheduler(0)


def test_scheduler_prefill_token_budget():
    s = SlotScheduler(n_slots=8, max_prefill_tokens=25)
    for n in (10, 10, 10, 40):
        s.submit([0] * n, 1)
    assert [len(r.prompt) for r in s.admit()] == [10, 10]
    assert [len(r.prompt) for r in s.admit()] == [10]
    assert [len(r.prompt) for r in s.admit()] == [40]   # an over-budget prompt still runs, alone
    assert s.admit() == [] and not s.idle


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _rank_main(rank, world, port, V, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from qllm2_b200.fused_ce import _combine_stats
    gen = torch.Generator().manual_seed(0)
    N, F = 37, 8
    h = torch.randn(N, F, generator=gen, dtype=torch.float64)
    w = torch.randn(V, F, generator=gen, dtype=torch.float64)
    t = torch.randint(0, V, (N,), generator=gen)
    lo, hi = rank * V // world, (rank + 1) * V // world
    z = h @ w[lo:hi].T                                           # this rank's logits (stand-in for the kernel)
    row_max = z.max(1).values
    row_sum = torch.exp(z - row_max[:, None]).sum(1)
    own = (t >= lo) & (t < hi)
    row_tgt = torch.where(own, z[torch.arange(N), (t - lo).clamp(0, hi - lo - 1)], torch.zeros(N, dtype=torch.float64))
    row_arg = z.argmax(1) + lo
    gmax, gsum, gtgt, garg = _combine_stats((row_max, row_sum, row_tgt, row_arg), None)
    if rank == 0:
        ref = ce_oracle.linear_ce(h.numpy(), w.numpy(), t.numpy(), want_grads=False)
        lse = (gmax + torch.log(gsum)).numpy()
        ret["lse_err"] = float(np.abs(lse - ref["lse"]).max())
        ret["loss_err"] = float(abs((lse - gtgt.numpy()).mean() - ref["loss"]))
        ret["argmax_ok"] = bool(np.array_equal(garg.numpy(), ref["argmax"]))
    dist.destroy_process_group()


def test_vocab_parallel_stats_two_ranks():
    """Sharded (max, sum-exp, target logit, arg-max) combine to the unsharded values."""
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, 101, ret), nprocs=2, join=True)
    assert ret["lse_err"] < 1e-12 and ret["loss_err"] < 1e-12 and ret["argmax_ok"]


# ------------------------------------------------------------------ sequence-parallel prefill (2 gloo ranks)
def _oracle_scan(q, k, v, gamma, coef=None, s0=None, head_dim=None, eps=1e-6, chunk=64):
    from oracle import pam_oracle as po
    cz = None if coef is None else po.to_complex(coef.numpy())
    sz = None if s0 is None else po.to_complex(s0.double().numpy())
    Y, S = po.scan_recurrence(po.to_complex(q.numpy()), po.to_complex(k.numpy()), po.to_complex(v.numpy()), gamma.numpy(),
                              head_dim=head_dim, eps=eps, s0=sz, coef=cz)
    return torch.from_numpy(po.to_split(Y)), torch.from_numpy(po.to_split(S))


def _oracle_states(k, v, gamma, eps=1e-6, chunk=64):
    return _oracle_scan(torch.zeros_like(k), k, v, gamma, eps=eps)[1]


def _seqpar_rank(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from qllm2_b200.seq_parallel import pam_scan_sequence_parallel
    gen = torch.Generator().manual_seed(0)
    B, H, T, d, K = 2, 2, 23, 4, 3
    q, k, v = (torch.randn(B, H, T, d, 2, generator=gen, dtype=torch.float64) * 0.5 for _ in range(3))
    gamma = torch.sigmoid(torch.randn(K, B, H, T, generator=gen, dtype=torch.float64) + 2)
    coef = torch.randn(K, B, H, T, 2, generator=gen, dtype=torch.float64)
    s0 = torch.randn(K, B, H, d, d, 2, generator=gen, dtype=torch.float64) * 0.1
    cut = [0, 9, T]                                                   # ragged split: 9 and 14 tokens
    sl = slice(cut[rank], cut[rank + 1])
    y, s = pam_scan_sequence_parallel(q[:, :, sl], k[:, :, sl], v[:, :, sl], gamma[..., sl], coef=coef[:, :, :, sl], s0=s0,
                                      scan=_oracle_scan, scan_states=_oracle_states)
    y_full, s_full = _oracle_scan(q, k, v, gamma, coef=coef, s0=s0)
    ret[f"y{rank}"] = float((y - y_full[:, :, sl]).abs().max())
    if rank == world - 1:
        ret["s"] = float((s.double() - s_full).abs().max())
    dist.destroy_process_group()


def test_sequence_parallel_prefill_two_ranks():
    """Two segments of one sequence, (decay, state) exchanged once: outputs and final state equal the
    unsplit scan (oracle arithmetic, float64)."""
    ret = mp.Manager().dict()
    mp.spawn(_seqpar_rank, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["y0"] < 1e-6 and ret["y1"] < 1e-6 and ret["s"] < 1e-6, dict(ret)


def test_fold_segment_states_is_the_linear_recurrence():
    from qllm2_b200.seq_parallel import fold_segment_states, segment_decay
    gen = torch.Generator().manual_seed(1)
    W = 4
    states = torch.randn(W, 2, 1, 3, 2, 2, 2, generator=gen, dtype=torch.float64)
    decays = torch.rand(W, 2, 1, 3, generator=gen, dtype=torch.float64)
    s0 = torch.randn(2, 1, 3, 2, 2, 2, generator=gen, dtype=torch.float64)
    cur = s0.clone()
    for r in range(W):
        assert torch.allclose(fold_segment_states(states, decays, r, s0), cur)
        cur = cur * decays[r][..., None, None, None] + states[r]
    g = torch.rand(2, 1, 3, 50, generator=gen) * 0.5 + 0.5
    assert torch.allclose(segment_decay(g, 1e-6), (g.double() + 1e-6).prod(-1).float(), rtol=1e-5)


def test_scheduler_chunked_prefill_plan():
    """With chunked prefill a prompt longer than the budget is absorbed over several steps, resumed pieces
    first, and the budget is never exceeded."""
    s = SlotScheduler(n_slots=2, max_prefill_tokens=25, chunked_prefill=True)
    a, b, c = s.submit([0] * 40, 1), s.submit([0] * 10, 1), s.submit([0] * 7, 1)
    plan = s.plan_prefill()
    assert [(r.rid, st, n) for r, st, n in plan] == [(a, 0, 25)]          # budget spent on the first piece
    for r, st, n in plan:
        r.prefilled = st + n
    plan = s.plan_prefill()
    assert [(r.rid, st, n) for r, st, n in plan] == [(a, 25, 15), (b, 0, 10)]
    for r, st, n in plan:
        r.prefilled = st + n
    assert s.plan_prefill() == []                                          # both slots taken, nothing left to prefill
    assert not s.live[0].prefilling and not s.live[1].prefilling and len(s.waiting) == 1
    for r in s.live_requests():
        r.generated.append(1)
    s.retire_finished()
    assert [(r.rid, st, n) for r, st, n in s.plan_prefill()] == [(c, 0, 7)]
    # whole-prompt mode keeps the old contract
    w = SlotScheduler(n_slots=4, max_prefill_tokens=25)
    for n in (10, 10, 10):
        w.submit([0] * n, 1)
    assert [(st, n) for _, st, n in w.plan_prefill()] == [(0, 10), (0, 10)]
    with pytest.raises(ValueError):
        SlotScheduler(1, max_prefill_tokens=0)
