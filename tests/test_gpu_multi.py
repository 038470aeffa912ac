"""Multi-GPU paths (skipped on a single-GPU box): vocabulary-parallel fused cross-entropy over NCCL
equals the single-GPU result; the scan shards by (batch, head) with no collective."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]


def _ce_rank(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from qllm2_b200 import fused_ce, synthetic
    c = synthetic.ce_inputs(1000, 64, 5003, seed=1, dtype=torch.bfloat16)
    dev = f"cuda:{rank}"
    V = c.w.shape[0]
    lo, hi = rank * V // world, (rank + 1) * V // world
    h = c.h.to(dev).requires_grad_(True)
    w_full = (c.w.float() * 20).bfloat16()
    w = w_full[lo:hi].contiguous().to(dev).requires_grad_(True)
    t = c.targets.to(dev)
    loss = fused_ce.fused_linear_cross_entropy(h, w, t, group=dist.group.WORLD, vocab_start=lo)
    loss.backward()
    if rank == 0:
        h1 = c.h.to(dev).requires_grad_(True)
        w1 = w_full.to(dev).requires_grad_(True)
        l1 = fused_ce.fused_linear_cross_entropy(h1, w1, t)
        l1.backward()
        ret["loss"] = (float(loss.detach()), float(l1.detach()))
        ret["dh_err"] = float((h.grad.float() - h1.grad.float()).norm() / h1.grad.float().norm())
        ret["dw_err"] = float((w.grad.float() - w1.grad[lo:hi].float()).norm() / w1.grad[lo:hi].float().norm())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_vocab_parallel_ce_two_gpus():
    ret = mp.Manager().dict()
    mp.spawn(_ce_rank, args=(2, _free_port(), ret), nprocs=2, join=True)
    a, b = ret["loss"]
    assert abs(a - b) <= 1e-5 * abs(b), (a, b)
    assert ret["dh_err"] < 1e-2 and ret["dw_err"] < 1e-2, dict(ret)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_scan_head_shards_equal_unsharded():
    """Heads split over two GPUs (no exchange) reproduce the single-GPU result bit for bit."""
    from qllm2_b200 import ops, synthetic
    inp = synthetic.scan_inputs(1, 4, 700, 64, seed=3, dtype=torch.bfloat16)
    full, _ = ops.pam_scan(inp.q.cuda(0), inp.k.cuda(0), inp.v.cuda(0), inp.gamma.cuda(0))
    parts = []
    for r in range(2):
        torch.cuda.set_device(r)
        sl = slice(2 * r, 2 * r + 2)
        y, _ = ops.pam_scan(inp.q[:, sl].contiguous().cuda(r), inp.k[:, sl].contiguous().cuda(r),
                            inp.v[:, sl].contiguous().cuda(r), inp.gamma[:, sl].contiguous().cuda(r))
        parts.append(y.cpu())
    torch.cuda.set_device(0)
    assert torch.equal(torch.cat(parts, dim=1), full.cpu())


def _seqpar_rank(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from qllm2_b200 import ops
    from qllm2_b200.seq_parallel import pam_scan_sequence_parallel
    dev = f"cuda:{rank}"
    for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        gen = torch.Generator().manual_seed(5)
        B, H, T, d, K = 1, 3, 1000, 64, 3
        q, k, v = (torch.randn(B, H, T, d, 2, generator=gen).mul(0.125).to(dtype) for _ in range(3))
        gamma = torch.sigmoid(torch.randn(K, B, H, T, generator=gen) + 3)
        coef = torch.randn(K, B, H, T, 2, generator=gen)
        cut = [0, 437, T]                                              # segments need not align with the kernels' chunks
        sl = slice(cut[rank], cut[rank + 1])
        y, s = pam_scan_sequence_parallel(q[:, :, sl].contiguous().to(dev), k[:, :, sl].contiguous().to(dev),
                                          v[:, :, sl].contiguous().to(dev), gamma[..., sl].contiguous().to(dev),
                                          coef=coef[:, :, :, sl].contiguous().to(dev), group=dist.group.WORLD)
        y_full, s_full = ops.pam_scan(q.to(dev), k.to(dev), v.to(dev), gamma.to(dev), coef=coef.to(dev))
        ref = y_full[:, :, sl].float()
        ret[f"y_{tag}_{rank}"] = float((y.float() - ref).norm() / ref.norm())
        if rank == world - 1:
            ret[f"s_{tag}"] = float((s - s_full).norm() / s_full.norm())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sequence_parallel_prefill_two_gpus():
    """One sequence split 437 + 563 tokens over two GPUs with a single (decay, state) all-gather: every
    segment's output and the final state equal the unsplit scan (fp32 1e-4, bf16 2e-2)."""
    ret = mp.Manager().dict()
    mp.spawn(_seqpar_rank, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        assert ret[f"y_f32_{r}"] < 1e-4 and ret[f"y_bf16_{r}"] < 2e-2, dict(ret)
    assert ret["s_f32"] < 1e-4 and ret["s_bf16"] < 2e-2, dict(ret)
