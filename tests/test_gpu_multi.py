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
