"""Tensor-core (tcgen05) path of the fused cross-entropy: bf16 inputs of assorted shapes vs the
fp64 oracle on the same bf16-rounded values.  Loss 1e-5 relative, gradients 2e-2 relative."""
import numpy as np
import pytest
import torch

from oracle import ce_oracle
from qllm2_b200 import _lib, fused_ce, ops, synthetic
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("N,D,V", [(128, 32, 256), (300, 64, 1000), (64, 32, 130), (1000, 96, 5003), (129, 8, 257)])
def test_bf16_shapes(N, D, V):
    c = synthetic.ce_inputs(N, D, V, seed=N + V, dtype=torch.bfloat16)
    w_host = (c.w.float() * 20).bfloat16()          # spread the logits so softmax is not flat
    t_host = c.targets.clone()
    t_host[::5] = -100
    h = c.h.to(DEV).requires_grad_(True)
    w = w_host.to(DEV).requires_grad_(True)
    t = t_host.to(DEV)
    loss = fused_ce.fused_linear_cross_entropy(h, w, t)
    loss.backward()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    r = ce_oracle.linear_ce(c.h.float().numpy(), w_host.float().numpy(), t_host.numpy())
    assert abs(float(loss.detach()) - r["loss"]) <= 1e-5 * abs(r["loss"]), (float(loss.detach()), r["loss"])
    assert_close(h.grad.float().cpu().numpy(), r["dH"], 2e-2, "dH")
    assert_close(w.grad.float().cpu().numpy(), r["dW"], 2e-2, "dW")
    ids, best = ops.head_argmax(h.detach(), w.detach())
    z = ce_oracle.head_logits(c.h.float().numpy(), w_host.float().numpy())
    top2 = np.sort(z, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 1e-4       # ignore numerically tied rows
    assert np.array_equal(ids.cpu().numpy()[clear], z.argmax(1)[clear])
    assert_close(best.cpu().numpy(), z.max(1), 1e-5, "best logit")


def test_masked_and_scaled():
    c = synthetic.ce_inputs(260, 64, 700, seed=3, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(1)
    mask = (torch.rand(260, generator=gen) > 0.4).float()
    h = c.h.to(DEV).requires_grad_(True)
    w = (c.w.float() * 20).bfloat16().to(DEV).requires_grad_(True)
    loss = fused_ce.fused_linear_cross_entropy(h, w, c.targets.to(DEV), mask=mask.to(DEV))
    (2.5 * loss).backward()
    r = ce_oracle.linear_ce(c.h.float().numpy(), w.detach().float().cpu().numpy(), c.targets.numpy(),
                            mask=mask.numpy(), grad_output=2.5)
    assert abs(float(loss.detach()) - r["loss"]) <= 1e-5 * abs(r["loss"])
    assert_close(h.grad.float().cpu().numpy(), r["dH"], 2e-2, "dH")
    assert_close(w.grad.float().cpu().numpy(), r["dW"], 2e-2, "dW")
    assert _lib.device_status() == 0


@pytest.mark.parametrize("N", [8192 + 300, 4 * 8192 + 200])
def test_many_row_chunks(N):
    """Backward over several row chunks: two chunks sum dW in buffers of their own, a fifth chunk adds into the
    first buffer again.  Checked against fp64 arithmetic on the same bf16 values (numpy, vectorised)."""
    D, V = 32, 520
    c = synthetic.ce_inputs(N, D, V, seed=11, dtype=torch.bfloat16)
    w_host = (c.w.float() * 20).bfloat16()
    t_host = c.targets.clone()
    t_host[::7] = -100
    h = c.h.to(DEV).requires_grad_(True)
    w = w_host.to(DEV).requires_grad_(True)
    loss = fused_ce.fused_linear_cross_entropy(h, w, t_host.to(DEV))
    loss.backward()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    r = ce_oracle.linear_ce(c.h.float().numpy(), w_host.float().numpy(), t_host.numpy())
    assert abs(float(loss.detach()) - r["loss"]) <= 1e-5 * abs(r["loss"])
    assert_close(h.grad.float().cpu().numpy(), r["dH"], 2e-2, "dH")
    assert_close(w.grad.float().cpu().numpy(), r["dW"], 2e-2, "dW")


@pytest.mark.parametrize("N,D,V", [(8191, 32, 1000), (257, 4, 9), (640, 100, 4099), (5, 32, 100000), (127, 36, 255)])
def test_odd_shapes_masked_scaled(N, D, V):
    """Rows one short of a chunk, fewer columns than one tile, a vocabulary of one row tile of logits per
    hundred thousand columns, widths that are not a power of two; mask, ignored rows and an upstream factor."""
    c = synthetic.ce_inputs(N, D, V, seed=N + 3 * V, dtype=torch.bfloat16)
    w_host = (c.w.float() * 20).bfloat16()
    t_host = c.targets.clone()
    t_host[::9] = -100
    gen = torch.Generator().manual_seed(N)
    mask = (torch.rand(N, generator=gen) > 0.2).float()
    h = c.h.to(DEV).requires_grad_(True)
    w = w_host.to(DEV).requires_grad_(True)
    loss = fused_ce.fused_linear_cross_entropy(h, w, t_host.to(DEV), mask=mask.to(DEV))
    (1.7 * loss).backward()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    r = ce_oracle.linear_ce(c.h.float().numpy(), w_host.float().numpy(), t_host.numpy(), mask=mask.numpy(),
                            grad_output=1.7)
    assert abs(float(loss.detach()) - r["loss"]) <= 1e-5 * abs(r["loss"])
    assert_close(h.grad.float().cpu().numpy(), r["dH"], 2e-2, "dH")
    assert_close(w.grad.float().cpu().numpy(), r["dW"], 2e-2, "dW")


def test_vocabulary_shard_statistics_with_ragged_last_group():
    """Row statistics of a vocabulary shard whose width is not a multiple of 32, with targets that live in the
    OTHER shard just past its last column: max, sum-exp and arg-max match the shard's logits, the target logit is
    the logit for rows whose target is inside the shard and exactly 0 otherwise (never a padding value)."""
    N, F, V = 300, 64, 1003
    g = torch.Generator().manual_seed(31)
    h = (torch.randn(N, F, generator=g) * 0.5).bfloat16().to("cuda")
    w = (torch.randn(V, F, generator=g) * 0.5).bfloat16().to("cuda")
    split = 501                                                        # 501 = 15 * 32 + 21
    t = torch.randint(0, V, (N,), generator=g)
    t[:40] = torch.arange(split, split + 40) % V                        # targets in the first columns of shard 1
    t = t.to("cuda")
    for a, b in ((0, split), (split, V)):
        ws = w[a:b].contiguous()
        m, s, tz, arg = ops.ce_row_stats(h, ws, t, v_offset=a)
        lg = h.float() @ ws.float().T
        mr = lg.max(1).values
        assert torch.isfinite(tz).all() and torch.isfinite(s).all()
        assert float((m - mr).abs().max()) < 1e-4
        assert float(((s - torch.exp(lg - mr[:, None]).sum(1)) / s).abs().max()) < 1e-4
        assert torch.equal(arg, lg.argmax(1) + a)
        inside = (t >= a) & (t < b)
        want = torch.where(inside, lg.gather(1, (t - a).clamp(0, b - a - 1)[:, None])[:, 0], torch.zeros_like(mr))
        assert float((tz - want).abs().max()) < 1e-4


@pytest.mark.parametrize("N,F,V", [(256, 1536, 50261), (1, 64, 9), (130, 72, 1001), (300, 768, 4096)])
def test_head_logits_bf16_tiles(N, F, V):
    """Sampling decode head: bf16 logits of the tensor-core GEMM against the fp64 product of the same bf16 inputs
    (relative to the largest logit: 2^-8, one bf16 rounding of the output)."""
    g = torch.Generator().manual_seed(N + V)
    h = torch.randn(N, F, generator=g).bfloat16()
    w = (torch.randn(V, F, generator=g) * (4.0 / F ** 0.5)).bfloat16()
    z = ops.head_logits(h.to(DEV), w.to(DEV))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert z.shape == (N, V) and z.dtype == torch.bfloat16
    ref = ce_oracle.head_logits(h.float().numpy(), w.float().numpy())
    err = np.abs(z.float().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err <= 2.0 ** -8, err
