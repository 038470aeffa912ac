"""GPU parity of the fused tied-head cross-entropy (v11/fused_ce.py) against oracle + goldens.
Tolerances: loss 1e-5 relative; fp32 grads 1e-4; bf16 grads 2e-2."""
import os

import numpy as np
import pytest
import torch

from oracle import ce_oracle
from qllm2_b200 import fused_ce, ops, synthetic
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_small_golden_ignore_and_mask(golden_dir):
    g = np.load(os.path.join(golden_dir, "ce_small.npz"))
    t = torch.from_numpy(g["t"]).to(DEV)
    for tag, mask in (("", None), ("m_", torch.from_numpy(g["mask"]).float().to(DEV))):
        h = torch.from_numpy(g["h"]).float().to(DEV).requires_grad_(True)
        w = torch.from_numpy(g["w"]).float().to(DEV).requires_grad_(True)
        loss = fused_ce.fused_linear_cross_entropy(h, w, t, mask=mask, chunk=32)
        assert loss.dtype == torch.float32 and loss.dim() == 0
        loss.backward()
        ref = float(g[tag + "loss"])
        assert abs(float(loss) - ref) <= 1e-5 * abs(ref), (float(loss), ref)
        assert_close(h.grad.cpu().numpy(), g[tag + "dh"], 1e-4, tag + "dH")
        assert_close(w.grad.cpu().numpy(), g[tag + "dw"], 1e-4, tag + "dW")
    h = torch.from_numpy(g["h"]).float().to(DEV)
    w = torch.from_numpy(g["w"]).float().to(DEV)
    per = fused_ce.linear_ce_per_token(h, w, t, chunk=32)
    assert_close(per.cpu().numpy(), g["per_token"], 1e-5, "per-token")
    np.testing.assert_allclose(fused_ce.linear_ce_stats(h, w, t), g["stats"], rtol=1e-5)
    np.testing.assert_allclose(fused_ce.linear_ce_stats(h, w, t, mask=torch.from_numpy(g["mask"]).to(DEV)),
                               g["stats_m"], rtol=1e-5)


def test_grad_output_scaling_and_all_ignored():
    gen = torch.Generator().manual_seed(3)
    h = torch.randn(70, 40, generator=gen).to(DEV).requires_grad_(True)
    w = torch.randn(130, 40, generator=gen).to(DEV).requires_grad_(True)
    t = torch.randint(0, 130, (70,), generator=gen).to(DEV)
    (3.0 * fused_ce.fused_linear_cross_entropy(h, w, t)).backward()
    r = ce_oracle.linear_ce(h.detach().cpu().numpy(), w.detach().cpu().numpy(), t.cpu().numpy(), grad_output=3.0)
    assert_close(h.grad.cpu().numpy(), r["dH"], 1e-4, "dH x3")
    assert_close(w.grad.cpu().numpy(), r["dW"], 1e-4, "dW x3")
    h.grad = None
    w.grad = None
    loss = fused_ce.fused_linear_cross_entropy(h, w, torch.full_like(t, -100))
    loss.backward()
    assert float(loss) == 0.0 and float(h.grad.abs().max()) == 0.0 and float(w.grad.abs().max()) == 0.0


def test_config2_bf16(golden_dir):
    """N=8192, F=768, V=50261 bf16: loss within 1e-5 of the reference; grads within 2e-2."""
    g = np.load(os.path.join(golden_dir, "ce_c2.npz"))
    c2 = synthetic.config2()
    h = c2.h.to(DEV).requires_grad_(True)
    w = c2.w.to(DEV).requires_grad_(True)
    loss = fused_ce.fused_linear_cross_entropy(h, w, c2.targets.to(DEV))
    loss.backward()
    ref = float(g["loss32"])
    assert abs(float(loss) - ref) <= 1e-5 * ref, (float(loss), ref)
    assert h.grad.dtype == torch.bfloat16 and w.grad.dtype == torch.bfloat16
    rows, vrows = torch.from_numpy(g["rows"]), torch.from_numpy(g["vrows"])
    assert_close(h.grad[rows.to(DEV)].float().cpu().numpy(), g["dh32"], 2e-2, "dH rows")
    assert_close(w.grad[vrows.to(DEV)].float().cpu().numpy(), g["dw32"], 2e-2, "dW rows")
    assert abs(float(h.grad.float().norm()) - float(g["dh_norm"])) <= 2e-2 * float(g["dh_norm"])
    assert abs(float(w.grad.float().norm()) - float(g["dw_norm"])) <= 2e-2 * float(g["dw_norm"])


def test_head_argmax_and_vocab_shards():
    """Greedy head ids equal the oracle's argmax; shard statistics with v_offset combine exactly."""
    c = synthetic.ce_inputs(96, 24, 1000, seed=9, dtype=torch.float32)
    h, w, t = c.h.to(DEV), c.w.to(DEV) * 50, c.targets.to(DEV)
    ids, best = ops.head_argmax(h, w)
    z = ce_oracle.head_logits(h.cpu().numpy(), w.cpu().numpy())
    assert np.array_equal(ids.cpu().numpy(), z.argmax(1))
    assert_close(best.cpu().numpy(), z.max(1), 1e-5, "best logit")
    full = ops.ce_row_stats(h, w, t)
    a = ops.ce_row_stats(h, w[:437].contiguous(), t, v_offset=0)
    b = ops.ce_row_stats(h, w[437:].contiguous(), t, v_offset=437)
    m = torch.maximum(a[0], b[0])
    s = a[1] * torch.exp(a[0] - m) + b[1] * torch.exp(b[0] - m)
    lse_full = full[0] + torch.log(full[1])
    assert_close((m + torch.log(s)).cpu().numpy(), lse_full.cpu().numpy(), 1e-6, "sharded lse")
    assert_close((a[2] + b[2]).cpu().numpy(), full[2].cpu().numpy(), 1e-6, "sharded target logit")
    arg = torch.where(a[0] >= b[0], a[3], b[3])
    assert np.array_equal(arg.cpu().numpy(), full[3].cpu().numpy())


def test_empty_batch():
    h = torch.zeros(0, 16, device=DEV, requires_grad=True)
    w = torch.randn(33, 16, device=DEV, requires_grad=True)
    t = torch.zeros(0, dtype=torch.int64, device=DEV)
    loss = fused_ce.fused_linear_cross_entropy(h, w, t)
    loss.backward()
    assert float(loss) == 0.0 and float(w.grad.abs().max()) == 0.0
