"""Seeded random shapes of the fused tied-head cross-entropy (bf16, tensor-core path; fp32, CUDA-core path) against the
fp64 oracle: loss, dH, dW with ignored targets, a per-row mask and a scaled upstream gradient.  The reference is
`_FusedLinearCE` (v11/fused_ce.py:26-94).  Shapes are drawn so that rows, features and vocabulary are rarely a multiple
of any tile size (128-row tiles, 256-column tiles, 64-deep K blocks, 8192-row chunks of the backward)."""
import numpy as np
import pytest
import torch

from oracle import ce_oracle
from tests.helpers import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _shape(seed):
    rng = np.random.default_rng(4000 + seed)
    fixed = [(8193, 64, 1000), (257, 8, 9), (4097, 128, 5003), (5, 64, 20011), (127, 72, 255), (129, 24, 513)]
    if seed < len(fixed):
        return fixed[seed]
    return int(rng.integers(1, 3000)), 8 * int(rng.integers(1, 40)), int(rng.integers(2, 9000))


@pytest.mark.parametrize("seed,dtype", [(i, torch.bfloat16) for i in range(12)] + [(i, torch.float32) for i in (1, 7, 9)])
def test_random_shape_loss_and_gradients(seed, dtype):
    from qllm2_b200 import _lib, fused_ce
    N, F, V = _shape(seed)
    g = torch.Generator().manual_seed(seed)
    h_host = torch.randn(N, F, generator=g).to(dtype)
    w_host = (torch.randn(V, F, generator=g) * (4.0 / F ** 0.5)).to(dtype)      # logits of a few units: softmax not flat
    t_host = torch.randint(0, V, (N,), generator=g)
    t_host[::9] = -100
    mask_host = (torch.rand(N, generator=g) > 0.2).float()
    h = h_host.to(DEV).requires_grad_(True)
    w = w_host.to(DEV).requires_grad_(True)
    loss = fused_ce.fused_linear_cross_entropy(h, w, t_host.to(DEV), mask=mask_host.to(DEV))
    (1.7 * loss).backward()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    r = ce_oracle.linear_ce(h_host.float().numpy(), w_host.float().numpy(), t_host.numpy(), mask=mask_host.numpy(),
                            grad_output=1.7)
    what = f"seed {seed} {dtype}: N={N} F={F} V={V}"
    ltol, gtol = (1e-5, 2e-2) if dtype == torch.bfloat16 else (1e-5, 1e-4)
    assert abs(float(loss.detach()) - r["loss"]) <= ltol * max(abs(r["loss"]), 1e-9), (what, float(loss.detach()), r["loss"])
    for name, got, ref in (("dH", h.grad, r["dH"]), ("dW", w.grad, r["dW"])):
        got = got.float().cpu().numpy()
        assert np.isfinite(got).all(), f"{what}: {name} not finite"
        if not np.any(ref):
            assert not np.any(got), f"{what}: {name} should be zero"
            continue
        e = rel_err(got, ref)
        assert e <= gtol, f"{what}: {name} rel {e:.3e} > {gtol:.0e}"
