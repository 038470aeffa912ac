"""GPU parity of the recurrent decode step over a slot pool (v11/model.py:927-965)."""
import os

import numpy as np
import pytest
import torch

from oracle import pam_oracle as po
from qllm2_b200 import ops
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_step_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "recur_step.npz"))
    B, H, d = g["S"].shape[:3]
    pool = torch.zeros(B + 3, 1, 1, H, d, d, 2, device=DEV)
    slots = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    ops.pam_pool_store(pool, slots, torch.from_numpy(g["S"]).float()[None].to(DEV))
    f = lambda name: torch.from_numpy(g[name]).float().to(DEV)
    y = ops.pam_decode_step(pool, slots, f("q"), f("k"), f("v"), f("gamma"))
    assert_close(y.cpu().numpy(), g["y"], 1e-5, "y")
    assert_close(pool[slots.long(), 0, 0].cpu().numpy(), g["S_new"], 1e-5, "S_new")
    untouched = [i for i in range(B + 3) if i not in (4, 1)]
    assert float(pool[untouched].abs().max()) == 0.0


@pytest.mark.parametrize("d,K,state_dtype,io_dtype", [
    (64, 3, torch.float32, torch.float32), (64, 3, torch.bfloat16, torch.bfloat16),
    (32, 1, torch.float32, torch.bfloat16), (16, 2, torch.bfloat16, torch.float32),
    (64, 1, torch.float32, torch.float32)])
def test_multi_step_vs_oracle(d, K, state_dtype, io_dtype):
    """Several steps with sequences joining/leaving (slot ids change between steps)."""
    n_slots, L, H = 9, 2, 3
    gen = torch.Generator().manual_seed(d + K)
    pool = torch.zeros(n_slots, L, K, H, d, d, 2, dtype=state_dtype, device=DEV)
    ref = np.zeros((n_slots, L, K, H, d, d), dtype=np.complex128)
    tol = 1e-5 if (state_dtype == torch.float32 and io_dtype == torch.float32) else 2e-2
    live_sets = [[0, 5, 2], [0, 5, 2, 7], [5, 7], [8, 5, 7, 1, 3]]
    for step, live in enumerate(live_sets):
        n = len(live)
        layer = step % L
        q, k, v = (torch.randn(n, H, d, 2, generator=gen).to(io_dtype) * 0.3 for _ in range(3))
        gamma = torch.sigmoid(torch.randn(K, n, H, generator=gen) + 2)
        coef = torch.randn(K, n, H, 2, generator=gen)
        slots = torch.tensor(live, dtype=torch.int32)
        y = ops.pam_decode_step(pool, slots.to(DEV), q.to(DEV), k.to(DEV), v.to(DEV), gamma.to(DEV),
                                coef.to(DEV), layer=layer)
        S_in = np.transpose(ref[live, layer], (1, 0, 2, 3, 4))          # [K,n,H,d,d]
        y_ref, S_new = po.recurrent_step(S_in, gamma.double().numpy(), po.to_complex(v.float().numpy()),
                                         po.to_complex(k.float().numpy()), po.to_complex(q.float().numpy()),
                                         coef=po.to_complex(coef.numpy()))
        if state_dtype == torch.bfloat16:   # the pool rounds the stored state
            S_new = po.to_complex(torch.from_numpy(po.to_split(S_new)).bfloat16().double().numpy())
        ref[live, layer] = np.transpose(S_new, (1, 0, 2, 3, 4))
        assert_close(y.float().cpu().numpy(), po.to_split(y_ref), tol, f"y step {step}")
    assert_close(pool.float().cpu().numpy(), po.to_split(ref), tol, "pool")


def test_out_of_range_slot_is_skipped():
    pool = torch.zeros(2, 1, 1, 1, 16, 16, 2, device=DEV)
    x = torch.ones(2, 1, 16, 2, device=DEV)
    ops.pam_decode_step(pool, torch.tensor([-1, 1], dtype=torch.int32, device=DEV), x, x, x,
                        torch.ones(1, 2, 1, device=DEV))
    assert float(pool[0].abs().max()) == 0.0 and float(pool[1].abs().max()) > 0.0


@pytest.mark.parametrize("state_dtype,tol", [(torch.float32, 2e-2), (torch.bfloat16, 3e-2)])
def test_full_size_decode_steps_equal_the_scan(state_dtype, tol):
    """Config-5 size (256 slots, 12 layers, H=12, d=64, K=3, bf16 tokens): a run of decode steps from empty slots
    equals the chunked scan over the same tokens -- last output and final state -- in one layer of the pool,
    and leaves every other layer untouched.  (The recurrent step takes gamma as is, the scan gamma + 1e-6.)"""
    n, L, K, H, d, steps, layer = 256, 12, 3, 12, 64, 6, 7
    g = torch.Generator(device=DEV).manual_seed(3)
    q, k, v = (torch.randn(n, H, steps, d, 2, device=DEV, generator=g).mul_(0.125).bfloat16() for _ in range(3))
    gamma = torch.sigmoid(torch.randn(K, n, H, steps, device=DEV, generator=g) + 2.0)
    coef = torch.randn(K, n, H, steps, 2, device=DEV, generator=g)
    pool = torch.zeros(n, L, K, H, d, d, 2, dtype=state_dtype, device=DEV)
    slots = torch.randperm(n, device=DEV, generator=g).int()           # sequence i lives in slot slots[i]
    for t in range(steps):
        y = ops.pam_decode_step(pool, slots, (q[:, :, t].float() * d ** -0.5).bfloat16().contiguous(), k[:, :, t].contiguous(),
                                v[:, :, t].contiguous(), gamma[..., t].contiguous(), coef[:, :, :, t].contiguous(), layer=layer)
    with torch.no_grad():
        y_ref, s_ref = ops.pam_scan(q, k, v, gamma, coef=coef, eps=0.0)
    ref = y_ref[:, :, -1].float()
    assert float((y.float() - ref).norm() / ref.norm()) < tol
    got = pool[slots.long(), layer].float().permute(1, 0, 2, 3, 4, 5)    # [K,n,H,d,d,2]
    assert float((got - s_ref).norm() / s_ref.norm()) < tol
    others = [i for i in range(L) if i != layer]
    assert float(pool[:, others].float().abs().max()) == 0.0


def test_long_horizon_state_rounding_is_bounded():
    """2048 recurrent steps at gamma = 0.999 (memory of ~1000 tokens): a state pool that rounds the d x d state to
    bf16 on every step -- what the reference's recurrent path does when the model runs in half precision, its
    states being tensors of the model dtype -- is compared with the complex128 recurrence and with a float32 pool.
    Rounding errors of relative size 2^-9 enter at every step and decay like the state itself, so the expected
    error of y is about 2^-9 / sqrt(3) * sqrt(1 / (1 - gamma^2)) ~ 2.5e-2 of the output norm; the bar is 6e-2 for
    the bf16 pool and 2e-3 for the float32 pool (bf16 token inputs in both)."""
    n, H, d, steps = 2, 2, 64, 2048
    gen = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(n, H, steps, d, 2, generator=gen).mul_(0.125).bfloat16() for _ in range(3))
    gamma = torch.full((1, n, H, steps), 0.999)
    y_ref, _ = po.scan_recurrence(po.to_complex(q.float().numpy()), po.to_complex(k.float().numpy()),
                                  po.to_complex(v.float().numpy()), gamma[0].double().numpy(), eps=0.0)
    y_ref = po.to_split(y_ref)                                              # [n,H,T,d,2]
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    qd, kd, vd, gd = q.to(DEV), k.to(DEV), v.to(DEV), gamma.to(DEV)
    drift = {}
    for state_dtype in (torch.float32, torch.bfloat16):
        pool = torch.zeros(n, 1, 1, H, d, d, 2, dtype=state_dtype, device=DEV)
        ys = []
        for t in range(steps):
            ys.append(ops.pam_decode_step(pool, slots, qd[:, :, t] * d ** -0.5, kd[:, :, t], vd[:, :, t], gd[:, :, :, t]))
        got = torch.stack(ys, dim=2).float().cpu().numpy()
        tail = slice(steps - 256, steps)
        err = np.linalg.norm(got[:, :, tail] - y_ref[:, :, tail]) / np.linalg.norm(y_ref[:, :, tail])
        drift[str(state_dtype)] = float(err)
    print("relative error of the last 256 outputs after 2048 steps:", drift)
    assert drift["torch.float32"] < 2e-3, drift
    assert drift["torch.bfloat16"] < 6e-2, drift
