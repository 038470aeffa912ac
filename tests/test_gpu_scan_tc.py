"""Tensor-core (tcgen05) scan kernels: bf16 token tensors, head dim 64, one state.
Reference = fp64 oracle on the same bf16-rounded inputs; tolerance 2e-2 relative."""
import numpy as np
import pytest
import torch

from oracle import pam_oracle as po
from qllm2_b200 import _lib, ops, synthetic
from tests.helpers import assert_close, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 2e-2


@pytest.mark.parametrize("B,H,T", [(1, 1, 128), (2, 3, 300), (1, 2, 1), (1, 1, 129), (2, 2, 1024), (1, 1, 77)])
def test_forward_shapes(B, H, T):
    inp = synthetic.scan_inputs(B, H, T, 64, seed=60 + T, dtype=torch.bfloat16)
    y, s = ops.pam_scan(inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV), inp.gamma.to(DEV))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    q, k, v = (po.to_complex(t.float().numpy()) for t in (inp.q, inp.k, inp.v))
    y_ref, s_ref = po.scan_recurrence(q, k, v, inp.gamma.double().numpy())
    assert_close(y.float().cpu().numpy(), po.to_split(y_ref), TOL, "Y")
    assert_close(s.cpu().numpy(), po.to_split(s_ref), TOL, "S")
    # typical error is far below the bar; catch silent degradations early
    assert rel_err(y.float().cpu().numpy(), po.to_split(y_ref)) < 8e-3


def test_forward_initial_state_and_varlen():
    p = synthetic.packed_inputs(4, 100, 600, 3, 64, seed=9, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(2)
    s0 = torch.randn(1, 4, 3, 64, 64, 2, generator=gen) * 0.05
    q, k, v = (t.unsqueeze(0).to(DEV) for t in (p.q, p.k, p.v))
    y, s = ops.pam_scan(q, k, v, p.gamma.unsqueeze(0).to(DEV), s0=s0.to(DEV), cu_seqlens=p.cu_seqlens)
    assert _lib.device_status() == 0
    qc, kc, vc = (po.to_complex(t.float().numpy()) for t in (p.q, p.k, p.v))
    y_ref, s_ref = po.scan_varlen(qc, kc, vc, p.gamma.double().numpy(), p.cu_seqlens.numpy(),
                                  s0=po.to_complex(s0.numpy()))
    assert_close(y[0].float().cpu().numpy(), po.to_split(y_ref), TOL, "Y packed")
    assert_close(s.cpu().numpy(), po.to_split(s_ref), TOL, "S packed")


def test_forward_then_backward_mixed_paths():
    """Forward on tensor cores, backward on its own chunking: gradients still match the oracle."""
    inp = synthetic.scan_inputs(1, 2, 260, 64, seed=70, dtype=torch.bfloat16)
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (inp.q, inp.k, inp.v))
    g = inp.g.to(DEV).requires_grad_(True)
    y, _ = ops.pam_scan(q, k, v, torch.sigmoid(g))
    dq, dk, dv, dg = torch.autograd.grad(y, [q, k, v, g], inp.dy.to(DEV))
    qc, kc, vc, dyc = (po.to_complex(t.float().numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
    gam = torch.sigmoid(inp.g.double()).numpy()
    b = po.scan_backward(qc, kc, vc, gam, dyc)
    assert_close(dq.float().cpu().numpy(), po.to_split(b["dq"]), TOL, "dq")
    assert_close(dk.float().cpu().numpy(), po.to_split(b["dk"]), TOL, "dk")
    assert_close(dv.float().cpu().numpy(), po.to_split(b["dv"]), TOL, "dv")
    assert_close(dg.cpu().numpy(), b["dgamma"][0] * gam * (1 - gam), TOL, "dg")


def _grads_vs_oracle(inp, s0=None, ds_final=None, cu=None, packed=False):
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (inp.q, inp.k, inp.v))
    g = inp.g.to(DEV).requires_grad_(True)
    s0d = None if s0 is None else s0.to(DEV).requires_grad_(True)
    y, s = ops.pam_scan(q, k, v, torch.sigmoid(g), s0=s0d)
    outs, gos = [y], [inp.dy.to(DEV)]
    if ds_final is not None:
        outs.append(s)
        gos.append(ds_final.to(DEV))
    leaves = [q, k, v, g] + ([s0d] if s0 is not None else [])
    grads = torch.autograd.grad(outs, leaves, gos)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    qc, kc, vc, dyc = (po.to_complex(t.float().numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
    gam = torch.sigmoid(inp.g.double()).numpy()
    b = po.scan_backward(qc, kc, vc, gam, dyc, s0=None if s0 is None else po.to_complex(s0.numpy()),
                         dS_final=None if ds_final is None else po.to_complex(ds_final.numpy()))
    assert_close(grads[0].float().cpu().numpy(), po.to_split(b["dq"]), TOL, "dq")
    assert_close(grads[1].float().cpu().numpy(), po.to_split(b["dk"]), TOL, "dk")
    assert_close(grads[2].float().cpu().numpy(), po.to_split(b["dv"]), TOL, "dv")
    assert_close(grads[3].cpu().numpy(), b["dgamma"][0] * gam * (1 - gam), TOL, "dg")
    if s0 is not None:
        assert_close(grads[4].cpu().numpy(), po.to_split(b["dS0"]), TOL, "ds0")


@pytest.mark.parametrize("B,H,T", [(1, 1, 128), (2, 2, 300), (1, 1, 50), (1, 2, 1024), (1, 1, 129), (1, 1, 4096)])
def test_backward_shapes(B, H, T):
    _grads_vs_oracle(synthetic.scan_inputs(B, H, T, 64, seed=80 + T, dtype=torch.bfloat16))


def test_backward_with_state_gradients():
    gen = torch.Generator().manual_seed(6)
    s0 = torch.randn(1, 1, 2, 64, 64, 2, generator=gen) * 0.05
    dsf = torch.randn(1, 1, 2, 64, 64, 2, generator=gen) * 0.05
    _grads_vs_oracle(synthetic.scan_inputs(1, 2, 400, 64, seed=91, dtype=torch.bfloat16), s0=s0, ds_final=dsf)


def test_backward_is_deterministic():
    inp = synthetic.scan_inputs(2, 2, 500, 64, seed=95, dtype=torch.bfloat16)
    res = []
    for _ in range(2):
        q, k, v = (t.to(DEV).requires_grad_(True) for t in (inp.q, inp.k, inp.v))
        g = inp.g.to(DEV).requires_grad_(True)
        y, _ = ops.pam_scan(q, k, v, torch.sigmoid(g))
        res.append([y.detach()] + list(torch.autograd.grad(y, [q, k, v, g], inp.dy.to(DEV))))
    for a, b in zip(*res):
        assert torch.equal(a, b)


def test_multistate_bf16_on_tensor_cores(golden_dir):
    """K=3 phase-routed scan, bf16, d=64: the sum of K single-state tensor-core scans equals the oracle's
    K-state scan (forward, final states, and every gradient incl. dgamma_k and dcoef)."""
    B, H, T, d, K = 1, 2, 300, 64, 3
    inp = synthetic.scan_inputs(B, H, T, d, seed=33, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(4)
    gamma = torch.sigmoid(torch.randn(K, B, H, T, generator=gen) + torch.tensor([1.0, 3.0, 5.0]).view(K, 1, 1, 1))
    phase = torch.randn(K, B, H, T, generator=gen)
    alpha = 0.5 + torch.rand(K, B, H, T, generator=gen)
    coef = torch.stack([alpha * torch.cos(phase), alpha * torch.sin(phase)], dim=-1)
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (inp.q, inp.k, inp.v))
    gd = gamma.to(DEV).requires_grad_(True)
    cd = coef.to(DEV).requires_grad_(True)
    y, s = ops.pam_scan(q, k, v, gd, coef=cd)
    dq, dk, dv, dgam, dcoef = torch.autograd.grad(y, [q, k, v, gd, cd], inp.dy.to(DEV))
    assert _lib.device_status() == 0
    qc, kc, vc, dyc = (po.to_complex(t.float().numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
    cf = po.to_complex(coef.numpy())
    y_ref, s_ref = po.scan_recurrence(qc, kc, vc, gamma.double().numpy(), coef=cf)
    b = po.scan_backward(qc, kc, vc, gamma.double().numpy(), dyc, coef=cf)
    assert_close(y.detach().float().cpu().numpy(), po.to_split(y_ref), TOL, "Y")
    assert_close(s.detach().cpu().numpy(), po.to_split(s_ref), TOL, "S")
    assert_close(dq.float().cpu().numpy(), po.to_split(b["dq"]), TOL, "dq")
    assert_close(dk.float().cpu().numpy(), po.to_split(b["dk"]), TOL, "dk")
    assert_close(dv.float().cpu().numpy(), po.to_split(b["dv"]), TOL, "dv")
    assert_close(dgam.cpu().numpy(), b["dgamma"], TOL, "dgamma")
    assert_close(dcoef.cpu().numpy(), po.to_split(b["dcoef"]), TOL, "dcoef")


def _k_state_inputs(B, H, T, K, seed):
    inp = synthetic.scan_inputs(B, H, T, 64, seed=seed, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(seed + 1)
    shift = torch.tensor([1.0, 3.0, 5.0, 2.0])[:K].view(K, 1, 1, 1)
    gamma = torch.sigmoid(torch.randn(K, B, H, T, generator=gen) + shift)
    phase = torch.randn(K, B, H, T, generator=gen)
    alpha = 0.5 + torch.rand(K, B, H, T, generator=gen)
    coef = torch.stack([alpha * torch.cos(phase), alpha * torch.sin(phase)], dim=-1)
    return inp, gamma, coef


@pytest.mark.parametrize("K,B,H,T", [(3, 1, 2, 300), (2, 2, 1, 128), (4, 1, 1, 515), (3, 2, 3, 1), (2, 1, 2, 77)])
def test_fused_k_state_forward(K, B, H, T):
    """Inference (no gradient needed): K states in ONE output kernel against the fp64 oracle, with and without
    read-out weights and an initial state."""
    inp, gamma, coef = _k_state_inputs(B, H, T, K, seed=70 + T)
    gen = torch.Generator().manual_seed(5)
    s0 = torch.randn(K, B, H, 64, 64, 2, generator=gen) * 0.05
    qc, kc, vc = (po.to_complex(t.float().numpy()) for t in (inp.q, inp.k, inp.v))
    for use_coef, use_s0 in ((True, False), (True, True), (False, False)):
        with torch.no_grad():
            y, s = ops.pam_scan(inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV), gamma.to(DEV),
                                coef=coef.to(DEV) if use_coef else None, s0=s0.to(DEV) if use_s0 else None)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        y_ref, s_ref = po.scan_recurrence(qc, kc, vc, gamma.double().numpy(),
                                          coef=po.to_complex(coef.numpy()) if use_coef else None,
                                          s0=po.to_complex(s0.numpy()) if use_s0 else None)
        assert_close(y.float().cpu().numpy(), po.to_split(y_ref), TOL, f"Y coef={use_coef} s0={use_s0}")
        assert_close(s.cpu().numpy(), po.to_split(s_ref), TOL, "S")
        assert rel_err(y.float().cpu().numpy(), po.to_split(y_ref)) < 8e-3


def test_fused_k_state_forward_packed_and_launch_count():
    """Packed ragged sequences through the fused K-state kernel; the output pass is ONE launch for all states."""
    K = 3
    p = synthetic.packed_inputs(4, 60, 500, 2, 64, seed=19, dtype=torch.bfloat16)
    total = p.q.shape[1]
    gen = torch.Generator().manual_seed(6)
    gamma = torch.sigmoid(torch.randn(K, 2, total, generator=gen) + torch.tensor([1.0, 3.0, 5.0]).view(K, 1, 1))
    coef = torch.randn(K, 2, total, 2, generator=gen)
    q, k, v = (t.unsqueeze(0).to(DEV) for t in (p.q, p.k, p.v))
    with torch.no_grad():
        n0 = _lib.launch_count()
        y, s = ops.pam_scan(q, k, v, gamma.unsqueeze(1).to(DEV), coef=coef.unsqueeze(1).to(DEV), cu_seqlens=p.cu_seqlens)
        launches = _lib.launch_count() - n0
    assert _lib.device_status() == 0
    assert launches == 4              # chunk prefix, state sums (grid z = K), carry, fused output
    qc, kc, vc = (po.to_complex(t.float().numpy()) for t in (p.q, p.k, p.v))
    y_ref, s_ref = po.scan_varlen(qc, kc, vc, gamma.double().numpy(), p.cu_seqlens.numpy(), coef=po.to_complex(coef.numpy()))
    assert_close(y[0].float().cpu().numpy(), po.to_split(y_ref), TOL, "Y packed")
    assert_close(s.cpu().numpy(), po.to_split(s_ref), TOL, "S packed")


def test_full_size_adjoint_identity_headline_shape():
    """Headline shape (B=8, H=6, T=2048, d=64, bf16), tensor-core forward and backward: Y is linear in V, so
    <dY, Y(V)> = <dV(dY), V>; and with Y = Y(Q) linear in Q, <dY, Y> = <dQ, Q>.  (Size-independent checks of
    the gradients at the size the benchmark runs; bf16 bar 2e-2.)"""
    inp = synthetic.scan_inputs(8, 6, 2048, 64, seed=51, dtype=torch.bfloat16)
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (inp.q, inp.k, inp.v))
    gam = inp.gamma.to(DEV).requires_grad_(True)
    dy = inp.dy.to(DEV)
    y, _ = ops.pam_scan(q, k, v, gam)
    dq, dk, dv, dg = torch.autograd.grad(y, [q, k, v, gam], dy)
    assert _lib.device_status() == 0
    lhs = float((dy.double() * y.detach().double()).sum())
    for name, g, x in (("V", dv, v), ("Q", dq, q)):
        rhs = float((g.double() * x.detach().double()).sum())
        assert abs(lhs - rhs) <= 2e-2 * abs(lhs), (name, lhs, rhs)
    # conj-linearity in K gives the same pairing for dK
    rhs = float((dk.double() * k.detach().double()).sum())
    assert abs(lhs - rhs) <= 2e-2 * abs(lhs), ("K", lhs, rhs)
    assert torch.isfinite(dg).all()


def test_full_size_packed_prefill_properties():
    """Config-4 size (32 packed sequences of 512..16384 tokens, H=16, d=64, bf16): a sequence scanned inside the
    packed batch equals the same sequence scanned alone (chunks never straddle a boundary: bit for bit), and a
    sequence split at a chunk boundary and chained through its state equals the unsplit scan."""
    gen = torch.Generator().manual_seed(0)
    lens = torch.randint(512, 16385, (32,), generator=gen)
    cu = torch.zeros(33, dtype=torch.int32)
    cu[1:] = lens.cumsum(0).int()
    total, H = int(cu[-1]), 16
    g2 = torch.Generator(device=DEV).manual_seed(1)
    q, k, v = (torch.randn(1, H, total, 64, 2, device=DEV, generator=g2).mul_(128 ** -0.5).bfloat16() for _ in range(3))
    gamma = torch.sigmoid(torch.randn(1, H, total, device=DEV, generator=g2) + 3.0)
    with torch.no_grad():
        y, s = ops.pam_scan(q, k, v, gamma, cu_seqlens=cu)
        assert _lib.device_status() == 0
        for i in (0, 13, 31):
            a, b = int(cu[i]), int(cu[i + 1])
            yi, si = ops.pam_scan(q[:, :, a:b].contiguous(), k[:, :, a:b].contiguous(), v[:, :, a:b].contiguous(),
                                  gamma[:, :, a:b].contiguous())
            assert torch.equal(yi, y[:, :, a:b]) and torch.equal(si[:, 0], s[:, i])
        a, b = int(cu[5]), int(cu[6])
        m = a + 128 * ((b - a) // 256)                      # a chunk boundary inside sequence 5
        _, s_head = ops.pam_scan(q[:, :, a:m].contiguous(), k[:, :, a:m].contiguous(), v[:, :, a:m].contiguous(),
                                 gamma[:, :, a:m].contiguous())
        y_tail, s_tail = ops.pam_scan(q[:, :, m:b].contiguous(), k[:, :, m:b].contiguous(), v[:, :, m:b].contiguous(),
                                      gamma[:, :, m:b].contiguous(), s0=s_head)
    ref = y[:, :, m:b].float()
    assert float((y_tail.float() - ref).norm() / ref.norm()) < 2e-3
    assert float((s_tail[:, 0] - s[:, 5]).norm() / s[:, 5].norm()) < 1e-4
