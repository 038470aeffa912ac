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


@pytest.mark.parametrize("lo,hi", [(0.05, 0.3), (0.02, 0.999), (0.45, 0.6)])
def test_strong_decay_is_exact(lo, hi):
    """gamma far below the usual sigmoid(N(3,1)) range: a 128-token chunk then decays by more than e^-80 and the
    factored decay of the fast path would overflow; the kernels must switch to the per-score form.  Forward,
    final state and every gradient against the oracle, with an initial state and a gradient into the final one."""
    B, H, T = 1, 2, 300
    inp = synthetic.scan_inputs(B, H, T, 64, seed=123, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(11)
    gamma = lo + (hi - lo) * torch.rand(B, H, T, generator=gen)
    inp.g = torch.log(gamma / (1 - gamma))
    s0 = torch.randn(1, B, H, 64, 64, 2, generator=gen) * 0.05
    dsf = torch.randn(1, B, H, 64, 64, 2, generator=gen) * 0.05
    _grads_vs_oracle(inp, s0=s0, ds_final=dsf)
    with torch.no_grad():
        y, s = ops.pam_scan(inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV), inp.gamma.to(DEV), s0=s0.to(DEV))
    q, k, v = (po.to_complex(t.float().numpy()) for t in (inp.q, inp.k, inp.v))
    y_ref, s_ref = po.scan_recurrence(q, k, v, inp.gamma.double().numpy(), s0=po.to_complex(s0.numpy()))
    assert_close(y.float().cpu().numpy(), po.to_split(y_ref), TOL, "Y")
    assert_close(s.cpu().numpy(), po.to_split(s_ref), TOL, "S")


def test_strong_decay_k_states_forward():
    """The fused K-state output kernel under strong decay in one of its states."""
    K, B, H, T = 3, 1, 2, 300
    inp, gamma, coef = _k_state_inputs(B, H, T, K, seed=170)
    gen = torch.Generator().manual_seed(12)
    gamma[1] = 0.05 + 0.3 * torch.rand(B, H, T, generator=gen)
    s0 = torch.randn(K, B, H, 64, 64, 2, generator=gen) * 0.05
    with torch.no_grad():
        y, s = ops.pam_scan(inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV), gamma.to(DEV), coef=coef.to(DEV), s0=s0.to(DEV))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    qc, kc, vc = (po.to_complex(t.float().numpy()) for t in (inp.q, inp.k, inp.v))
    y_ref, s_ref = po.scan_recurrence(qc, kc, vc, gamma.double().numpy(), coef=po.to_complex(coef.numpy()),
                                      s0=po.to_complex(s0.numpy()))
    assert_close(y.float().cpu().numpy(), po.to_split(y_ref), TOL, "Y")
    assert_close(s.cpu().numpy(), po.to_split(s_ref), TOL, "S")


def test_packed_backward_matches_oracle():
    """Gradients through the packed (cu_seqlens) layout: ragged sequences, one of them shorter than a chunk."""
    p = synthetic.packed_inputs(4, 40, 500, 2, 64, seed=29, dtype=torch.bfloat16)
    total = p.q.shape[1]
    gen = torch.Generator().manual_seed(7)
    dy = (torch.randn(2, total, 64, 2, generator=gen) / 2 ** 0.5).bfloat16()
    q, k, v = (t.unsqueeze(0).to(DEV).requires_grad_(True) for t in (p.q, p.k, p.v))
    gam = p.gamma.unsqueeze(0).to(DEV).requires_grad_(True)
    y, _ = ops.pam_scan(q, k, v, gam, cu_seqlens=p.cu_seqlens)
    dq, dk, dv, dgam = torch.autograd.grad(y, [q, k, v, gam], dy.unsqueeze(0).to(DEV))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    cu = p.cu_seqlens.numpy()
    for i in range(4):
        a, b = int(cu[i]), int(cu[i + 1])
        qc, kc, vc, dyc = (po.to_complex(t[:, a:b].float().numpy())[None] for t in (p.q, p.k, p.v, dy))
        ref = po.scan_backward(qc, kc, vc, p.gamma[:, a:b].double().numpy()[None], dyc)
        assert_close(dq[0, :, a:b].float().cpu().numpy(), po.to_split(ref["dq"])[0], TOL, f"dq seq {i}")
        assert_close(dk[0, :, a:b].float().cpu().numpy(), po.to_split(ref["dk"])[0], TOL, f"dk seq {i}")
        assert_close(dv[0, :, a:b].float().cpu().numpy(), po.to_split(ref["dv"])[0], TOL, f"dv seq {i}")
        assert_close(dgam[0, :, a:b].cpu().numpy(), ref["dgamma"][0][0], TOL, f"dgamma seq {i}")


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


def test_headline_shape_against_oracle():
    """Headline shape (B=8, H=6, T=2048, d=64, bf16), forward and backward through the tensor-core kernels:
    two of the 48 (batch, head) pairs compared with the oracle's exact recurrence and its adjoint."""
    inp = synthetic.scan_inputs(8, 6, 2048, 64, seed=0, dtype=torch.bfloat16)
    q, k, v = (t.to(DEV).requires_grad_(True) for t in (inp.q, inp.k, inp.v))
    g = inp.g.to(DEV).requires_grad_(True)
    y, s = ops.pam_scan(q, k, v, torch.sigmoid(g))
    dq, dk, dv, dg = torch.autograd.grad(y, [q, k, v, g], inp.dy.to(DEV))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for b, h in ((0, 0), (5, 3)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        qc, kc, vc, dyc = (po.to_complex(t[sl].float().numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
        gam = torch.sigmoid(inp.g[sl].double()).numpy()
        y_ref, s_ref = po.scan_recurrence(qc, kc, vc, gam)
        ref = po.scan_backward(qc, kc, vc, gam, dyc)
        assert_close(y[sl].detach().float().cpu().numpy(), po.to_split(y_ref), TOL, f"Y {b},{h}")
        assert_close(s.detach()[0][sl].cpu().numpy(), po.to_split(s_ref)[0], TOL, f"S {b},{h}")
        assert_close(dq[sl].float().cpu().numpy(), po.to_split(ref["dq"]), TOL, f"dq {b},{h}")
        assert_close(dk[sl].float().cpu().numpy(), po.to_split(ref["dk"]), TOL, f"dk {b},{h}")
        assert_close(dv[sl].float().cpu().numpy(), po.to_split(ref["dv"]), TOL, f"dv {b},{h}")
        assert_close(dg[sl].cpu().numpy(), ref["dgamma"][0] * gam * (1 - gam), TOL, f"dg {b},{h}")


def test_config4_sequences_against_oracle():
    """The packed ragged prefill at its configured size (32 sequences of 512..16384 tokens, H=16, d=64, bf16,
    seed 0): the shortest, the median and the longest sequence, outputs and final states of four heads,
    against the oracle."""
    p = synthetic.config4()
    q, k, v = (t.unsqueeze(0).to(DEV) for t in (p.q, p.k, p.v))
    with torch.no_grad():
        y, s = ops.pam_scan(q, k, v, p.gamma.unsqueeze(0).to(DEV), cu_seqlens=p.cu_seqlens, chunk=128)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    order = torch.argsort(p.lengths)
    cu = p.cu_seqlens.numpy()
    heads = [0, 5, 10, 15]
    for i in (int(order[0]), int(order[16]), int(order[31])):
        a, b = int(cu[i]), int(cu[i + 1])
        qc, kc, vc = (po.to_complex(t[heads, a:b].float().numpy())[None] for t in (p.q, p.k, p.v))
        y_ref, s_ref = po.scan_recurrence(qc, kc, vc, p.gamma[heads, a:b].double().numpy()[None])
        assert_close(y[0, heads, a:b].float().cpu().numpy(), po.to_split(y_ref)[0], TOL, f"Y seq {i} ({b - a} tokens)")
        assert_close(s[0, i][heads].cpu().numpy(), po.to_split(s_ref)[0, 0], TOL, f"S seq {i}")


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


def _direct_forward(q, k, v, gamma, cu, y, s_final):
    """qpam_scan_fwd through the C ABI with caller-made output buffers (so that they can be poisoned first)."""
    import ctypes as C
    L = _lib.lib()
    H, T = q.shape[1], q.shape[2]
    a = _lib.ScanArgs()
    a.q, a.k, a.v, a.gamma = q.data_ptr(), k.data_ptr(), v.data_ptr(), gamma.data_ptr()
    a.cu_seqlens = cu.data_ptr() if cu is not None else None
    a.y, a.s_final = y.data_ptr(), s_final.data_ptr()
    a.B, a.H, a.T, a.d, a.K = q.shape[0], H, T, 64, 1
    a.S = cu.numel() - 1 if cu is not None else q.shape[0]
    a.chunk, a.io_dtype, a.q_scale, a.gamma_eps = 128, _lib.QPAM_BF16, 64 ** -0.5, 1e-6
    ws = torch.empty(L.qpam_scan_workspace_bytes(C.byref(a), 0), dtype=torch.uint8, device=DEV)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    rc = L.qpam_scan_fwd(C.byref(a), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return rc


@pytest.mark.parametrize("bad", [[0, 100, 90, 300], [5, 100, 200, 300], [0, 100, 200, 400], [0, -3, 200, 300]])
def test_bad_cu_seqlens_is_reported_not_followed(bad):
    """A device-side cu_seqlens that decreases, does not start at 0 or runs past T: the call touches nothing
    through it (outputs keep their poison) and the status word says 301; the next good call works."""
    assert _lib.device_status() == 0
    p = synthetic.packed_inputs(3, 100, 100, 2, 64, seed=3, dtype=torch.bfloat16)     # T = 300
    q, k, v = (t.unsqueeze(0).to(DEV) for t in (p.q, p.k, p.v))
    gamma = p.gamma.unsqueeze(0).unsqueeze(0).to(DEV).contiguous()
    y = torch.full_like(q, float("nan"))
    cu = torch.tensor(bad, dtype=torch.int32, device=DEV)
    s_final = torch.full((1, 3, 2, 64, 64, 2), float("nan"), device=DEV)
    assert _direct_forward(q, k, v, gamma, cu, y, s_final) == 0
    assert _lib.device_status(clear=False) == 301
    assert torch.isnan(y).all()
    assert _lib.device_status(clear=True) == 301 and _lib.device_status() == 0
    good = torch.tensor([0, 100, 200, 300], dtype=torch.int32, device=DEV)
    assert _direct_forward(q, k, v, gamma, good, y, s_final) == 0
    assert _lib.device_status() == 0 and torch.isfinite(y.float()).all()
    with pytest.raises(_lib.QPamError):                   # the same descriptor on the host is refused before any launch
        ops.pam_scan(q, k, v, gamma[0], cu_seqlens=torch.tensor(bad, dtype=torch.int32))


def test_expired_wait_sets_status_and_later_launches_skip():
    """A bounded wait that runs out (a barrier nobody arrives at, 2 ms limit): the status word is set, a scan
    launched while it is set leaves its outputs untouched, clearing the word restores normal service."""
    assert _lib.device_status() == 0
    assert _lib.lib().qpam_selftest_wait_expiry(2_000_000, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert _lib.device_status(clear=False) == 299
    inp = synthetic.scan_inputs(1, 2, 300, 64, seed=5, dtype=torch.bfloat16)
    q, k, v = (t.to(DEV) for t in (inp.q, inp.k, inp.v))
    gamma = inp.gamma.unsqueeze(0).to(DEV).contiguous()
    y = torch.full_like(q, float("nan"))
    s_final = torch.zeros(1, 1, 2, 64, 64, 2, device=DEV)
    assert _direct_forward(q, k, v, gamma, None, y, s_final) == 0
    assert torch.isnan(y).all()                          # skipped
    with pytest.raises(_lib.QPamError):
        _lib.raise_on_device_error("test")
    assert _lib.device_status() == 0
    assert _direct_forward(q, k, v, gamma, None, y, s_final) == 0
    assert _lib.device_status() == 0 and torch.isfinite(y.float()).all()


def test_long_memory_decay_does_not_drift():
    """16,384 tokens at a decay of 0.9999 per token (every token still weighs 0.19 at the end): an error in the
    per-token log-decay that all tokens share would add up 16,384 times.  Final state and the last 512 outputs stay
    at the bf16 level against the fp64 recurrence (v11/model.py:378-417)."""
    T, H = 16384, 1
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(1, H, T, 64, 2, generator=g).mul(0.125).bfloat16() for _ in range(3))
    gamma = torch.full((1, H, T), 0.9999)
    y, s = ops.pam_scan(q.to(DEV), k.to(DEV), v.to(DEV), gamma.to(DEV))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    qc, kc, vc = (po.to_complex(t.float().numpy()) for t in (q, k, v))
    y_ref, s_ref = po.scan_recurrence(qc, kc, vc, gamma.double().numpy())
    assert rel_err(s.cpu().numpy(), po.to_split(s_ref)) < 4e-3
    assert rel_err(y[0, :, -512:].float().cpu().numpy(), po.to_split(y_ref[0, :, -512:])) < 6e-3
