"""GPU parity of the chunked PAM scan (forward + backward) against the CPU oracle and the
golden fixtures made by the reference.  Tolerances: fp32 1e-4 relative, bf16 2e-2 relative."""
import os

import numpy as np
import pytest
import torch

from oracle import pam_oracle as po
from qllm2_b200 import ops, synthetic
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL32, TOL16 = 1e-4, 2e-2


def _run_gpu(q, k, v, g, dy, dtype=torch.float32, coef=None, gamma=None, s0=None, cu=None, ds_final=None,
             save_states=True):
    """Returns dict of numpy outputs.  gamma = sigmoid(g) unless gamma [K,..] given directly."""
    qd, kd, vd = (t.to(DEV, dtype).requires_grad_(True) for t in (q, k, v))
    leaves = [qd, kd, vd]
    if gamma is None:
        gd = g.to(DEV).requires_grad_(True)
        gam = torch.sigmoid(gd)
        leaves.append(gd)
    else:
        gam = gamma.to(DEV).float().requires_grad_(True)
        leaves.append(gam)
    cd = None
    if coef is not None:
        cd = coef.to(DEV).float().requires_grad_(True)
        leaves.append(cd)
    s0d = None
    if s0 is not None:
        s0d = s0.to(DEV).float().requires_grad_(True)
        leaves.append(s0d)
    y, s = ops.pam_scan(qd, kd, vd, gam, coef=cd, s0=s0d, cu_seqlens=cu, save_states=save_states)
    outs = [y]
    gos = [dy.to(DEV, dtype)]
    if ds_final is not None:
        outs.append(s)
        gos.append(ds_final.to(DEV))
    grads = torch.autograd.grad(outs, leaves, gos)
    r = dict(y=y, s=s, dq=grads[0], dk=grads[1], dv=grads[2], dg=grads[3])
    i = 4
    if coef is not None:
        r["dcoef"] = grads[i]; i += 1
    if s0 is not None:
        r["ds0"] = grads[i]
    return {k_: v_.detach().float().cpu().numpy() for k_, v_ in r.items()}


def _oracle(q, k, v, gamma, dy, coef=None, s0=None, ds_final=None):
    qc, kc, vc, dyc = (po.to_complex(t.float().numpy()) for t in (q, k, v, dy))
    cf = None if coef is None else po.to_complex(coef.numpy())
    s0c = None if s0 is None else po.to_complex(s0.numpy())
    dsf = None if ds_final is None else po.to_complex(ds_final.numpy())
    y, s = po.scan_recurrence(qc, kc, vc, gamma, coef=cf, s0=s0c)
    b = po.scan_backward(qc, kc, vc, gamma, dyc, coef=cf, s0=s0c, dS_final=dsf)
    return dict(y=po.to_split(y), s=po.to_split(s), dq=po.to_split(b["dq"]), dk=po.to_split(b["dk"]),
                dv=po.to_split(b["dv"]), dgamma=b["dgamma"], dcoef=po.to_split(b["dcoef"]), ds0=po.to_split(b["dS0"]))


def _check(r, o, gam, tol, with_dg=True):
    for key in ("y", "s", "dq", "dk", "dv"):
        assert_close(r[key], o[key].reshape(r[key].shape), tol, key)
    if with_dg:
        dg_ref = (o["dgamma"] * gam * (1 - gam)).reshape(r["dg"].shape)
        assert_close(r["dg"], dg_ref, tol * 5, "dg")


def test_config1_fp32_vs_oracle_and_golden(golden_dir):
    """B=2,H=4,d=32,T=512, complex64: Y, S, dQ, dK, dV, dg within 1e-4 of the reference."""
    inp = synthetic.config1()
    r = _run_gpu(inp.q, inp.k, inp.v, inp.g, inp.dy)
    gam = torch.sigmoid(inp.g.double()).numpy()
    o = _oracle(inp.q, inp.k, inp.v, gam, inp.dy)
    _check(r, o, gam, TOL32)
    g = np.load(os.path.join(golden_dir, "scan_c1.npz"))
    st = int(g["stride"])
    for key in ("y", "dq", "dk", "dv"):
        assert_close(r[key][:, :, ::st], g[key + "64"], TOL32, "golden " + key)
    assert_close(r["s"][0], g["s64"], TOL32, "golden s")
    assert_close(r["dg"], g["dg64"], TOL32 * 5, "golden dg")


@pytest.mark.parametrize("B,H,T,d", [(2, 2, 80, 16), (1, 1, 7, 64), (1, 3, 64, 32), (2, 1, 193, 64), (1, 2, 1, 16)])
def test_shapes_fp32(B, H, T, d):
    """Ragged tails (T not a multiple of 64), T < 64, a single (b,h), T = 1."""
    inp = synthetic.scan_inputs(B, H, T, d, seed=10 + T)
    gam = torch.sigmoid(inp.g.double()).numpy()
    r = _run_gpu(inp.q, inp.k, inp.v, inp.g, inp.dy)
    _check(r, _oracle(inp.q, inp.k, inp.v, gam, inp.dy), gam, TOL32)
    r2 = _run_gpu(inp.q, inp.k, inp.v, inp.g, inp.dy, save_states=False)   # recompute path
    for key in r:
        assert np.array_equal(r[key], r2[key]), f"{key}: not bit-identical between runs"


def test_small_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "scan_small.npz"))
    inp = synthetic.scan_inputs(2, 2, 80, 16, seed=1)
    r = _run_gpu(inp.q, inp.k, inp.v, inp.g, inp.dy)
    for key in ("y", "dq", "dk", "dv", "dg"):
        assert_close(r[key], g[key], TOL32 * (5 if key == "dg" else 1), "golden " + key)
    assert_close(r["s"][0], g["s"], TOL32, "golden s")


def test_multistate_e3(golden_dir):
    """K=3 phase-routed scan vs the reference's fused E3 path (v11/model.py:739-781)."""
    g = np.load(os.path.join(golden_dir, "e3_small.npz"))
    inp = synthetic.scan_inputs(2, 3, 80, 16, seed=2)
    phase = torch.from_numpy(np.transpose(g["phase"], (3, 0, 2, 1)).copy()).float()
    alpha = torch.from_numpy(np.transpose(g["alpha"], (3, 0, 2, 1)).copy()).float()
    coef = torch.stack([alpha * torch.cos(phase), alpha * torch.sin(phase)], dim=-1)
    gamma = torch.from_numpy(g["gamma_all"]).float()
    r = _run_gpu(inp.q, inp.k, inp.v, None, inp.dy, coef=coef, gamma=gamma)
    for key in ("y", "s", "dq", "dk", "dv"):
        assert_close(r[key], g[key], TOL32, "golden " + key)
    assert_close(r["dg"], g["dgamma"], TOL32 * 5, "golden dgamma")
    o = _oracle(inp.q, inp.k, inp.v, gamma.double().numpy(), inp.dy, coef=coef.double())
    assert_close(r["dcoef"], o["dcoef"], TOL32, "dcoef")


def test_initial_state_and_state_gradient():
    """Two chained halves (s_final of the first feeds s0 of the second) equal one full scan,
    and gradients flow through s_final / s0."""
    inp = synthetic.scan_inputs(1, 2, 150, 32, seed=21)
    gam = torch.sigmoid(inp.g.double()).numpy()
    gen = torch.Generator().manual_seed(5)
    s0 = torch.randn(1, 1, 2, 32, 32, 2, generator=gen) * 0.1
    dsf = torch.randn(1, 1, 2, 32, 32, 2, generator=gen) * 0.1
    r = _run_gpu(inp.q, inp.k, inp.v, inp.g, inp.dy, s0=s0, ds_final=dsf)
    o = _oracle(inp.q, inp.k, inp.v, gam, inp.dy, s0=s0.double(), ds_final=dsf.double())
    _check(r, o, gam, TOL32)
    assert_close(r["ds0"], o["ds0"].reshape(r["ds0"].shape), TOL32, "ds0")


def test_packed_varlen_matches_per_sequence():
    """cu_seqlens: state restarts at every boundary; includes an empty sequence."""
    p = synthetic.packed_inputs(5, 3, 200, 2, 32, seed=7, dtype=torch.float32)
    lens = p.lengths.clone()
    cu = torch.zeros(7, dtype=torch.int32)
    cu[1:4] = torch.cumsum(lens[:3], 0).int()
    cu[4] = cu[3]                                  # empty sequence
    cu[5:] = cu[4] + torch.cumsum(lens[3:], 0).int()
    gen = torch.Generator().manual_seed(8)
    dy = torch.randn(p.q.shape, generator=gen) / 2 ** 0.5
    q, k, v = (t.unsqueeze(0) for t in (p.q, p.k, p.v))
    gamma = p.gamma.unsqueeze(0).unsqueeze(0)      # [K=1,B=1,H,T]
    r = _run_gpu(q, k, v, None, dy.unsqueeze(0), gamma=gamma, cu=cu)
    qc, kc, vc, dyc = (po.to_complex(t.numpy()) for t in (p.q, p.k, p.v, dy))
    y_ref, s_ref = po.scan_varlen(qc, kc, vc, p.gamma.double().numpy(), cu.numpy())
    assert_close(r["y"][0], po.to_split(y_ref), TOL32, "Y")
    assert_close(r["s"], po.to_split(s_ref), TOL32, "S per sequence")
    cul = cu.tolist()
    for i in range(6):
        a, b = cul[i], cul[i + 1]
        if a == b:
            continue
        bo = po.scan_backward(qc[None, :, a:b], kc[None, :, a:b], vc[None, :, a:b],
                              p.gamma.double().numpy()[None, :, a:b], dyc[None, :, a:b])
        assert_close(r["dq"][0, :, a:b], po.to_split(bo["dq"][0]), TOL32, f"dq seq {i}")
        assert_close(r["dk"][0, :, a:b], po.to_split(bo["dk"][0]), TOL32, f"dk seq {i}")
        assert_close(r["dv"][0, :, a:b], po.to_split(bo["dv"][0]), TOL32, f"dv seq {i}")
        assert_close(r["dg"][0, 0, :, a:b], bo["dgamma"][0, 0], TOL32 * 5, f"dgamma seq {i}")


@pytest.mark.parametrize("B,H,T,d", [(2, 3, 300, 64), (1, 2, 130, 32)])
def test_bf16_io(B, H, T, d):
    """bf16 token tensors: compare with fp64 math on the same bf16-rounded inputs, 2e-2."""
    inp = synthetic.scan_inputs(B, H, T, d, seed=30, dtype=torch.bfloat16)
    gam = torch.sigmoid(inp.g.double()).numpy()
    r = _run_gpu(inp.q, inp.k, inp.v, inp.g, inp.dy, dtype=torch.bfloat16)
    o = _oracle(inp.q, inp.k, inp.v, gam, inp.dy)
    _check(r, o, gam, TOL16)


def test_gamma_above_one_is_clamped_in_forward():
    """gamma + eps > 1 engages the min(.,0) clamp of the decay matrix (v11/triton_kernels.py:528)."""
    inp = synthetic.scan_inputs(1, 1, 64, 16, seed=40)
    gamma = torch.full((1, 1, 1, 64), 1.0)
    qd, kd, vd = (t.to(DEV) for t in (inp.q, inp.k, inp.v))
    y, s = ops.pam_scan(qd, kd, vd, gamma.to(DEV))
    qc, kc, vc = (po.to_complex(t.numpy()) for t in (inp.q, inp.k, inp.v))
    y_ref, s_ref = po.scan_dual_chunked(qc, kc, vc, gamma[0].double().numpy(), 64)
    assert_close(y.cpu().numpy(), po.to_split(y_ref), TOL32, "Y clamp")
    assert_close(s.cpu().numpy(), po.to_split(s_ref), TOL32, "S clamp")


def test_large_property_linearity_in_v():
    """Full-size property check (B=8,H=6,T=2048,d=64, bf16): the scan is linear in V."""
    inp = synthetic.scan_inputs(8, 6, 2048, 64, seed=50, dtype=torch.bfloat16)
    q, k, v, gam = inp.q.to(DEV), inp.k.to(DEV), inp.v.to(DEV), inp.gamma.to(DEV)
    v2 = torch.flip(v, dims=[2])
    y1, s1 = ops.pam_scan(q.float(), k.float(), v.float(), gam)
    y2, s2 = ops.pam_scan(q.float(), k.float(), v2.float(), gam)
    y3, s3 = ops.pam_scan(q.float(), k.float(), (v.float() + 2 * v2.float()), gam)
    assert_close(y3.cpu().numpy(), (y1 + 2 * y2).cpu().numpy(), 1e-4, "linearity Y")
    assert_close(s3.cpu().numpy(), (s1 + 2 * s2).cpu().numpy(), 1e-4, "linearity S")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_states_only_scan_equals_the_full_scan_state(dtype):
    """`pam_scan_states` (no output kernel) returns the state `pam_scan` returns, batch and packed."""
    from qllm2_b200 import ops
    g = torch.Generator().manual_seed(17)
    B, H, T, d, K = 2, 2, 300, 64, 2
    k, v, q = (torch.randn(B, H, T, d, 2, generator=g).mul(0.125).to("cuda").to(dtype) for _ in range(3))
    gamma = torch.sigmoid(torch.randn(K, B, H, T, generator=g) + 3).to("cuda")
    s0 = (torch.randn(K, B, H, d, d, 2, generator=g) * 0.1).to("cuda")
    _, s_ref = ops.pam_scan(q, k, v, gamma, s0=s0)
    assert torch.equal(ops.pam_scan_states(k, v, gamma, s0=s0), s_ref)
    cu = torch.tensor([0, 120, 120, 300], dtype=torch.int32)
    _, s_ref = ops.pam_scan(q[:1], k[:1], v[:1], gamma[:, :1], cu_seqlens=cu)
    assert torch.equal(ops.pam_scan_states(k[:1], v[:1], gamma[:, :1], cu_seqlens=cu), s_ref)
