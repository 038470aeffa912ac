"""Seeded random cases of the packed scan against the fp64 oracle, sequence by sequence: output, final states and
every gradient (dq, dk, dv, dgamma_k, dcoef_k) -- the tensor-core kernels (bf16, d = 64) and the fp32 kernels
(d = 16, 32 or 64).

Each case draws its own number of heads, states (1..4), sequences and sequence lengths (zero-length sequences and
lengths that are not a multiple of the 128-token chunk included), an optional initial state, and a decay range that
sometimes drives whole chunks below e^-80 (the exact slow path of the chunk kernels).  The reference behaviour is
`V11PAMLayer._forward_chunked_head` / `_forward_multistate_fused` (v11/model.py:378-417, 739-781) applied to every
sequence on its own."""
import numpy as np
import pytest
import torch

from oracle import pam_oracle as po
from tests.helpers import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.bfloat16: 2e-2,     # bf16 tokens in, bf16 outputs: relative Frobenius error per tensor
       torch.float32: 1e-4}


def _case(seed, dtype=torch.bfloat16):
    rng = np.random.default_rng(1000 + seed + (0 if dtype == torch.bfloat16 else 500))
    d = 64 if dtype == torch.bfloat16 else int(rng.choice([16, 32, 64]))
    H = int(rng.integers(1, 4))
    K = int(rng.choice([1, 1, 2, 3, 4]))
    S = int(rng.integers(1, 5))
    lens = rng.integers(0, 420, size=S)
    if seed % 5 == 0:
        lens[int(rng.integers(0, S))] = 128 * int(rng.integers(1, 4))      # a sequence of whole chunks
    if lens.sum() == 0:
        lens[0] = 5
    T = int(lens.sum())
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    g = torch.Generator().manual_seed(seed)
    q, k, v, dy = (torch.randn(1, H, T, d, 2, generator=g).mul(0.125).to(dtype) for _ in range(4))
    # decay: sigmoid(N(0,1) + shift); shift < 0 puts 128-token products below e^-80
    shift = float(rng.choice([-1.0, 0.5, 2.0, 4.0]))
    gamma = torch.sigmoid(torch.randn(K, 1, H, T, generator=g) + shift)
    coef = torch.randn(K, 1, H, T, 2, generator=g) if K > 1 else None
    s0 = torch.randn(K, S, H, d, d, 2, generator=g) * 0.05 if bool(rng.integers(0, 2)) else None
    return dict(d=d, H=H, K=K, S=S, T=T, lens=lens, cu=cu, q=q, k=k, v=v, dy=dy, gamma=gamma, coef=coef, s0=s0, shift=shift)


@pytest.mark.parametrize("seed,dtype", [(i, torch.bfloat16) for i in range(14)] + [(i, torch.float32) for i in range(8)])
def test_random_packed_case_forward_and_gradients(seed, dtype):
    from qllm2_b200 import _lib, ops
    c = _case(seed, dtype)
    K, S, T, d = c["K"], c["S"], c["T"], c["d"]
    cu_t = torch.from_numpy(c["cu"])
    qd, kd, vd = (c[n].to(DEV).requires_grad_(True) for n in ("q", "k", "v"))
    gd = c["gamma"].to(DEV).requires_grad_(True)
    cd = None if c["coef"] is None else c["coef"].to(DEV).requires_grad_(True)
    s0d = None if c["s0"] is None else c["s0"].to(DEV)
    y, s = ops.pam_scan(qd, kd, vd, gd, coef=cd, s0=s0d, cu_seqlens=cu_t)
    wrt = [qd, kd, vd, gd] + ([cd] if cd is not None else [])
    grads = torch.autograd.grad(y, wrt, c["dy"].to(DEV))
    assert _lib.device_status() == 0
    with torch.no_grad():   # the inference route (fused K-state kernel for K > 1) must give the same tokens
        y_inf, s_inf = ops.pam_scan(qd.detach(), kd.detach(), vd.detach(), gd.detach(),
                                    coef=None if cd is None else cd.detach(), s0=s0d, cu_seqlens=cu_t)
    got = dict(y=y.detach()[0].float().cpu().numpy(), s=s.detach().cpu().numpy(),
               y_inf=y_inf[0].float().cpu().numpy(), s_inf=s_inf.cpu().numpy(),
               dq=grads[0][0].float().cpu().numpy(), dk=grads[1][0].float().cpu().numpy(),
               dv=grads[2][0].float().cpu().numpy(), dgamma=grads[3][:, 0].cpu().numpy(),
               dcoef=None if cd is None else grads[4][:, 0].cpu().numpy())
    assert all(np.isfinite(x).all() for x in got.values() if x is not None)
    qc, kc, vc, dyc = (po.to_complex(c[n][0].float().numpy()) for n in ("q", "k", "v", "dy"))
    gam = c["gamma"][:, 0].double().numpy()
    cf = None if c["coef"] is None else po.to_complex(c["coef"][:, 0].numpy())
    ref = {n: np.zeros_like(got[n], dtype=np.float64) for n in ("y", "dq", "dk", "dv", "dgamma")}
    ref["dcoef"] = None if cf is None else np.zeros_like(got["dcoef"], dtype=np.float64)
    ref["s"] = np.zeros_like(got["s"], dtype=np.float64)
    for i in range(S):
        a, b = int(c["cu"][i]), int(c["cu"][i + 1])
        s0c = None if c["s0"] is None else po.to_complex(c["s0"][:, i].numpy())[:, None]     # [K, 1, H, d, d]
        if b == a:       # an empty sequence keeps its initial state
            if s0c is not None:
                ref["s"][:, i] = po.to_split(s0c[:, 0])
            continue
        sl = (slice(None), slice(a, b))
        kw = dict(coef=None if cf is None else cf[:, None, :, a:b], s0=s0c)
        y_ref, s_ref = po.scan_recurrence(qc[None][(slice(None),) + sl], kc[None][(slice(None),) + sl],
                                          vc[None][(slice(None),) + sl], gam[:, None, :, a:b], **kw)
        bw = po.scan_backward(qc[None][(slice(None),) + sl], kc[None][(slice(None),) + sl],
                              vc[None][(slice(None),) + sl], gam[:, None, :, a:b], dyc[None][(slice(None),) + sl], **kw)
        ref["y"][:, a:b] = po.to_split(y_ref[0])
        ref["s"][:, i] = po.to_split(np.asarray(s_ref).reshape(K, 1, c["H"], d, d)[:, 0])
        for n in ("dq", "dk", "dv"):
            ref[n][:, a:b] = po.to_split(bw[n][0])
        ref["dgamma"][:, :, a:b] = bw["dgamma"][:, 0]
        if cf is not None:
            ref["dcoef"][:, :, a:b] = po.to_split(bw["dcoef"][:, 0])
    what = f"seed {seed} {dtype}: d={d} H={c['H']} K={K} lens={list(c['lens'])} s0={c['s0'] is not None} shift={c['shift']}"
    for n in ("y", "y_inf", "s", "s_inf", "dq", "dk", "dv", "dgamma", "dcoef"):
        if got[n] is None:
            continue
        r = ref[n.replace("_inf", "")]
        if not np.any(r):          # nothing to compare (e.g. every state of an all-empty batch)
            assert not np.any(got[n]), f"{what}: {n} should be zero"
            continue
        e = rel_err(got[n], r)
        assert e <= TOL[dtype], f"{what}: {n} rel {e:.3e} > {TOL[dtype]:.0e}"
