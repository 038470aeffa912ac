"""Pin the CPU oracle against outputs of the reference itself (tests/golden/*.npz)."""
import os

import numpy as np
import pytest
import torch

from oracle import ce_oracle, pam_oracle as po
from qllm2_b200 import synthetic
from tests.helpers import assert_close, checksum


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_inputs_reproduce(golden_dir):
    """The seeded generators give the tensors the fixtures were made from."""
    g = _load(golden_dir, "scan_c1.npz")
    inp = synthetic.config1()
    np.testing.assert_allclose(checksum(inp.q, inp.k, inp.v, inp.g, inp.dy), g["insum"], rtol=1e-12)
    g2 = _load(golden_dir, "ce_c2.npz")
    c2 = synthetic.config2()
    np.testing.assert_allclose(checksum(c2.h.float(), c2.w.float(), c2.targets.float()), g2["insum"], rtol=1e-12)


def test_scan_small_fwd_bwd(golden_dir):
    g = _load(golden_dir, "scan_small.npz")
    inp = synthetic.scan_inputs(2, 2, 80, 16, seed=1)
    q, k, v, dy = (po.to_complex(t.numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
    gamma = torch.sigmoid(inp.g.double()).numpy()
    y, s = po.scan_recurrence(q, k, v, gamma)
    assert_close(po.to_split(y), g["y"], 1e-12, "Y")
    assert_close(po.to_split(s[0]), g["s"], 1e-12, "S")
    y2, s2 = po.scan_dual_chunked(q, k, v, gamma, 24)
    assert_close(po.to_split(y2), g["y"], 1e-12, "Y chunked")
    assert_close(po.to_split(s2[0]), g["s"], 1e-12, "S chunked")
    assert_close(g["flash_y"], g["y"], 1e-12, "flash == chunked in the reference")
    b = po.scan_backward(q, k, v, gamma, dy)
    assert_close(po.to_split(b["dq"]), g["dq"], 1e-11, "dq")
    assert_close(po.to_split(b["dk"]), g["dk"], 1e-11, "dk")
    assert_close(po.to_split(b["dv"]), g["dv"], 1e-11, "dv")
    assert_close(b["dgamma"][0], g["dgamma"], 1e-10, "dgamma")
    gam = torch.sigmoid(inp.g.double()).numpy()
    assert_close(b["dgamma"][0] * gam * (1 - gam), g["dg"], 1e-10, "dg")


def test_scan_c1(golden_dir):
    g = _load(golden_dir, "scan_c1.npz")
    st = int(g["stride"])
    inp = synthetic.config1()
    q, k, v, dy = (po.to_complex(t.numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
    gam = torch.sigmoid(inp.g.double()).numpy()
    y, s = po.scan_recurrence(q, k, v, gam)
    b = po.scan_backward(q, k, v, gam, dy)
    sub = lambda z: po.to_split(z)[:, :, ::st]
    # fp64 reference run: tight; fp32 reference run: its own rounding noise (~1e-6)
    for tol, sfx in ((1e-11, "64"), (5e-6, "")):
        assert_close(sub(y), g["y" + sfx], tol, "Y" + sfx)
        assert_close(po.to_split(s[0]), g["s" + sfx], tol, "S" + sfx)
        assert_close(sub(b["dq"]), g["dq" + sfx], tol, "dq" + sfx)
        assert_close(sub(b["dk"]), g["dk" + sfx], tol, "dk" + sfx)
        assert_close(sub(b["dv"]), g["dv" + sfx], tol, "dv" + sfx)
        assert_close(b["dgamma"][0] * gam * (1 - gam), g["dg" + sfx], tol * 10, "dg" + sfx)


def test_e3_small(golden_dir):
    g = _load(golden_dir, "e3_small.npz")
    B, H, T, d, K = 2, 3, 80, 16, 3
    inp = synthetic.scan_inputs(B, H, T, d, seed=2)
    q, k, v, dy = (po.to_complex(t.numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
    phase = np.transpose(g["phase"].astype(np.float64), (3, 0, 2, 1))   # [B,T,H,K] -> [K,B,H,T]
    alpha = np.transpose(g["alpha"].astype(np.float64), (3, 0, 2, 1))
    coef = alpha * np.exp(1j * phase)
    y, s = po.scan_recurrence(q, k, v, g["gamma_all"], coef=coef)
    assert_close(po.to_split(y), g["y"], 1e-12, "Y")
    assert_close(po.to_split(s), g["s"], 1e-12, "S")
    y2, s2 = po.scan_dual_chunked(q, k, v, g["gamma_all"], 24, coef=coef)
    assert_close(po.to_split(y2), g["y"], 1e-12, "Y chunked")
    b = po.scan_backward(q, k, v, g["gamma_all"], dy, coef=coef)
    assert_close(po.to_split(b["dq"]), g["dq"], 1e-11, "dq")
    assert_close(po.to_split(b["dk"]), g["dk"], 1e-11, "dk")
    assert_close(po.to_split(b["dv"]), g["dv"], 1e-11, "dv")
    assert_close(b["dgamma"], g["dgamma"], 1e-10, "dgamma")
    # c = alpha e^{i phi}:  dalpha = Re(conj(e^{i phi}) dc),  dphi = Re(conj(i c) dc)
    dc = b["dcoef"]
    dalpha = (np.conj(np.exp(1j * phase)) * dc).real
    dphase = (np.conj(1j * coef) * dc).real
    assert_close(np.transpose(dalpha, (1, 3, 2, 0)), g["dalpha"], 1e-10, "dalpha")
    assert_close(np.transpose(dphase, (1, 3, 2, 0)), g["dphase"], 1e-10, "dphase")


def test_recurrent_step(golden_dir):
    g = _load(golden_dir, "recur_step.npz")
    y, s = po.recurrent_step(po.to_complex(g["S"]), g["gamma"], po.to_complex(g["v"]),
                             po.to_complex(g["k"]), po.to_complex(g["q"]))
    assert_close(po.to_split(y), g["y"], 1e-13, "y")
    assert_close(po.to_split(s), g["S_new"], 1e-13, "S_new")


def test_scan_varlen_matches_per_sequence():
    p = synthetic.packed_inputs(4, 5, 70, 2, 16, seed=5, dtype=torch.float32)
    q, k, v = (po.to_complex(t.numpy()) for t in (p.q, p.k, p.v))
    y, s = po.scan_varlen(q, k, v, p.gamma.numpy(), p.cu_seqlens.numpy())
    cu = p.cu_seqlens.tolist()
    for i in range(4):
        a, b = cu[i], cu[i + 1]
        yi, si = po.scan_dual_chunked(q[None, :, a:b], k[None, :, a:b], v[None, :, a:b],
                                      p.gamma.numpy()[None, :, a:b], 32)
        assert_close(po.to_split(y[:, a:b]), po.to_split(yi[0]), 1e-12, f"seq {i} Y")
        assert_close(po.to_split(s[0, i]), po.to_split(si[0, 0]), 1e-12, f"seq {i} S")


def test_ce_small(golden_dir):
    # the reference computes logits in fp32 even for fp64 inputs (v11/fused_ce.py:39), so its
    # own outputs carry ~1e-7 rounding; tolerances reflect that, not the oracle's precision
    g = _load(golden_dir, "ce_small.npz")
    r = ce_oracle.linear_ce(g["h"], g["w"], g["t"])
    assert abs(r["loss"] - float(g["loss"])) <= 2e-6 * abs(float(g["loss"]))
    assert_close(r["dH"], g["dh"], 2e-6, "dH")
    assert_close(r["dW"], g["dw"], 2e-6, "dW")
    rm = ce_oracle.linear_ce(g["h"], g["w"], g["t"], mask=g["mask"])
    assert abs(rm["loss"] - float(g["m_loss"])) <= 2e-6 * abs(float(g["m_loss"]))
    assert_close(rm["dH"], g["m_dh"], 2e-6, "masked dH")
    assert_close(rm["dW"], g["m_dw"], 2e-6, "masked dW")
    assert_close(ce_oracle.linear_ce_per_token(g["h"], g["w"], g["t"]), g["per_token"], 2e-6, "per-token")
    np.testing.assert_allclose(ce_oracle.linear_ce_stats(g["h"], g["w"], g["t"]), g["stats"], rtol=2e-6)
    np.testing.assert_allclose(ce_oracle.linear_ce_stats(g["h"], g["w"], g["t"], mask=g["mask"]),
                               g["stats_m"], rtol=2e-6)


def test_ce_c2_loss(golden_dir):
    """Config 2 (N=8192, V=50261): oracle loss vs the reference's fp32 run; sampled grads."""
    g = _load(golden_dir, "ce_c2.npz")
    c2 = synthetic.config2()
    r = ce_oracle.linear_ce(c2.h.float().numpy(), c2.w.float().numpy(), c2.targets.numpy())
    assert abs(r["loss"] - float(g["loss32"])) <= 2e-6 * float(g["loss32"])
    assert_close(r["dH"][g["rows"]], g["dh32"], 1e-5, "dH rows")
    assert_close(r["dW"][g["vrows"]], g["dw32"], 1e-5, "dW rows")
    assert_close(r["dH"][g["rows"]], g["dh"], 1e-2, "dH rows (reference bf16 grads)")


def test_torch_port_matches_oracle():
    """The multi-threaded CPU port used as the timed baseline computes what the oracle computes."""
    from oracle import torch_port
    inp = synthetic.scan_inputs(1, 2, 150, 16, seed=11)
    y, dq, dk, dv, dg = torch_port.scan_fwd_bwd(inp.q.double(), inp.k.double(), inp.v.double(), inp.g.double(),
                                                inp.dy.double(), 64)
    q, k, v, dy = (po.to_complex(t.numpy()) for t in (inp.q, inp.k, inp.v, inp.dy))
    gam = torch.sigmoid(inp.g.double()).numpy()
    y_ref, _ = po.scan_recurrence(q, k, v, gam)
    b = po.scan_backward(q, k, v, gam, dy)
    assert_close(y.numpy(), po.to_split(y_ref), 1e-10, "Y")
    assert_close(dq.numpy(), po.to_split(b["dq"]), 1e-10, "dq")
    assert_close(dk.numpy(), po.to_split(b["dk"]), 1e-10, "dk")
    assert_close(dv.numpy(), po.to_split(b["dv"]), 1e-10, "dv")
    assert_close(dg.numpy(), b["dgamma"][0] * gam * (1 - gam), 1e-9, "dg")
    c = synthetic.ce_inputs(100, 8, 300, seed=2, dtype=torch.float32)
    loss, dh, dw = torch_port.linear_ce_fwd_bwd(c.h, c.w, c.targets, chunk=32)
    r = ce_oracle.linear_ce(c.h.numpy(), c.w.numpy(), c.targets.numpy())
    assert abs(float(loss) - r["loss"]) < 1e-5 * r["loss"]
    assert_close(dh.numpy(), r["dH"], 1e-5, "dH")
    assert_close(dw.numpy(), r["dW"], 1e-5, "dW")
