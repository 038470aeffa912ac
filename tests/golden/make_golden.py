"""Generate golden fixtures by RUNNING THE REFERENCE ITSELF on seeded inputs.

Usage (only where a checkout of the reference is importable):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/qllm2

The reference has no stored golden vectors (its tests are self-consistency scripts),
so the fixtures written here ARE the pin: outputs of the reference's own functions
    V11PAMLayer._forward_chunked_head / flash_pam_chunked_head     (scan fwd + autograd)
    V11PAMLayer._forward_multistate_fused                          (K-state scan)
    V11PAMLayer._recur_step_additive                               (decode step)
    fused_linear_cross_entropy / linear_ce_per_token / linear_ce_stats
Large outputs are stored sub-sampled (every ``STRIDE``-th token) to keep fixtures small;
inputs are regenerated from the seed by qllm2_b200.synthetic and guarded by a checksum.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
if len(sys.argv) < 2:
    sys.exit("usage: python " + sys.argv[0] + " /path/to/qllm2   (a checkout of the reference)")
REF = sys.argv[1]
sys.path.insert(0, REF)
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
sys.dont_write_bytecode = True

from v11 import triton_kernels  # noqa: E402
from v11.flash_pam import flash_pam_chunked_head  # noqa: E402
from v11.fused_ce import fused_linear_cross_entropy, linear_ce_per_token, linear_ce_stats  # noqa: E402
from v11.model import V11Config, V11PAMLayer  # noqa: E402

from qllm2_b200 import synthetic  # noqa: E402

triton_kernels.set_triton_enabled(False)
STRIDE = 16


def checksum(*ts):
    return np.array([float(t.double().sum()) for t in ts] + [float(t.double().abs().sum()) for t in ts])


def layer_for(d, H, chunk, n_states=1):
    cfg = V11Config(vocab_size=64, dim=H * d, n_heads=H, head_dim=d, n_layers=1, dropout=0.0,
                    max_seq_len=64, chunk_size=chunk, n_states=n_states, gradient_checkpointing=False)
    return V11PAMLayer(cfg)


def run_scan(inp, chunk, dtype, use_flash=False):
    q, k, v = (t.to(dtype).clone().requires_grad_(True) for t in (inp.q, inp.k, inp.v))
    g = inp.g.to(dtype).clone().requires_grad_(True)
    gamma = torch.sigmoid(g)
    d = q.shape[-2]
    if use_flash:
        y, s = flash_pam_chunked_head(q, k, v, gamma, d, chunk)
    else:
        layer = layer_for(d, q.shape[1], chunk).to(dtype)
        y, s = layer._forward_chunked_head(q, k, v, gamma, d)
    gamma.retain_grad()
    dq, dk, dv, dg, dgamma = torch.autograd.grad(y, [q, k, v, g, gamma], inp.dy.to(dtype))
    return dict(y=y, s=s, dq=dq, dk=dk, dv=dv, dg=dg, dgamma=dgamma)


def save(name, **arrs):
    out = {}
    for key, val in arrs.items():
        if isinstance(val, torch.Tensor):
            val = val.detach().cpu().numpy()
        out[key] = val
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **out)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def golden_scan_small():
    """selftest-like shape with a ragged tail: T=80 = 3*24 + 8 (v11/selftest.py:16-38)."""
    inp = synthetic.scan_inputs(2, 2, 80, 16, seed=1)
    r = run_scan(inp, 24, torch.float64)
    rf = run_scan(inp, 24, torch.float64, use_flash=True)
    save("scan_small.npz", insum=checksum(inp.q, inp.k, inp.v, inp.g, inp.dy),
         **{k_: v_ for k_, v_ in r.items()}, flash_y=rf["y"], flash_dq=rf["dq"], flash_dgamma=rf["dgamma"])


def golden_scan_c1():
    inp = synthetic.config1()
    r = run_scan(inp, 64, torch.float32)
    r64 = run_scan(inp, 64, torch.float64)
    sub = lambda t: t[:, :, ::STRIDE]
    save("scan_c1.npz", insum=checksum(inp.q, inp.k, inp.v, inp.g, inp.dy), stride=STRIDE,
         y=sub(r["y"]), s=r["s"], dq=sub(r["dq"]), dk=sub(r["dk"]), dv=sub(r["dv"]), dg=r["dg"],
         y64=sub(r64["y"]), s64=r64["s"], dq64=sub(r64["dq"]), dk64=sub(r64["dk"]),
         dv64=sub(r64["dv"]), dg64=r64["dg"],
         norms=np.array([float(r64[k_].norm()) for k_ in ("y", "s", "dq", "dk", "dv", "dg")]))


def golden_e3_small():
    """K=3 phase-routed scan through the reference's fused E3 path (v11/model.py:739-781)."""
    B, H, T, d, K, chunk = 2, 3, 80, 16, 3, 24
    inp = synthetic.scan_inputs(B, H, T, d, seed=2)
    gen = torch.Generator().manual_seed(12)
    gk = torch.randn(K, B, H, T, generator=gen) + torch.tensor([1.0, 3.0, 5.0]).view(K, 1, 1, 1)
    phase = torch.randn(B, T, H, K, generator=gen)
    alpha = 0.5 + torch.rand(B, T, H, K, generator=gen)
    layer = layer_for(d, H, chunk, n_states=K).double()
    q, k, v = (t.double().clone().requires_grad_(True) for t in (inp.q, inp.k, inp.v))
    gamma_all = torch.sigmoid(gk.double()).requires_grad_(True)
    phase_l = phase.double().clone().requires_grad_(True)
    alpha_l = alpha.double().clone().requires_grad_(True)
    layer._gamma_all_and_vprime = lambda x, values: (gamma_all, values)
    layer._phase_and_alpha = lambda x: (phase_l, alpha_l)
    x_dummy = torch.zeros(B, T, H * d, 2, dtype=torch.float64)
    y, s = layer._forward_multistate_fused(x_dummy, q, k, v, d)
    dq, dk, dv, dgam, dph, dal = torch.autograd.grad(y, [q, k, v, gamma_all, phase_l, alpha_l], inp.dy.double())
    save("e3_small.npz", insum=checksum(inp.q, inp.k, inp.v, inp.dy), gamma_all=gamma_all,
         phase=phase, alpha=alpha, y=y, s=s, dq=dq, dk=dk, dv=dv, dgamma=dgam, dphase=dph, dalpha=dal)


def golden_recur_step():
    B, H, d = 2, 3, 16
    gen = torch.Generator().manual_seed(3)
    S = torch.randn(B, H, d, d, 2, generator=gen, dtype=torch.float64)
    gamma = torch.sigmoid(torch.randn(B, H, generator=gen, dtype=torch.float64) + 3)
    v, k, qs = (torch.randn(B, H, d, 2, generator=gen, dtype=torch.float64) for _ in range(3))
    layer = layer_for(d, H, 24)
    y, S2 = layer._recur_step_additive(S, gamma, v, k, qs)
    save("recur_step.npz", S=S, gamma=gamma, v=v, k=k, q=qs, y=y, S_new=S2)


def golden_ce_small():
    """v11/fused_ce.py:144-182 shape: N=200, F=48, V=512, every 7th row ignored; plus a masked run."""
    gen = torch.Generator().manual_seed(4)
    N, F, V = 200, 48, 512
    h = torch.randn(N, F, generator=gen, dtype=torch.float64)
    w = torch.randn(V, F, generator=gen, dtype=torch.float64)
    t = torch.randint(0, V, (N,), generator=gen)
    t[::7] = -100
    mask = (torch.rand(N, generator=gen) > 0.3).double()
    out = {}
    for tag, m in (("", None), ("m_", mask)):
        hh, ww = h.clone().requires_grad_(True), w.clone().requires_grad_(True)
        loss = fused_linear_cross_entropy(hh, ww, t, mask=m, chunk=32)
        loss.backward()
        out[tag + "loss"] = loss.detach()
        out[tag + "dh"] = hh.grad
        out[tag + "dw"] = ww.grad
    per_tok = linear_ce_per_token(h, w, t, chunk=32)
    stats = np.array(linear_ce_stats(h, w, t, chunk=32))
    stats_m = np.array(linear_ce_stats(h, w, t, mask=mask, chunk=32))
    save("ce_small.npz", h=h, w=w, t=t, mask=mask, per_token=per_tok, stats=stats, stats_m=stats_m, **out)


def golden_ce_c2():
    """Config 2 at full size: fp32 math on the bf16-rounded inputs (grads come back bf16)."""
    inp = synthetic.config2()
    h = inp.h.clone().requires_grad_(True)
    w = inp.w.clone().requires_grad_(True)
    loss = fused_linear_cross_entropy(h, w, inp.targets)
    loss.backward()
    # fp32-grad variant of the same math (no per-chunk bf16 rounding of grad_W)
    h32 = inp.h.float().requires_grad_(True)
    w32 = inp.w.float().requires_grad_(True)
    loss32 = fused_linear_cross_entropy(h32, w32, inp.targets)
    loss32.backward()
    rows = torch.arange(0, 8192, 64)
    vrows = torch.cat([torch.arange(0, 50261, 512), inp.targets[:64]])
    save("ce_c2.npz", insum=checksum(inp.h.float(), inp.w.float(), inp.targets.float()),
         loss=loss.detach().float(), loss32=loss32.detach(), rows=rows, vrows=vrows,
         dh=h.grad[rows].float(), dw=w.grad[vrows].float(),
         dh32=h32.grad[rows], dw32=w32.grad[vrows],
         dh_norm=float(h32.grad.double().norm()), dw_norm=float(w32.grad.double().norm()))


if __name__ == "__main__":
    torch.set_num_threads(os.cpu_count())
    which = sys.argv[2:] or ["scan_small", "scan_c1", "e3_small", "recur_step", "ce_small", "ce_c2"]
    for name in which:
        globals()["golden_" + name]()
