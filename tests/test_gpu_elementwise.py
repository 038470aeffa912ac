"""Fused element-wise complex operators against the reference's plain arithmetic.

Golden vectors (tests/golden/elementwise.npz) come from the reference's `_pt_*` functions in float64;
fp32 kernels must match to 1e-4 relative, bf16 to 2e-2.  Larger seeded cases compare with the same
arithmetic written in torch (fp32) on the device.
"""
import os

import numpy as np
import pytest
import torch

from qllm2_b200 import fused_elementwise as FE
from qllm2_b200._lib import QPamError

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    a, b = a.detach().double().flatten(), b.detach().double().flatten()
    return float((a - b).norm() / (b.norm() + 1e-30))


@pytest.fixture(scope="module")
def gold(golden_dir):
    return dict(np.load(os.path.join(golden_dir, "elementwise.npz")))


def _t(g, key, dtype=torch.float32, grad=False):
    return torch.from_numpy(g[key]).to(DEV).to(dtype).requires_grad_(grad)


CASES = {
    "norm": (lambda z, p: FE.fused_complex_norm(z, p["scale"], 1e-6), ["scale"]),
    "swish": (lambda z, p: FE.fused_mod_swish(z, p["bias"], p["beta"]), ["bias", "beta"]),
    "relu": (lambda z, p: FE.fused_mod_relu(z, p["bias"]), ["bias"]),
    "gate": (lambda z, p: FE.fused_cgu_gate(z, p["up"]), ["up"]),
}


@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("name", list(CASES))
def test_against_reference_golden(gold, tag, name):
    fn, wrt = CASES[name]
    z = _t(gold, f"{tag}_z", grad=True)
    p = {k: _t(gold, f"{tag}_{k}", grad=True) for k in wrt}
    dout = _t(gold, f"{tag}_dout")
    y = fn(z, p)
    assert y.dtype == torch.float32 and y.shape == z.shape
    grads = torch.autograd.grad((y * dout).sum(), [z] + [p[k] for k in wrt])
    assert rel(y, _t(gold, f"{tag}_{name}_out")) < 1e-4
    for i, g in enumerate(grads):
        assert rel(g, _t(gold, f"{tag}_{name}_grad{i}")) < 1e-4, (name, i)


@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("name", list(CASES))
def test_bf16_io_matches_fp32_on_the_same_rounded_inputs(gold, tag, name):
    """bf16 tensors in and out, fp32 arithmetic inside: against the fp32 kernels fed the bf16-rounded
    values, only the rounding of the results differs (2e-2 is the bf16 bar; parameters stay fp32)."""
    fn, wrt = CASES[name]
    outs = []
    for dtype in (torch.bfloat16, torch.float32):
        z = _t(gold, f"{tag}_z", torch.bfloat16).to(dtype).requires_grad_(True)
        p = {k: (_t(gold, f"{tag}_{k}", torch.bfloat16).to(dtype) if k == "up" else _t(gold, f"{tag}_{k}")).requires_grad_(True)
             for k in wrt}
        dout = _t(gold, f"{tag}_dout", torch.bfloat16).to(dtype)
        y = fn(z, p)
        assert y.dtype == dtype
        outs.append([y] + list(torch.autograd.grad((y.float() * dout.float()).sum(), [z] + [p[k] for k in wrt])))
    for a, b in zip(*outs):
        assert rel(a, b) < 2e-2


def _pt_norm(z, scale, eps=1e-6):
    mag = torch.sqrt(z[..., 0] ** 2 + z[..., 1] ** 2 + 1e-8)
    rms = torch.sqrt((mag ** 2).mean(-1, keepdim=True) + eps)
    return z / (mag.unsqueeze(-1) + 1e-8) * ((mag / rms) * scale).unsqueeze(-1)


def _pt_swish(z, bias, beta):
    mag = torch.sqrt(z[..., 0] ** 2 + z[..., 1] ** 2 + 1e-8)
    return z / (mag.unsqueeze(-1) + 1e-8) * (mag * torch.sigmoid(beta * mag + bias)).unsqueeze(-1)


def _pt_gate(gate, up):
    mag = torch.sqrt(gate[..., 0] ** 2 + gate[..., 1] ** 2 + 1e-8)
    ph = gate / (mag.unsqueeze(-1) + 1e-8)
    pr = ph[..., 0] * up[..., 0] - ph[..., 1] * up[..., 1]
    pi = ph[..., 0] * up[..., 1] + ph[..., 1] * up[..., 0]
    return torch.stack([pr, pi], -1) * torch.sigmoid(mag)[..., None]


@pytest.mark.parametrize("N,C", [(1, 384), (4099, 384), (777, 1152), (130, 2304)])
def test_large_rows_match_torch_arithmetic(N, C):
    g = torch.Generator().manual_seed(N + C)
    z = torch.randn(N, C, 2, generator=g).to(DEV).requires_grad_(True)
    up = torch.randn(N, C, 2, generator=g).to(DEV).requires_grad_(True)
    dout = torch.randn(N, C, 2, generator=g).to(DEV)
    scale = (1 + 0.2 * torch.randn(C, generator=g)).to(DEV).requires_grad_(True)
    bias = (0.5 * torch.randn(C, generator=g)).to(DEV).requires_grad_(True)
    beta = (1 + 0.2 * torch.randn(C, generator=g)).to(DEV).requires_grad_(True)
    pairs = [
        (lambda: FE.fused_complex_norm(z, scale), lambda: _pt_norm(z, scale), [z, scale]),
        (lambda: FE.fused_mod_swish(z, bias, beta), lambda: _pt_swish(z, bias, beta), [z, bias, beta]),
        (lambda: FE.fused_cgu_gate(z, up), lambda: _pt_gate(z, up), [z, up]),
    ]
    for ours, theirs, wrt in pairs:
        y, yr = ours(), theirs()
        assert rel(y, yr) < 1e-5
        ga = torch.autograd.grad((y * dout).sum(), wrt)
        gb = torch.autograd.grad((yr * dout).sum(), wrt)
        for a, b in zip(ga, gb):
            assert rel(a, b) < 1e-4


def test_norm_under_autocast_returns_bf16_and_matches():
    g = torch.Generator().manual_seed(5)
    z = torch.randn(3, 50, 384, 2, generator=g).to(DEV).requires_grad_(True)
    scale = torch.ones(384, device=DEV, requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = FE.fused_complex_norm(z, scale)
    assert y.dtype == torch.bfloat16
    yr = _pt_norm(z, scale)
    assert rel(y, yr) < 1e-2
    dout = torch.randn_like(yr)
    ga = torch.autograd.grad((y.float() * dout).sum(), [z, scale])
    gb = torch.autograd.grad((yr * dout).sum(), [z, scale])
    assert ga[0].dtype == torch.float32
    assert rel(ga[0], gb[0]) < 2e-2 and rel(ga[1], gb[1]) < 2e-2


def test_packed_gate_equals_two_tensor_gate_and_strided_views():
    g = torch.Generator().manual_seed(9)
    gu = torch.randn(5, 11, 2 * 96, 2, generator=g).to(DEV).requires_grad_(True)
    dout = torch.randn(5, 11, 96, 2, generator=g).to(DEV)
    y1 = FE.fused_cgu_gate_packed(gu)
    (g1,) = torch.autograd.grad((y1 * dout).sum(), [gu])
    y2 = FE.fused_cgu_gate(gu[..., :96, :], gu[..., 96:, :])     # strided views, no copies
    (g2,) = torch.autograd.grad((y2 * dout).sum(), [gu])
    y3 = _pt_gate(gu[..., :96, :], gu[..., 96:, :])
    (g3,) = torch.autograd.grad((y3 * dout).sum(), [gu])
    assert torch.equal(y1, y2) and torch.equal(g1, g2)
    assert rel(y1, y3) < 1e-5 and rel(g1, g3) < 1e-4


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,d", [(6, 64), (3, 32), (2, 128)])
def test_pam_prep_matches_torch_path(dtype, tol, H, d):
    from qllm2_b200.model import _complex_mul, build_rope_cache
    B, T = 2, 37
    g = torch.Generator().manual_seed(H * d)
    qkv32 = torch.randn(B, T, 3 * H * d, 2, generator=g).to(DEV)
    omp32 = torch.rand(B, T, H, generator=g).to(DEV)
    rope = build_rope_cache(128, d).to(DEV)
    douts = [torch.randn(B, H, T, d, 2, generator=g).to(DEV) for _ in range(3)]
    for positions, offset in ((None, 5), (torch.randint(0, 128, (B, T), generator=g).to(DEV), 0)):
        qkv = qkv32.to(dtype).requires_grad_(True)
        omp = omp32.clone().requires_grad_(True)
        q, k, v = FE.pam_prep(qkv, rope, omp, n_heads=H, head_dim=d, positions=positions, offset=offset)
        ga = torch.autograd.grad(sum((a.float() * b).sum() for a, b in zip((q, k, v), douts)), [qkv, omp])
        # the same stage with torch operators in fp32 (the module's own path)
        x = qkv32.clone().requires_grad_(True)
        o2 = omp32.clone().requires_grad_(True)
        parts = x.view(B, T, 3, H, d, 2)
        qr, kr, vr = (parts[:, :, i].transpose(1, 2) for i in range(3))
        rot = (rope[offset:offset + T] if positions is None else rope[positions].unsqueeze(1))
        qr, kr = _complex_mul(qr, rot), _complex_mul(kr, rot)
        vr = vr * o2.transpose(1, 2)[..., None, None]
        gb = torch.autograd.grad(sum((a * b).sum() for a, b in zip((qr, kr, vr), douts)), [x, o2])
        for a, b in zip((q, k, v), (qr, kr, vr)):
            assert a.shape == b.shape and rel(a, b) < tol
        assert rel(ga[0], gb[0]) < tol and rel(ga[1], gb[1]) < tol


def test_wrappers_refuse_bad_input_before_any_launch():
    z = torch.randn(4, 6, 2, device=DEV)          # 6 channels: not a multiple of 4
    with pytest.raises(QPamError):
        FE.fused_complex_norm(z, torch.ones(6, device=DEV))
    with pytest.raises(QPamError):
        FE.fused_mod_relu(torch.randn(4, 8, 2), torch.zeros(8))           # CPU tensor
    with pytest.raises(QPamError):
        FE.fused_cgu_gate(torch.randn(4, 8, 2, device=DEV), torch.randn(4, 12, 2, device=DEV))
    with pytest.raises(QPamError):
        FE.pam_prep(torch.randn(1, 4, 3 * 2 * 24, 2, device=DEV), None, None, n_heads=2, head_dim=24)
    with pytest.raises(QPamError):
        FE.fused_mod_swish(torch.randn(4, 8, 2, device=DEV), torch.zeros(8, device=DEV), torch.zeros(4, device=DEV))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("K,d", [(3, 64), (2, 32), (4, 128), (1, 16)])
def test_state_combine_matches_complex_sum(dtype, tol, K, d):
    g = torch.Generator().manual_seed(K * d)
    shape = (2, 3, 29)
    yks32 = [torch.randn(*shape, d, 2, generator=g).to(DEV) for _ in range(K)]
    coef32 = torch.randn(K, *shape, 2, generator=g).to(DEV)
    dy = torch.randn(*shape, d, 2, generator=g).to(DEV)
    yks = [t.to(dtype).requires_grad_(True) for t in yks32]
    coef = coef32.clone().requires_grad_(True)
    y = FE.state_combine(coef, yks)
    ga = torch.autograd.grad((y.float() * dy).sum(), [coef] + yks)
    ref_in = [t.clone().requires_grad_(True) for t in yks32]
    cr = coef32.clone().requires_grad_(True)
    yr = sum(torch.view_as_real(torch.view_as_complex(cr[k]).unsqueeze(-1) * torch.view_as_complex(ref_in[k]))
             for k in range(K))
    gb = torch.autograd.grad((yr * dy).sum(), [cr] + ref_in)
    assert y.dtype == dtype and rel(y, yr) < tol
    for a, b in zip(ga, gb):
        assert rel(a, b) < tol


@pytest.mark.parametrize("xd,dd", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                   (torch.bfloat16, torch.bfloat16)])
def test_scaled_residual_matches_torch(xd, dd):
    g = torch.Generator().manual_seed(11)
    x32 = torch.randn(37, 52, 2, generator=g).to(DEV)
    d32 = torch.randn(37, 52, 2, generator=g).to(DEV)
    dout = torch.randn(37, 52, 2, generator=g).to(DEV)
    s = torch.tensor(0.37, device=DEV, requires_grad=True)
    x = x32.to(xd).requires_grad_(True)
    d = d32.to(dd).requires_grad_(True)
    y = FE.scaled_residual(x, d, s)
    assert y.dtype == xd
    ga = torch.autograd.grad((y.float() * dout).sum(), [x, d, s])
    xr, dr, sr = x.detach().float().requires_grad_(True), d.detach().float().requires_grad_(True), s.detach().clone().requires_grad_(True)
    yr = xr + dr * sr
    gb = torch.autograd.grad((yr * dout).sum(), [xr, dr, sr])
    tol = 1e-6 if xd == torch.float32 and dd == torch.float32 else 1e-2
    assert rel(y, yr) < tol
    for a, b in zip(ga, gb):
        assert rel(a, b) < tol


@pytest.mark.parametrize("wd,od", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                   (torch.bfloat16, torch.bfloat16)])
def test_block_weight_is_the_complex_product(wd, od):
    g = torch.Generator().manual_seed(12)
    out_dim, in_dim = 24, 40
    wr = torch.randn(out_dim, in_dim, generator=g).to(DEV).to(wd).requires_grad_(True)
    wi = torch.randn(out_dim, in_dim, generator=g).to(DEV).to(wd).requires_grad_(True)
    x = torch.randn(9, in_dim, 2, generator=g).to(DEV)
    dy = torch.randn(9, out_dim, 2, generator=g).to(DEV)
    w = FE.block_weight(wr, wi, od)
    assert w.dtype == od and w.shape == (2 * out_dim, 2 * in_dim)
    y = (x.reshape(9, 2 * in_dim) @ w.float().T).view(9, out_dim, 2)
    ga = torch.autograd.grad((y * dy).sum(), [wr, wi])
    wr2, wi2 = wr.detach().float().requires_grad_(True), wi.detach().float().requires_grad_(True)
    yc = torch.view_as_complex(x) @ torch.complex(wr2, wi2).T
    gb = torch.autograd.grad((torch.view_as_real(yc) * dy).sum(), [wr2, wi2])
    tol = 1e-5 if od == torch.float32 else 1e-2
    assert rel(y, torch.view_as_real(yc)) < tol
    for a, b in zip(ga, gb):
        assert rel(a, b) < tol


def test_token_major_scan_equals_scan_then_head_merge():
    """`pam_scan_tokens` (inference: K bf16 scans + read-out written token-major) against `pam_scan` + transpose."""
    from qllm2_b200 import ops
    g = torch.Generator().manual_seed(21)
    B, H, T, d, K = 2, 3, 200, 64, 3
    q, k, v = (torch.randn(B, H, T, d, 2, generator=g).mul(0.125).to(DEV).bfloat16() for _ in range(3))
    gamma = torch.sigmoid(torch.randn(K, B, H, T, generator=g) + 3).to(DEV)
    coef = torch.randn(K, B, H, T, 2, generator=g).to(DEV)
    with torch.no_grad():
        y_ref, s_ref = ops.pam_scan(q, k, v, gamma, coef=coef)
        y_tok, s_tok = ops.pam_scan_tokens(q, k, v, gamma, coef=coef)
    assert y_tok.shape == (B, T, H * d, 2)
    assert torch.equal(y_tok, y_ref.transpose(1, 2).reshape(B, T, H * d, 2))
    assert torch.equal(s_tok, s_ref)
    # one state (single-state tensor-core kernel, token-major store) and packed sequences
    with torch.no_grad():
        y1, s1 = ops.pam_scan_tokens(q, k, v, gamma[0])
        r1, t1 = ops.pam_scan(q, k, v, gamma[0])
        cu = torch.tensor([0, 70, 70, 200], dtype=torch.int32)
        y2, s2 = ops.pam_scan_tokens(q[:1], k[:1], v[:1], gamma[:, :1], coef=coef[:, :1], cu_seqlens=cu)
        r2, t2 = ops.pam_scan(q[:1], k[:1], v[:1], gamma[:, :1], coef=coef[:, :1], cu_seqlens=cu)
    assert torch.equal(y1, r1.transpose(1, 2).reshape(B, T, H * d, 2)) and torch.equal(s1, t1)
    assert torch.equal(y2, r2.transpose(1, 2).reshape(1, T, H * d, 2)) and torch.equal(s2, t2)
    # fp32 (no fused read-out): same contract
    y32, _ = ops.pam_scan_tokens(q.float(), k.float(), v.float(), gamma, coef=coef)
    r32, _ = ops.pam_scan(q.float(), k.float(), v.float(), gamma, coef=coef)
    assert torch.equal(y32, r32.transpose(1, 2).reshape(B, T, H * d, 2))


@pytest.mark.parametrize("K,use_pg,use_score,floor", [(3, True, True, 0.0), (3, True, False, 0.05), (1, True, False, 0.0),
                                                      (2, False, True, 0.0), (1, False, False, 0.1), (4, True, True, 0.0)])
def test_pam_gates_match_torch_arithmetic(K, use_pg, use_score, floor):
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(K * 7 + int(use_pg))
    B, T, H = 2, 19, 3
    mk = lambda *s: torch.randn(*s, generator=g).to(DEV).requires_grad_(True)
    dt, bias = mk(B, T, H), mk(H)
    pg = mk(B, T, H) if use_pg else None
    phase = mk(B, T, H, K) if K > 1 else None
    score = mk(B, T, H, K) if (use_score and K > 1) else None
    off = mk(K) if K > 1 else None
    gamma, omp, coef = FE.pam_gates(dt, pg, phase, score, bias, off, floor, K)
    # the module's arithmetic (v11/model.py:630-655, 685-720) with torch operators
    x = (dt + bias).unsqueeze(0) + (off.view(K, 1, 1, 1) if off is not None else 0)
    base = torch.exp(-F.softplus(x)).permute(0, 1, 3, 2)                       # [K,B,H,T]
    if floor > 0:
        base = floor + (1 - floor) * base
    if use_pg:
        p = torch.sigmoid(pg)
        gamma_ref = base * (1 - p.transpose(1, 2)) + p.transpose(1, 2)
        omp_ref = 1 - p
    else:
        gamma_ref, omp_ref = base, None
    coef_ref = None
    if K > 1:
        w = F.softmax(score, dim=-1) * K if score is not None else torch.ones_like(phase)
        ph, w = phase.permute(3, 0, 2, 1), w.permute(3, 0, 2, 1)
        coef_ref = torch.stack([w * torch.cos(ph), w * torch.sin(ph)], dim=-1)
    assert gamma.shape == (K, B, H, T) and rel(gamma, gamma_ref) < 1e-5
    assert (omp is None) == (omp_ref is None) and (coef is None) == (coef_ref is None)
    outs, refs = [gamma], [gamma_ref]
    if omp is not None:
        assert rel(omp, omp_ref) < 1e-5
        outs.append(omp); refs.append(omp_ref)
    if coef is not None:
        assert rel(coef, coef_ref) < 1e-5
        outs.append(coef); refs.append(coef_ref)
    ups = [torch.randn(o.shape, generator=g).to(DEV) for o in outs]
    wrt = [t for t in (dt, pg, phase, score, bias, off) if t is not None]
    ga = torch.autograd.grad(sum((o * u).sum() for o, u in zip(outs, ups)), wrt)
    gb = torch.autograd.grad(sum((o * u).sum() for o, u in zip(refs, ups)), wrt)
    for a, b in zip(ga, gb):
        assert a.shape == b.shape and rel(a, b) < 1e-4


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-2)])
def test_complex_magnitude_matches_torch(dtype, tol):
    g = torch.Generator().manual_seed(31)
    z32 = torch.randn(3, 17, 24, 2, generator=g).to(DEV)
    z32[0, 0, :4] = 0                                     # the 1e-8 guard keeps the gradient finite at zero
    dm = torch.randn(3, 17, 24, generator=g).to(DEV)
    z = z32.to(dtype).requires_grad_(True)
    m = FE.complex_magnitude(z)
    (gz,) = torch.autograd.grad((m.float() * dm).sum(), [z])
    zr = z.detach().float().requires_grad_(True)
    mr = torch.sqrt(zr[..., 0] ** 2 + zr[..., 1] ** 2 + 1e-8)
    (gr,) = torch.autograd.grad((mr * dm).sum(), [zr])
    assert m.dtype == dtype and m.shape == (3, 17, 24)
    assert rel(m, mr) < tol and rel(gz, gr) < tol and torch.isfinite(gz.float()).all()


def test_state_combine_token_major_with_gradients():
    g = torch.Generator().manual_seed(41)
    B, H, T, d, K = 2, 3, 21, 64, 3
    yks = [torch.randn(B, H, T, d, 2, generator=g).to(DEV).requires_grad_(True) for _ in range(K)]
    coef = torch.randn(K, B, H, T, 2, generator=g).to(DEV).requires_grad_(True)
    dy = torch.randn(B, T, H * d, 2, generator=g).to(DEV)
    y_tm = FE.state_combine(coef, yks, token_major=True)
    y = FE.state_combine(coef, yks)
    assert y_tm.shape == (B, T, H * d, 2) and torch.equal(y_tm, y.transpose(1, 2).reshape(B, T, H * d, 2))
    ga = torch.autograd.grad((y_tm * dy).sum(), [coef] + yks)
    gb = torch.autograd.grad((y.transpose(1, 2).reshape(B, T, H * d, 2) * dy).sum(), [coef] + yks)
    for a, b in zip(ga, gb):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-5)
