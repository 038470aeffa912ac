"""Host-side logic of the packed inference forward and of the element-wise wrappers (no GPU).

The packed matrices must reproduce the modules' projections exactly when applied with plain
matmuls on the CPU: that is the algebra the GPU path relies on.
"""
import pytest
import torch
import torch.nn.functional as F

from qllm2_b200 import model as M
from qllm2_b200.fused_elementwise import _rows
from qllm2_b200.fused_forward import FusedForward
from qllm2_b200.model import _concat_planes, _magnitude

VARIANTS = {
    "k3_content_gate": dict(n_states=3, gate_content_aware=True),
    "k3_all_content_aware_compete": dict(n_states=3, gate_content_aware=True, routing_content_aware=True, state_compete=True),
    "k2_magnitude_inputs_compete": dict(n_states=2, state_compete=True),
    "k1_no_gsp": dict(n_states=1, use_gsp=False),
}


def _block(over):
    torch.manual_seed(0)
    cfg = M.V11Config(vocab_size=64, dim=24, n_heads=3, head_dim=8, n_layers=1, expand=2, dropout=0.0, **over)
    net = M.V11LM(cfg)
    with torch.no_grad():
        for p in net.parameters():
            p.add_(0.1 * torch.randn_like(p))
    return net.blocks[0], cfg


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_packed_matrices_reproduce_the_module_projections(variant):
    blk, cfg = _block(VARIANTS[variant])
    L = FusedForward.pack_block(blk, torch.float32)
    N, D, H, K = 7, cfg.dim, cfg.n_heads, cfg.n_states
    inner = cfg.n_heads * cfg.head_dim
    x = torch.randn(N, D, 2)
    flat = x.reshape(N, 2 * D)                                     # interleaved columns
    with torch.no_grad():
        # gate | up in one matrix, each half already interleaved complex
        gu = F.linear(flat, L.w_gu).view(N, 2, L.hidden, 2)
        assert torch.allclose(gu[:, 0], blk.cgu.gate_proj(x), atol=1e-5)
        assert torch.allclose(gu[:, 1], blk.cgu.up_proj(x), atol=1e-5)
        h = torch.randn(N, L.hidden, 2)
        assert torch.allclose(F.linear(h.reshape(N, -1), L.w_down).view(N, D, 2), blk.cgu.down_proj(h), atol=1e-5)
        y = torch.randn(N, inner, 2)
        assert torch.allclose(F.linear(y.reshape(N, -1), L.w_o).view(N, D, 2), blk.pam.o_proj(y), atol=1e-5)
        # the front projection: qkv, then every small Linear that reads the layer input
        raw = F.linear(flat, L.w_front, L.b_front)
        assert raw.shape[1] % 8 == 0
        assert torch.allclose(raw[:, :6 * inner].reshape(N, 3 * inner, 2), blk.pam.qkv_proj(x), atol=1e-5)
        rawm = F.linear(_magnitude(x), L.w_mag, L.b_mag) if L.w_mag is not None else None
        lin = {"dt": (blk.pam.dt_proj, True), "pg": (getattr(blk.pam, "protect_gate", None), blk.pam.gate_content_aware),
               "phase": (getattr(blk.pam, "phase_proj", None), blk.pam.routing_content_aware),
               "score": (getattr(blk.pam, "score_proj", None), blk.pam.routing_content_aware)}
        expected = {"dt"} | ({"pg"} if cfg.use_gsp else set()) | ({"phase"} if K > 1 else set()) \
            | ({"score"} if K > 1 and cfg.state_compete else set())
        assert set(L.cols) == expected
        for name, (src, off) in L.cols.items():
            mod, content = lin[name]
            assert (src == "a") == bool(content)
            ref = mod(_concat_planes(x)) if content else mod(_magnitude(x))
            got = (raw if src == "a" else rawm)[:, off:off + ref.shape[1]]
            assert torch.allclose(got, ref, atol=1e-5), name


def test_unsupported_configurations_are_named():
    torch.manual_seed(0)
    net = M.V11LM(M.V11Config(vocab_size=32, dim=16, n_heads=2, head_dim=8, n_layers=1, dropout=0.0))
    assert "CUDA" in FusedForward.unsupported_reason(net)            # a CPU model
    net2 = M.V11LM(M.V11Config(vocab_size=32, dim=16, n_heads=2, head_dim=8, n_layers=1, dropout=0.0, qk_norm=True))
    assert "qk_norm" in FusedForward.unsupported_reason(net2)
    net3 = M.V11LM(M.V11Config(vocab_size=32, dim=24, n_heads=2, head_dim=12, n_layers=1, dropout=0.0))
    assert "power of two" in FusedForward.unsupported_reason(net3)


def test_row_view_logic_of_the_elementwise_wrappers():
    base = torch.zeros(5, 11, 2 * 96, 2)
    t, N, C, ld = _rows(base[..., :96, :])                            # column block of a wider matrix: no copy
    assert (N, C, ld) == (55, 96, 4 * 96) and t.data_ptr() == base.data_ptr()
    t, N, C, ld = _rows(base)                                         # dense
    assert (N, C, ld) == (55, 192, 384)
    t, N, C, ld = _rows(base.transpose(0, 1)[..., 96:, :])            # leading dims not collapsible: copied
    assert (N, C, ld) == (55, 96, 192) and t.is_contiguous()
    t, N, C, ld = _rows(torch.zeros(8, 2))                            # a single row
    assert (N, C, ld) == (1, 8, 16)
    with pytest.raises(Exception):
        _rows(torch.zeros(4, 6, 2))                                   # 6 channels: not a multiple of 4
