"""Inference forward through packed weights and the fused block kernels vs the module path.

The module path (V11Block operators) is pinned to the reference by tests/test_gpu_model.py; here the
packed forward must reproduce its hidden states (fp32: 1e-4 relative; bf16: 2e-2) and greedy ids.
"""
import pytest
import torch

from qllm2_b200 import model as M, ops
from qllm2_b200.fused_forward import FusedForward
from qllm2_b200.serving import ContinuousBatcher

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _ScanMix:
    q_scale = 1.0

    def __call__(self, layer, q, k, v, gamma, coef):
        y, _ = ops.pam_scan(q, k, v, gamma, coef=coef, head_dim=q.shape[3])
        return y.transpose(1, 2).reshape(q.shape[2], -1)


def rel(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm())


VARIANTS = {
    "k1_swish": dict(n_states=1),
    "k3_content_gate": dict(n_states=3, gate_content_aware=True),
    "k3_compete_routed": dict(n_states=3, gate_content_aware=True, routing_content_aware=True, state_compete=True,
                              phase_init="spread"),
    "k2_compete_magnitude_routing": dict(n_states=2, state_compete=True, phase_init="ortho"),
    "k1_modrelu_no_gsp_floor": dict(n_states=1, activation="modrelu", use_gsp=False, gamma_floor=0.05),
    "k3_no_rope_d32": dict(n_states=3, use_rope=False, head_dim=32, n_heads=4),
}


def _net(over, dtype=torch.float32):
    torch.manual_seed(0)
    kw = dict(vocab_size=257, dim=64, n_heads=2, head_dim=32, n_layers=3, expand=2, dropout=0.0, max_seq_len=256,
              gradient_checkpointing=False, chunk_size=64)
    kw.update(over)
    net = M.V11LM(M.V11Config(**kw)).to(DEV).eval()
    with torch.no_grad():                      # move every gate and routing weight off its zero/constant init
        for p in net.parameters():
            if p.dim() <= 1:
                p.add_(0.2 * torch.randn_like(p))
        for blk in net.blocks:
            if hasattr(blk.pam, "score_proj"):
                blk.pam.score_proj.weight.normal_(std=0.3)
    return net.to(dtype)


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_hidden_and_head_match_module_path_fp32(variant):
    net = _net(VARIANTS[variant])
    ids = torch.randint(0, 257, (1, 150), generator=torch.Generator().manual_seed(1)).to(DEV)
    ff = FusedForward(net, max_position=512)
    xn = ff.hidden(ids, _ScanMix())
    with torch.no_grad():
        z = net._embed(ids, 0)
        z, _ = net._run_blocks(z, None, 0, False)
        ref = net.output_norm(z)[0]
        ref_lm = net._head_hidden(z)[0]
    assert rel(xn, ref) < 1e-4
    lm = ff.head_hidden(xn)
    assert rel(lm, ref_lm) < 1e-4
    assert torch.equal(ff.greedy_next(lm), net.greedy_next(ref_lm))


def test_long_prefill_uses_the_many_row_kernels():
    """More rows than one CTA per row covers (the warp-per-row sweep of the residual+norm kernel)."""
    net = _net(dict(VARIANTS["k3_compete_routed"], max_seq_len=2048))
    ids = torch.randint(0, 257, (1, 1500), generator=torch.Generator().manual_seed(3)).to(DEV)
    xn = FusedForward(net, max_position=2048).hidden(ids, _ScanMix())
    with torch.no_grad():
        z = net._embed(ids, 0)
        z, _ = net._run_blocks(z, None, 0, False)
        ref = net.output_norm(z)[0]
    assert rel(xn, ref) < 1e-4


def test_hidden_matches_module_path_bf16():
    net = _net(VARIANTS["k3_content_gate"], torch.bfloat16)
    ids = torch.randint(0, 257, (1, 130), generator=torch.Generator().manual_seed(2)).to(DEV)
    xn = FusedForward(net, max_position=512).hidden(ids, _ScanMix())
    with torch.no_grad():
        z = net._embed(ids, 0)
        z, _ = net._run_blocks(z, None, 0, False)
        ref = net.output_norm(z)[0]
    assert rel(xn, ref) < 2e-2


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("variant", ["k3_compete_routed", "k2_compete_magnitude_routing", "k1_modrelu_no_gsp_floor"])
def test_batcher_fused_equals_module_path(variant, graph):
    """Continuous batching through the packed forward (optionally replayed from a CUDA graph) yields the
    same token ids as the module path, sequence by sequence (fp32)."""
    net = _net(VARIANTS[variant])
    gen = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 257, (int(n),), generator=gen).tolist() for n in (3, 40, 25, 1, 70, 12)]
    outs = []
    for fused in (True, False):
        eng = ContinuousBatcher(net, n_slots=4, cuda_graph=graph and fused, fused=fused, max_position=512)
        assert (eng.ff is not None) == fused
        rids = [eng.submit(p, 6) for p in prompts]
        res = eng.run()
        outs.append([res[r] for r in rids])
    assert outs[0] == outs[1]


def test_positions_beyond_the_table_are_refused():
    net = _net(VARIANTS["k1_swish"])
    eng = ContinuousBatcher(net, n_slots=2, max_position=16)
    eng.submit(list(range(1, 30)), 2)
    with pytest.raises(RuntimeError):
        eng.run()


@pytest.mark.parametrize("variant", ["k3_compete_routed", "k1_swish"])
def test_generate_on_the_packed_forward_equals_the_module_loop(variant):
    net = _net(VARIANTS[variant])
    ids = torch.randint(0, 257, (3, 21), generator=torch.Generator().manual_seed(6)).to(DEV)
    fast = net.generate(ids, max_new_tokens=9, temperature=0.0)
    slow = net.generate(ids, max_new_tokens=9, temperature=0.0, fused=False)
    assert fast.shape == (3, 30) and torch.equal(fast, slow)
    one = net.generate(ids, max_new_tokens=1, temperature=0.0)
    assert torch.equal(one, slow[:, :22])
    # sampling path: logits come from the packed head; same seed, same path -> same tokens, all in range
    torch.manual_seed(3)
    a = net.generate(ids, max_new_tokens=6, temperature=0.8, top_k=20, top_p=0.9, repetition_penalty=1.1)
    torch.manual_seed(3)
    b = net.generate(ids, max_new_tokens=6, temperature=0.8, top_k=20, top_p=0.9, repetition_penalty=1.1)
    assert torch.equal(a, b) and int(a.max()) < 257 and torch.equal(a[:, :21], ids)
    # an end-of-sequence id stops the loop early
    eos = int(slow[0, 21])
    stopped = net.generate(ids[:1], max_new_tokens=9, temperature=0.0, eos_token_id=eos)
    assert stopped.shape[1] == 22


@pytest.mark.parametrize("fused", [True, False])
def test_chunked_prefill_equals_whole_prefill(fused):
    """Prompts absorbed in pieces of at most 16 tokens per step (each piece scanned from the state its
    predecessor left in the slot) decode to the same ids as whole-prompt prefill."""
    net = _net(VARIANTS["k3_compete_routed"])
    gen = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 257, (int(n),), generator=gen).tolist() for n in (70, 5, 33, 16, 41)]
    outs = []
    for chunked in (True, False):
        eng = ContinuousBatcher(net, n_slots=3, fused=fused, max_position=512, chunked_prefill=chunked,
                                max_prefill_tokens=16 if chunked else 1 << 16)
        rids = [eng.submit(p, 5) for p in prompts]
        res = eng.run()
        outs.append([res[r] for r in rids])
        if chunked:
            assert eng.steps > 10           # 165 prompt tokens at 16 per step
    assert outs[0] == outs[1]
