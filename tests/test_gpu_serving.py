"""Continuous-batching greedy decode: token ids equal the reference's per-sequence decode."""
import os

import numpy as np
import pytest
import torch

from qllm2_b200.serving import ContinuousBatcher
from tests.test_gpu_model import _load

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("name", ["k1", "k3", "d64"])
def test_batcher_matches_reference_greedy(golden_dir, name, fused):
    """The golden prompt decoded inside a busy batch (other sequences joining and leaving around it)."""
    g, net = _load(golden_dir, name)
    V = net.config.vocab_size
    eng = ContinuousBatcher(net, n_slots=3, fused=fused)
    assert (eng.ff is not None) == fused
    gen = torch.Generator().manual_seed(0)
    others = [torch.randint(0, V, (n,), generator=gen).tolist() for n in (5, 33, 64, 9, 17)]
    eng.submit(others[0], 3)
    eng.submit(others[1], 7)
    rid = eng.submit(g["ids"][0, :20].tolist(), len(g["greedy"]))
    for o in others[2:]:
        eng.submit(o, 5)
    out = eng.run()
    assert out[rid] == g["greedy"].tolist(), (out[rid], g["greedy"].tolist(), g["greedy_margin"])
    assert len(out) == 6 and all(len(v) > 0 for v in out.values())


@pytest.mark.parametrize("graph", [False, True])
def test_batcher_equals_sequential_generate(golden_dir, graph):
    """Every sequence decoded in the batch equals the same sequence decoded alone by V11LM.generate
    (graph=True: the decode step is replayed from one captured CUDA graph)."""
    g, net = _load(golden_dir, "k3")
    V = net.config.vocab_size
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, V, (int(n),), generator=gen) for n in (3, 40, 25, 1, 70, 12, 31)]
    eng = ContinuousBatcher(net, n_slots=4, cuda_graph=graph)
    rids = [eng.submit(p.tolist(), 6) for p in prompts]
    out = eng.run()
    mism = 0
    for rid, p in zip(rids, prompts):
        alone = net.generate(p[None].to(DEV), max_new_tokens=6, temperature=0.0)[0, len(p):].tolist()
        mism += int(alone != out[rid])
    assert mism == 0
