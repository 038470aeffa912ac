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


@pytest.mark.parametrize("graph,fused", [(False, True), (True, True), (False, False)])
def test_sampling_engine_with_top_k_one_equals_greedy(golden_dir, graph, fused):
    """The sampling kernel inside the step (history on the device, appended by the kernel): with top_k = 1 only the
    arg-max survives the filter, so the sampled tokens must equal greedy decoding whatever the random numbers."""
    g, net = _load(golden_dir, "k3")
    V = net.config.vocab_size
    gen = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, V, (int(n),), generator=gen).tolist() for n in (9, 30, 4, 55, 18)]
    greedy = ContinuousBatcher(net, n_slots=3, fused=fused)
    want = [greedy.submit(p, 7) for p in prompts]
    want_out = greedy.run()
    eng = ContinuousBatcher(net, n_slots=3, cuda_graph=graph, fused=fused,
                            sampling=dict(temperature=0.7, top_k=1, top_p=0.9, repetition_penalty=1.0))
    rids = [eng.submit(p, 7) for p in prompts]
    out = eng.run()
    assert [out[r] for r in rids] == [want_out[r] for r in want]
    # the histories on the device hold prompt + generated tokens of the sequences that used each slot last
    lens = eng._hist_len.cpu().tolist()
    assert all(0 < n <= 55 + 7 for n in lens)


def test_sampling_engine_is_reproducible(golden_dir):
    g, net = _load(golden_dir, "k3")
    V = net.config.vocab_size
    prompts = [[5, 6, 7, 8] * 6, list(range(10, 40))]

    def run(seed):
        torch.manual_seed(seed)
        eng = ContinuousBatcher(net, n_slots=2, sampling=dict(temperature=1.0, top_k=0, top_p=0.95, repetition_penalty=1.3))
        rids = [eng.submit(p, 24) for p in prompts]
        out = eng.run()
        hist, lens = eng._hist.cpu(), eng._hist_len.cpu().tolist()
        for slot, n_ in enumerate(lens):          # each slot's device history = prompt + generated of its sequence
            assert any(hist[slot, :n_].tolist() == p + out[r] for p, r in zip(prompts, rids))
        return [out[r] for r in rids]

    a, b, c = run(1), run(1), run(2)
    assert a == b and a != c
    assert all(0 <= t < V for seq in a for t in seq)


def test_session_export_import_continues_exactly(golden_dir):
    """A live sequence taken out of one engine (state block of its slot + tokens) and put into another continues
    with the tokens it would have produced where it was."""
    g, net = _load(golden_dir, "k3")
    V = net.config.vocab_size
    gen = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, V, (int(n),), generator=gen).tolist() for n in (21, 8, 40)]
    ref_eng = ContinuousBatcher(net, n_slots=3)
    ref_ids = [ref_eng.submit(p, 12) for p in prompts]
    ref = ref_eng.run()
    a = ContinuousBatcher(net, n_slots=3)
    rids = [a.submit(p, 12) for p in prompts]
    for _ in range(5):
        a.step()
    blob = a.export_session(rids[1])
    assert blob["state"].device.type == "cpu" and len(blob["generated"]) == 5
    assert len(a.sched.free) == 1
    with pytest.raises(KeyError):
        a.export_session(rids[1])
    b = ContinuousBatcher(net, n_slots=2, cuda_graph=True)
    other = b.submit(prompts[2], 3)
    new_rid = b.import_session(blob)
    out_b = b.run()
    out_a = a.run()
    assert out_b[new_rid] == ref[ref_ids[1]]
    assert out_b[other] == ref[ref_ids[2]][:3]
    assert out_a[rids[0]] == ref[ref_ids[0]] and out_a[rids[2]] == ref[ref_ids[2]] and rids[1] not in out_a
