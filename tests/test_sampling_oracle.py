"""The sampling oracle against the torch operators of the reference's sampling block (v11/model.py:1221-1244,
restated line by line below) on tie-free float64 logits: same surviving tokens, same probabilities."""
import numpy as np
import pytest
import torch

from oracle import sampling_oracle as so


def _reference_block(nl, out, temperature, top_k, top_p, repetition_penalty):
    nl = nl / temperature
    if repetition_penalty != 1.0:
        sc = torch.gather(nl, 1, out)
        nl.scatter_(1, out, torch.where(sc > 0, sc / repetition_penalty, sc * repetition_penalty))
    if top_k > 0:
        kth = nl.topk(min(top_k, nl.size(-1))).values[:, -1:]
        nl[nl < kth] = float("-inf")
    if top_p > 0:
        sl, si = nl.sort(descending=True)
        pr = sl.softmax(dim=-1)
        sl[(pr.cumsum(dim=-1) - pr) >= top_p] = float("-inf")
        nl = sl.scatter(1, si, sl)
    return nl.softmax(dim=-1)


@pytest.mark.parametrize("cfg", [
    dict(temperature=0.8, top_k=50, top_p=0.9, repetition_penalty=1.1),
    dict(temperature=1.0, top_k=0, top_p=0.95, repetition_penalty=1.0),
    dict(temperature=1.3, top_k=20, top_p=0.0, repetition_penalty=1.2),
    dict(temperature=0.5, top_k=0, top_p=0.0, repetition_penalty=2.0),
])
def test_filtered_distribution_equals_the_reference_block(cfg):
    g = torch.Generator().manual_seed(0)
    nl = torch.randn(5, 700, generator=g, dtype=torch.float64) * 3
    out = torch.randint(0, 700, (5, 30), generator=g)
    ref = _reference_block(nl.clone(), out, **cfg).numpy()
    for r in range(5):
        p = so.filtered_probs(nl[r].numpy(), out[r].tolist(), **cfg)
        assert ((p > 0) == (ref[r] > 0)).all()
        assert np.abs(p - ref[r]).max() < 1e-14


def test_draw_is_the_inverse_cdf():
    p = np.array([0.0, 0.25, 0.0, 0.5, 0.25, 0.0])
    assert [so.draw(p, u) for u in (0.0, 0.2499, 0.25, 0.7499, 0.75, 0.9999)] == [1, 1, 3, 3, 4, 4]
