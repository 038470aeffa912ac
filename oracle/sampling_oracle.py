"""CPU restatement (numpy, float64) of the token-sampling block of the reference's V11LM.generate
(v11/model.py:1221-1244).  TEST INFRASTRUCTURE: only tests/ and the smoke check may import this.

    x = logits / temperature
    x[h] = x[h] / penalty if x[h] > 0 else x[h] * penalty      for every token h already in the sequence
    top-k: x[x < k-th largest] = -inf
    top-p: sort descending, p = softmax(sorted), drop where cumsum(p) - p >= top_p
    draw from softmax(x)

The reference draws with torch.multinomial; here the draw is the inverse CDF, in vocabulary order, of a uniform
number given by the caller (same distribution).  Where several tokens tie with the value at which the nucleus
closes, a sort keeps an arbitrary subset of them; this restatement keeps the whole tie group.
"""
from __future__ import annotations

import numpy as np


def filtered_probs(logits, history=None, *, temperature=1.0, top_k=0, top_p=0.0, repetition_penalty=1.0):
    """Probabilities [V] (float64, zero where a token was filtered out) of one row of logits."""
    x = np.asarray(logits, dtype=np.float64) / temperature
    V = x.shape[0]
    if repetition_penalty != 1.0 and history is not None:
        for h in set(int(t) for t in history):
            if 0 <= h < V:
                x[h] = x[h] / repetition_penalty if x[h] > 0 else x[h] * repetition_penalty
    if 0 < top_k < V:
        kth = np.sort(x)[::-1][top_k - 1]
        x = np.where(x < kth, -np.inf, x)
    if 0 < top_p < 1:
        order = np.argsort(-x, kind="stable")
        xs = x[order]
        ps = np.exp(xs - xs[0])
        ps /= ps.sum()
        before = np.cumsum(ps) - ps
        keep_sorted = before < top_p
        threshold = xs[keep_sorted][-1]            # lowest kept value; its whole tie group stays
        x = np.where(x < threshold, -np.inf, x)
    p = np.exp(x - x.max())
    return p / p.sum()


def draw(probs, u):
    """Inverse CDF in vocabulary order: the first token whose cumulative probability exceeds u * total."""
    c = np.cumsum(probs)
    idx = int(np.searchsorted(c, u * c[-1], side="right"))
    kept = np.nonzero(probs > 0)[0]
    return int(min(idx, kept[-1]))
