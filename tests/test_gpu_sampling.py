"""Device-side token sampling (qpam_sample_logits) against the CPU restatement of the reference's sampling block
(v11/model.py:1221-1244): the filtered distribution (kept count, kept mass) and the inverse-CDF draw."""
import numpy as np
import pytest
import torch

from oracle import sampling_oracle as so
from qllm2_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check_rows(logits, hist, hist_len, u, ids, stats, cfg, count_exact=True):
    """Kept count: exact where only integer logic decides it (top-k, no filter).  Where the nucleus closes, the
    float32 mass sums of the kernel and the float64 sums here may put the boundary a few negligible tokens apart
    (the tail tokens there weigh ~1e-6 of the total, the rounding noise of any float32 cumulative sum, the
    reference's included): then the kept MASS must agree to 5e-5 of the total."""
    lg = logits.float().cpu().numpy()
    nucleus = 0 < cfg["top_p"] < 1
    for r in range(lg.shape[0]):
        h = None if hist is None else hist[r, :(hist.shape[1] if hist_len is None else int(hist_len[r]))].tolist()
        p = so.filtered_probs(lg[r], h, **cfg)
        kept = int((p > 0).sum())
        if count_exact and not nucleus:
            assert int(stats[r, 2]) == kept, (r, int(stats[r, 2]), kept)
        else:
            full = so.filtered_probs(lg[r], h, **{**cfg, "top_p": 0.0})       # distribution before the nucleus filter
            assert abs(float(stats[r, 1]) / float(stats[r, 3]) - full[p > 0].sum()) < 5e-5, (r, stats[r], kept)
            assert abs(int(stats[r, 2]) - kept) <= max(3, 0.02 * kept), (r, int(stats[r, 2]), kept)
        c = np.cumsum(p)
        i = int(ids[r])
        if int(stats[r, 2]) == kept:
            assert p[i] > 0, (r, i)
        lo, hi = (c[i - 1] if i > 0 else 0.0), c[i]
        assert lo - 5e-5 <= float(u[r]) <= hi + 5e-5, (r, i, lo, float(u[r]), hi)


@pytest.mark.parametrize("cfg", [
    dict(temperature=0.8, top_k=50, top_p=0.9, repetition_penalty=1.1),
    dict(temperature=1.0, top_k=0, top_p=0.95, repetition_penalty=1.0),
    dict(temperature=1.3, top_k=20, top_p=0.0, repetition_penalty=1.2),
    dict(temperature=1.0, top_k=0, top_p=0.0, repetition_penalty=1.0),
    dict(temperature=0.7, top_k=1, top_p=0.5, repetition_penalty=1.0),
])
@pytest.mark.parametrize("V", [50261, 97, 70001])
def test_rows_match_reference_filter_and_inverse_cdf(cfg, V):
    n = 24
    g = torch.Generator().manual_seed(V + int(cfg["top_k"]))
    logits = (torch.randn(n, V, generator=g) * 3.0).to(DEV)
    hist = torch.randint(0, V, (n, 40), generator=g)
    u = torch.rand(n, generator=g)
    ids, stats = ops.sample_logits(logits, u.to(DEV), history=hist.to(DEV), return_stats=True, **cfg)
    _check_rows(logits, hist.numpy(), None, u.numpy(), ids.cpu().numpy(), stats.cpu().numpy(), cfg)


def test_bf16_logits_with_ties():
    """bf16 logits repeat values many times over 50k entries: the whole tie group at either threshold stays."""
    n, V = 16, 50261
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(n, V, generator=g) * 2.0).bfloat16().to(DEV)
    u = torch.rand(n, generator=g)
    cfg = dict(temperature=0.9, top_k=40, top_p=0.9, repetition_penalty=1.0)
    ids, stats = ops.sample_logits(logits, u.to(DEV), return_stats=True, **cfg)
    _check_rows(logits, None, None, u.numpy(), ids.cpu().numpy(), stats.cpu().numpy(), cfg, count_exact=False)


def test_frequencies_follow_the_filtered_distribution():
    """One row, 8192 evenly spaced uniforms: every token is drawn as often as its probability says (to 2 / n)."""
    V, n = 1000, 8192
    g = torch.Generator().manual_seed(9)
    row = torch.randn(V, generator=g) * 2.5
    cfg = dict(temperature=1.1, top_k=64, top_p=0.92, repetition_penalty=1.0)
    u = (torch.arange(n, dtype=torch.float32) + 0.5) / n
    ids = ops.sample_logits(row[None].expand(n, V).contiguous().to(DEV), u.to(DEV), **cfg).cpu().numpy()
    p = so.filtered_probs(row.numpy(), None, **cfg)
    freq = np.bincount(ids, minlength=V) / n
    assert np.abs(freq - p).max() <= 2.0 / n + 2e-5, float(np.abs(freq - p).max())
    assert set(np.nonzero(freq)[0]) <= set(np.nonzero(p)[0])


def test_slots_lengths_and_append():
    """Rows map to history rows through slot ids; only hist_len[slot] entries count for the penalty; the drawn id is
    appended behind them; a slot of -1 is a padded row (id 0, nothing appended)."""
    V, rows, cap = 311, 6, 12
    g = torch.Generator().manual_seed(21)
    logits = torch.randn(4, V, generator=g) * 4.0
    hist = torch.randint(0, V, (rows, cap), generator=g)
    hist_len = torch.tensor([3, 0, 12, 5, 7, 1], dtype=torch.int32)
    slots = torch.tensor([4, -1, 0, 2], dtype=torch.int32)
    u = torch.rand(4, generator=g)
    cfg = dict(temperature=1.0, top_k=0, top_p=0.0, repetition_penalty=1.5)
    hd, ld = hist.to(DEV), hist_len.to(DEV)
    ids = ops.sample_logits(logits.to(DEV), u.to(DEV), history=hd, hist_len=ld, slot_ids=slots.to(DEV), append=True, **cfg)
    ids = ids.cpu().numpy()
    assert ids[1] == 0
    new_len, new_hist = ld.cpu().numpy(), hd.cpu().numpy()
    for r, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        ln = int(hist_len[s])
        p = so.filtered_probs(logits[r].numpy(), hist[s, :ln].tolist(), **cfg)
        c = np.cumsum(p)
        lo, hi = (c[ids[r] - 1] if ids[r] > 0 else 0.0), c[ids[r]]
        assert lo - 2e-5 <= float(u[r]) <= hi + 2e-5
        if ln < cap:
            assert new_len[s] == ln + 1 and new_hist[s, ln] == ids[r]
        else:       # a full row keeps its length and its entries
            assert new_len[s] == ln and (new_hist[s] == hist[s].numpy()).all()
    untouched = [s for s in range(rows) if s not in slots.tolist()]
    assert (new_len[untouched] == hist_len.numpy()[untouched]).all()


def test_bad_arguments_are_refused():
    from qllm2_b200._lib import QPamError
    logits = torch.zeros(2, 10, device=DEV)
    with pytest.raises(QPamError):
        ops.sample_logits(logits, temperature=0.0)
    with pytest.raises(QPamError):
        ops.sample_logits(logits, torch.zeros(3, device=DEV))
    with pytest.raises(QPamError):
        ops.sample_logits(logits, append=True)
