"""The sampler's candidate path for the top-k pivot (ops/csrc/sampling.cu), restated with numpy:
the k-th largest of the 256 group maxima is a lower bound of the k-th largest value, so the
entries at or above it contain the whole top-k set and the pivot can be picked among them."""
import numpy as np
import pytest

THREADS, GROUPS = 1024, 256


def _pivot_by_candidates(row: np.ndarray, k: int):
    v = len(row)
    # per-thread maxima over a strided walk, then per-group maxima (threads t, t + 256, ...)
    tmax = np.full(THREADS, -np.inf)
    for t in range(THREADS):
        part = row[t::THREADS]
        if len(part):
            tmax[t] = part.max()
    gmax = tmax.reshape(THREADS // GROUPS, GROUPS).max(axis=0)
    # rank by (value desc, group index asc): the group of rank k - 1 gives the bound
    order = sorted(range(GROUPS), key=lambda j: (-gmax[j], j))
    bound = gmax[order[k - 1]]
    cand = row[row >= bound]
    # the candidate with fewer than k values above it and at least k at or above it
    pivots = {c for c in cand if (cand > c).sum() < k <= (cand >= c).sum()}
    assert len(pivots) == 1
    return pivots.pop(), len(cand), v


@pytest.mark.parametrize("seed", range(12))
@pytest.mark.parametrize("k", [1, 5, 50, 256])
def test_candidate_pivot_is_the_kth_largest(seed, k):
    rng = np.random.default_rng(seed)
    v = int(rng.choice([1500, 32016, 40000]))
    row = rng.standard_normal(v).astype(np.float32) * 2
    if seed % 3 == 0:                       # ties, also at the pivot
        row[rng.integers(0, v, 200)] = 3.25
        row[rng.integers(0, v, 40)] = 9.0
    pivot, n_cand, _ = _pivot_by_candidates(row, k)
    assert pivot == np.sort(row)[-k]
    assert n_cand >= k
    if seed % 3:
        assert n_cand <= 2048               # the list the kernel keeps is long enough
