"""The work split of the decode attention kernel (ops/csrc/attn_decode.cu), restated in Python and
checked on the CPU: every 32-key chunk of every (sequence, kv head) pair is taken by exactly one
CTA, a pair is never shared by more CTAs than the partial-result buffer has slots for, and the
slot a CTA writes is the slot the merging CTA reads."""
import random

import pytest

K_CHUNK = 32


def _chunks(pos, smax, left_pad):
    pos = min(max(pos, 0), smax - 1)
    out = []
    for lp in left_pad:
        start = min(max(lp, 0), pos)
        out.append((pos - start + K_CHUNK) // K_CHUNK)
    return out


def _runs(nc, n_kv, grid, max_parts, fixed_parts):
    """[(lo, hi)] per CTA in the numbering (sequence, head, chunk), as the kernel computes it."""
    pre = [0]
    for c in nc:
        pre.append(pre[-1] + c)
    total = pre[-1] * n_kv
    runs, per_of = [], []
    for cta in range(grid):
        if fixed_parts > 0:
            item, part = divmod(cta, fixed_parts)
            b, hk = divmod(item, n_kv)
            per = -(-nc[b] // fixed_parts)
            lo = pre[b] * n_kv + hk * nc[b] + part * per
            hi = min(pre[b] * n_kv + (hk + 1) * nc[b], lo + per)
        else:
            per = -(-total // grid)
            per = max(per, -(-max(nc) // (max_parts - 1)))
            lo = min(total, cta * per)
            hi = min(total, lo + per)
        runs.append((lo, hi))
        per_of.append(per)
    return pre, total, runs, per_of


def _grid(B, n_kv, resident, max_parts):
    if max_parts <= 1:
        return B * n_kv, 1
    if B * n_kv <= resident:
        fixed = min(max_parts, resident // (B * n_kv))
        return B * n_kv * fixed, fixed
    return resident, 0


@pytest.mark.parametrize("seed", range(40))
def test_every_chunk_once_and_parts_fit(seed):
    rnd = random.Random(seed)
    B = rnd.choice([1, 2, 3, 7, 64, 200, 512])
    n_kv = rnd.choice([1, 2, 4, 8, 32])
    smax = rnd.choice([64, 300, 768, 4096])
    pos = rnd.randrange(0, smax)
    left_pad = [rnd.randrange(0, max(1, pos // rnd.choice([1, 2, 5]) + 1)) for _ in range(B)]
    max_parts = rnd.choice([1, 2, 3, 8])
    resident = rnd.choice([148 * 3, 148 * 4, 20, 1])
    nc = _chunks(pos, smax, left_pad)
    grid, fixed = _grid(B, n_kv, resident, max_parts)
    pre, total, runs, per_of = _runs(nc, n_kv, grid, max(max_parts, 2), fixed)

    covered = [0] * total
    parts_of = {}                     # (b, hk) -> list of (cta, part index as the kernel computes)
    for cta, (lo, hi) in enumerate(runs):
        P = lo
        while P < hi:
            b = max(i for i in range(B) if pre[i] * n_kv <= P)
            rem = P - pre[b] * n_kv
            hk, ch = divmod(rem, nc[b])
            n_here = min(nc[b] - ch, hi - P)
            for c in range(P, P + n_here):
                covered[c] += 1
            whole = ch == 0 and n_here == nc[b]
            if not whole:
                per = per_of[cta]
                if fixed > 0:
                    part, parts = cta % fixed, -(-nc[b] // per)
                else:
                    item_lo = pre[b] * n_kv + hk * nc[b]
                    first, last = item_lo // per, (item_lo + nc[b] - 1) // per
                    part, parts = cta - first, last - first + 1
                parts_of.setdefault((b, hk), []).append((part, parts))
            P += n_here
    assert all(c == 1 for c in covered)
    for key, lst in parts_of.items():
        parts = lst[0][1]
        assert all(p[1] == parts for p in lst), key          # every CTA expects the same count
        assert sorted(p[0] for p in lst) == list(range(parts)), key   # slots 0..parts-1, once each
        assert 2 <= parts <= max(max_parts, 2), key
    if max_parts <= 1:
        assert not parts_of
