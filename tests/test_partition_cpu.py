"""Invariants of the unit-range plan (host restatement of the in-kernel integer logic)."""
import random

import partition_plan as P


def _check(ctx, qls, group, n_hg, tok_stage, ctas, weighted):
    per, units, owners, segs = P.plan(ctx, qls, group=group, n_head_groups=n_hg, tok_stage=tok_stage,
                                      num_ctas=ctas, weighted=weighted)
    n_units = sum(-(-c // tok_stage) * n_hg for c, q in zip(ctx, qls) if c > 0 and q > 0)
    assert len(units) == n_units                                   # every unit exactly once
    assert all(0 <= c < ctas for c in owners)                      # ... on an existing CTA
    assert owners == sorted(owners)                                # ranges are contiguous and ordered
    cost = {}
    for u, c in zip(units, owners):
        cost[c] = cost.get(c, 0) + u.weight
    if cost:
        assert max(cost.values()) <= per + 1                       # no CTA carries more than its share
    for (s, hg), (first, n) in segs.items():                       # the merge reads CTAs first .. first+n-1:
        mine = {c for u, c in zip(units, owners) if (u.seq, u.head_group) == (s, hg)}
        assert mine == set(range(first, first + n)), (s, hg, first, n, sorted(mine))


def test_llama_shaped_batch():
    rng = random.Random(0)
    ctx = [rng.randint(1024, 8192) for _ in range(64)]
    _check(ctx, [1] * 64, 4, 1, 32, 148, False)


def test_mixed_rows_weighted():
    rng = random.Random(1)
    for trial in range(200):
        n = rng.randint(1, 40)
        ctx = [rng.choice([0, 1, 15, 16, 17, 31, 32, 33, 100, 700, 5000]) for _ in range(n)]
        qls = [rng.choice([0, 1, 1, 1, 4]) for _ in range(n)]
        _check(ctx, qls, 4, rng.choice([1, 2, 4]), 32, rng.choice([1, 2, 3, 7, 33, 148]), True)


def test_unweighted_random():
    rng = random.Random(2)
    for trial in range(200):
        n = rng.randint(1, 30)
        ctx = [rng.choice([0, 1, 16, 17, 128, 129, 1000, 9000]) for _ in range(n)]
        _check(ctx, [1] * n, rng.choice([1, 4, 8]), rng.choice([1, 4, 8]), rng.choice([16, 32, 64, 128]),
               rng.choice([1, 5, 148]), False)
