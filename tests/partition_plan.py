"""Host-side restatement of the unit-range plan the decode kernel computes on the device.

The kernel cuts all (sequence, head group, tile) units of a launch into contiguous ranges of equal
*cost*, one per CTA, with integer arithmetic only (``paged_decode_kernel.cuh``, "plan").  This module
states the same rules in Python so that their invariants can be checked on the CPU and the table the
kernel writes can be compared with them entry by entry on the GPU.  Test infrastructure only.

Rules (all positions in cost units):

* a unit (one stage: ``tok_stage`` tokens of ``HG`` KV heads) costs ``w``: 2 where a query of 9..16
  rows runs on the 8-bit 16-row kernels, else 1;
* every (sequence, head group) is preceded by a gap of ``SEG_GAP`` cost units (what finishing one
  segment and starting the next was measured to cost);
* CTA ``c`` of ``G`` owns the units whose start position lies in ``[c * per, (c + 1) * per)`` with
  ``per = max(ceil(total / G), w_max)``;
* the CTAs that leave partial rows for a segment are ``first .. last`` = the owners of its first
  and last unit; every CTA in between owns at least one of its units.
"""
from __future__ import annotations

import dataclasses
from typing import List, Sequence, Tuple

SEG_GAP = 2


@dataclasses.dataclass(frozen=True)
class Unit:
    seq: int
    head_group: int
    tile: int
    pos: int      # cost position of the unit's start
    weight: int


def unit_weight(group: int, q_len: int, sixteen_row_8bit_kernel: bool) -> int:
    return 2 if (sixteen_row_8bit_kernel and group * q_len > 8) else 1


def enumerate_units(context_lens: Sequence[int], q_lens: Sequence[int], *, group: int, n_head_groups: int,
                    tok_stage: int, weighted: bool) -> Tuple[List[Unit], int]:
    """All units in launch order with their cost positions, and the total cost."""
    units: List[Unit] = []
    pos = 0
    for s, (ctx, ql) in enumerate(zip(context_lens, q_lens)):
        if ctx <= 0 or ql <= 0:
            continue
        tiles = -(-ctx // tok_stage)
        w = unit_weight(group, ql, weighted)
        for hg in range(n_head_groups):
            pos += SEG_GAP
            for t in range(tiles):
                units.append(Unit(s, hg, t, pos, w))
                pos += w
    return units, pos


def plan(context_lens: Sequence[int], q_lens: Sequence[int], *, group: int, n_head_groups: int, tok_stage: int,
         num_ctas: int, weighted: bool = False):
    """Returns (per_cta, owner_of_unit list, {(seq, head_group): (first_cta, n_ctas)})."""
    units, total = enumerate_units(context_lens, q_lens, group=group, n_head_groups=n_head_groups,
                                   tok_stage=tok_stage, weighted=weighted)
    per = max(-(-total // num_ctas) if total else 0, 2 if weighted else 1)
    owners = [u.pos // per for u in units]
    segments = {}
    for u, c in zip(units, owners):
        key = (u.seq, u.head_group)
        first, last = segments.get(key, (c, c))
        segments[key] = (min(first, c), max(last, c))
    return per, units, owners, {k: (f, l - f + 1) for k, (f, l) in segments.items()}
