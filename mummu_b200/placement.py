"""Hit counters -> hot-expert placement for the expert-parallel layer.

The reference closes this loop for its tiered pool: `ExpertPool::take_hits`
(crates/mummu/src/nn/moe.rs:1527-1535) drains per-expert routing hits, `smooth_hotness`
(crates/mummu/src/tier.rs:417-431) folds them into a moving average, and `plan_tiers`
(tier.rs:353-411) promotes experts hottest first (`promotion_order`, tier.rs:231-242) onto its
devices under their byte budgets.  Its devices differ in speed and precision; the ranks of an
NVLink box are equal, so the plan here answers the question that remains: WHICH RANK holds which
expert, and which experts are held TWICE OR MORE, so that no rank is the critical path of a layer
whose routing is skewed.

A rank offers `slots` bank slots (>= experts / world; the surplus is room for replicas).  The plan
  1. gives every expert one copy and hands the spare slots, one at a time, to the expert whose
     load per copy is largest, while that load is above a stated share of a rank's fair load;
  2. places the copies, heaviest first, on the least loaded rank that still has a slot and does not
     hold that expert yet (longest-processing-time-first);
  3. gives each source rank a table expert -> slot: its own copy where it has one, otherwise the
     copies are dealt out over the remaining source ranks in turn.
Everything is plain Python over float64 so that it runs, and is tested, without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np


def smooth_hotness(prev: List[float], hits: Sequence[int], alpha: float) -> List[float]:
    """tier.rs:417-431: exponential moving average of per-expert hits, normalised per request.
    `prev` of another length starts from zeros; a request without hits changes nothing.  The two
    products are rounded separately before the sum (the reference's test pins the averages
    exactly, tier.rs:643-650).  Returns the updated list (also written back into `prev`)."""
    if len(prev) != len(hits):
        prev[:] = [0.0] * len(hits)
    total = int(sum(int(h) for h in hits))
    if total == 0:
        return prev
    inv = 1.0 / float(total)
    for i, h in enumerate(hits):
        kept = (1.0 - alpha) * prev[i]
        fresh = alpha * (float(int(h)) * inv)
        prev[i] = kept + fresh
    return prev


def promotion_order(hotness: Sequence[float], experts: int) -> List[int]:
    """tier.rs:231-242: hottest first, ties (and an empty hotness) in expert order."""
    order = list(range(experts))
    if len(hotness):
        order.sort(key=lambda e: (-float(hotness[e]), e))
    return order


@dataclass
class Placement:
    world: int
    slots: int                      # bank slots per rank
    experts: int                    # real experts
    slot_expert: np.ndarray         # [world, slots] expert held by a slot, -1 = empty
    hosts: List[List[int]]          # per expert: the ranks that hold a copy, ascending

    @property
    def virtual_experts(self) -> int:
        return self.world * self.slots

    def slot_of(self, expert: int, rank: int) -> int:
        (where,) = np.nonzero(self.slot_expert[rank] == expert)
        return int(where[0])

    def serving_rank(self, expert: int, source: int) -> int:
        """The copy that serves `source`'s tokens: its own where it holds one; the other source
        ranks take the copies in turn."""
        hs = self.hosts[expert]
        if source in hs:
            return source
        others = [s for s in range(self.world) if s not in hs]
        return hs[others.index(source) % len(hs)]

    def route_table(self, source: int) -> np.ndarray:
        """int32 [experts]: the slot id (rank * slots + slot) that serves `source`'s tokens."""
        out = np.empty(self.experts, dtype=np.int32)
        for e in range(self.experts):
            r = self.serving_rank(e, source)
            out[e] = r * self.slots + self.slot_of(e, r)
        return out

    def rank_experts(self, rank: int) -> np.ndarray:
        """int64 [slots]: which expert's weights go into each slot of `rank` (an empty slot gets
        expert 0's: it is never routed to, it only has to be readable)."""
        e = self.slot_expert[rank].astype(np.int64)
        return np.where(e < 0, 0, e)

    def rank_loads(self, hotness: Sequence[float]) -> np.ndarray:
        """Load per rank when tokens are spread evenly over the source ranks."""
        loads = np.zeros(self.world, dtype=np.float64)
        for e in range(self.experts):
            for s in range(self.world):
                loads[self.serving_rank(e, s)] += float(hotness[e]) / self.world
        return loads

    def fold_hits(self, slot_hits: Sequence[int]) -> np.ndarray:
        """Per-slot counters of a bank handle -> per-expert hits."""
        out = np.zeros(self.experts, dtype=np.uint64)
        flat = self.slot_expert.reshape(-1)
        for v, h in enumerate(slot_hits):
            if flat[v] >= 0:
                out[flat[v]] += np.uint64(h)
        return out


def contiguous_placement(experts: int, world: int) -> Placement:
    """The plain sharding: rank r holds experts [r * E / world, (r + 1) * E / world)."""
    if experts % world:
        raise ValueError(f"placement: {experts} experts do not divide over {world} ranks")
    el = experts // world
    slot_expert = np.arange(experts, dtype=np.int64).reshape(world, el)
    return Placement(world, el, experts, slot_expert, [[e // el] for e in range(experts)])


def plan_placement(hotness: Sequence[float], experts: int, world: int, slots: int,
                   min_copy_share: float = 0.5) -> Placement:
    """Hotness (any non-negative scale; empty = uniform, as in tier.rs:340) -> placement.

    A spare slot goes to the expert with the largest load per copy, as long as that load exceeds
    `min_copy_share` of a rank's fair load (total / world): lighter copies no longer move the
    maximum, they only split an expert's rows into smaller groups.  Errors, never silent drops
    (tier.rs:342-346): no ranks, hotness of the wrong length or negative, too few slots."""
    if world < 1:
        raise ValueError("placement: no ranks")
    if len(hotness) not in (0, experts):
        raise ValueError(f"placement: {len(hotness)} hotness values for {experts} experts")
    if world * slots < experts:
        raise ValueError(f"placement: {world} ranks x {slots} slots cannot hold {experts} experts "
                         f"({experts - world * slots} short)")
    h = np.asarray(hotness if len(hotness) else [1.0] * experts, dtype=np.float64)
    if not np.all(np.isfinite(h)) or np.any(h < 0):
        raise ValueError("placement: hotness must be finite and non-negative")
    total = float(h.sum())
    if total == 0.0:
        h, total = np.ones(experts), float(experts)
    fair = total / world
    order = promotion_order(h, experts)
    copies = np.ones(experts, dtype=np.int64)
    spare = world * slots - experts
    while spare > 0:
        best = max(order, key=lambda e: (h[e] / copies[e] if copies[e] < world else -1.0, -e))
        if copies[best] >= world or h[best] / copies[best] <= min_copy_share * fair:
            break
        copies[best] += 1
        spare -= 1
    while True:
        units = sorted(((h[e] / copies[e], e, c) for e in range(experts) for c in range(copies[e])),
                       key=lambda u: (-u[0], u[1], u[2]))
        slot_expert = -np.ones((world, slots), dtype=np.int64)
        used = np.zeros(world, dtype=np.int64)
        load = np.zeros(world, dtype=np.float64)
        hosts: List[List[int]] = [[] for _ in range(experts)]
        failed = -1
        for share, e, _ in units:
            ranks = [r for r in range(world) if used[r] < slots and r not in hosts[e]]
            if not ranks:
                failed = e
                break
            r = min(ranks, key=lambda q: (load[q], q))
            slot_expert[r, used[r]] = e
            used[r] += 1
            load[r] += share
            hosts[e].append(r)
        if failed < 0:
            break
        copies[failed] -= 1             # a copy that fits on no new rank is given up; plan again
    for e in range(experts):
        hosts[e].sort()
    return Placement(world, slots, experts, slot_expert, hosts)
