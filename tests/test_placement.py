"""Hit counters -> placement: the host-side planner (no GPU)."""
import numpy as np
import pytest

from mummu_b200 import placement as P


def test_smoothing_matches_the_reference_vectors():
    """crates/mummu/src/tier.rs:643-650 (`smoothing_normalizes_per_request`), exact equality."""
    h = []
    P.smooth_hotness(h, [3, 1], 1.0)
    assert h == [0.75, 0.25]
    P.smooth_hotness(h, [0, 4], 0.5)
    assert h == [0.375, 0.625]
    P.smooth_hotness(h, [0, 0], 0.5)            # an empty request changes nothing
    assert h == [0.375, 0.625]
    P.smooth_hotness(h, [1, 1, 2], 1.0)         # another length starts from zeros (tier.rs:418-420)
    assert h == [0.25, 0.25, 0.5]


def test_promotion_order_hottest_first_ties_by_id():
    """tier.rs:231-242."""
    assert P.promotion_order([0.1, 0.5, 0.5, 0.0], 4) == [1, 2, 0, 3]
    assert P.promotion_order([], 3) == [0, 1, 2]


def zipf(E, s=1.2):
    h = 1.0 / np.arange(1, E + 1) ** s
    return h / h.sum()


@pytest.mark.parametrize("E,world,slots", [(64, 8, 10), (128, 8, 20), (64, 2, 34), (8, 4, 2)])
def test_plan_is_a_valid_placement(E, world, slots):
    h = zipf(E)
    plan = P.plan_placement(h, E, world, slots)
    assert plan.slot_expert.shape == (world, slots)
    held = plan.slot_expert[plan.slot_expert >= 0]
    assert set(held.tolist()) == set(range(E))                       # every expert somewhere
    for r in range(world):                                           # at most one copy per rank
        row = plan.slot_expert[r][plan.slot_expert[r] >= 0]
        assert len(set(row.tolist())) == len(row)
    for e in range(E):
        assert plan.hosts[e] == sorted(r for r in range(world) if e in plan.slot_expert[r])
    for s in range(world):
        table = plan.route_table(s)
        assert table.dtype == np.int32 and table.shape == (E,)
        for e in range(E):
            r, slot = divmod(int(table[e]), slots)
            assert plan.slot_expert[r, slot] == e
            if s in plan.hosts[e]:
                assert r == s                                        # a rank's own copy serves its tokens
    # every copy of an expert serves somebody
    for e in range(E):
        served = {plan.serving_rank(e, s) for s in range(world)}
        assert served == set(plan.hosts[e])


def test_plan_flattens_a_zipf_skew():
    E, world = 64, 8
    h = zipf(E)
    plain = P.contiguous_placement(E, world).rank_loads(h)
    placed = P.plan_placement(h, E, world, E // world + 2).rank_loads(h)
    assert abs(plain.sum() - 1) < 1e-12 and abs(placed.sum() - 1) < 1e-12
    assert plain.max() > 3.0 / world                                 # rank 0 carries the head of the curve
    assert placed.max() < 1.15 / world                               # within 15 % of the fair share
    moved_only = P.plan_placement(h, E, world, E // world).rank_loads(h)   # no spare slot: placement alone
    assert moved_only.max() < plain.max()


def test_uniform_hotness_needs_no_copies():
    plan = P.plan_placement([], 16, 4, 6)
    assert all(len(hs) == 1 for hs in plan.hosts)
    assert (plan.slot_expert >= 0).sum() == 16


def test_refusals_name_the_shortfall():
    with pytest.raises(ValueError, match="no ranks"):
        P.plan_placement([], 8, 0, 8)
    with pytest.raises(ValueError, match="3 hotness values for 8 experts"):
        P.plan_placement([1, 2, 3], 8, 2, 4)
    with pytest.raises(ValueError, match="2 short"):
        P.plan_placement([], 8, 2, 3)
    with pytest.raises(ValueError, match="non-negative"):
        P.plan_placement([1, -1], 2, 2, 1)


def test_fold_hits_sums_the_copies():
    plan = P.plan_placement([10, 1, 1, 1], 4, 2, 3)
    assert len(plan.hosts[0]) == 2
    slot_hits = np.zeros(6, dtype=np.uint64)
    for r in plan.hosts[0]:
        slot_hits[r * 3 + plan.slot_of(0, r)] = 5
    assert plan.fold_hits(slot_hits).tolist() == [10, 0, 0, 0]


def test_random_plans_are_valid_and_conserve_load():
    """Random shapes and hotness (zeros, spikes, ties included): every plan is a valid placement,
    the loads it predicts add up to the total, and the folded slot hits of a simulated routing
    give the experts' own counts back."""
    hyp = pytest.importorskip("hypothesis")
    st = hyp.strategies

    @hyp.settings(max_examples=120, deadline=None, derandomize=True)
    @hyp.given(st.data())
    def run(data):
        world = data.draw(st.integers(1, 8))
        E = data.draw(st.integers(1, 40))
        need = -(-E // world)
        slots = data.draw(st.integers(need, need + 4))
        kind = data.draw(st.sampled_from(["floats", "spike", "ties", "zeros", "empty"]))
        if kind == "floats":
            h = data.draw(st.lists(st.floats(0.0, 1e6, allow_nan=False), min_size=E, max_size=E))
        elif kind == "spike":
            h = [1.0] * E
            h[data.draw(st.integers(0, E - 1))] = 1e4
        elif kind == "ties":
            h = [float(data.draw(st.integers(0, 2))) for _ in range(E)]
        elif kind == "zeros":
            h = [0.0] * E
        else:
            h = []
        plan = P.plan_placement(h, E, world, slots)
        assert plan.slot_expert.shape == (world, slots)
        for r in range(world):
            row = plan.slot_expert[r][plan.slot_expert[r] >= 0]
            assert len(set(row.tolist())) == len(row)
        for e in range(E):
            assert plan.hosts[e] and plan.hosts[e] == sorted(r for r in range(world) if e in plan.slot_expert[r])
        tables = [plan.route_table(s) for s in range(world)]
        for s in range(world):
            for e in range(E):
                r, slot = divmod(int(tables[s][e]), slots)
                assert plan.slot_expert[r, slot] == e
        hh = np.asarray(h if len(h) else [1.0] * E, dtype=np.float64)
        assert np.isclose(plan.rank_loads(hh).sum(), hh.sum(), rtol=1e-9, atol=1e-12)
        # a routing drawn per source rank, counted per slot, folds back to the experts' counts
        seed = data.draw(st.integers(0, 2**31 - 1))
        rng = np.random.default_rng(seed)
        slot_hits = np.zeros(plan.virtual_experts, dtype=np.int64)
        per_expert = np.zeros(E, dtype=np.int64)
        for s in range(world):
            ids = rng.integers(0, E, size=50)
            np.add.at(per_expert, ids, 1)
            np.add.at(slot_hits, tables[s][ids], 1)
        assert np.array_equal(plan.fold_hits(slot_hits).astype(np.int64), per_expert)

    run()
