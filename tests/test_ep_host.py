"""CPU tests of the expert-parallel exchange: plan arithmetic, and the whole dispatch / combine
round trip over two gloo ranks with a stand-in expert (no GPU, no CUDA library)."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_exchange_arithmetic():
    from mummu_b200.ep import plan_exchange
    rng = np.random.default_rng(0)
    R, E = 4, 16
    all_counts = rng.integers(0, 5, size=(R, E))
    all_counts[:, 3] = 0                                         # an expert nobody routes to
    for rank in range(R):
        p = plan_exchange(all_counts, rank, R)
        el = E // R
        assert p.send_splits == [int(all_counts[rank, d * el:(d + 1) * el].sum()) for d in range(R)]
        assert p.recv_splits == [int(all_counts[s, rank * el:(rank + 1) * el].sum()) for s in range(R)]
        assert np.array_equal(p.local_counts, all_counts[:, rank * el:(rank + 1) * el].sum(0))
        # the permutation is a bijection of the received rows and groups them by expert
        assert sorted(p.to_expert_major.tolist()) == list(range(sum(p.recv_splits)))
        label = np.concatenate([np.repeat(np.arange(el), all_counts[s, rank * el:(rank + 1) * el]) for s in range(R)]) \
            if sum(p.recv_splits) else np.zeros(0, int)
        grouped = label[p.to_expert_major]
        assert np.array_equal(grouped, np.sort(grouped, kind="stable"))


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from mummu_b200.ep import plan_exchange
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, K, T, H = 8, 2, 11 + rank, 4
        rng = np.random.default_rng(100 + rank)
        ids = np.stack([rng.choice(E, size=K, replace=False) for _ in range(T)]).astype(np.int64)
        w = rng.random((T, K)).astype(np.float32)
        x = rng.normal(size=(T, H)).astype(np.float32)
        flat = ids.reshape(-1)
        order = np.argsort(flat, kind="stable")                  # what mummu_moe_permute produces
        row_token = order // K
        pos = np.empty(T * K, np.int64)
        pos[order] = np.arange(T * K)
        counts = np.bincount(flat, minlength=E).astype(np.int32)
        allc = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(allc, torch.from_numpy(counts))
        plan = plan_exchange(torch.stack(allc).numpy(), rank, world)
        send = torch.from_numpy(x[row_token])
        recv = torch.empty(sum(plan.recv_splits), H)
        dist.all_to_all_single(recv, send, plan.recv_splits, plan.send_splits)
        xs = recv[torch.from_numpy(plan.to_expert_major)]
        # stand-in expert e: y = (global expert id + 1) * x
        el = E // world
        gid = np.repeat(np.arange(el) + rank * el, plan.local_counts)
        ys = xs * torch.from_numpy((gid + 1).astype(np.float32))[:, None]
        back = torch.empty_like(recv)
        back[torch.from_numpy(plan.to_expert_major)] = ys
        out_rows = torch.empty(T * K, H)
        dist.all_to_all_single(out_rows, back, plan.send_splits, plan.recv_splits)
        got = np.zeros((T, H), np.float32)
        for t in range(T):
            for s in np.argsort(ids[t]):                         # ascending expert id
                got[t] += w[t, s] * out_rows[pos[t * K + s]].numpy()
        want = np.zeros((T, H), np.float32)
        for t in range(T):
            for s in np.argsort(ids[t]):
                want[t] += w[t, s] * (np.float32(ids[t, s] + 1) * x[t])
        q.put((rank, bool(np.array_equal(got, want))))
    finally:
        dist.destroy_process_group()


def test_dispatch_combine_round_trip_two_gloo_ranks():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def _placed_worker(rank, world, port, q):
    """The placed exchange: expert ids go through this rank's expert -> slot table, rows travel to
    the rank that holds the slot, the stand-in expert there answers with the REAL expert of the
    slot, and the sum keeps the order of the real ids.  Slot hits folded over the ranks give the
    per-expert counts back."""
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from mummu_b200.ep import plan_exchange
    from mummu_b200.placement import plan_placement
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, K, T, H, slots = 8, 2, 13 + rank, 4, 6
        hot = [40.0, 1, 1, 1, 20.0, 1, 1, 1]
        pl = plan_placement(hot, E, world, slots)
        assert len(pl.hosts[0]) == 2                             # the hottest expert is held twice
        V = pl.virtual_experts
        table = pl.route_table(rank)
        rng = np.random.default_rng(300 + rank)
        p_e = np.asarray(hot) / sum(hot)
        ids = np.stack([rng.choice(E, size=K, replace=False, p=p_e) for _ in range(T)]).astype(np.int64)
        w = rng.random((T, K)).astype(np.float32)
        x = rng.normal(size=(T, H)).astype(np.float32)
        vids = table[ids]                                        # what mummu_ep_place writes
        assert np.all(vids // slots == np.vectorize(lambda e: pl.serving_rank(int(e), rank))(ids))
        flat = vids.reshape(-1)
        order = np.argsort(flat, kind="stable")
        row_token = order // K
        pos = np.empty(T * K, np.int64)
        pos[order] = np.arange(T * K)
        counts = np.bincount(flat, minlength=V).astype(np.int32)
        allc = [torch.zeros(V, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(allc, torch.from_numpy(counts))
        plan = plan_exchange(torch.stack(allc).numpy(), rank, world)
        send = torch.from_numpy(x[row_token])
        recv = torch.empty(sum(plan.recv_splits), H)
        dist.all_to_all_single(recv, send, plan.recv_splits, plan.send_splits)
        xs = recv[torch.from_numpy(plan.to_expert_major)]
        real = pl.rank_experts(rank)                             # the weights each slot was loaded with
        gid = np.repeat(real, plan.local_counts)
        ys = xs * torch.from_numpy((gid + 1).astype(np.float32))[:, None]
        back = torch.empty_like(recv)
        back[torch.from_numpy(plan.to_expert_major)] = ys
        out_rows = torch.empty(T * K, H)
        dist.all_to_all_single(out_rows, back, plan.send_splits, plan.recv_splits)
        got = np.zeros((T, H), np.float32)
        want = np.zeros((T, H), np.float32)
        for t in range(T):
            for s in np.argsort(ids[t]):                         # ascending REAL expert id
                got[t] += w[t, s] * out_rows[pos[t * K + s]].numpy()
                want[t] += w[t, s] * (np.float32(ids[t, s] + 1) * x[t])
        # hit counters: each rank counts the rows its slots served; folded and summed over the
        # ranks they are the routing counts of the real experts
        slot_hits = np.zeros(V, np.int64)
        slot_hits[rank * slots:(rank + 1) * slots] = plan.local_counts
        folded = torch.from_numpy(pl.fold_hits(slot_hits).astype(np.int64))
        dist.all_reduce(folded)
        mine = torch.from_numpy(np.bincount(ids.reshape(-1), minlength=E).astype(np.int64))
        dist.all_reduce(mine)
        q.put((rank, bool(np.array_equal(got, want)) and bool(torch.equal(folded, mine))))
    finally:
        dist.destroy_process_group()


def test_placed_exchange_two_gloo_ranks():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_placed_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
