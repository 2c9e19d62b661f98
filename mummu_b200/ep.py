"""Expert-parallel form of the MoE layer: experts sharded in contiguous blocks over the ranks of a
`torch.distributed` group, token rows exchanged with two all-to-alls per layer.

The reference has no collectives (its devices exchange through host memory,
crates/mummu/src/backend.rs:128-143, nn/moe.rs:1219-1272); expert parallelism is how this path
shards on an NVLink box.  Per layer and rank:
  1. route the rank's own tokens (replicated router)                     mummu_moe_route
  2. group (token, slot) pairs by GLOBAL expert id = by destination rank mummu_moe_permute
  3. all-gather the per-expert row counts, plan the exchange             plan_exchange (host)
  4. all-to-all the routed rows to the ranks that own their experts      all_to_all_single
  5. re-order received rows (source-major -> expert-major), run the local experts
                                                                         mummu_moe_experts_grouped
  6. all-to-all the outputs back, weighted un-permute on the owner       mummu_moe_combine
`plan_exchange` and the index arithmetic are plain numpy so that they run (and are tested) on CPU
ranks with the gloo backend; only steps 1, 2, 5 and 6 touch the CUDA library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np


@dataclass
class ExchangePlan:
    send_splits: list          # rows this rank sends to each rank (sorted rows are already in that order)
    recv_splits: list          # rows this rank receives from each rank
    local_counts: np.ndarray   # [experts_local] rows per local expert, all sources together
    to_expert_major: np.ndarray  # index: expert-major position -> position in the received (source-major) buffer


def plan_exchange(all_counts: np.ndarray, rank: int, world: int) -> ExchangePlan:
    """all_counts[src, e] = rows rank `src` routes to global expert e.  Experts are sharded in
    contiguous blocks of E / world.  Rows arrive source-major (per source: ascending local expert,
    ascending token); the expert bank wants them expert-major, sources in rank order inside an
    expert, which keeps every expert's rows in a fixed, reproducible order."""
    all_counts = np.asarray(all_counts, dtype=np.int64)
    assert all_counts.shape[0] == world and all_counts.shape[1] % world == 0
    el = all_counts.shape[1] // world
    mine = all_counts[rank].reshape(world, el)
    send_splits = mine.sum(axis=1).tolist()
    recv = all_counts[:, rank * el:(rank + 1) * el]            # [src, e_local]
    recv_splits = recv.sum(axis=1).tolist()
    local_counts = recv.sum(axis=0)
    # start of (src, e) block in the received buffer
    flat = recv.reshape(-1)
    starts = np.concatenate([[0], np.cumsum(flat)[:-1]]).reshape(world, el)
    order = []
    for e in range(el):
        for src in range(world):
            n = int(recv[src, e])
            if n:
                order.append(np.arange(starts[src, e], starts[src, e] + n))
    to_expert_major = np.concatenate(order) if order else np.zeros(0, dtype=np.int64)
    return ExchangePlan(send_splits, recv_splits, local_counts.astype(np.int32), to_expert_major.astype(np.int64))


class PeerWorkspace:
    """The buffers of a rank, shared by every layer of a stack: rows received for its experts, the
    expert outputs of its own (token, slot) pairs that come back, and the block of flags and counts
    the ranks signal each other through - those three allocated by the CUDA library, exported as
    IPC handles, exchanged through the process group and mapped by every peer - plus the private
    buffer its experts write into.  cap_rows: rows that may arrive (every rank's tokens * top_k);
    back_rows: this rank's own tokens * top_k."""

    def __init__(self, group, device: int, cap_rows: int, hidden: int, experts: int = 256, back_rows: int = 0):
        import ctypes as C
        import torch.distributed as dist
        from . import _lib as L
        self.L, self.device, self.group = L, device, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.cap_rows, self.bytes = cap_rows, cap_rows * hidden * 2
        self.back_rows = back_rows or -(-cap_rows // self.world)
        self.own, self.opened, handles = [], [], []
        sync_bytes = int(L.lib.mummu_ep_sync_bytes(self.world, experts))
        for nbytes in (self.bytes, self.back_rows * hidden * 2, sync_bytes, self.bytes):
            ptr, h = C.c_void_p(), C.create_string_buffer(64)
            rc = L.lib.mummu_ep_alloc(device, max(nbytes, 16), C.byref(ptr), h)
            if rc:
                raise RuntimeError(L.last_error())
            self.own.append(ptr.value)
            handles.append(h.raw)
        handles = handles[:3]                      # the fourth buffer is private
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles, group=group)
        self.tables = []
        for which in range(3):
            table = (C.c_void_p * self.world)()
            for r in range(self.world):
                if r == self.rank:
                    table[r] = self.own[which]
                else:
                    ptr = C.c_void_p()
                    rc = L.lib.mummu_ep_open(device, gathered[r][which], C.byref(ptr))
                    if rc:
                        raise RuntimeError(L.last_error())
                    self.opened.append(ptr.value)
                    table[r] = ptr.value
            self.tables.append(table)
        self.recv_table, self.back_table, self.sync_table = self.tables
        self.recv_ptr, self.back_ptr, self.sync_ptr, self.ys_ptr = self.own
        self.experts = experts
        dist.barrier(group=group)          # every peer has mapped every (zeroed) block

    def reset(self):
        """After a timed-out step: every rank zeroes its own block of flags and epochs, between two
        host barriers (nobody signals into a block that is about to be zeroed)."""
        import torch.distributed as dist
        dist.barrier(group=self.group)
        rc = self.L.lib.mummu_ep_reset(self.device, self.sync_ptr, self.world, self.experts)
        if rc:
            raise RuntimeError(self.L.last_error())
        dist.barrier(group=self.group)

    def close(self):
        """Unmap the peers' blocks, wait until every rank has done so, then free the own blocks:
        freeing exported memory that a peer still has mapped is undefined."""
        import torch.distributed as dist
        for p in self.opened:
            self.L.lib.mummu_ep_close(p)
        self.opened = []
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for p in self.own:
            self.L.lib.mummu_ep_free(p)
        self.own = []


class LocalWorkspaces:
    """`world` rank workspaces on ONE device in one process (no process group, no IPC): the peers'
    blocks are plain device pointers.  For running the rank handles of a group stage by stage on a
    single stream (tests on one GPU; never several streams or processes: a stage that waits for a
    kernel that has not been scheduled would only run into its bound)."""

    def __init__(self, device: int, world: int, cap_rows: int, hidden: int, experts: int, back_rows: int = 0):
        import ctypes as C
        from . import _lib as L
        self.L, self.device, self.world, self.experts = L, device, world, experts
        self.cap_rows = cap_rows
        self.back_rows = back_rows or -(-cap_rows // world)
        sync_bytes = int(L.lib.mummu_ep_sync_bytes(world, experts))
        self.ptrs = [[], [], [], []]                   # recv, back, sync, ys per rank
        for _ in range(world):
            sizes = (cap_rows * hidden * 2, self.back_rows * hidden * 2, sync_bytes, cap_rows * hidden * 2)
            for which, nbytes in enumerate(sizes):
                ptr, h = C.c_void_p(), C.create_string_buffer(64)
                rc = L.lib.mummu_ep_alloc(device, max(nbytes, 16), C.byref(ptr), h)
                if rc:
                    raise RuntimeError(L.last_error())
                self.ptrs[which].append(ptr.value)
        self.views = [_RankView(self, r) for r in range(world)]

    def reset(self):
        for p in self.ptrs[2]:
            rc = self.L.lib.mummu_ep_reset(self.device, p, self.world, self.experts)
            if rc:
                raise RuntimeError(self.L.last_error())

    def close(self):
        for lst in self.ptrs:
            for p in lst:
                self.L.lib.mummu_ep_free(p)
        self.ptrs = [[], [], [], []]


class _RankView:
    def __init__(self, ws: LocalWorkspaces, rank: int):
        import ctypes as C
        self.world, self.rank, self.cap_rows, self.experts = ws.world, rank, ws.cap_rows, ws.experts
        self.back_rows = ws.back_rows
        mk = lambda lst: (C.c_void_p * ws.world)(*lst)
        self.recv_table, self.back_table, self.sync_table = mk(ws.ptrs[0]), mk(ws.ptrs[1]), mk(ws.ptrs[2])
        self.recv_ptr, self.back_ptr, self.sync_ptr = ws.ptrs[0][rank], ws.ptrs[1][rank], ws.ptrs[2][rank]
        self.ys_ptr = ws.ptrs[3][rank]


class ExpertParallelMoe:
    """One MoE layer sharded over `group`; each rank calls forward on its own tokens.

    With a workspace (16-bit activations) rows move by peer stores and loads over NVLink and
    nothing waits for the host; without one the exchange is two NCCL all-to-alls whose split sizes
    are read back to the host.  `rank`/`world` given explicitly (with a `LocalWorkspaces` view)
    build one rank of a group that lives on a single device."""

    def __init__(self, cfg, group=None, device: Optional[int] = None, act_dtype: int = 2,
                 weight_dtype: Optional[int] = None, max_tokens: int = 0, workspace=None,
                 scratch_donor=None, rank: Optional[int] = None, world: Optional[int] = None,
                 placement=None):
        import torch
        from . import moe
        self.group = group
        if rank is None:
            import torch.distributed as dist
            self.dist = dist
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.dist, self.rank, self.world = None, rank, world
        self.cfg = cfg
        self.placement = placement
        if placement is None:
            assert cfg.num_experts % self.world == 0, "experts must divide evenly over the ranks"
            self.el = cfg.num_experts // self.world
            self.slots_total = cfg.num_experts
        else:
            # the bank handles of the group run over SLOTS; a second, bank-less handle routes over
            # the real experts and its ids are turned into slot ids (mummu_ep_place)
            assert placement.world == self.world and placement.experts == cfg.num_experts
            assert workspace is not None, "a placed layer moves rows through a peer workspace"
            self.el = placement.slots
            self.slots_total = placement.virtual_experts
        dev = torch.cuda.current_device() if device is None else device
        self.device = torch.device("cuda", dev)
        # scratch for the local experts must hold the rows that can arrive: every rank's tokens * k
        self.workspace = workspace
        if workspace is not None:
            assert self.slots_total <= workspace.experts, "workspace sync block too small for this group"
        self.moe = moe.SparseMoeConfig(cfg.hidden_size, cfg.expert_intermediate_size, self.slots_total,
                                       cfg.num_experts_per_tok).init(
            device=dev, act_dtype=act_dtype, weight_dtype=weight_dtype,
            max_tokens=0 if scratch_donor is not None else max_tokens * self.world,
            expert_first=self.rank * self.el, experts_local=self.el)
        if scratch_donor is not None:
            self.moe.adopt_scratch(scratch_donor.moe)
        self.router = self.moe
        if placement is not None:
            self.router = moe.SparseMoeConfig(cfg.hidden_size, cfg.expert_intermediate_size, cfg.num_experts,
                                              cfg.num_experts_per_tok).init(
                device=dev, act_dtype=act_dtype, weight_dtype=weight_dtype, max_tokens=max_tokens,
                expert_first=0, experts_local=1)
            self.table = torch.from_numpy(placement.route_table(self.rank)).to(self.device)

    def set_router(self, weight, layout: int = 0, bias=None):
        self.router.set_router(weight, layout, bias)

    def set_local_banks(self, gate, up, down):
        """Banks of this rank's experts only: [experts / world, out, in]; with a placement, of its
        slots: bank[placement.rank_experts(rank)]."""
        self.moe.set_banks(gate, up, down)

    def take_hits(self):
        """Per (real) expert routing hits of this rank's tokens since the last call
        (`ExpertPool::take_hits`, nn/moe.rs:1527-1535): the planner's input."""
        return self.router.take_hits()

    # ---- the four stages (see include/mummu_cuda.h); a rank runs them in this order ------------
    def stage_route(self, x, top_k: int, norm_topk_prob: bool):
        import torch
        m, ws = self.moe, self.workspace
        T = x.shape[0]
        assert T * top_k * self.world <= ws.cap_rows, "workspace too small for the rows that may arrive"
        assert T * top_k <= ws.back_rows, "workspace too small for the rows that come back"
        st = dict(x=x, top_k=top_k)
        i32 = dict(dtype=torch.int32, device=x.device)
        if self.placement is None:
            st["ids"], st["w"], st["counts"], st["offsets"], st["row_token"], st["pos"] = m.route_grouped(x, top_k, norm_topk_prob)
        else:
            st["expert_ids"], st["w"] = self.router.route_flat(x, top_k, norm_topk_prob)
            st["ids"] = torch.empty_like(st["expert_ids"])
            m.ep_place(st["expert_ids"], self.table, self.cfg.num_experts, st["ids"])
            V = self.slots_total
            st["counts"], st["offsets"] = torch.empty(V, **i32), torch.empty(V + 1, **i32)
            st["row_token"], st["pos"] = torch.empty(T * top_k, **i32), torch.empty(T * top_k, **i32)
            m.permute(st["ids"], st["counts"], st["offsets"], st["row_token"], st["pos"])
        m.ep_post_counts(st["counts"], ws.sync_table, self.rank, self.world)
        st["dst_base"], st["local_counts"] = torch.empty(self.slots_total, **i32), torch.empty(self.el, **i32)
        return st

    def stage_dispatch(self, st):
        ws = self.workspace
        self.moe.ep_dispatch(st["x"], st["row_token"], st["offsets"], ws.sync_table, ws.recv_table, self.rank,
                             self.world, ws.cap_rows, st["dst_base"], st["local_counts"])

    def stage_experts(self, st):
        ws = self.workspace
        self.moe.ep_experts(ws.sync_table, ws.back_table, self.rank, self.world, ws.recv_ptr, st["local_counts"],
                            ws.cap_rows, ws.ys_ptr, ws.back_rows)

    def stage_combine(self, st):
        import torch
        ws = self.workspace
        y = torch.empty_like(st["x"])
        self.moe.ep_combine(ws.sync_table, ws.back_ptr, st["ids"], st["w"], st["pos"], self.rank, self.world, y,
                            order_ids=st.get("expert_ids"))
        return y

    # ---- small-batch form: every rank gets every token, routes them all, runs its own experts -----
    def gathered_supported(self, tokens: int, top_k: int) -> bool:
        from . import _lib as L
        ws = self.workspace
        return (ws is not None and self.placement is None and self.moe.weight_dtype == L.Q4_K
                and self.moe.act_dtype == L.F16 and self.world * tokens * top_k <= min(8192, ws.back_rows)
                and self.world * tokens <= ws.cap_rows)

    def stage_gather(self, x, top_k: int, norm_topk_prob: bool):
        ws = self.workspace
        self.moe.ep_gather_tokens(x, ws.sync_table, ws.recv_table, self.rank, self.world)
        return dict(x=x, top_k=top_k, norm=norm_topk_prob)

    def stage_route_all(self, st):
        ws, m, T, k = self.workspace, self.moe, st["x"].shape[0], st["top_k"]
        m.ep_wait(ws.sync_table, self.rank, self.world, 0)
        st["ids"], st["w"], st["counts"], st["offsets"], st["row_token"], st["pos"] = m.route_grouped_ptr(
            ws.recv_ptr, self.world * T, k, st["norm"], st["x"].device)
        m.ep_experts_gathered(ws.sync_table, ws.back_table, ws.recv_ptr, st["row_token"], st["counts"], st["offsets"],
                              self.rank, self.world, T, k, ws.back_rows)

    def stage_combine_own(self, st):
        import torch
        ws, T = self.workspace, st["x"].shape[0]
        own = slice(self.rank * T, (self.rank + 1) * T)
        y = torch.empty_like(st["x"])
        self.moe.ep_combine(ws.sync_table, ws.back_ptr, st["ids"][own], st["w"][own],
                            st["pos"].view(-1, st["top_k"])[own], self.rank, self.world, y)
        return y

    def forward_gathered(self, x, top_k: int, norm_topk_prob: bool):
        st = self.stage_gather(x, top_k, norm_topk_prob)
        self.stage_route_all(st)
        return self.stage_combine_own(st)

    def forward_p2p(self, x, top_k: int, norm_topk_prob: bool):
        st = self.stage_route(x, top_k, norm_topk_prob)
        self.stage_dispatch(st)
        self.stage_experts(st)
        return self.stage_combine(st)

    def forward(self, x, top_k: int, norm_topk_prob: bool):
        if self.workspace is not None:
            if self.gathered_supported(x.shape[0], top_k):
                return self.forward_gathered(x, top_k, norm_topk_prob)
            return self.forward_p2p(x, top_k, norm_topk_prob)
        import torch
        dist, m = self.dist, self.moe
        T, H = x.shape
        E, R = self.cfg.num_experts, self.world
        ids, w = m.route_flat(x, top_k, norm_topk_prob)
        counts = torch.empty(E, dtype=torch.int32, device=x.device)
        row_token = torch.empty(T * top_k, dtype=torch.int32, device=x.device)
        pos = torch.empty(T * top_k, dtype=torch.int32, device=x.device)
        m.permute(ids, counts, None, row_token, pos)
        send = x.index_select(0, row_token.long())                   # rows sorted by destination expert
        all_counts = torch.empty(R, E, dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(all_counts, counts, group=self.group)
        plan = plan_exchange(all_counts.cpu().numpy(), self.rank, R)  # host sync: split sizes are host integers
        n_recv = int(sum(plan.recv_splits))
        recv = torch.empty(n_recv, H, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, send, plan.recv_splits, plan.send_splits, group=self.group)
        order = torch.from_numpy(plan.to_expert_major).to(x.device)
        xs = recv.index_select(0, order)                              # expert-major
        ys = torch.empty_like(xs)
        if n_recv:
            m.experts_grouped(xs, torch.from_numpy(plan.local_counts).to(x.device), ys)
        back = torch.empty_like(recv)
        back.index_copy_(0, order, ys)                                # source-major again
        out_rows = torch.empty(T * top_k, H, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out_rows, back, plan.send_splits, plan.recv_splits, group=self.group)
        y = torch.empty_like(x)
        m.combine(out_rows, ids, w, pos, y)
        return y

    def close(self):
        if self.router is not self.moe:
            self.router.close()
        self.moe.close()
