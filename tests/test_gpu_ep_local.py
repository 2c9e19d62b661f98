"""The expert-parallel exchange on ONE GPU: every rank of a group is a handle on the same device,
and the four stages (post counts, dispatch, experts, combine) are issued stage by stage on a single
stream - rank 0's stage, rank 1's stage, ... - so no kernel ever waits for one that has not run.
These are the kernels the multi-GPU layer runs (peer stores, flags, epochs, peer loads); the peers'
buffers are simply on the same device.  Checked against the same layer on a single handle, and the
single handle against the CPU oracle on sampled tokens."""
import numpy as np
import pytest

from oracle import oracle as O
from mummu_b200 import synth

pytestmark = pytest.mark.gpu


def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.view(np.float32)


def run_group(torch, group, ws_views, xs, K, norm):
    """One layer of the whole group, stage by stage on the current stream."""
    states = [ep.stage_route(x, K, norm) for ep, x in zip(group, xs)]
    for ep, st in zip(group, states):
        ep.stage_dispatch(st)
    for ep, st in zip(group, states):
        ep.stage_experts(st)
    return [ep.stage_combine(st) for ep, st in zip(group, states)]


def build_group(torch, L, moe, epmod, cfg, world, act, wdt, banks_dev, router, T_per_rank, bias=None):
    H, E, K = cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok
    el = E // world
    ws = epmod.LocalWorkspaces(0, world, world * T_per_rank * K, H, E)
    group = []
    for r in range(world):
        ep = epmod.ExpertParallelMoe(cfg, device=0, act_dtype=act, weight_dtype=wdt, max_tokens=T_per_rank,
                                     workspace=ws.views[r], rank=r, world=world)
        ep.set_router(router, bias=bias)
        ep.set_local_banks(*(b[r * el:(r + 1) * el] for b in banks_dev))
        group.append(ep)
    return ws, group


@pytest.mark.parametrize("world,Tr", [(2, 48), (8, 48), (2, 160)])
def test_ep_stages_bf16_qwen3_layer_shape(cuda_lib, world, Tr):
    """The expert-parallel configuration's layer: hidden 2048, 128 experts, top-8, intermediate 768,
    bf16; 48 tokens per rank (ragged segments, some experts without rows), and 160 per rank (1280
    rows: enough for the dispatch to move its rows through the copy engine)."""
    import torch
    from mummu_b200 import ep as epmod, moe
    L = cuda_lib
    H, I, E, K = 2048, 768, 128, 8
    cfg = moe.SparseMoeConfig(H, I, E, K)
    g = torch.Generator(device="cuda").manual_seed(50 + world)
    rnd = lambda *s: (torch.randn(*s, generator=g, device="cuda") * 0.02)
    router = rnd(H, E).cpu().numpy()
    banks = [rnd(E, I, H).to(torch.bfloat16), rnd(E, I, H).to(torch.bfloat16), rnd(E, H, I).to(torch.bfloat16)]
    xs = [torch.randn(Tr, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    ws, group = build_group(torch, L, moe, epmod, cfg, world, L.BF16, L.BF16, banks, router, Tr)
    single = cfg.init(act_dtype=L.BF16, weight_dtype=L.BF16, max_tokens=Tr * world)
    single.set_router(router)
    single.set_banks(*banks)
    ys = run_group(torch, group, ws.views, xs, K, False)
    ys2 = run_group(torch, group, ws.views, xs, K, False)        # epochs advance: a second layer call
    torch.cuda.synchronize()
    for ep in group:
        ep.moe.sync()                                            # no wait ran out, no row left its buffer
    want = single.forward(torch.cat(xs), K, False)
    single.sync()
    for r in range(world):
        a, b = ys[r].float(), want[r * Tr:(r + 1) * Tr].float()
        assert (a - b).abs().max().item() / b.abs().max().item() < 2e-2
        assert torch.equal(ys[r], ys2[r])
    # the single handle against the oracle on sampled tokens (tokens are independent)
    pick = [0, 1, Tr, Tr * world - 1]
    xf = torch.cat(xs)[pick].float().cpu().numpy()
    gate, up, down = (b.float().cpu().numpy() for b in banks)
    ref, _, _ = O.moe_forward(xf, router, gate, up, down, K, False)
    got = want[pick].float().cpu().numpy()
    assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-2
    for ep in group:
        ep.close()
    single.close()
    ws.close()


@pytest.mark.parametrize("world,Tr", [(2, 24), (8, 64)])
def test_ep_stages_q4k_decode_shape(cuda_lib, world, Tr):
    """The decode benchmark's layer sharded: hidden 2048, 64 experts, top-8, intermediate 1024, Q4_K
    experts, f16 activations; with 8 ranks and 64 tokens each an expert sees about 64 rows (several
    passes of the token tile)."""
    import torch
    from mummu_b200 import ep as epmod, moe
    L = cuda_lib
    H, I, E, K = 2048, 1024, 64, 8
    cfg = moe.SparseMoeConfig(H, I, E, K)
    g = torch.Generator(device="cuda").manual_seed(70 + world)
    rnd = lambda *s: (torch.randn(*s, generator=g, device="cuda") * 0.02)
    router = rnd(H, E).cpu().numpy()
    banks = [moe.q4k_quantize_device(rnd(E, I, H)).view(E, -1), moe.q4k_quantize_device(rnd(E, I, H)).view(E, -1),
             moe.q4k_quantize_device(rnd(E, H, I)).view(E, -1)]
    xs = [torch.randn(Tr, H, generator=g, device="cuda").to(torch.float16) for _ in range(world)]
    ws, group = build_group(torch, L, moe, epmod, cfg, world, L.F16, L.Q4_K, banks, router, Tr)
    ys = run_group(torch, group, ws.views, xs, K, False)
    torch.cuda.synchronize()
    for ep in group:
        ep.moe.sync()
    # reference: the CPU oracle on sampled tokens of every rank
    gq, uq, dq = (b.cpu().numpy() for b in banks)
    for r in (0, world - 1):
        pick = [0, Tr // 2, Tr - 1]
        xf = xs[r][pick].float().cpu().numpy()
        ref, _, _ = O.moe_forward(xf, router, gq, uq, dq, K, False, q4k=True)
        got = ys[r][pick].float().cpu().numpy()
        assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-2
    # and the same layer on one handle, every token (token batches of at most 256 rows per call)
    single = cfg.init(act_dtype=L.F16, weight_dtype=L.Q4_K, max_tokens=256)
    single.set_router(router)
    single.set_banks(*banks)
    for r in range(world):
        want = single.forward(xs[r], K, False).float()
        a = ys[r].float()
        assert (a - want).abs().max().item() / want.abs().max().item() < 2e-2
    single.sync()
    for ep in group:
        ep.close()
    single.close()
    ws.close()


def test_ep_receive_buffer_too_small_is_reported_not_written(cuda_lib):
    """A receive buffer smaller than the rows routed to it: the rows beyond it are dropped and the
    next sync reports it; nothing is stored outside the buffer."""
    import torch
    from mummu_b200 import ep as epmod, moe
    L = cuda_lib
    H, I, E, K, Tr, world = 256, 128, 8, 2, 16, 2
    cfg = moe.SparseMoeConfig(H, I, E, K)
    router, gate, up, down, _ = synth.moe_layer(H, I, E, 1, cfg_seed=5)
    banks = [torch.from_numpy(b).cuda().to(torch.bfloat16) for b in (gate, up, down)]
    ws, group = build_group(torch, L, moe, epmod, cfg, world, L.BF16, L.BF16, banks, router, Tr)
    xs = [torch.from_numpy(synth.normal(100 + r, (Tr, H), 1.0)).cuda().to(torch.bfloat16) for r in range(world)]
    for v in ws.views:
        v.cap_rows = 8                     # the buffers really hold world * Tr * K = 64 rows
    states = []
    for ep, x in zip(group, xs):           # stage_route without its host-side size check
        st = dict(x=x, top_k=K)
        st["ids"], st["w"], st["counts"], st["offsets"], st["row_token"], st["pos"] = ep.moe.route_grouped(x, K, False)
        ep.moe.ep_post_counts(st["counts"], ep.workspace.sync_table, ep.rank, world)
        i32 = dict(dtype=torch.int32, device="cuda")
        st["dst_base"], st["local_counts"] = torch.empty(E, **i32), torch.empty(E // world, **i32)
        states.append(st)
    for ep, st in zip(group, states):
        ep.stage_dispatch(st)
    torch.cuda.synchronize()
    with pytest.raises(moe.MoeContractError, match="left its buffer"):
        group[0].moe.sync()
    for ep in group:
        ep.close()
    ws.close()


def test_ep_return_buffer_too_small_is_reported_not_written(cuda_lib):
    """The way back: a rank whose buffer for returning outputs is smaller than its own rows gets
    the rows that fit; the rest are dropped by the sender and the sender's next sync reports it."""
    import torch
    from mummu_b200 import ep as epmod, moe
    L = cuda_lib
    H, I, E, K, Tr, world = 256, 128, 8, 2, 16, 2
    cfg = moe.SparseMoeConfig(H, I, E, K)
    router, gate, up, down, _ = synth.moe_layer(H, I, E, 1, cfg_seed=5)
    banks = [torch.from_numpy(b).cuda().to(torch.bfloat16) for b in (gate, up, down)]
    ws, group = build_group(torch, L, moe, epmod, cfg, world, L.BF16, L.BF16, banks, router, Tr)
    xs = [torch.from_numpy(synth.normal(100 + r, (Tr, H), 1.0)).cuda().to(torch.bfloat16) for r in range(world)]
    states = [ep.stage_route(x, K, False) for ep, x in zip(group, xs)]
    for ep, st in zip(group, states):
        ep.stage_dispatch(st)
    for v in ws.views:
        v.back_rows = 4                    # the buffers really hold Tr * K = 32 rows
    for ep, st in zip(group, states):
        ep.stage_experts(st)
    torch.cuda.synchronize()
    reported = 0
    for ep in group:
        try:
            ep.moe.sync()
        except moe.MoeContractError as exc:
            assert "left its buffer" in str(exc)
            reported += 1
    assert reported >= 1
    for ep in group:
        ep.close()
    ws.close()


def test_ep_wait_runs_out_and_the_group_recovers(cuda_lib):
    """Failure detection without a fault: rank 1 never posts its counts, so rank 0's dispatch stage
    runs into the (shortened) bound of its wait.  The kernel returns, moves no row, the next sync
    reports MUMMU_ERR_TIMEOUT, and after the sync blocks are re-zeroed the group runs a normal
    layer."""
    import torch
    from mummu_b200 import ep as epmod, moe
    L = cuda_lib
    H, I, E, K, Tr, world = 256, 128, 8, 2, 16, 2
    cfg = moe.SparseMoeConfig(H, I, E, K)
    router, gate, up, down, _ = synth.moe_layer(H, I, E, 1, cfg_seed=6)
    banks = [torch.from_numpy(b).cuda().to(torch.bfloat16) for b in (gate, up, down)]
    ws, group = build_group(torch, L, moe, epmod, cfg, world, L.BF16, L.BF16, banks, router, Tr)
    xs = [torch.from_numpy(synth.normal(200 + r, (Tr, H), 1.0)).cuda().to(torch.bfloat16) for r in range(world)]
    group[0].moe.set_switch("WAIT_POLLS", 2000)          # about a millisecond instead of seconds
    st = group[0].stage_route(xs[0], K, False)
    group[0].stage_dispatch(st)                           # rank 1 is silent
    torch.cuda.synchronize()
    with pytest.raises(TimeoutError):
        group[0].moe.sync()
    group[0].moe.sync()                                   # the status word was cleared: usable again
    ws.reset()
    group[0].moe.set_switch("WAIT_POLLS", 0)
    ys = run_group(torch, group, ws.views, xs, K, False)
    torch.cuda.synchronize()
    for ep in group:
        ep.moe.sync()
    single = cfg.init(act_dtype=L.BF16, weight_dtype=L.BF16, max_tokens=Tr * world)
    single.set_router(router)
    single.set_banks(*banks)
    want = single.forward(torch.cat(xs), K, False)
    for r in range(world):
        a, b = ys[r].float(), want[r * Tr:(r + 1) * Tr].float()
        assert (a - b).abs().max().item() / b.abs().max().item() < 2e-2
    for ep in group:
        ep.close()
    single.close()
    ws.close()


@pytest.mark.parametrize("weights", ["bf16", "q4k"])
def test_ep_hot_expert_placement_changes_loads_not_results(cuda_lib, weights):
    """A router with a Zipf bias over 64 experts on 8 ranks: hits -> smoothed hotness -> placement
    with two spare slots per rank.  The placed group (experts moved between ranks, hot ones held
    several times) must return bit for bit what the plainly sharded group returns - the same
    weights give the same numbers wherever they sit - while the busiest rank's rows drop."""
    import torch
    from mummu_b200 import ep as epmod, moe, placement as P
    L = cuda_lib
    H, I, E, K, world, Tr = 1024, 512, 64, 8, 8, 64
    cfg = moe.SparseMoeConfig(H, I, E, K)
    g = torch.Generator(device="cuda").manual_seed(91)
    rnd = lambda *s: (torch.randn(*s, generator=g, device="cuda") * 0.02)
    router = rnd(H, E).cpu().numpy()
    bias = synth.zipf_router_bias(E, 1.0, 1.2, seed=5)
    if weights == "bf16":
        act, wdt = L.BF16, L.BF16
        banks = [rnd(E, I, H).to(torch.bfloat16), rnd(E, I, H).to(torch.bfloat16), rnd(E, H, I).to(torch.bfloat16)]
        xs = [torch.randn(Tr, H, generator=g, device="cuda").to(torch.bfloat16) for _ in range(world)]
    else:
        act, wdt = L.F16, L.Q4_K
        banks = [moe.q4k_quantize_device(rnd(E, I, H)).view(E, -1), moe.q4k_quantize_device(rnd(E, I, H)).view(E, -1),
                 moe.q4k_quantize_device(rnd(E, H, I)).view(E, -1)]
        xs = [torch.randn(Tr, H, generator=g, device="cuda").to(torch.float16) for _ in range(world)]
    ws, group = build_group(torch, L, moe, epmod, cfg, world, act, wdt, banks, router, Tr, bias=bias)
    if weights == "q4k":
        # 8 experts per rank would take the expand-to-f16 path, 10 slots per rank the packed-weight
        # kernels: pin both groups to the same kernels, the comparison below is bit for bit
        for ep in group:
            ep.moe.set_switch("NO_TC", 1)
    ys = run_group(torch, group, ws.views, xs, K, True)
    torch.cuda.synchronize()
    hits = np.zeros(E, dtype=np.uint64)
    for ep in group:
        ep.moe.sync()
        hits += ep.take_hits()
    assert int(hits.sum()) == world * Tr * K
    hot = P.smooth_hotness([], hits.tolist(), 1.0)
    plan = P.plan_placement(hot, E, world, E // world + 2)
    assert max(len(h) for h in plan.hosts) >= 2                       # the head of the curve is held more than once
    S = plan.slots
    ws2 = epmod.LocalWorkspaces(0, world, world * Tr * K, H, plan.virtual_experts)
    placed = []
    for r in range(world):
        ep = epmod.ExpertParallelMoe(cfg, device=0, act_dtype=act, weight_dtype=wdt, max_tokens=Tr,
                                     workspace=ws2.views[r], rank=r, world=world, placement=plan)
        ep.set_router(router, bias=bias)
        if weights == "q4k":
            ep.moe.set_switch("NO_TC", 1)
        idx = torch.from_numpy(plan.rank_experts(r)).cuda()
        ep.set_local_banks(*(b.index_select(0, idx).contiguous() for b in banks))
        placed.append(ep)
    states = [ep.stage_route(x, K, True) for ep, x in zip(placed, xs)]
    for ep, st in zip(placed, states):
        ep.stage_dispatch(st)
    rows_placed = [int(st["local_counts"].sum().item()) for st in states]
    for ep, st in zip(placed, states):
        ep.stage_experts(st)
    ys2 = [ep.stage_combine(st) for ep, st in zip(placed, states)]
    torch.cuda.synchronize()
    for ep in placed:
        ep.moe.sync()
    for r in range(world):
        assert torch.equal(ys[r], ys2[r])
    el = E // world
    rows_plain = [int(hits[r * el:(r + 1) * el].sum()) for r in range(world)]
    assert sum(rows_placed) == sum(rows_plain) == world * Tr * K
    assert max(rows_placed) < 0.6 * max(rows_plain)
    # the routing hits of the placed group are still per real expert
    hits2 = np.zeros(E, dtype=np.uint64)
    for ep in placed:
        hits2 += ep.take_hits()
    assert np.array_equal(hits, hits2)
    # a table entry outside the slots is reported, not followed
    bad = placed[0].table.clone()
    ids_real, _ = placed[0].router.route_flat(xs[0], K, True)
    bad[int(ids_real[0, 0].item())] = plan.virtual_experts + 3
    out = torch.empty_like(ids_real)
    placed[0].moe.ep_place(ids_real, bad, E, out)
    with pytest.raises(moe.MoeContractError, match="left its buffer"):
        placed[0].moe.sync()
    assert int(out.max().item()) < plan.virtual_experts
    placed[0].moe.sync()                                              # the report does not stick
    for ep in placed + group:
        ep.close()
    ws.close()
    ws2.close()


@pytest.mark.parametrize("world,Tr", [(2, 24), (8, 64)])
def test_ep_gathered_decode_form(cuda_lib, world, Tr):
    """The small-batch form: tokens to every rank, every rank routes them all and runs its own
    experts, outputs back.  Stage by stage on one stream; bit-equal to the three-hop form where
    both run the packed-weight kernels (same rows of an expert in the same order), and checked
    against the oracle."""
    import torch
    from mummu_b200 import ep as epmod, moe
    L = cuda_lib
    H, I, E, K = 2048, 1024, 64, 8
    cfg = moe.SparseMoeConfig(H, I, E, K)
    g = torch.Generator(device="cuda").manual_seed(170 + world)
    rnd = lambda *s: (torch.randn(*s, generator=g, device="cuda") * 0.02)
    router = rnd(H, E).cpu().numpy()
    banks = [moe.q4k_quantize_device(rnd(E, I, H)).view(E, -1), moe.q4k_quantize_device(rnd(E, I, H)).view(E, -1),
             moe.q4k_quantize_device(rnd(E, H, I)).view(E, -1)]
    xs = [torch.randn(Tr, H, generator=g, device="cuda").to(torch.float16) for _ in range(world)]
    el = E // world
    rows = world * Tr * K
    ws = epmod.LocalWorkspaces(0, world, rows, H, E, back_rows=rows)
    group = []
    for r in range(world):
        ep = epmod.ExpertParallelMoe(cfg, device=0, act_dtype=L.F16, weight_dtype=L.Q4_K, max_tokens=Tr,
                                     workspace=ws.views[r], rank=r, world=world)
        ep.set_router(router)
        ep.set_local_banks(*(b[r * el:(r + 1) * el] for b in banks))
        assert ep.gathered_supported(Tr, K)
        group.append(ep)

    def gathered():
        states = [ep.stage_gather(x, K, False) for ep, x in zip(group, xs)]
        for ep, st in zip(group, states):
            ep.stage_route_all(st)
        return [ep.stage_combine_own(st) for ep, st in zip(group, states)]

    ys = gathered()
    ys_again = gathered()                                         # epochs advance
    ys_hops = run_group(torch, group, ws.views, xs, K, False)      # the three-hop form on the same handles
    torch.cuda.synchronize()
    for ep in group:
        ep.moe.sync()
    for r in range(world):
        assert torch.equal(ys[r], ys_again[r])
        if world == 2:
            assert torch.equal(ys[r], ys_hops[r])
        else:
            # 8 experts with about 64 rows each per rank: the three-hop form expands them to f16 for
            # the tensor cores, this form keeps the packed-weight kernels - same layer, other roundings
            a, b = ys[r].float(), ys_hops[r].float()
            assert (a - b).abs().max().item() / b.abs().max().item() < 2e-2
    gq, uq, dq = (b.cpu().numpy() for b in banks)
    for r in (0, world - 1):
        pick = [0, Tr // 2, Tr - 1]
        ref, _, _ = O.moe_forward(xs[r][pick].float().cpu().numpy(), router, gq, uq, dq, K, False, q4k=True)
        got = ys[r][pick].float().cpu().numpy()
        assert np.abs(got - ref).max() / np.abs(ref).max() < 2e-2
    for ep in group:
        ep.close()
    ws.close()
