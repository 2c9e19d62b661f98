"""Expert parallelism on 2 GPUs: the sharded layer against the same layer on one GPU."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q, act, wdt_name):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from mummu_b200 import _lib as L, moe, q4k, synth
        from mummu_b200.ep import ExpertParallelMoe
        H, I, E, K, T = 512, 256, 16, 4, 96 if wdt_name == "bf16" else 24
        router, gate, up, down, _ = synth.moe_layer(H, I, E, 1, cfg_seed=41)
        x = synth.normal(synth.layer_seed(41, 0, 10 + rank), (T, H), 1.0)
        if wdt_name == "q4k":
            act_code, wcode, tdt = L.F16, L.Q4_K, torch.float16
            enc = lambda a: q4k.quantize(a).reshape(a.shape[0], -1)
        else:
            act_code, wcode, tdt = L.BF16, L.BF16, torch.bfloat16
            enc = lambda a: torch.from_numpy(a).to(torch.bfloat16).cuda()
        el = E // world
        cfg = moe.SparseMoeConfig(H, I, E, K)
        from mummu_b200.ep import PeerWorkspace
        bias, plan = None, None
        if act == "placed":
            # a skewed router and a placement with two spare slots per rank: experts move between the
            # ranks and the hottest are held on both
            from mummu_b200 import placement as P
            bias = synth.zipf_router_bias(E, 1.0, 1.5, seed=3)
            hot = np.exp(bias.astype(np.float64))
            plan = P.plan_placement(hot / hot.sum(), E, world, el + 2)
            assert max(len(h) for h in plan.hosts) == 2
        slots_total = plan.virtual_experts if plan else E
        ws = (PeerWorkspace(None, rank, world * T * K, H, slots_total, back_rows=world * T * K if act == "gathered" else 0)
              if act != "nccl" else None)
        ep = ExpertParallelMoe(cfg, device=rank, act_dtype=act_code, weight_dtype=wcode, max_tokens=T, workspace=ws,
                               placement=plan)
        ep.set_router(router, bias=bias)
        sl = plan.rank_experts(rank) if plan else slice(rank * el, (rank + 1) * el)
        ep.set_local_banks(enc(gate[sl]), enc(up[sl]), enc(down[sl]))
        assert ep.gathered_supported(T, K) == (act == "gathered")
        xd = torch.from_numpy(x).cuda().to(tdt)
        y_ep = ep.forward(xd, K, False)
        y_ep2 = ep.forward(xd, K, False)
        ep.moe.sync()                      # raises if a bounded device-side wait ran out
        # the same layer, all experts on this GPU
        single = cfg.init(device=rank, act_dtype=act_code, weight_dtype=wcode, max_tokens=T)
        single.set_router(router, bias=bias)
        single.set_banks(enc(gate), enc(up), enc(down))
        y_one = single.forward(xd, K, False)
        single.sync()
        err = (y_ep.float() - y_one.float()).abs().max().item() / y_one.float().abs().max().item()
        q.put((rank, err, bool(torch.equal(y_ep, y_ep2))))
        ep.close()
        single.close()
        torch.cuda.synchronize()
        dist.barrier()
        if ws is not None:
            ws.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl", "p2p", "placed", "gathered"])
@pytest.mark.parametrize("wdt_name", ["bf16", "q4k"])
def test_expert_parallel_matches_single_gpu(cuda_lib, wdt_name, mode):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    if mode == "gathered" and wdt_name != "q4k":
        pytest.skip("the small-batch form serves the Q4_K decode layer")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, mode, wdt_name)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, same in results:
        assert err < 2e-2, (rank, err)
        assert same, "two identical calls must give identical results"
