"""The allocation-free router entry point against the handle-based one.

`mummu_moe_route_noalloc` serves callers that may not allocate device memory (a serving loop with
a fixed memory plan, a host framework that owns all device memory, a process whose GPU is already
full): its scratch is a fixed array inside the library.  This file is named to be collected last,
so a run that stops at the first failure has already run every other test.  It passes on its own
in a fresh process and after the rest of the suite."""
import numpy as np
import pytest

from mummu_b200 import synth

pytestmark = pytest.mark.gpu


def _route_both(L, moe, torch, T, H, E, K, norm, seed, act):
    router = synth.normal(synth.layer_seed(seed, 0, 0), (H, E), 0.02)
    x = synth.normal(synth.layer_seed(seed, 0, 4), (T, H), 1.0)
    tdt, code = {"f32": (torch.float32, L.F32), "f16": (torch.float16, L.F16)}[act]
    xd = torch.from_numpy(x).cuda().to(tdt)
    wd = torch.from_numpy(router).cuda()
    # the existing entry point, through a handle (allocates its own scratch)
    m = moe.SparseMoeConfig(H, 1, E, K).init(act_dtype=code, weight_dtype=L.F32)
    m.set_router(router)
    ids_ref, w_ref = m.route_flat(xd, K, norm)
    m.sync()
    # the new entry point: caller-owned inputs and outputs, nothing else
    ids = torch.full((T, K), -1, dtype=torch.int32, device="cuda")
    w = torch.full((T, K), -1.0, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = L.lib.mummu_moe_route_noalloc(xd.data_ptr(), code, wd.data_ptr(), None, T, H, E, K, int(norm),
                                       ids.data_ptr(), w.data_ptr(), 0, stream)
    assert rc == L.OK, L.last_error()
    torch.cuda.synchronize()
    m.close()
    return ids.cpu().numpy(), w.cpu().numpy(), ids_ref.cpu().numpy(), w_ref.cpu().numpy()


def test_noalloc_router_matches_handle_router_twice_in_a_row(cuda_lib):
    import torch
    from mummu_b200 import moe
    L = cuda_lib
    # two calls in a row share the fixed scratch: the second must not see the first's leftovers
    for T, H, E, K, norm, seed, act in [(333, 2048, 64, 8, False, 21, "f32"), (64, 2048, 64, 8, True, 22, "f16"),
                                        (1, 512, 128, 4, False, 23, "f32")]:
        ids, w, ids_ref, w_ref = _route_both(L, moe, torch, T, H, E, K, norm, seed, act)
        assert np.array_equal(ids, ids_ref)                                  # integer work: bit-exact
        assert np.array_equal(w.view(np.uint32), w_ref.view(np.uint32))      # same kernel, same bits


def test_noalloc_router_refuses_sizes_beyond_its_fixed_scratch(cuda_lib):
    import torch
    L = cuda_lib
    x = torch.zeros(8, 64, device="cuda")
    wd = torch.zeros(64, 16, device="cuda")
    ids = torch.zeros(8, 2, dtype=torch.int32, device="cuda")
    w = torch.zeros(8, 2, device="cuda")
    rc = L.lib.mummu_moe_route_noalloc(x.data_ptr(), L.F32, wd.data_ptr(), None, 1025, 64, 16, 2, 0,
                                       ids.data_ptr(), w.data_ptr(), 0, None)
    assert rc == L.ERR_CONTRACT and "exceed the fixed scratch" in L.last_error()
    rc = L.lib.mummu_moe_route_noalloc(x.data_ptr(), L.F32, wd.data_ptr(), None, 1024, 64, 257, 2, 0,
                                       ids.data_ptr(), w.data_ptr(), 0, None)
    assert rc == L.ERR_CONTRACT
    rc = L.lib.mummu_moe_route_noalloc(x.data_ptr(), L.F32, wd.data_ptr(), None, 8, 64, 16, 17, 0,
                                       ids.data_ptr(), w.data_ptr(), 0, None)
    assert rc == L.ERR_CONTRACT and "top_k" in L.last_error()


def test_noalloc_router_refuses_a_misaligned_weight_pointer(cuda_lib):
    """A router weight that starts in the middle of a packed buffer (4-byte but not 16-byte
    aligned) is refused on the host: the kernel would read it in 128-bit words.  Only the host-side
    check runs here; nothing is launched with the bad pointer."""
    import torch
    L = cuda_lib
    x = torch.zeros(8, 64, device="cuda")
    packed = torch.zeros(64 * 16 + 4, device="cuda")
    ids = torch.zeros(8, 2, dtype=torch.int32, device="cuda")
    w = torch.zeros(8, 2, device="cuda")
    rc = L.lib.mummu_moe_route_noalloc(x.data_ptr(), L.F32, packed.data_ptr() + 4, None, 8, 64, 16, 2, 0,
                                       ids.data_ptr(), w.data_ptr(), 0, None)
    assert rc == L.ERR_CONTRACT and "16-byte aligned" in L.last_error()
    rc = L.lib.mummu_moe_route_noalloc(x.data_ptr(), L.F32, packed.data_ptr(), None, 8, 64, 16, 2, 0,
                                       ids.data_ptr(), w.data_ptr(), 0, None)
    assert rc == L.OK, L.last_error()
    torch.cuda.synchronize()
