"""The allocation-free decode entry point (hb_moe_decode_routed_static), called through the C ABI.

It exists for hosts that are not allowed to allocate device memory at call time (memory budget handed out at start-up,
latency-critical loops, plugin hosts that keep the allocator): its scratch is a fixed array inside the library.  The file name
sorts last on purpose: if this test fails under `pytest -x`, every other test has already run.

Checked here: two calls in a row give exactly the output of hb_moe_decode_routed with a caller workspace (same kernels, same
arithmetic, so equality is bit for bit — tighter than the 2e-2 x RMS the other decode tests allow); the second call finds the
first call's leftovers in the shared array and must not be disturbed by them; a problem larger than the array is refused with
a clear error; no torch allocation happens inside the calls."""
import numpy as np
import pytest

from util import bf16_tensor, random_records, rel_rms_err, upload

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_workspace_entry(oracle):
    import torch

    import eke_hive_b200 as E
    H, I, Ex, K = 2048, 512, 24, 4
    rng = np.random.default_rng(2026)
    recs = random_records(oracle, H, I, Ex, seed=17)
    drecs = upload(recs)
    tab = E.rec_table(drecs)
    assert E.static_max_pairs(H, I) >= 16 * K
    # everything the calls need is allocated up front: outputs, inputs, routing
    cases = []
    for M in (16, 5):                                               # the second call is smaller: stale groups of the first stay behind it
        x = bf16_tensor(oracle.bf16r(rng.normal(0, 1, (M, H)).astype(np.float32)))
        ids_np = np.stack([rng.permutation(Ex)[:K] for _ in range(M)]).astype(np.int32)
        if M > 8:
            ids_np[:, 0] = 3                                        # one expert takes every row (two groups)
            ids_np[:, 1:][ids_np[:, 1:] == 3] = 7
            for m in range(M):                                      # keep experts distinct within a row
                if len(set(ids_np[m])) < K:
                    ids_np[m] = np.concatenate([[3], rng.permutation([e for e in range(Ex) if e != 3])[:K - 1]])
        ids_np[-1, -1] = -1                                         # an invalid id contributes nothing
        ids = torch.from_numpy(ids_np).cuda()
        w = torch.from_numpy(rng.uniform(0.05, 0.5, (M, K)).astype(np.float32)).cuda()
        shared = bf16_tensor(oracle.bf16r(rng.normal(0, 0.1, (M, H)).astype(np.float32)))
        lg = torch.from_numpy(rng.normal(0, 1, (M, 2)).astype(np.float32)).cuda()
        out_ws = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
        out_st = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device="cuda")
        cases.append((M, x, ids, w, shared, lg, out_ws, out_st, ids_np))
    ws = torch.empty(E.moe_decode_ws_bytes(16 * K, H, I), dtype=torch.uint8, device="cuda")
    ctx = E.Context(flags=8)     # HB_FLAG_DECODE_MMA_SYNC: the workspace entry point pinned to the streaming kernels, which the static entry always runs
    # a first call resolves the array's address once (no allocation either, but it is the only call that asks the runtime anything)
    M0, x0, ids0, w0, shared0, lg0, _, out_st0, _ = cases[0]
    E.fn_moe_decode_routed_static(ids0, w0, tab, 0, Ex, x0, H, I, shared=shared0, lg=lg0, col=1, out=out_st0, ctx=ctx)
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    free_before = torch.cuda.mem_get_info()[0]                      # the driver's count: sees a cudaMalloc inside the library too
    for M, x, ids, w, shared, lg, out_ws, out_st, _ in cases:       # two calls in a row on the static array
        E.fn_moe_decode_routed_static(ids, w, tab, 0, Ex, x, H, I, shared=shared, lg=lg, col=1, out=out_st, ctx=ctx)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before              # no device memory was taken by the calls, by anybody
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before   # nor through torch's allocator
    for M, x, ids, w, shared, lg, out_ws, out_st, _ in cases:
        E.fn_moe_decode_routed(ids, w, tab, 0, Ex, x, H, I, shared=shared, lg=lg, col=1, out=out_ws, ws=ws, ctx=ctx)
    torch.cuda.synchronize()
    ctx.check_device()
    for M, x, ids, w, shared, lg, out_ws, out_st, ids_np in cases:
        assert torch.equal(out_st, out_ws), f"M={M}: static-scratch output differs from the workspace entry point (streaming engine)"
    # and both agree with the CPU oracle (first case)
    M, x, ids, w, shared, lg, out_ws, out_st, ids_np = cases[0]
    acc = oracle.moe_routed(H, I, ids_np, w.cpu().numpy(), recs, x.float().cpu().numpy(), 0.0, 0)
    ref = oracle.bf16_to_f32(oracle.moe_combine(acc, shared.float().cpu().numpy(), lg.cpu().numpy(), 1, True))
    assert rel_rms_err(out_st.float().cpu().numpy(), ref) <= 2e-2
    # an unpinned context may run the same call on its other gate/up engine (64 pairs here: the tensor-memory kernel): same tolerance
    out_def = E.fn_moe_decode_routed(ids, w, tab, 0, Ex, x, H, I, shared=shared, lg=lg, col=1, ws=ws)
    torch.cuda.synchronize()
    E.context().check_device()
    assert rel_rms_err(out_def.float().cpu().numpy(), ref) <= 2e-2
    ctx.close()


def test_static_scratch_rejects_oversize():
    import torch

    import eke_hive_b200 as E
    H, I = 4096, 1536
    limit = E.static_max_pairs(H, I)
    assert 0 < limit < 4096
    M, K = 64, 8                                                    # 512 pairs > limit (371)
    assert M * K > limit
    ids = torch.zeros((M, K), dtype=torch.int32, device="cuda"); w = torch.zeros((M, K), dtype=torch.float32, device="cuda")
    x = torch.zeros((M, H), dtype=torch.bfloat16, device="cuda"); out = torch.zeros((M, H), dtype=torch.bfloat16, device="cuda")
    tab = torch.zeros(4, dtype=torch.int64, device="cuda")
    with pytest.raises(E.HbError) as ei:
        E.fn_moe_decode_routed_static(ids, w, tab, 0, 4, x, H, I, shared=x, out=out)
    assert ei.value.status == -2 and "scratch" in str(ei.value) and str(limit) in str(ei.value)
