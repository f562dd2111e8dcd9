"""A bounded wait that runs out: the rank's gather flag is local memory that nobody sets, the context's wait limit is small, so the
wait kernel gives up after its polls, sets the context's device error word and returns; hb_check_device reports
HB_ERR_DEVICE_FLAG and clears the word, the context stays usable, and a wait whose flag IS set passes.  Nothing hangs and
nothing faults: the kernel ends by itself (one GPU, world size 1)."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
HB_ERR_DEVICE_FLAG = -6


def test_wait_runs_out_reports_and_recovers():
    import eke_hive_b200 as E
    B, H, K, Ex = 4, 256, 2, 8
    ctx = E.Context(wait_polls=3000)
    _, total, _ = E.PeerExchange.layout(1, B, H, K)
    mine = torch.zeros(total, dtype=torch.uint8, device="cuda")
    ex = E.PeerExchange(mine, lambda o: [o], 0, 1, B, H, K, ctx=ctx)
    try:
        torch.cuda.synchronize()
        for _ in range(2):                                    # the second wait runs out just as quickly: nothing is left latched
            t0 = time.perf_counter()
            ex.wait_rows()                                    # no push before it: the flag stays 0
            with pytest.raises(E.HbError) as ei:
                ctx.check_device()
            assert ei.value.status == HB_ERR_DEVICE_FLAG and "0x40000" in str(ei.value)
            assert time.perf_counter() - t0 < 1.0
        ctx.check_device()                                    # the word was cleared by the failing check
        # the same context still computes: the rows are pushed (to this rank itself), the wait passes
        x = torch.randn(B, H, device="cuda").to(torch.bfloat16)
        lg = torch.randn(B, Ex, device="cuda")
        ids = torch.empty(B, K, dtype=torch.int32, device="cuda"); w = torch.empty(B, K, device="cuda")
        ex.route_push(lg, x, ids, w, Ex)
        ex.wait_rows()
        ctx.check_device()
        ref_ids, ref_w = E.router_softmax_topk(lg, K, renorm=True, logits_bf16=True)
        assert torch.equal(ids, ref_ids) and torch.equal(w, ref_w)
    finally:
        torch.cuda.synchronize()
        ex.close()
        ctx.close()
