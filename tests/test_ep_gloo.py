"""Expert-parallel exchange logic on CPU: two gloo ranks, the CPU oracle standing in for the GPU operators (same function names
and argument meaning).  The sharded layer must reproduce the unsharded oracle layer: identical routing, outputs equal up to the
fp32 reassociation of the cross-rank sum."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
H, I, E, K, B = 128, 64, 8, 3, 4


class OracleOps:
    """The three operators ExpertParallelMoE calls, computed by the CPU oracle on CPU tensors.  Records are numpy arrays kept in
    a registry; the 'pointer table' holds registry keys."""

    def __init__(self, O, registry):
        self.O, self.reg = O, registry

    def router_softmax_topk(self, logits, k, renorm, logits_bf16, E=None, ids=None, w=None, ctx=None):
        i, ww = self.O.router_softmax_topk(logits.numpy(), k, renorm, logits_bf16, 0, E=E)
        ids.copy_(torch.from_numpy(i)); w.copy_(torch.from_numpy(ww))
        return ids, w

    def moe_decode_ep_local(self, ids, w, tab, li, E, x, H_, I_, routed_out, shared_ptr=0, sh_row0=0, sh_rows=0, shared_out=None, limit=0.0,
                            ws=None, ctx=None):
        recs = [self.reg.get(int(p)) for p in tab[li * E:(li + 1) * E]]
        xs = np.ascontiguousarray(x.float().numpy())
        acc = self.O.moe_routed(H_, I_, np.ascontiguousarray(ids.numpy()), np.ascontiguousarray(w.numpy()), recs, xs, limit, 0)
        routed_out.copy_(torch.from_numpy(acc))
        if shared_ptr:
            rec = self.reg[int(shared_ptr)]
            sh = np.stack([self.O.expert_forward(rec, H_, I_, xs[sh_row0 + m], 1.0, limit, 0) for m in range(sh_rows)])
            shared_out.copy_(torch.from_numpy(sh).to(torch.bfloat16))
        return routed_out

    def fn_moe_prefill(self, tab, li, E, ids, w, x, H_, I_, out=None, ws=None, S=None, limit=0.0, ctx=None):
        recs = [self.reg.get(int(p)) for p in tab[li * E:(li + 1) * E]]
        xs, idn, wn = x.float().numpy(), ids.numpy(), w.numpy()
        acc = np.zeros((xs.shape[0], H_), np.float32)
        for m in range(xs.shape[0]):
            for k in range(idn.shape[1]):
                e = int(idn[m, k])
                if 0 <= e < E and recs[e] is not None:
                    acc[m] += self.O.expert_forward_a4(recs[e], H_, I_, xs[m], limit) * np.float32(wn[m, k])
        out.copy_(torch.from_numpy(acc))
        return out

    def moe_combine(self, routed, shared, lg, col, out=None, ctx=None):
        bits = self.O.moe_combine(routed.numpy(), shared.float().numpy(), None if lg is None else lg.numpy(), col, True)
        out.copy_(torch.from_numpy(self.O.bf16_to_f32(bits)).to(torch.bfloat16))
        return out


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), FAKE_NUMA_NODES="1")
    sys.path.insert(0, str(ROOT)); sys.path.insert(0, str(ROOT / "tests"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from util import make_records
        spec = __import__("importlib.util").util.spec_from_file_location("hb_ep", ROOT / "eke_hive_b200" / "ep.py")
        ep_mod = __import__("importlib.util").util.module_from_spec(spec)
        spec.loader.exec_module(ep_mod)                                  # the module alone: no CUDA library needed for this test
        recs = make_records(O, H, I, E + 1, seed=123)                     # every rank builds the same experts; index E = shared
        registry = {1000 + e: recs[e] for e in range(E + 1)}
        lo, hi = ep_mod.expert_range(E, world, rank)
        assert (lo, hi) == (rank * E // world, (rank + 1) * E // world)
        tab = torch.tensor(ep_mod.local_table(E, world, rank, lambda j: 1000 + lo + j), dtype=torch.int64)
        assert int((tab != 0).sum()) == hi - lo
        rng = np.random.default_rng(7)                                    # same stream on every rank: the global batch
        x_all = O.bf16r(rng.normal(0, 1, (world * B, H)).astype(np.float32))
        lg_all = rng.normal(0, 1, (world * B, E + 1)).astype(np.float32)
        x = torch.from_numpy(x_all[rank * B:(rank + 1) * B]).to(torch.bfloat16)
        lg = torch.from_numpy(lg_all[rank * B:(rank + 1) * B].copy())
        layer = ep_mod.ExpertParallelMoE(OracleOps(O, registry), None, H, I, E, K, B, world, rank, torch.device("cpu"))
        ids = torch.empty((B, K), dtype=torch.int32); w = torch.empty((B, K), dtype=torch.float32)
        out = torch.empty((B, H), dtype=torch.bfloat16)
        layer.layer(lg, x, tab, 0, 1000 + E, E, ids, w, out)
        # unsharded oracle on the local rows
        rids, rw, rout = O.moe_layer(H, I, lg.numpy(), x.float().numpy(), recs[:E], K, shared_rec=recs[E], gate_logits=lg.numpy(), gate_col=E)
        ref = O.bf16_to_f32(rout)
        got = out.float().numpy()
        ok_ids = bool(np.array_equal(ids.numpy(), rids)) and ids.numpy().tobytes() == rids.tobytes()
        err = float(np.max(np.abs(got - ref)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))
        touched = layer.local_records_touched([layer.ids_all])
        # prefill form: the same rows through the grouped-GEMM operator's stand-in (NVFP4 activations), sharded vs unsharded
        full = torch.tensor([1000 + e for e in range(E)], dtype=torch.int64)
        ids_pf = ids.clone()
        ids_pf[0, 0] = -1; ids_pf[1, 1] = E + 2                          # ids outside [0, E) go nowhere and add nothing
        ref_pf = OracleOps(O, registry).fn_moe_prefill(full, 0, E, ids_pf, w, x, H, I, out=torch.empty((B, H), dtype=torch.float32)).numpy()
        err_pf, sent = 0.0, {}
        for exchange in ("a2a", "allgather"):
            pf = ep_mod.ExpertParallelPrefill(OracleOps(O, registry), None, H, I, E, K, B, world, rank, torch.device("cpu"), exchange=exchange)
            got_pf = pf.layer(ids_pf, w, x, tab, 0).numpy().copy()
            err_pf = max(err_pf, float(np.max(np.abs(got_pf - ref_pf)) / (np.sqrt(np.mean(ref_pf ** 2)) + 1e-30)))
            sent[exchange] = pf.stats["rows_sent"]
        # the dispatch sends a row to the other rank only when one of its valid ids lives there
        other = [(int(e) >= 0 and int(e) < E and not (lo <= int(e) < hi)) for e in ids_pf.reshape(-1)]
        want_sent = int(np.array(other).reshape(B, K).any(axis=1).sum())
        assert sent["a2a"] == want_sent and sent["allgather"] == (world - 1) * B, (sent, want_sent)
        q.put((rank, ok_ids, err, touched, err_pf))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_two_ranks_match_unsharded_oracle():
    world = 2
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_ids, err, touched, err_pf in res:
        assert err_pf <= 1e-5, f"rank {rank}: sharded prefill differs from unsharded by {err_pf} x RMS"      # fp32 reassociation of the cross-rank sum
        assert ok_ids, f"rank {rank}: routing differs"
        assert err <= 8e-3, f"rank {rank}: error {err} x RMS"            # bf16 output ulp after fp32 reassociation
        assert 1 <= touched <= E // world + 1


def test_partition_helpers():
    spec = __import__("importlib.util").util.spec_from_file_location("hb_ep", ROOT / "eke_hive_b200" / "ep.py")
    ep_mod = __import__("importlib.util").util.module_from_spec(spec)
    spec.loader.exec_module(ep_mod)
    for E_, G in ((512, 8), (160, 8), (256, 8), (512, 3), (7, 2)):
        ranges = [ep_mod.expert_range(E_, G, r) for r in range(G)]
        assert ranges[0][0] == 0 and ranges[-1][1] == E_
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(G - 1))
        sizes = [b - a for a, b in ranges]
        assert max(sizes) - min(sizes) <= 1
        tabs = [ep_mod.local_table(E_, G, r, lambda j: j + 1) for r in range(G)]
        owners = np.array([[t != 0 for t in tab] for tab in tabs]).sum(0)
        assert (owners == 1).all()                                        # every expert lives on exactly one rank
