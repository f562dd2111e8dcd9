"""Expert-parallel decode MoE layer over torch.distributed (one process per GPU, NCCL over NVLink / NVSwitch).

The reference engine has no multi-GPU code; this is the sharded form of its MoE layer.  Rank r of G owns the routed experts
[r·E/G, (r+1)·E/G) of every layer; the router and the shared expert are replicated; every rank brings its own B rows.

    route (local rows) → ONE all-gather of [row | ids | w] records → local experts over all G·B rows (pairs whose expert
    lives elsewhere are skipped through NULL table entries) → reduce-scatter of the fp32 routed sums → shared expert and
    combine on the local rows.

Remote data always lands in local memory through the collective before a kernel reads it; no kernel touches a peer's memory.
The fp32 routed sum of a row is then a sum over ranks of per-rank sums in k order, which differs from the single-GPU k order
only by fp32 reassociation; routing indices are unaffected.

`ops` is the operator module (eke_hive_b200 itself on GPUs).  The CPU tests pass a stand-in with the same four functions, so the
exchange logic runs under the gloo backend without a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def expert_range(E: int, world: int, rank: int) -> tuple[int, int]:
    """Experts [lo, hi) owned by `rank`."""
    return rank * E // world, (rank + 1) * E // world


def local_table(E: int, world: int, rank: int, ptr_of) -> list[int]:
    """Global expert id → record pointer on this rank, 0 for experts owned elsewhere.  ptr_of(local_index) gives the pointer."""
    lo, hi = expert_range(E, world, rank)
    return [ptr_of(e - lo) if lo <= e < hi else 0 for e in range(E)]


class ExpertParallelMoE:
    def __init__(self, ops, ctx, H: int, I: int, E: int, K: int, B: int, world: int, rank: int, device, group=None, renorm=True,
                 logits_bf16=True, limit=0.0):
        self.ops, self.ctx, self.H, self.I, self.E, self.K, self.B = ops, ctx, H, I, E, K, B
        self.world, self.rank, self.dev, self.group = world, rank, device, group
        self.renorm, self.logits_bf16, self.limit = renorm, logits_bf16, limit
        self.rec_bytes = H * 2 + K * 8                                    # one row's record: bf16 row | int32 ids | fp32 weights
        self.send = torch.empty((B, self.rec_bytes), dtype=torch.uint8, device=device)
        self.recv = torch.empty((world * B, self.rec_bytes), dtype=torch.uint8, device=device)
        self.x_all = torch.empty((world * B, H), dtype=torch.bfloat16, device=device)
        self.ids_all = torch.empty((world * B, K), dtype=torch.int32, device=device)
        self.w_all = torch.empty((world * B, K), dtype=torch.float32, device=device)
        self.part = torch.empty((world * B, H), dtype=torch.float32, device=device)
        self.routed = torch.empty((B, H), dtype=torch.float32, device=device)
        self.shared_f32 = torch.empty((B, H), dtype=torch.float32, device=device)
        self.one_id = torch.zeros((B, 1), dtype=torch.int32, device=device)
        self.one_w = torch.ones((B, 1), dtype=torch.float32, device=device)
        self.shared_tab = torch.zeros(1, dtype=torch.int64, device=device)
        self.reduce_scatter = dist.get_backend(group) != "gloo"            # gloo has no reduce-scatter: all-reduce and slice there
        ws_bytes = getattr(ops, "moe_decode_ws_bytes", lambda n, h, i: 256)(world * B * K, H, I)
        self.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)

    def layer(self, logits, x, tab, li: int, shared_ptr: int, gate_col: int, ids_out, w_out, out):
        """logits fp32 [B, ≥E(+1)], x bf16 [B, H] local rows; tab: device table [L·E] of local record pointers (0 = elsewhere);
        shared_ptr: this layer's shared-expert record (0 = none).  Writes ids_out / w_out [B, K] and out bf16 [B, H]."""
        ops, B, H, K, G = self.ops, self.B, self.H, self.K, self.world
        ops.router_softmax_topk(logits, K, self.renorm, self.logits_bf16, E=self.E, ids=ids_out, w=w_out, ctx=self.ctx)
        # pack [row | ids | w] per row, one all-gather, unpack into dense arrays
        self.send[:, :H * 2].copy_(x.view(torch.uint8).view(B, H * 2))
        self.send[:, H * 2:H * 2 + K * 4].copy_(ids_out.view(torch.uint8).view(B, K * 4))
        self.send[:, H * 2 + K * 4:].copy_(w_out.view(torch.uint8).view(B, K * 4))
        dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        self.x_all.view(torch.uint8).view(G * B, H * 2).copy_(self.recv[:, :H * 2])
        self.ids_all.view(torch.uint8).view(G * B, K * 4).copy_(self.recv[:, H * 2:H * 2 + K * 4])
        self.w_all.view(torch.uint8).view(G * B, K * 4).copy_(self.recv[:, H * 2 + K * 4:])
        # local experts over every rank's rows
        ops.moe_decode_routed_f32(self.ids_all, self.w_all, tab, li, self.E, self.x_all, H, self.I, out=self.part, limit=self.limit, ws=self.ws,
                                  ctx=self.ctx)
        if self.reduce_scatter:
            dist.reduce_scatter_tensor(self.routed, self.part, op=dist.ReduceOp.SUM, group=self.group)
        else:
            dist.all_reduce(self.part, op=dist.ReduceOp.SUM, group=self.group)
            self.routed.copy_(self.part[self.rank * B:(self.rank + 1) * B])
        # shared expert (replicated) on the local rows, then the combine
        if shared_ptr:
            self.shared_tab.fill_(shared_ptr)
            ops.moe_decode_routed_f32(self.one_id, self.one_w, self.shared_tab, 0, 1, x, H, self.I, out=self.shared_f32, limit=self.limit,
                                      ws=self.ws, ctx=self.ctx)
            shared = self.shared_f32.to(torch.bfloat16)                     # exact: the values are bf16 already
            ops.moe_combine(self.routed, shared, logits if gate_col >= 0 else None, gate_col if gate_col >= 0 else 0, out=out, ctx=self.ctx)
        else:
            ops.moe_combine(self.routed, torch.zeros_like(out), None, 0, out=out, ctx=self.ctx)
        return out

    def local_records_touched(self, ids_all_sets) -> float:
        """Mean number of distinct local expert records (plus the shared copy) one layer call streams, from gathered ids."""
        lo, hi = expert_range(self.E, self.world, self.rank)
        n = []
        for ids in ids_all_sets:
            v = ids[(ids >= lo) & (ids < hi)]
            n.append(int(torch.unique(v).numel()) + 1)
        return float(sum(n)) / max(len(n), 1)
