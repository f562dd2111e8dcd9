"""Expert-parallel MoE layers (decode and prefill) over torch.distributed (one process per GPU, NCCL over NVLink / NVSwitch).

The reference engine has no multi-GPU code; this is the sharded form of its MoE layer.  Rank r of G owns the routed experts
[r·E/G, (r+1)·E/G) of every layer; the router and the shared expert are replicated; every rank brings its own B rows.

    route (local rows) → ONE all-gather of [row | ids | w] records → ONE operator pass: local experts over all G·B rows, read in
    place from the gathered buffer (pairs whose expert lives elsewhere are skipped through NULL table entries), plus the shared
    expert on the local rows → reduce-scatter of the fp32 routed sums → combine on the local rows.

Two transports.  "nccl": all-gather and reduce-scatter of torch.distributed; remote data lands in local memory through the
collective before a kernel reads it.  "peer" (default on GPUs; HIVE_B200_EP=nccl selects the other): the library's own kernels write the rows and the
partial sums straight into the other GPUs' exchange buffers over NVLink (plain peer stores, buffers mapped through CUDA IPC) and
announce them with step-number flags — no collective launch on the layer's critical path, and the cross-rank sum is added in
rank order by the combine kernel.  Reads of exchanged data are always local.
The fp32 routed sum of a row is then a sum over ranks of per-rank sums in k order, which differs from the single-GPU k order
only by fp32 reassociation; routing indices are unaffected.

`ops` is the operator module (eke_hive_b200 itself on GPUs).  The CPU tests pass a stand-in with the same three functions, so the
exchange logic runs under the gloo backend without a GPU.
"""
from __future__ import annotations

import os
import sys

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
                 logits_bf16=True, limit=0.0, transport: str | None = None, router: str = "softmax", bias=None, sigmoid_scale: float = 1.0):
        """router: "softmax" (top-k of softmax over bf16-rounded logits, renormalised) or "sigmoid" (GLM: top-k of sigmoid + bias,
        weights s / Σs · sigmoid_scale; bias fp32 [E] on the device or None)."""
        self.ops, self.ctx, self.H, self.I, self.E, self.K, self.B = ops, ctx, H, I, E, K, B
        self.router, self.bias, self.sigmoid_scale = router, bias, sigmoid_scale
        self.world, self.rank, self.dev, self.group = world, rank, device, group
        self.renorm, self.logits_bf16, self.limit = renorm, logits_bf16, limit
        # one row's exchange record: bf16 row | int32 ids | fp32 weights, padded to 16 bytes so every field of every gathered
        # row stays aligned for the kernels that read the gathered buffer in place
        self.rec_bytes = (H * 2 + K * 8 + 15) // 16 * 16
        self.send = torch.zeros((B, self.rec_bytes), dtype=torch.uint8, device=device)
        self.recv = torch.zeros((world * B, self.rec_bytes), dtype=torch.uint8, device=device)
        # strided views of the gathered buffer: no unpacking copies
        self.x_all = self.recv[:, :H * 2].view(torch.bfloat16)
        self.ids_all = self.recv[:, H * 2:H * 2 + K * 4].view(torch.int32)
        self.w_all = self.recv[:, H * 2 + K * 4:H * 2 + K * 8].view(torch.float32)
        self.part = torch.empty((world * B, H), dtype=torch.float32, device=device)
        self.routed = torch.empty((B, H), dtype=torch.float32, device=device)
        self.shared = torch.zeros((B, H), dtype=torch.bfloat16, device=device)
        self.reduce_scatter = dist.get_backend(group) != "gloo"            # gloo has no reduce-scatter: all-reduce and slice there
        want_peer = (transport or os.environ.get("HIVE_B200_EP", "peer")) == "peer" and self.reduce_scatter and hasattr(ops, "PeerExchange")
        self.peer = self._setup_peer() if want_peer else None
        self.transport = "peer" if self.peer is not None else "nccl"
        ws_bytes = getattr(ops, "moe_decode_ws_bytes", lambda n, h, i: 256)(world * B * (K + 1), H, I)
        self.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)

    def _setup_peer(self):
        """Maps every rank's exchange memory into this process (CUDA IPC) and builds the hb_ep object.  All ranks agree on the
        outcome: if any rank fails, every rank falls back to the NCCL transport."""
        ops, G, B, H, K = self.ops, self.world, self.B, self.H, self.K
        peer, err = None, ""
        try:
            off, total, rec = ops.PeerExchange.layout(G, B, H, K)
            assert rec == self.rec_bytes
            mine = torch.zeros(total, dtype=torch.uint8, device=self.dev)
            torch.cuda.synchronize(self.dev)

            def exchange(obj):
                got = [None] * G
                dist.all_gather_object(got, obj, group=self.group)
                return got
            peer = ops.PeerExchange(mine, exchange, self.rank, G, B, H, K, ctx=self.ctx)
            # the gathered rows are read in place from this rank's own buffer
            view = mine[off["recv"]:off["recv"] + G * B * rec].view(G * B, rec)
            self.recv = view
            self.x_all = view[:, :H * 2].view(torch.bfloat16)
            self.ids_all = view[:, H * 2:H * 2 + K * 4].view(torch.int32)
            self.w_all = view[:, H * 2 + K * 4:H * 2 + K * 8].view(torch.float32)
        except Exception as e:  # noqa: BLE001 - any failure means "use the collective library"
            err = f"{type(e).__name__}: {e}"
            peer = None
        ok = torch.tensor([1 if peer is not None else 0], dtype=torch.int32, device=self.dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            if err and self.rank == 0:
                print(f"[ep] peer-memory transport unavailable ({err}); using NCCL collectives", file=sys.stderr, flush=True)
            if peer is not None:                                           # another rank failed: drop the views into the exchange memory
                self.recv = torch.zeros((G * B, self.rec_bytes), dtype=torch.uint8, device=self.dev)
                self.x_all = self.recv[:, :H * 2].view(torch.bfloat16)
                self.ids_all = self.recv[:, H * 2:H * 2 + K * 4].view(torch.int32)
                self.w_all = self.recv[:, H * 2 + K * 4:H * 2 + K * 8].view(torch.float32)
            return None
        dist.barrier(group=self.group)                                     # nobody pushes before everybody has mapped and zeroed
        return peer

    def layer(self, logits, x, tab, li: int, shared_ptr: int, gate_col: int, ids_out, w_out, out):
        """logits fp32 [B, ≥E(+1)], x bf16 [B, H] local rows; tab: device table [L·E] of local record pointers (0 = elsewhere);
        shared_ptr: this layer's shared-expert record (0 = none).  Writes ids_out / w_out [B, K] and out bf16 [B, H]."""
        ops, B, H, K = self.ops, self.B, self.H, self.K
        if self.peer is not None:
            # three calls, six kernels: [route + push rows] → [wait + group] → gate/up → down → [reduce + push sums] → [wait + combine]
            if self.router == "sigmoid":
                ops.router_topk(logits[:, :self.E].contiguous() if logits.shape[1] != self.E else logits, self.bias, K, self.sigmoid_scale, ctx=self.ctx, ids=ids_out,
                                w=w_out)
                self.peer.push_rows(x, ids_out, w_out)
            else:
                self.peer.route_push(logits, x, ids_out, w_out, self.E, self.renorm, self.logits_bf16)
            self.peer.layer_local(tab, li, self.E, self.I, shared_ptr, self.shared, self.ws, self.limit)
            self.peer.combine(self.shared if shared_ptr else None, logits if (shared_ptr and gate_col >= 0) else None, max(gate_col, 0), out)
            return out
        if self.router == "sigmoid":
            ops.router_topk(logits[:, :self.E].contiguous() if logits.shape[1] != self.E else logits, self.bias, K, self.sigmoid_scale, ctx=self.ctx, ids=ids_out,
                            w=w_out)
        else:
            ops.router_softmax_topk(logits, K, self.renorm, self.logits_bf16, E=self.E, ids=ids_out, w=w_out, ctx=self.ctx)
        # pack [row | ids | w] per row (one kernel), one all-gather
        torch.cat([x.view(torch.uint8).view(B, H * 2), ids_out.view(torch.uint8).view(B, K * 4), w_out.view(torch.uint8).view(B, K * 4)], dim=1,
                  out=self.send[:, :H * 2 + K * 8])
        dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        # local experts over every rank's rows, read in place from the gathered buffer, and the (replicated) shared expert on the
        # local rows in the same pass
        ops.moe_decode_ep_local(self.ids_all, self.w_all, tab, li, self.E, self.x_all, H, self.I, self.part, shared_ptr=shared_ptr,
                                sh_row0=self.rank * B, sh_rows=B, shared_out=self.shared, limit=self.limit, ws=self.ws, ctx=self.ctx)
        if self.reduce_scatter:
            dist.reduce_scatter_tensor(self.routed, self.part, op=dist.ReduceOp.SUM, group=self.group)
        else:
            dist.all_reduce(self.part, op=dist.ReduceOp.SUM, group=self.group)
            self.routed.copy_(self.part[self.rank * B:(self.rank + 1) * B])
        if shared_ptr:
            ops.moe_combine(self.routed, self.shared, logits if gate_col >= 0 else None, gate_col if gate_col >= 0 else 0, out=out, ctx=self.ctx)
        else:
            ops.moe_combine(self.routed, torch.zeros_like(out), None, 0, out=out, ctx=self.ctx)
        return out

    def close(self):
        """Drops the mappings of the peers' exchange memory (peer transport).  Every rank calls it, with no exchange in flight."""
        if self.peer is not None:
            dist.barrier(group=self.group)
            self.peer.close()
            self.peer = None

    def local_records_touched(self, ids_all_sets) -> float:
        """Mean number of distinct local expert records (plus the shared copy) one layer call streams, from gathered ids."""
        lo, hi = expert_range(self.E, self.world, self.rank)
        n = []
        for ids in ids_all_sets:
            v = ids[(ids >= lo) & (ids < hi)]
            n.append(int(torch.unique(v).numel()) + 1)
        return float(sum(n)) / max(len(n), 1)


class ExpertParallelPrefill:
    """Expert-parallel prefill of one MoE layer: every rank holds T_local rows and the experts [r·E/G, (r+1)·E/G).

    exchange = "a2a": token dispatch and combine as two all-to-all-v exchanges.
        dispatch   a row goes ONCE to every rank that owns at least one of its k experts (de-duplicated per destination), as the
                   bf16 row plus its k ids and weights; the rows for one destination travel in row order
        experts    the grouped-GEMM operator (fn_moe_prefill) over the received rows with the local experts only (NULL table
                   entries: a row's pairs of experts held elsewhere contribute nothing) → one fp32 partial sum per received row
        combine    the partial sums travel back the way the rows came; the home rank adds them in rank order
      Per direction a rank moves (rows × distinct destination ranks) records instead of every row to every rank, and the
      operator pass works on the rows that have business on this rank, not on all G·T_local rows.  The split sizes of the
      exchanges are data-dependent: one small all-gather of the per-destination counts and one host read per layer.
    exchange = "allgather" (what "auto", the default, picks — see __init__): all-gather of rows, ids and weights → the operator over
      ALL G·T_local rows → reduce-scatter of the fp32 sums.

    Either way the routed sum of a row is a sum over ranks of per-rank sums in k order: it differs from the single-GPU sum by fp32
    reassociation only, and routing is unaffected."""

    def __init__(self, ops, ctx, H: int, I: int, E: int, K: int, T_local: int, world: int, rank: int, device, group=None, limit: float = 0.0,
                 exchange: str = "auto"):
        self.ops, self.ctx, self.H, self.I, self.E, self.K, self.T = ops, ctx, H, I, E, K, T_local
        if exchange == "auto":
            # The de-duplicated dispatch moves (1 - (1 - 1/G)^K) of what the all-gather moves under even routing (0.66 at 8 ranks and
            # top-8, 1.0 at 2 ranks), but its split sizes need a host read in the middle of the layer, which lets the GPU run dry.
            # Measured on 8 B200 over NVSwitch (T = 8192, H = 7168) the all-gather form is the faster one at 2 and at 8 ranks, so it is
            # what "auto" picks; "a2a" is the form for fabrics where the bytes, not the host read, are the cost.
            exchange = "allgather"
        self.world, self.rank, self.group, self.limit, self.exchange = world, rank, group, limit, exchange
        G = world
        cap = G * T_local                                               # a rank can receive every row of every rank at worst
        self.x_all = torch.empty((cap, H), dtype=torch.bfloat16, device=device)
        self.ids_all = torch.empty((cap, K), dtype=torch.int32, device=device)
        self.w_all = torch.empty((cap, K), dtype=torch.float32, device=device)
        self.part = torch.empty((cap, H), dtype=torch.float32, device=device)
        self.routed = torch.empty((T_local, H), dtype=torch.float32, device=device)
        self.reduce_scatter = dist.get_backend(group) != "gloo"
        ws_bytes = getattr(ops, "moe_prefill_ws_bytes", lambda s, k, e, h, i: 256)(cap, K, E, H, I)
        self.ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        if exchange == "a2a":
            # send side: at most T_local rows per destination
            self.sx = torch.empty((cap, H), dtype=torch.bfloat16, device=device)
            self.smeta = torch.empty((cap, 2 * K), dtype=torch.int32, device=device)
            self.rmeta = torch.empty((cap, 2 * K), dtype=torch.int32, device=device)
            self.back = torch.empty((cap, H), dtype=torch.float32, device=device)
            self.counts_all = torch.empty((G, G), dtype=torch.int64, device=device)
            # owner of expert e = the rank r with r·E//G ≤ e < (r+1)·E//G
            self.bounds = torch.tensor([(r + 1) * E // G for r in range(G - 1)], dtype=torch.int32, device=device)
        self.stats = {}

    def _dispatch_plan(self, ids):
        """(rows to send ordered by destination then row, counts per destination [G] on the device)."""
        G = self.world
        valid = (ids >= 0) & (ids < self.E)
        owner = torch.bucketize(ids, self.bounds, right=True)                       # [T, K] in [0, G)
        owner = torch.where(valid, owner, torch.full_like(owner, G))                # invalid ids go nowhere
        wants = torch.zeros((self.T, G + 1), dtype=torch.bool, device=ids.device)
        wants.scatter_(1, owner.long(), True)
        wants = wants[:, :G]
        # (destination, row) pairs that are wanted, in destination-then-row order, without a data-dependent shape (which would make
        # the host wait): a stable sort brings them to the front; the caller cuts the list at the total it reads with the counts
        order = torch.argsort((~wants.t().reshape(-1)).to(torch.uint8), stable=True)
        return order % self.T, wants.sum(0)

    def layer(self, ids, w, x, tab, li: int, shared=None, lg=None, col: int = 0, out=None):
        """ids int32 / w fp32 [T_local, K], x bf16 [T_local, H]: this rank's rows; tab: device table [L·E] of local record pointers.
        Returns fp32 routed sums [T_local, H], or with `shared` (bf16 [T_local, H]) the combined bf16 rows written to `out`."""
        ops, G, T, K = self.ops, self.world, self.T, self.K
        if self.exchange == "a2a":
            rows, counts = self._dispatch_plan(ids)
            dist.all_gather_into_tensor(self.counts_all.view(-1), counts, group=self.group)
            c = self.counts_all.cpu()                                               # the one host read of the layer: split sizes
            send = [int(v) for v in c[self.rank]]
            recv = [int(v) for v in c[:, self.rank]]
            ns, nr = sum(send), sum(recv)
            rows = rows[:ns]
            sx, smeta = self.sx[:ns], self.smeta[:ns]
            torch.index_select(x, 0, rows, out=sx)
            smeta[:, :K] = ids.index_select(0, rows)
            smeta[:, K:] = w.index_select(0, rows).view(torch.int32)
            xr, mr = self.x_all[:nr], self.rmeta[:nr]
            dist.all_to_all_single(xr, sx, recv, send, group=self.group)
            dist.all_to_all_single(mr, smeta, recv, send, group=self.group)
            part = self.part[:nr]
            if nr:
                self.ids_all[:nr] = mr[:, :K]
                self.w_all[:nr] = mr[:, K:].view(torch.float32)
                ops.fn_moe_prefill(tab, li, self.E, self.ids_all[:nr], self.w_all[:nr], xr, self.H, self.I, out=part, ws=self.ws, S=max(nr, 1), limit=self.limit,
                                   ctx=self.ctx)
            back = self.back[:ns]
            dist.all_to_all_single(back, part, send, recv, group=self.group)
            self.routed.zero_()
            o = 0
            for g in range(G):                                                      # rank order: the sum is the same on every run
                if send[g]:
                    self.routed.index_add_(0, rows[o:o + send[g]], back[o:o + send[g]])   # the rows of one destination are distinct
                o += send[g]
            self.stats = {"rows_sent": ns - send[self.rank], "rows_received": nr - recv[self.rank], "rows_local": send[self.rank],
                          "bytes_dispatch": (ns - send[self.rank]) * (self.H * 2 + K * 8), "bytes_combine": (ns - send[self.rank]) * self.H * 4}
        else:
            dist.all_gather_into_tensor(self.x_all, x.contiguous(), group=self.group)
            dist.all_gather_into_tensor(self.ids_all, ids.contiguous(), group=self.group)
            dist.all_gather_into_tensor(self.w_all, w.contiguous(), group=self.group)
            ops.fn_moe_prefill(tab, li, self.E, self.ids_all, self.w_all, self.x_all, self.H, self.I, out=self.part, ws=self.ws, S=G * T, limit=self.limit,
                               ctx=self.ctx)
            if self.reduce_scatter:
                dist.reduce_scatter_tensor(self.routed, self.part, op=dist.ReduceOp.SUM, group=self.group)
            else:
                dist.all_reduce(self.part, op=dist.ReduceOp.SUM, group=self.group)
                self.routed.copy_(self.part[self.rank * T:(self.rank + 1) * T])
            self.stats = {"rows_sent": (G - 1) * T, "rows_received": (G - 1) * T, "rows_local": T,
                          "bytes_dispatch": (G - 1) * T * (self.H * 2 + K * 8), "bytes_combine": (G - 1) * T * self.H * 4}
        if shared is None:
            return self.routed
        out = torch.empty((T, self.H), dtype=torch.bfloat16, device=x.device) if out is None else out
        ops.moe_combine(self.routed, shared, lg, col, out=out, ctx=self.ctx)
        return out
