#!/usr/bin/env python
"""Benchmark of the quantized routed-expert decode path (Qwen3-Next-shaped MoE, NVFP4 weights, bf16 activations).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload prefill [--tokens T]      one DeepSeek-shaped prefill MoE layer (tcgen05 FP4 grouped GEMM), FP4 roofline
    python bench.py --workload dense                     the dense 27B-style MLP GEMVs (NVFP4, 3-bit, 2-bit), HBM roofline
    python bench.py --workload records                   expert records assembled on the device from checkpoint-form tensors (compressed scales)

One "step" is one decode step of B tokens through the 48 MoE layers (router → routed NVFP4 experts → NVFP4 shared expert →
combine), each layer with its own weights, so a step streams ≈ 48 × U × 1.77 MB of distinct expert records (far more than the
126 MB L2).  The metric is MoE-layer tokens/s = B · layers / step time, whole job.  Printed: ONE JSON line.

  value        device-resident inputs, the 48 layers replayed from one CUDA graph, timed with CUDA events on the launching stream
  e2e          the same step through the Python mirror of the C ABI with pinned HOST inputs and outputs: H2D of logits and
               activations, the layers, D2H of the layer outputs, all inside the timed region
  roofline     the dominant kernel (gate/up weight stream): algorithmic bytes per launch ÷ its mean duration from the library's
               per-kernel event timing, against the measured HBM copy bandwidth of this pool
  cpu_baseline the reference engine's own CPU code (oracle/_ref, make_mat + matmul_multi in its CPU daemon's order) on the
               host cores, on a bounded sample (two layers' worth of experts), reported beside the GPU number
  --impl reference   times that CPU path alone with the same metric / unit / config

At N > 1 the experts of every layer are sharded over the ranks (expert parallel), each rank brings its own B tokens
(weak scaling): rows and routing go to every rank → local experts → the fp32 routed sums go to the row's rank → combine there.
The exchange runs in the library's own kernels over NVLink peer memory (HIVE_B200_EP=nccl: NCCL all-gather + reduce-scatter).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(H=2048, I=512, E=512, K=10, L=48, batches=(1, 4, 8, 16), headline_batch=16, sigma=0.02, seed=2)
WORKLOAD = "qwen3-next-shaped MoE decode: hidden 2048, 512 routed experts top-10 + 1 shared, intermediate 512, 48 layers, NVFP4 W4A16"


def rec_bytes(H, I):
    return 3 * H * I * 9 // 16 + 12


def layer_algorithmic_bytes(H, I, E, K, B, U):
    """Algorithmic bytes of one decode layer: U records (incl. the shared expert) + x + out + logits + ids/w."""
    return U * rec_bytes(H, I) + B * H * 2 + B * H * 2 + B * (E + 1) * 4 + B * K * 8


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and clock-event reasons through NVML (read-only) while `active` is set."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap", 0x80: "hw_power_brake",
               0x2: "applications_clocks_setting", 0x10: "sync_boost", 0x100: "display_clock_setting"}

    def __init__(self, uuid: str, index: int):
        self.samples, self.reasons, self.active, self._stop = [], set(), False, False
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.t = threading.Thread(target=self._run, daemon=True)
            self.t.start()
        except Exception as e:  # NVML missing: the line says so instead of inventing numbers
            self.nv = None
            self.err = str(e)

    def _run(self):
        nv = self.nv
        while not self._stop:
            if self.active:
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    for bit, name in self.REASONS.items():
                        if r & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(0.005)

    def result(self):
        self._stop = True
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": getattr(self, "err", "nvml unavailable")}
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz, "samples": len(self.samples),
                "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------------------ CPU reference arm
def cpu_reference(B: int, steps: int, warmup: int, budget_s: float | None, seed: int = 0):
    """Times the reference's CPU expert path (oracle/_ref) on a bounded sample: two layers' worth of expert records
    (2 × 513 × 1.77 MB ≈ 1.8 GB, beyond any L3), B tokens, routing from seeded N(0,1) logits.  Returns (tokens_per_s, info)."""
    os.environ.setdefault("FAKE_NUMA_NODES", "1")
    from oracle import oracle as O
    if not O.have_ref():
        O.build(ref=True)
    if not O.have_ref():
        raise RuntimeError("oracle/_ref/libhive_ref.so is not built and the reference tree is not present")
    H, I, E, K = CFG["H"], CFG["I"], CFG["E"], CFG["K"]
    n_layers = 2
    rng = np.random.default_rng(seed)
    pool = []
    for _ in range(8):                                            # 8 distinct quantized experts, replicated into distinct memory
        mats = [O.nvfp4_quantize(rng.normal(0, CFG["sigma"], sh).astype(np.float32), False) for sh in ((I, H), (I, H), (H, I))]
        pool.append(O.pack_record(H, I, *mats))
    R = O.ref()
    threads = int(R.ref_pool_threads())
    layers = []
    import ctypes as C
    off = O.rec_layout(H, I)
    for li in range(n_layers):
        recs = [pool[(li * 3 + e) % len(pool)] for e in range(E + 1)]
        layers.append(R.ref_layer_create(H, I, E + 1, C.cast(O._rec_ptrs(recs), C.POINTER(C.c_void_p)), O._ptr(off, O._u64p)))
    sets = []
    for s in range(4):
        logits = rng.normal(0, 1, (n_layers, B, E)).astype(np.float32)
        x = O.bf16r(rng.normal(0, 1, (n_layers, B, H)).astype(np.float32))
        routed = []
        for li in range(n_layers):
            ids, w = O.router_softmax_topk(logits[li], K, True, True, 1)
            ids = np.concatenate([ids, np.full((B, 1), E, np.int32)], axis=1)       # the shared expert: one more record, weight 1
            w = np.concatenate([w, np.ones((B, 1), np.float32)], axis=1)
            routed.append((np.ascontiguousarray(ids), np.ascontiguousarray(w)))
        sets.append((x, routed))
    acc = np.zeros((B, H), np.float32)

    def one_step(i):
        x, routed = sets[i % len(sets)]
        for li in range(n_layers):
            ids, w = routed[li]
            R.ref_layer_routed(layers[li], B, K + 1, O._ptr(ids, O._i32p), O._ptr(w, O._f32p), O._ptr(x[li], O._f32p), C.c_float(0.0), O._ptr(acc, O._f32p))

    t0 = time.perf_counter()
    one_step(0)
    t1 = time.perf_counter() - t0
    if budget_s is not None:
        steps = int(min(max(budget_s / max(t1, 1e-6), 3), 400))
        warmup = min(warmup, 2)
    for i in range(warmup):
        one_step(i)
    t0 = time.perf_counter()
    for i in range(steps):
        one_step(warmup + i)
    dt = time.perf_counter() - t0
    for h in layers:
        R.ref_layer_destroy(h)
    ms = dt / steps * 1e3
    value = B * n_layers / (dt / steps)
    u = float(np.mean([len(np.unique(r[0])) for _, routed in sets for r in routed]))
    info = {"value": value, "unit": "tokens/s", "cores": threads, "kind": "reference",
            "sample": f"{n_layers} layers x {E}+1 experts ({n_layers * (E + 1) * rec_bytes(H, I) / 1e9:.2f} GB of records, 8 distinct quantized experts "
                      f"replicated into distinct memory), B={B} tokens, {steps} timed passes after {warmup}; routed + shared experts via "
                      f"make_mat/matmul_multi (router and combine left out: <1% of the time)",
            "ms_per_layer": ms / n_layers, "weight_GBps": u * rec_bytes(H, I) / (ms / n_layers * 1e-3) / 1e9, "numa_nodes": int(R.ref_pool_nodes())}
    return value, ms, steps, warmup, info


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B = args.batch or CFG["headline_batch"]
    value, ms, steps, warmup, info = cpu_reference(B, args.steps, args.warmup, None)
    line = {"impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 accumulate over NVFP4 weights",
            "data": "synthetic", "config": {"workload": WORKLOAD, "batch_tokens": B, "step": "bounded sample: 2 of the 48 layers per step (see cpu_baseline.sample)"},
            "cpu_baseline": info, "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ GPU arm
class Layers:
    """All expert records of the model resident in HBM: [L, E_local + 1, record] (last = the shared expert), quantised on the device
    from seeded fp32 ~N(0, sigma) with the library's quantiser."""

    def __init__(self, E_mod, H, I, L, experts, sigma, seed, device):
        import torch
        self.lay = E_mod.ExpertRecLayout.make(H, I)
        self.n = len(experts) + 1                                      # local routed experts + shared
        self.buf = torch.empty((L, self.n, self.lay.total), dtype=torch.uint8, device=device)
        for li in range(L):
            for j in range(self.n):
                # seeded per (layer, global expert id): a rank's shard holds the same weights the single-GPU run has
                self.fill_record(E_mod, self.buf[li, j], H, I, li, experts[j] if j < len(experts) else self.SHARED_ID, sigma, seed)
        torch.cuda.synchronize()

    SHARED_ID = 10 ** 6

    @staticmethod
    def fill_record(E_mod, rec, H, I, li, gid, sigma, seed):
        """Writes the record of (layer li, global expert id gid) into `rec` (device uint8 of the record's size)."""
        import torch
        lay = E_mod.ExpertRecLayout.make(H, I)
        gen = torch.Generator(device=rec.device)
        gen.manual_seed(seed * 1000003 + li * 4099 + gid)
        w = torch.empty((3, H * I), dtype=torch.float32, device=rec.device)
        w.normal_(0.0, sigma, generator=gen)
        g = rec[lay.g:lay.g + 12].view(torch.float32)
        for m, (ow, osc, shape) in enumerate(((lay.w1, lay.s1, (I, H)), (lay.w3, lay.s3, (I, H)), (lay.w2, lay.s2, (H, I)))):
            N_, K_ = shape
            E_mod.nvfp4_quantize(w[m].view(N_, K_), q=rec[ow:ow + N_ * K_ // 2], s=rec[osc:osc + N_ * K_ // 16], g=g[m:m + 1])

    def ptr(self, li, j):
        return self.buf[li, j].data_ptr()


def parity_check(E_mod, torch, H, I, Ex, K, L, B, logits, x, ids, out, n_rows=2):
    """Rows 0 and B-1 of the first and the last layer of input set 0, after the timed runs: the routing the device produced against the
    oracle's router, and the layer outputs against the oracle's layer on the same logits and activations, with the experts those rows
    touch regenerated from their seeds.  Returns {ids_equal, max_err_x_rms, rows, layers}; the caller fails the run above 2e-2."""
    from oracle import oracle as O
    rows = sorted({0, B - 1})[:n_rows]
    worst, beyond, ids_equal = 0.0, 0.0, True
    layers = sorted({0, L - 1})
    for li in layers:
        lg = logits[0, li][rows].float().cpu().numpy()
        xr = x[0, li][rows].float().cpu().numpy()
        rids, _ = O.router_softmax_topk(lg[:, :Ex], K, True, True, 0, E=Ex)
        ids_equal = ids_equal and bool(np.array_equal(rids, ids[0, li][rows].cpu().numpy()))
        lay = E_mod.ExpertRecLayout.make(H, I)
        tab = [None] * Ex
        scratch = torch.empty(lay.total, dtype=torch.uint8, device=x.device)
        for gid in sorted(set(int(v) for v in rids.ravel())) + [Layers.SHARED_ID]:
            scratch.zero_()
            Layers.fill_record(E_mod, scratch, H, I, li, gid, CFG["sigma"], CFG["seed"])
            rec = scratch.cpu().numpy().copy()
            if gid == Layers.SHARED_ID:
                shared = rec
            else:
                tab[gid] = rec
        _, _, ref = O.moe_layer(H, I, lg, xr, tab, K, shared_rec=shared, gate_logits=lg, gate_col=Ex)
        ref = O.bf16_to_f32(ref).astype(np.float64)
        got = out[0, li][rows].float().cpu().numpy().astype(np.float64)
        rms = np.sqrt(np.mean(ref ** 2, axis=-1)) + 1e-30
        diff = np.abs(got - ref)
        worst = max(worst, float(np.max(np.max(diff, axis=-1) / rms)))
        # The outputs are bf16 by the operator's contract: where the fp32 sums differ only by their order (sharded runs add per-rank sums),
        # a result may land on the neighbouring bf16 value, and one bf16 step of a 4-sigma element is already 1.6-3 % of the row RMS.
        # `beyond` is what is left of the difference after one such step of the reference value.
        step = np.where(ref != 0, 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 1e-300))) - 7), 0.0)
        beyond = max(beyond, float(np.max(np.max(np.maximum(diff - step, 0.0), axis=-1) / rms)))
    return {"ids_equal": ids_equal, "max_err_x_rms": worst, "max_err_beyond_one_bf16_step_x_rms": beyond, "rows": rows, "layers": layers, "bar": 2e-2,
            "what": "device routing vs the oracle router; layer outputs (bf16) vs the CPU oracle's layer on the same inputs, touched experts regenerated "
                    "from their seeds; ok = routing equal and the error beyond one bf16 step of the reference value within the bar"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    import eke_hive_b200 as E
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    t_start = time.perf_counter()

    def trace(msg):
        """Progress lines on stderr when BENCH_TRACE is set (stdout stays one JSON line)."""
        if os.environ.get("BENCH_TRACE"):
            print(f"[bench r{rank} +{time.perf_counter() - t_start:6.1f}s] {msg}", file=sys.stderr, flush=True)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        trace("process group up")
    H, I, Ex, K, L = CFG["H"], CFG["I"], CFG["E"], CFG["K"], args.layers or CFG["L"]
    ctx = E.context()
    sampler = ClockSampler(str(torch.cuda.get_device_properties(local).uuid), local)

    if world > 1:
        from eke_hive_b200.ep import ExpertParallelMoE
        e_lo, e_hi = rank * Ex // world, (rank + 1) * Ex // world
        experts = list(range(e_lo, e_hi))
    else:
        experts = list(range(Ex))
    t_setup = time.perf_counter()
    layers = Layers(E, H, I, L, experts, CFG["sigma"], CFG["seed"], dev)
    n_loc = len(experts)
    # per-layer device tables of record pointers (global expert id → record or 0) and the shared record
    tab_host = np.zeros((L, Ex), np.int64)
    for li in range(L):
        for j, gid in enumerate(experts):
            tab_host[li, gid] = layers.ptr(li, j)
    tab = torch.from_numpy(tab_host.reshape(-1)).to(dev)
    shared_ptr = [layers.ptr(li, n_loc) for li in range(L)]
    setup_s = time.perf_counter() - t_setup
    trace(f"weights ready in {setup_s:.1f}s")

    results = {}
    batches = [args.batch] if args.batch else list(CFG["batches"])
    head_B = args.batch or CFG["headline_batch"]
    NSETS = 2
    gen = torch.Generator(device=dev)
    gen.manual_seed(CFG["seed"] * 7919 + rank)
    for B in batches:
        logits = torch.randn((NSETS, L, B, Ex + 1), dtype=torch.float32, device=dev, generator=gen)     # column E: shared-expert gate logit
        x = torch.randn((NSETS, L, B, H), dtype=torch.float32, device=dev, generator=gen).to(torch.bfloat16)
        out = torch.empty((NSETS, L, B, H), dtype=torch.bfloat16, device=dev)         # one output buffer per input set (the copies of a step overlap the next step)
        ids = torch.empty((NSETS, L, B, K), dtype=torch.int32, device=dev)
        wts = torch.empty((NSETS, L, B, K), dtype=torch.float32, device=dev)
        if world > 1:
            ep = ExpertParallelMoE(E, ctx, H, I, Ex, K, B, world, rank, dev)
            ep_transport = ep.transport + (" (library kernels over NVLink peer memory, no collective library)" if ep.transport == "peer" else " (all-gather + reduce-scatter)")

            def run_layers(s):
                for li in range(L):
                    ep.layer(logits[s, li], x[s, li], tab, li, shared_ptr[li], Ex, ids[s, li], wts[s, li], out[s, li])
        else:
            ws = torch.empty(E.moe_decode_ws_bytes(B * (K + 1), H, I), dtype=torch.uint8, device=dev)

            def run_layers(s):
                for li in range(L):
                    E.moe_layer_decode(logits[s, li], x[s, li], tab, li, Ex, K, H, I, shared_rec=shared_ptr[li], gate_col=Ex, ids=ids[s, li],
                                       w=wts[s, li], out=out[s, li], ws=ws, ctx=ctx)
        # warm every kernel once outside capture, then one graph per input set
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graphs = []
        with torch.cuda.stream(side):
            run_layers(0)
            side.synchronize()
            trace(f"B={B}: eager pass done")
            n0 = ctx.launches
            for s in range(NSETS):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    run_layers(s)
                graphs.append(g)
            launches_per_step = (ctx.launches - n0) // NSETS
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        trace(f"B={B}: graphs captured")

        def timed(nsteps, fn, finish=None):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(nsteps + 1)] if finish is None else None
            e0.record()
            for i in range(nsteps):
                if marks:
                    marks[i].record()
                fn(i)
            if marks:
                marks[nsteps].record()
            if finish:
                finish()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if marks:                                            # the spread over the timed steps (events between the steps cost nothing on the device)
                per = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(nsteps))
                timed.spread = {"min_ms": per[0], "median_ms": per[len(per) // 2], "max_ms": per[-1]}
            if world > 1:
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

        for i in range(args.warmup):
            graphs[i % NSETS].replay()
        sampler.active = B == head_B
        ms = timed(args.steps, lambda i: graphs[i % NSETS].replay())
        spread_B = getattr(timed, "spread", None)
        sampler.active = False
        ctx.check_device()
        ms_step = ms / args.steps
        trace(f"B={B}: timed {ms_step:.3f} ms/step")
        ids_h = ids.cpu().numpy()
        U = np.array([[len(np.unique(ids_h[s, li])) + 1 for li in range(L)] for s in range(NSETS)], np.float64)   # + shared
        if world > 1:
            # records streamed per layer, summed over ranks: each rank's distinct local experts over the gathered batch + its shared copy
            ids_g = torch.empty((world,) + tuple(ids.shape), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(ids_g, ids.contiguous())
            ids_g = ids_g.permute(1, 2, 0, 3, 4).reshape(NSETS * L, -1)
            u_loc = ep.local_records_touched([ids_g[j] for j in range(ids_g.shape[0])])
            t = torch.tensor([u_loc], dtype=torch.float64, device=dev); dist.all_reduce(t); u_total = float(t.item())
        else:
            u_total = float(U.mean())
        bytes_step = L * layer_algorithmic_bytes(H, I, Ex, K, B * world, u_total)
        results[B] = {"batch": B, "ms_per_step": ms_step, "us_per_layer": ms_step * 1e3 / L, "tokens_per_s": B * world * L / (ms_step * 1e-3),
                      "records_per_layer": u_total, "algorithmic_GB_per_step": bytes_step / 1e9, "achieved_GBps": bytes_step / (ms_step * 1e-3) / 1e9,
                      "launches_per_step": launches_per_step, "step_spread": spread_B}

        if B == head_B:
            # ---- end to end: pinned host inputs → H2D → layers → D2H of the outputs, every step
            hl = [torch.randn((L, B, Ex + 1), dtype=torch.float32).pin_memory() for _ in range(NSETS)]
            hx = [torch.randn((L, B, H), dtype=torch.float32).to(torch.bfloat16).pin_memory() for _ in range(NSETS)]
            hout = [torch.empty((L, B, H), dtype=torch.bfloat16).pin_memory() for _ in range(NSETS)]
            # Every step copies its inputs from pinned host memory and its outputs back, inside the timed region.  The copies run on a
            # second stream so that step i+1's upload and step i's download overlap step i's / i+1's compute (two input sets, two
            # output buffers); events order upload → compute → download per set, and the timed region ends only when the last
            # download has finished.
            main, cps = torch.cuda.current_stream(), torch.cuda.Stream()
            up = [torch.cuda.Event() for _ in range(NSETS)]; comp = [torch.cuda.Event() for _ in range(NSETS)]; down = [torch.cuda.Event() for _ in range(NSETS)]

            def upload(s):
                with torch.cuda.stream(cps):
                    cps.wait_event(comp[s])                          # the previous compute on this set has read its inputs
                    logits[s].copy_(hl[s], non_blocking=True)
                    x[s].copy_(hx[s], non_blocking=True)
                    up[s].record(cps)

            def e2e_step(i):
                s = i % NSETS
                main.wait_event(up[s])                               # this step's inputs are on the device
                main.wait_event(down[s])                             # the previous results of this set have left its output buffer
                graphs[s].replay()
                comp[s].record(main)
                upload((i + 1) % NSETS)                              # next step's inputs, while this step computes
                with torch.cuda.stream(cps):
                    cps.wait_event(comp[s])
                    hout[s].copy_(out[s], non_blocking=True)
                    down[s].record(cps)

            def e2e_finish():
                main.wait_stream(cps)

            for s0 in range(NSETS):
                comp[s0].record(main); down[s0].record(main)
            upload(0)
            for i in range(max(3, args.warmup)):
                e2e_step(i)
            torch.cuda.synchronize()
            sampler.active = True
            ms_e = timed(args.steps, e2e_step, e2e_finish) / args.steps
            sampler.active = False
            e2e = {"value": B * world * L / (ms_e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e,
                   "h2d_bytes_per_step": hl[0].numel() * 4 + hx[0].numel() * 2, "d2h_bytes_per_step": hout[0].numel() * 2,
                   "overlap": "copies on a second stream: step i+1's upload and step i's download overlap compute; all inside the timed region"}
            # ---- per-kernel durations (library event pairs, PDL off, no graph) for the roofline of the dominant kernel
            prof = None
            if world == 1 or os.environ.get("BENCH_PROFILE_EP"):
                ctx.profile(True)
                nprof = max(1, min(args.steps, 8192 // (launches_per_step + 1)))
                for i in range(nprof):
                    run_layers(i % NSETS)
                prof = ctx.profile_read()
                ctx.profile(False)
                prof = {k: {"launches": v[0], "total_ms": v[1], "mean_us": v[1] * 1e3 / max(v[0], 1)} for k, v in prof.items()}
        if B == head_B:
            # ---- correctness of what was timed, outside every timed region: one more replay of set 0, then sampled rows against the CPU oracle
            graphs[0].replay()
            torch.cuda.synchronize()
            ctx.check_device()
            parity = parity_check(E, torch, H, I, Ex, K, L, B, logits, x, ids, out)
            first = out[0].clone()
            graphs[0].replay()
            torch.cuda.synchronize()
            parity["run_to_run_equal"] = bool(torch.equal(first, out[0]))      # the same graph on the same inputs: the same bits
            if not parity["run_to_run_equal"]:
                parity["run_to_run_max_diff_x_rms"] = float(((first.float() - out[0].float()).abs().max() / (out[0].float().pow(2).mean().sqrt() + 1e-30)).item())
            if world > 1:
                t = torch.tensor([parity["max_err_x_rms"], 0.0 if parity["ids_equal"] else 1.0, parity["max_err_beyond_one_bf16_step_x_rms"]], dtype=torch.float64,
                                 device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                parity["max_err_x_rms"] = float(t[0].item()); parity["ids_equal"] = bool(t[1].item() == 0.0); parity["ranks_checked"] = world
                parity["max_err_beyond_one_bf16_step_x_rms"] = float(t[2].item())
                t2 = torch.tensor([0.0 if parity["run_to_run_equal"] else 1.0], dtype=torch.float64, device=dev)
                dist.all_reduce(t2, op=dist.ReduceOp.MAX)
                parity["run_to_run_equal"] = bool(t2.item() == 0.0)
            parity["ok"] = bool(parity["ids_equal"] and parity["run_to_run_equal"] and parity["max_err_beyond_one_bf16_step_x_rms"] <= parity["bar"])
        if world > 1:
            torch.cuda.synchronize()
            ep.close()
        del logits, x, out, ids, wts, graphs, g
        torch.cuda.empty_cache()

    head = results[head_B]
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured copy bandwidth of this pool (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s (earlier measurement on this pool)"
    roofline = None
    gu_key = "moe_gate_up_tc" if prof and "moe_gate_up_tc" in prof else "moe_gate_up"
    if world == 1 and prof and gu_key in prof:
        U = head["records_per_layer"]
        gu_bytes = U * (2 * H * I * 9 // 16) + head_B * H * 2                     # gate+up halves of U records + the activation rows
        ach = gu_bytes / (prof[gu_key]["mean_us"] * 1e-6) / 1e9
        gu_label = ("moe_gate_up_tc (moe_dtc_layer_kernel, gate/up form: tcgen05 block-scaled FP4 MMAs over digit planes of the activations)"
                    if gu_key == "moe_gate_up_tc" else "moe_gate_up (moe_stream_kernel<8,1,false>)")
        roofline = {"bound": "hbm", "kernel": gu_label, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "peak_source": peak_src, "traffic": gu_bytes, "traffic_source": "algorithmic (an ncu capture of this kernel on a 4-layer case read 1.018 x algorithmic DRAM bytes; not measured in this run)", "algorithmic_bytes_per_launch": gu_bytes, "mean_us": prof[gu_key]["mean_us"]}
    clocks = sampler.result()
    line = {"metric": "moe_layer_tokens_per_s", "value": head["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e2m1·e4m3 weights x bf16 activations, exact products (gate/up: FP4 MMAs over base-8 digit planes of the activations; down: f16 mma.sync), f32 accumulate",
            "data": "synthetic", "config": {"workload": WORKLOAD, "batch_tokens_per_gpu": head_B, "layers": L,
                                            "l2": "inputs larger than L2: every step streams %.1f GB of distinct expert records" % head["algorithmic_GB_per_step"],
                                            "parallelism": "single GPU" if world == 1 else f"expert-parallel ep{world}: experts sharded, rows+routing gathered, fp32 sums sent to the row's rank; transport: {ep_transport}"},
            "layer": {"achieved_GBps": head["achieved_GBps"], "frac_of_measured_hbm": head["achieved_GBps"] / world / peak, "us_per_layer": head["us_per_layer"],
                      "records_per_layer": head["records_per_layer"]},
            "per_batch": [results[b] for b in sorted(results)], "roofline": roofline, "e2e": e2e, "gpu_launches": head["launches_per_step"] * args.steps,
            "clocks": clocks, "kernels": prof, "setup_s": setup_s, "parity": parity}
    if not args.batch and not args.layers and not args.no_extras:
        # the other workloads the path is judged on, each a bounded measurement with its own sampled-row check: the GLM-shaped decode
        # layer (strong scaling, skewed routing) and the DeepSeek-shaped prefill layer at every N, the dense low-bit GEMVs at N = 1
        del layers, tab
        torch.cuda.empty_cache()
        from oracle import oracle as O
        per_config = {}
        trace("extras: glm")
        per_config["glm_b8_zipf"] = glm_measure(args, torch, dist, E, O, ctx, dev, rank, world)
        trace("extras: prefill")
        pa = argparse.Namespace(**vars(args)); pa.steps = 5; pa.warmup = 3
        pl, prc = prefill_measure(pa, torch, dist, E, O, ctx, dev, rank, world, with_dense=(world == 1))
        per_config["prefill_t8192"] = {k: pl.get(k) for k in ("value", "unit", "ms_per_layer", "layer_TFLOPs", "scaling", "config", "roofline", "roofline_hbm", "exchange",
                                                              "parity", "w4a4_vs_w4a16", "w4a16", "dense_gemm_a4", "kernels")}
        line["per_config"] = per_config
        line["prefill"] = {"tokens_per_s": pl["value"], "ms_per_layer": pl["ms_per_layer"], "frac_of_measured_fp4_peak": pl["roofline"]["frac"],
                           "peak_TFLOPs": pl["roofline"]["peak"], "dense_gemm_a4": pl.get("dense_gemm_a4"), "parity_ok": pl["parity"]["ok"]}
        if pl.get("w4a16"):
            w16 = pl["w4a16"]      # the same layer with bf16 activations (the reference's default prefill arithmetic) on the kind::f16 grouped GEMM
            line["prefill"]["w4a16"] = {"tokens_per_s": w16["tokens_per_s"], "ms_per_layer": w16["ms_per_layer"], "frac_of_measured_bf16_peak": w16["roofline"]["frac"],
                                        "peak_TFLOPs": w16["roofline"]["peak"], "parity_ok": w16["parity"]["ok"], "max_err_x_rms": w16["parity"]["max_err_x_rms"]}
        if world == 1:
            trace("extras: dense")
            da = argparse.Namespace(**vars(args)); da.steps = 20
            dl = dense_measure(da, torch, E, ctx, dev)
            line["dense"] = {"per_case": dl["per_case"], "roofline": dl["roofline"]}
        if not (per_config["glm_b8_zipf"].get("parity", {"ok": True})["ok"] and pl["parity"]["ok"]):
            parity["ok"] = False
    if world == 1 and not args.no_cpu:
        try:
            _, _, _, _, info = cpu_reference(head_B, 0, 1, args.cpu_budget)
            line["cpu_baseline"] = info
        except Exception as ex:  # the reference library was never built on this machine
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "reference", "sample": f"unavailable: {ex}"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    rc = 0 if parity["ok"] else 3                                     # a run whose sampled rows miss the oracle fails
    if world > 1:
        # Tearing down an NCCL communicator waits for every CUDA graph that captured its collectives to be destroyed, and a graph
        # that is still referenced somewhere makes that wait endless.  Release what this function holds, and do not let the
        # teardown outlive a short grace period: the result is printed, the process may simply exit.
        dist.barrier()
        torch.cuda.synchronize()
        g = graphs = ep = run_layers = e2e_step = None
        import gc
        gc.collect()
        threading.Timer(20.0, lambda: os._exit(rc)).start()
        try:
            dist.destroy_process_group()
        finally:
            sys.stdout.flush()
            os._exit(rc)
    if rc:
        sys.exit(rc)


# ------------------------------------------------------------------------------------------------ side workloads (one GPU)
def _timed(torch, fn, n):
    fn(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def glm_measure(args, torch, dist, E, O, ctx, dev, rank, world):
    """The GLM-shaped decode workload, strong scaling: hidden 4096, 160 routed experts top-8 + 1 shared, intermediate 1536, 8 tokens per
    step IN ALL (8 / N per rank), sigmoid router over N(0,1) logits plus a per-expert Zipf(1.1) log-weight bias (hot experts), clamp
    10.  Experts are sharded over the ranks; 6 layers' records (larger than L2) are cycled.  Returns a dict for the bench line."""
    H, I, Ex, K, L, Btot, scale, limit = 4096, 1536, 160, 8, 6, 8, 2.5, 10.0
    if Btot % world:
        return {"skipped": f"{Btot} rows do not split over {world} ranks"}
    B = Btot // world
    e_lo, e_hi = rank * Ex // world, (rank + 1) * Ex // world
    experts = list(range(e_lo, e_hi))
    layers = Layers(E, H, I, L, experts, CFG["sigma"], CFG["seed"] + 3, dev)
    n_loc = len(experts)
    tab_host = np.zeros((L, Ex), np.int64)
    for li in range(L):
        for j, gid in enumerate(experts):
            tab_host[li, gid] = layers.ptr(li, j)
    tab = torch.from_numpy(tab_host.reshape(-1)).to(dev)
    shared_ptr = [layers.ptr(li, n_loc) for li in range(L)]
    rng = np.random.default_rng(11)                                   # the same global batch on every rank
    zipf = 1.0 / np.arange(1, Ex + 1) ** 1.1
    bias_h = np.log(zipf / zipf.sum())[rng.permutation(Ex)].astype(np.float32)
    bias = torch.from_numpy(bias_h).to(dev)
    NS = 2
    lg_all = rng.normal(0, 1, (NS, L, Btot, Ex)).astype(np.float32)
    x_all = O.bf16r(rng.normal(0, 1, (NS, L, Btot, H)).astype(np.float32))
    sl = slice(rank * B, (rank + 1) * B)
    logits = torch.from_numpy(lg_all[:, :, sl].copy()).to(dev)
    x = torch.from_numpy(x_all[:, :, sl].copy()).to(torch.bfloat16).to(dev)
    out = torch.empty((NS, L, B, H), dtype=torch.bfloat16, device=dev)
    ids = torch.empty((NS, L, B, K), dtype=torch.int32, device=dev); wts = torch.empty((NS, L, B, K), dtype=torch.float32, device=dev)
    ep = None
    if world > 1:
        from eke_hive_b200.ep import ExpertParallelMoE
        ep = ExpertParallelMoE(E, ctx, H, I, Ex, K, B, world, rank, dev, limit=limit, router="sigmoid", bias=bias, sigmoid_scale=scale)

        def run_layers(s):
            for li in range(L):
                ep.layer(logits[s, li], x[s, li], tab, li, shared_ptr[li], -1, ids[s, li], wts[s, li], out[s, li])
    else:
        ws = torch.empty(E.moe_decode_ws_bytes(B * (K + 1), H, I), dtype=torch.uint8, device=dev)

        def run_layers(s):
            for li in range(L):
                E.moe_layer_decode(logits[s, li], x[s, li], tab, li, Ex, K, H, I, shared_rec=shared_ptr[li], gate_col=-1, bias=bias, sigmoid_scale=scale,
                                   limit=limit, ids=ids[s, li], w=wts[s, li], out=out[s, li], ws=ws, ctx=ctx)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graphs = []
    with torch.cuda.stream(side):
        run_layers(0)
        side.synchronize()
        for s_ in range(NS):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                run_layers(s_)
            graphs.append(g)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for i in range(4):
        graphs[i % NS].replay()
    if world > 1:
        dist.barrier()
    it = [0]

    def step():
        graphs[it[0] % NS].replay(); it[0] += 1
    ms = _timed(torch, step, max(args.steps, 10))
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
    ctx.check_device()
    # parity: this rank's first row of layer 0 and last row of the last layer against the CPU oracle's whole layer (experts remade from seeds)
    graphs[0].replay(); torch.cuda.synchronize()
    lay = E.ExpertRecLayout.make(H, I)
    tmp = torch.empty(lay.total, dtype=torch.uint8, device=dev)
    err, raw, ids_ok = 0.0, 0.0, True
    for li, m in ((0, 0), (L - 1, B - 1)):
        lg_r = logits[0, li, m:m + 1].cpu().numpy(); x_r = x[0, li, m:m + 1].float().cpu().numpy()
        rid, rw = O.router_sigmoid_topk(lg_r, bias_h, K, scale)
        ids_ok = ids_ok and bool(np.array_equal(rid, ids[0, li, m:m + 1].cpu().numpy()))
        recs = [None] * Ex
        for e in sorted(set(int(v) for v in rid.reshape(-1))):
            Layers.fill_record(E, tmp, H, I, li, e, CFG["sigma"], CFG["seed"] + 3); recs[e] = tmp.cpu().numpy().copy()
        Layers.fill_record(E, tmp, H, I, li, Layers.SHARED_ID, CFG["sigma"], CFG["seed"] + 3); shared = tmp.cpu().numpy().copy()
        _, _, ref = O.moe_layer(H, I, lg_r, x_r, recs, K, shared_rec=shared, router="sigmoid", bias=bias_h, scale=scale, limit=limit)
        ref = O.bf16_to_f32(ref)[0].astype(np.float64); got = out[0, li, m].float().cpu().numpy().astype(np.float64)
        step = np.where(ref != 0, 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 1e-300))) - 7), 0.0)      # one bf16 step of the reference value (see parity_check)
        raw = max(raw, float(np.abs(got - ref).max() / (np.sqrt((ref ** 2).mean()) + 1e-30)))
        err = max(err, float(np.maximum(np.abs(got - ref) - step, 0.0).max() / (np.sqrt((ref ** 2).mean()) + 1e-30)))
    # load balance: pairs per rank of the global batch, records each rank streams per layer
    gid, _ = O.router_sigmoid_topk(lg_all.reshape(-1, Ex), bias_h, K, scale)
    gid = gid.reshape(NS * L, Btot * K)
    bounds = [(r + 1) * Ex // world for r in range(world)]
    owner = np.searchsorted(bounds, gid, side="right")
    ppr = np.array([(owner == r).sum() for r in range(world)], np.float64) / (NS * L)
    rec_r = np.array([np.mean([len(np.unique(row[(owner[j] == r)])) for j, row in enumerate(gid)]) + 1 for r in range(world)])   # + the shared copy
    us_layer = ms * 1e3 / L
    rec_bytes_ = 3 * H * I * 9 // 16
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    res = {"workload": "glm-shaped MoE decode: hidden 4096, 160 routed experts top-8 + shared, intermediate 1536, 8 tokens per step in all, sigmoid router + Zipf(1.1) bias",
           "scaling": "strong", "n_gpus": world, "rows_per_rank": B, "us_per_layer": us_layer, "tokens_per_s": Btot / (us_layer * 1e-6),
           "records_per_rank_per_layer_max": float(rec_r.max()), "records_per_rank_per_layer_mean": float(rec_r.mean()),
           "achieved_GBps_per_gpu_max": float(rec_r.max()) * rec_bytes_ / (us_layer * 1e-6) / 1e9, "frac_of_measured_hbm_busiest_gpu": float(rec_r.max()) * rec_bytes_ / (us_layer * 1e-6) / 1e9 / peak,
           "pairs_per_rank_max": float(ppr.max()), "pairs_per_rank_mean": float(ppr.mean()),
           "transport": ep.transport if ep is not None else "single GPU",
           "parity": {"ids_equal": ids_ok, "max_err_x_rms": raw, "max_err_beyond_one_bf16_step_x_rms": err, "bar": 2e-2, "ok": bool(ids_ok and err <= 2e-2)}}
    if world > 1:
        t = torch.tensor([err, 0.0 if ids_ok else 1.0, raw], dtype=torch.float64, device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["parity"] = {"ids_equal": bool(t[1].item() == 0.0), "max_err_x_rms": float(t[2].item()), "max_err_beyond_one_bf16_step_x_rms": float(t[0].item()),
                         "bar": 2e-2, "ranks_checked": world, "ok": bool(t[1].item() == 0.0 and t[0].item() <= 2e-2)}
        torch.cuda.synchronize()
        ep.close()
    del graphs, layers
    torch.cuda.empty_cache()
    return res


def run_prefill(args):
    """--workload prefill: the DeepSeek-shaped prefill layer alone, its own JSON line (see prefill_measure)."""
    import torch
    import torch.distributed as dist
    import eke_hive_b200 as E
    from oracle import oracle as O                                     # the checker of the sampled rows, outside the timed region
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line, rc = prefill_measure(args, torch, dist, E, O, E.context(), dev, rank, world)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()
    return rc


def prefill_measure(args, torch, dist, E, O, ctx, dev, rank, world, with_dense=True):
    """The DeepSeek-shaped prefill workload: one MoE layer, H 7168, I 2048, 256 routed experts (5.6 GB), top-8, T tokens, NVFP4
    weights and NVFP4 activations; plus a dense W4A4 GEMM and the measured FP4 tensor-pipe ceiling.  With N > 1 ranks the experts are
    sharded over the ranks and every rank brings T / N tokens (strong scaling on the same total problem); rows travel by all-to-all-v
    dispatch and combine (eke_hive_b200/ep.py).  Returns (JSON line as a dict, return code)."""
    H, I, Ex, K, T = 7168, 2048, args.experts, 8, args.tokens
    assert Ex % world == 0 and T % world == 0
    peak = E.fp4_peak_probe(8192)
    rb = E.ExpertRecLayout.make(H, I)
    e_lo, e_hi = rank * Ex // world, (rank + 1) * Ex // world
    n_loc = e_hi - e_lo
    def fill_expert(rec, e):
        """The record of global expert e, the same bytes on whichever rank makes it: e2m1 codes are any bytes, e4m3 scales 2^-2 .. 2."""
        gg = torch.Generator(device=dev); gg.manual_seed(90001 + e)
        rec.copy_(torch.randint(0, 256, (rb.total,), dtype=torch.uint8, device=dev, generator=gg))
        for off, n in ((rb.s1, I * H // 16), (rb.s3, I * H // 16), (rb.s2, H * I // 16)):
            rec[off:off + n] = torch.randint(0x28, 0x48, (n,), dtype=torch.uint8, device=dev, generator=gg)
        rec[rb.g:rb.g + 12] = torch.from_numpy(np.array([0.003, 0.003, 0.004], np.float32).view(np.uint8)).to(dev)
    blob = torch.empty((n_loc, rb.total), dtype=torch.uint8, device=dev)
    for e in range(e_lo, e_hi):
        fill_expert(blob[e - e_lo], e)
    tab = torch.tensor([blob[e - e_lo].data_ptr() if e_lo <= e < e_hi else 0 for e in range(Ex)], dtype=torch.int64, device=dev)
    g = torch.Generator(device=dev); g.manual_seed(4 + rank)
    Tl = T // world
    sets = []
    for _ in range(2):
        logits = torch.randn((Tl, Ex), device=dev, generator=g)
        w, ids = torch.topk(torch.softmax(logits, -1), K)
        sets.append((ids.to(torch.int32).contiguous(), w.contiguous(), torch.randn((Tl, H), device=dev, generator=g).to(torch.bfloat16)))
    it = [0]
    if world == 1:
        ws = torch.empty(E.moe_prefill_ws_bytes(T, K, Ex, H, I), dtype=torch.uint8, device=dev)
        out = torch.empty((T, H), dtype=torch.float32, device=dev)

        def layer():
            ids, w, x = sets[it[0] % 2]; it[0] += 1
            E.fn_moe_prefill(tab, 0, Ex, ids, w, x, H, I, out=out, ws=ws, S=T, ctx=ctx)
    else:
        from eke_hive_b200.ep import ExpertParallelPrefill
        epp = ExpertParallelPrefill(E, ctx, H, I, Ex, K, Tl, world, rank, dev, exchange=os.environ.get("HIVE_B200_PF_EXCHANGE", "auto"))

        def layer():
            ids, w, x = sets[it[0] % 2]; it[0] += 1
            epp.layer(ids, w, x, tab, 0)
    for _ in range(max(args.warmup, 3)):
        layer()
    if world > 1:
        dist.barrier()
    ms = _timed(torch, layer, args.steps)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms = float(t.item())
    ctx.profile(True); layer(); layer(); prof = ctx.profile_read(); ctx.profile(False)
    ctx.check_device()
    prof = {k: {"launches": v[0], "mean_us": v[1] * 1e3 / max(v[0], 1)} for k, v in prof.items()}
    flops = 2.0 * T * K * 3 * H * I
    gemm_us = prof["pf_gemm_gu"]["mean_us"] + prof["pf_gemm_down"]["mean_us"]
    line = {"metric": "moe_prefill_layer_tokens_per_s", "value": T / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "ms_per_layer": ms,
            "dtype": "e2m1 x e2m1 with ue4m3 block scales, f32 accumulate", "data": "synthetic", "scaling": "strong",
            "config": {"workload": f"deepseek-shaped MoE prefill layer: hidden 7168, {Ex} routed experts top-8, intermediate 2048, T={T}, NVFP4 W4A4",
                       "l2": f"{Ex * rb.total / 1e9:.1f} GB of expert records per layer (larger than L2)",
                       "parallelism": "single GPU" if world == 1 else f"expert-parallel ep{world}: experts sharded, tokens exchanged by {epp.exchange} (NCCL)"},
            "layer_TFLOPs": flops / (ms * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "kernel": "pf_gemm_kernel (gate/up + down), this rank's share", "achieved": flops / world / (gemm_us * 1e-6) / 1e12, "peak": peak,
                         "unit": "TFLOP/s", "frac": flops / world / (gemm_us * 1e-6) / 1e12 / peak,
                         "peak_source": "hb_fp4_peak_probe on this GPU (dense FP4, resident operands)", "traffic": None},
            "kernels": prof}
    if world > 1:
        # pairs per rank (load balance) and what the exchange moved and cost on this rank
        owner = torch.bucketize(sets[0][0], torch.tensor([(r + 1) * Ex // world for r in range(world - 1)], dtype=torch.int32, device=dev), right=True)
        ppr = torch.bincount(owner.reshape(-1).long(), minlength=world).double()
        dist.all_reduce(ppr)
        k_ms = sum(v["mean_us"] * v["launches"] for v in prof.values()) / 2 / 1e3          # two profiled layer calls
        st = dict(epp.stats)
        t = torch.tensor([float(st["bytes_dispatch"]), float(st["bytes_combine"]), k_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        line["exchange"] = {"kind": epp.exchange, "max_bytes_dispatch_per_rank": float(t[0].item()), "max_bytes_combine_per_rank": float(t[1].item()),
                            "max_kernels_ms_per_rank": float(t[2].item()), "exchange_and_host_ms": ms - float(t[2].item()),
                            "exchange_share_of_layer": (ms - float(t[2].item())) / ms,
                            "pairs_per_rank_max": float(ppr.max().item()), "pairs_per_rank_mean": float(ppr.mean().item())}
    # the same two GEMMs against HBM: at ~256 rows per expert every weight byte serves 256 rows, so even at the FP4 peak the expert
    # records would have to stream at 2·256 / (9/16) flop per byte — more than HBM gives.  Both views are reported.
    hbm = {}
    try:
        hbm = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    hbm_peak = float(hbm.get("hbm_gbs", 6650.0))
    wbytes = n_loc * (3 * H * I * 9 // 16) + (T * K // world) * ((H + I) * 9 // 16) + (T * K // world) * (I + H) * 2      # records + quantised rows + y, part
    line["roofline_hbm"] = {"bound": "hbm", "kernel": "pf_gemm_kernel (gate/up + down), this rank's share", "achieved": wbytes / (gemm_us * 1e-6) / 1e9,
                            "peak": hbm_peak, "unit": "GB/s", "frac": wbytes / (gemm_us * 1e-6) / 1e9 / hbm_peak,
                            "note": "expert records read once + quantised activation rows + bf16 outputs; min time at peak %.2f ms vs %.2f ms at the FP4 peak"
                                    % (wbytes / hbm_peak / 1e6, flops / world / peak / 1e9)}
    if world == 1 and with_dense:
        M, N, Kd = 16384, 8192, 8192
        xq, xs, xg = E.a4_quant(torch.randn((M, Kd), device=dev, generator=g).to(torch.bfloat16))
        W = E.GMat(E.FMT_NVFP4, N, Kd, torch.randint(0, 256, (N, Kd // 2), dtype=torch.uint8, device=dev),
                   torch.randint(0x28, 0x48, (N, Kd // 16), dtype=torch.uint8, device=dev), None, 0.01)
        y = torch.empty((M, N), dtype=torch.float32, device=dev)
        dms = _timed(torch, lambda: E.nvfp4_gemm_a4(W, xq, xs, xg, y=y, ctx=ctx), args.steps)
        line["dense_gemm_a4"] = {"M": M, "N": N, "K": Kd, "ms": dms, "TFLOPs": 2.0 * M * N * Kd / (dms * 1e-3) / 1e12,
                                 "frac_of_measured_fp4_peak": 2.0 * M * N * Kd / (dms * 1e-3) / 1e12 / peak}
    # ---- correctness, outside the timed region: two of this rank's rows of the last layer call against the CPU oracle (their experts are
    # made again from their seeds, so any rank can check rows whose experts live elsewhere), with the W4A4 rounding points; and how far
    # W4A4 is from the reference's default W4A16 arithmetic on the same rows (its own gate for that is cosine > 0.98)
    ids_l, w_l, x_l = sets[(it[0] - 1) % 2]
    got = (out if world == 1 else epp.routed).float()
    rows = sorted({0, Tl - 1})
    # ---- the same layer with bf16 activations (W4A16, the reference's default prefill arithmetic): the kind::f16 grouped GEMM
    got16 = None
    if world == 1:
        ctx16 = E.Context(flags=4)
        out16 = torch.empty((T, H), dtype=torch.float32, device=dev)
        def layer16():
            E.fn_moe_prefill(tab, 0, Ex, ids_l, w_l, x_l, H, I, out=out16, ws=ws, S=T, ctx=ctx16)
        for _ in range(3):
            layer16()
        ms16 = _timed(torch, layer16, args.steps)
        ctx16.profile(True); layer16(); layer16(); prof16 = ctx16.profile_read(); ctx16.profile(False)
        ctx16.check_device()
        prof16 = {k: {"launches": v[0], "mean_us": v[1] * 1e3 / max(v[0], 1)} for k, v in prof16.items()}
        g16_us = prof16["a16_gemm_gu"]["mean_us"] + prof16["a16_gemm_down"]["mean_us"]
        bf16_peak = float(hbm.get("bf16_tflops", 1590.0))
        line["w4a16"] = {"ms_per_layer": ms16, "tokens_per_s": T / (ms16 * 1e-3), "layer_TFLOPs": flops / (ms16 * 1e-3) / 1e12, "kernels": prof16,
                         "dtype": "bf16 x bf16 (weights dequantised exactly from e2m1 x e4m3), f32 accumulate",
                         "roofline": {"bound": "tensor", "kernel": "a16_gemm_kernel (gate/up + down)", "achieved": flops / (g16_us * 1e-6) / 1e12, "peak": bf16_peak,
                                      "unit": "TFLOP/s", "frac": flops / (g16_us * 1e-6) / 1e12 / bf16_peak,
                                      "peak_source": "MEASURED_PEAKS.json bf16_tflops (cuBLAS bf16 GEMM, burst)" if "bf16_tflops" in hbm else "fallback 1590"}}
        got16 = out16.float()
        ctx16.close()
    tmp = torch.empty(rb.total, dtype=torch.uint8, device=dev)
    err = 0.0; cos_min = 1.0; dev_max = 0.0; err16 = 0.0
    for m in rows:
        ref4 = np.zeros(H, np.float64); ref16 = np.zeros(H, np.float64)
        xr = x_l[m].float().cpu().numpy()
        for k in range(K):
            e = int(ids_l[m, k]); wk = float(w_l[m, k])
            fill_expert(tmp, e)
            rec = tmp.cpu().numpy()
            ref4 += wk * O.expert_forward_a4(rec, H, I, xr, 0.0).astype(np.float64)
            ref16 += wk * O.expert_forward(rec, H, I, xr, 1.0, 0.0).astype(np.float64)
        g_m = got[m].double().cpu().numpy()
        rms = float(np.sqrt((ref4 ** 2).mean())) + 1e-30
        err = max(err, float(np.abs(g_m - ref4).max()) / rms)
        cos_min = min(cos_min, float((g_m * ref16).sum() / (np.linalg.norm(g_m) * np.linalg.norm(ref16) + 1e-30)))
        dev_max = max(dev_max, float(np.abs(g_m - ref16).max()) / (float(np.sqrt((ref16 ** 2).mean())) + 1e-30))
        if got16 is not None:
            err16 = max(err16, float(np.abs(got16[m].double().cpu().numpy() - ref16).max()) / (float(np.sqrt((ref16 ** 2).mean())) + 1e-30))
    if world > 1:
        t = torch.tensor([err, -cos_min, dev_max], dtype=torch.float64, device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err, cos_min, dev_max = float(t[0].item()), -float(t[1].item()), float(t[2].item())
    parity = {"max_err_x_rms": err, "bar": 2e-2, "rows_per_rank": rows, "ranks_checked": world,
              "what": "routed sums of sampled rows vs the CPU oracle's W4A4 expert (NVFP4 activations), experts regenerated from their seeds",
              "ok": bool(err <= 2e-2)}
    line["parity"] = parity
    line["w4a4_vs_w4a16"] = {"cos_min": cos_min, "max_err_x_rms": dev_max, "gate": "cosine > 0.98", "ok": bool(cos_min > 0.98),
                             "what": "the same rows' W4A4 results against the oracle's W4A16 expert (bf16 activations, the reference's default prefill arithmetic)"}
    if got16 is not None:
        line["w4a16"]["parity"] = {"max_err_x_rms": err16, "bar": 2e-2, "rows": rows, "ok": bool(err16 <= 2e-2),
                                   "what": "routed sums of the sampled rows vs the CPU oracle's W4A16 expert (bf16 activations)"}
    rc = 0 if parity["ok"] and line["w4a4_vs_w4a16"]["ok"] and (got16 is None or line["w4a16"]["parity"]["ok"]) else 3      # a run whose sampled rows miss the oracle fails
    return line, rc


def run_dense(args):
    """--workload dense: the dense low-bit MLP GEMVs alone, their own JSON line (see dense_measure)."""
    import torch
    import eke_hive_b200 as E
    print(json.dumps(dense_measure(args, torch, E, E.context(), torch.device("cuda", 0))), flush=True)


def dense_measure(args, torch, E, ctx, dev, Ms=(1, 8)):
    """The dense 27B-style MLP decode workload: one FFN layer = fused gate/up GEMV + down GEMV, hidden 5120, FFN 17408, M rows,
    for the NVFP4, 3-bit and 2-bit group-64 formats; 12 distinct layers' matrices cycled so L2 cannot serve repeats."""
    H, I, n = 5120, 17408, 12
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))

    def mk(fmt, N, K):
        mats = []
        for _ in range(n):
            if fmt == E.FMT_NVFP4:
                mats.append(E.GMat(fmt, N, K, torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev),
                                   torch.randint(0x28, 0x48, (N, K // 16), dtype=torch.uint8, device=dev), None, 0.003))
            else:
                nb = N * K // 4 + (N * K // 8 if fmt == E.FMT_LB3_G64 else 0)
                mats.append(E.GMat(fmt, N, K, torch.randint(0, 256, (nb,), dtype=torch.uint8, device=dev),
                                   (torch.rand((N, K // 64), device=dev) * 0.01 + 0.005).to(torch.float16), (torch.rand((N, K // 64), device=dev) * 3).to(torch.float16)))
        return mats
    res = []
    for fmt, name, bpe in ((E.FMT_NVFP4, "nvfp4", 0.5625), (E.FMT_LB3_G64, "lb3_g64", 0.4375), (E.FMT_LB2_G64, "lb2_g64", 0.3125)):
        gs, us, ds = mk(fmt, I, H), mk(fmt, I, H), mk(fmt, H, I)
        for M in Ms:
            x = torch.randn((M, H), device=dev).to(torch.bfloat16)
            ws = torch.empty(max(E.dense_gemv_ws_bytes(fmt, I, H, 2), E.dense_gemv_ws_bytes(fmt, H, I, 1)), dtype=torch.uint8, device=dev)
            act = torch.empty((M, I), dtype=torch.bfloat16, device=dev); y = torch.empty((M, H), dtype=torch.bfloat16, device=dev)

            def layer(i):
                E.dense_gemv_gu(gs[i % n], us[i % n], x, act=act, ws=ws, ctx=ctx); E.dense_gemv(ds[i % n], act, y=y, ws=ws, ctx=ctx)
            for i in range(4):
                layer(i)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for i in range(n):
                    layer(i)
            us_layer = _timed(torch, gr.replay, max(args.steps // 4, 5)) * 1e3 / n
            by = 3 * H * I * bpe + M * (2 * H + I) * 2
            res.append({"fmt": name, "M": M, "us_per_ffn_layer": us_layer, "algorithmic_MB": by / 1e6, "achieved_GBps": by / us_layer / 1e3,
                        "frac_of_measured_hbm": by / us_layer / 1e3 / peak})
            del gr
        del gs, us, ds
        torch.cuda.empty_cache()
    ctx.check_device()
    head = res[0]
    return {"metric": "dense_ffn_layer_GBps", "value": head["achieved_GBps"], "unit": "GB/s", "n_gpus": 1, "data": "synthetic",
            "config": {"workload": "dense 27B-style MLP decode: hidden 5120, FFN 17408, gate/up + down GEMV, M in %s" % (list(Ms),),
                       "l2": "12 layers' matrices cycled (1.2-1.8 GB, larger than L2)"},
            "roofline": {"bound": "hbm", "kernel": "dense_stream_kernel", "achieved": head["achieved_GBps"], "peak": peak, "unit": "GB/s",
                         "frac": head["frac_of_measured_hbm"], "traffic": None},
            "per_case": res}


def run_records(args):
    """The step in front of the path: n experts (Qwen3-Next shape, hidden 2048, FFN 512) assembled into records on the device from
    checkpoint-form tensors whose block scales are stored compressed; one hb_record_pack_batch call per step."""
    import torch
    import eke_hive_b200 as E
    dev = torch.device("cuda", 0)
    ctx = E.context()
    H, I, n, distinct = 2048, 512, 256, 8

    def synth(rng, R, C):
        """e4m3 codes around one level with a 2 % tail of outliers, compressed as a checkpoint stores them (base = row minimum, entries
        more than 15 above it as exception words)"""
        s = np.minimum(40 + rng.integers(0, 12, (R, C)) + np.where(rng.integers(0, 50, (R, C)) == 0, rng.integers(0, 70, (R, C)), 0), 0x7E).astype(np.uint8)
        base = s.min(axis=1)
        d = s.astype(np.int32) - base[:, None]
        flat = np.flatnonzero(d.reshape(-1) > 15)
        exc = ((s.reshape(-1)[flat].astype(np.uint32) << 24) | flat.astype(np.uint32)).astype(np.uint32)
        d[d > 15] = 0
        nib = d.reshape(R // 16, 16 * C).astype(np.uint8)
        fixed = np.zeros((R // 16, 16 + 8 * C), dtype=np.uint8)
        fixed[:, :16] = base.reshape(R // 16, 16)
        fixed[:, 16:] = nib[:, 0::2] | (nib[:, 1::2] << 4)
        return fixed, exc
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    rng = np.random.default_rng(0)
    L = E.ExpertRecLayout(H, I)
    host, src_bytes = [], 0
    for _ in range(distinct):                                  # a few distinct compressed scale tensors, every expert its own copy on the device
        pr = []
        for rows, K in ((I, H), (I, H), (H, I)):
            fx, ex = synth(rng, rows, K // 16)
            pr.append((fx, ex.view(np.int32)))
        host.append(pr)
    experts = []
    for r in range(n):
        projs = []
        for j, (rows, K) in enumerate(((I, H), (I, H), (H, I))):
            fx, ex = host[r % distinct][j]
            projs.append({"weight": torch.randint(0, 256, (rows, K // 2), dtype=torch.uint8, device=dev), "csf_fixed": torch.from_numpy(fx).to(dev),
                          "csf_exc": torch.from_numpy(ex).to(dev), "global": 1e-4})
            src_bytes += rows * K // 2 + fx.size + ex.size * 4
        experts.append(projs)
    recs = torch.zeros((n, int(L.total)), dtype=torch.uint8, device=dev)
    jobs = E.record_jobs(experts, recs)
    status = torch.empty((n, 3, 2), dtype=torch.int32, device=dev)
    ws = torch.empty(E.record_pack_ws_bytes(H, I, n), dtype=torch.uint8, device=dev)
    ms = _timed(torch, lambda: E.record_pack_batch(jobs, n, H, I, status=status, ws=ws, ctx=ctx), max(args.steps, 10))
    ctx.check_device()
    assert int(status.abs().sum()) == 0
    by = src_bytes + n * (int(L.g) + 12)                        # sources read once, records written once
    # CPU arm: the same assembly by the oracle port on one host thread, as many experts as fit in 3 s
    from oracle import oracle as O
    t0 = time.perf_counter(); m = 0
    while time.perf_counter() - t0 < 3.0:
        pr = host[m % distinct]
        projs = [{"weight": np.zeros((rows, K // 2), np.uint8), "csf_fixed": pr[j][0], "csf_exc": pr[j][1].view(np.uint32), "global": 1e-4}
                 for j, (rows, K) in enumerate(((I, H), (I, H), (H, I)))]
        code, _ = O.record_pack(H, I, projs); assert code == 0
        m += 1
    cpu_rps = m / (time.perf_counter() - t0)
    print(json.dumps({"metric": "record_pack_records_per_s", "value": n / ms * 1e3, "unit": "records/s", "n_gpus": 1, "ms_per_step": ms, "data": "synthetic",
                      "config": {"workload": f"{n} experts, hidden {H}, FFN {I}, NVFP4 with compressed block scales → records; one batch call per step",
                                 "l2": f"{by / 1e6:.0f} MB read + written per step (larger than L2)"},
                      "roofline": {"bound": "hbm", "kernel": "record_main_kernel + csf_tail_kernel", "achieved": by / ms / 1e6, "peak": peak, "unit": "GB/s",
                                   "frac": by / ms / 1e6 / peak, "traffic": by,
                                   "traffic_source": "algorithmic (an ncu capture of record_main + csf_tail on this workload read 908.8 MB of DRAM traffic; not measured in this run)",
                                   "algorithmic_bytes": by},
                      "cpu_baseline": {"value": cpu_rps, "unit": "records/s", "cores": 1, "kind": "port", "sample": f"{m} experts in 3 s"}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=0, help="run one batch size only (default: 1, 4, 8, 16; headline 16)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than 48 (development only; the number is then not the benchmark's)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "dense", "records"],
                    help="decode = the benchmark proper (Qwen3-Next-shaped MoE decode); prefill = one DeepSeek-shaped MoE layer on the FP4 tensor cores; "
                         "dense = the dense 27B-style MLP GEMVs; records = record assembly in front of the path (one GPU each; their own JSON line)")
    ap.add_argument("--tokens", type=int, default=8192, help="--workload prefill: tokens per layer call")
    ap.add_argument("--experts", type=int, default=256, help="--workload prefill: routed experts resident (fewer = a smaller case for profiling)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the per_config / prefill / dense sub-measurements of the default run")
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work for the baseline leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload == "prefill":
        sys.exit(run_prefill(args) or 0)
    elif args.workload == "dense":
        run_dense(args)
    elif args.workload == "records":
        run_records(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
