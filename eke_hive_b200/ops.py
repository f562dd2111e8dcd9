"""Host-side mirror of the reference engine's expert-compute operators over the C ABI.

Names and argument meaning follow the reference's C++ free functions (engine/include/hive/glm/nvfp4.h, glm/glm_moe.h,
qwen/fn_moe.h, qwen/qwen_kernels.h, glm/glm_kernels.h); tensors are torch CUDA tensors used as typed device pointers.
Every call is asynchronous on the current torch CUDA stream and raises HbError on a negative status.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

from . import _lib
from ._lib import Config, HbError, MoePair, PfCombine, RecLayout

__all__ = ["Context", "context", "ExpertRecLayout", "nvfp4_dequant", "nvfp4_gemv", "nvfp4_quantize", "requant_nvfp4", "a4_quant", "router_softmax_topk",
           "router_topk", "build_moe_pairs", "moe_combine", "moe_decode_ws_bytes", "moe_decode", "fn_moe_decode_routed", "fn_moe_decode_routed_static", "static_max_pairs", "moe_decode_routed_f32", "moe_layer_decode",
           "moe_decode_supported", "GMat", "dense_gemv", "dense_gemv_gu", "dense_gemv_ws_bytes", "lb_dequant", "dispatch_plan", "moe_layer", "moe_layer_ws_bytes", "PeerExchange", "moe_decode_ep_local", "moe_prefill_supported", "moe_prefill_ws_bytes", "fn_moe_prefill", "nvfp4_gemm_a4", "fp4_peak_probe", "FMT_NVFP4", "FMT_LB3_G64", "FMT_LB2_G64", "expert_dequant", "csf_decode", "record_pack", "record_pack_ws_bytes", "record_jobs", "record_pack_batch", "CSF_OK", "CSF_EXC_INDEX", "CSF_EXC_DELTA", "CSF_EXC_VALUE", "CSF_CODE", "gather_rows", "swiglu_rows", "scatter_add_rows", "add_f32", "make_pairs", "rec_table", "HbError"]


def _L():
    from . import lib
    return lib


def _p(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        assert t.is_cuda, "device tensors only"
        return t.data_ptr()
    return int(t)


def _stream():
    return torch.cuda.current_stream().cuda_stream


class Context:
    """One hb_ctx: a device, its SM count and the device error word.  Calls on one context must not overlap."""

    def __init__(self, device: int | None = None, max_ctas: int = 0, flags: int = 0, wait_polls: int = 0):
        if not torch.cuda.is_available():
            raise HbError(-4, "no CUDA device: the library has no CPU path")
        self.device = torch.cuda.current_device() if device is None else device
        self._h = C.c_void_p()
        cfg = Config(self.device, max_ctas, flags, wait_polls)
        st = _L().hb_create(C.byref(cfg), C.byref(self._h))
        if st != 0:
            raise HbError(st, _L().hb_status_string(st).decode())

    def check(self, st: int):
        if st != 0:
            raise HbError(st, _L().hb_last_error(self._h).decode())

    @property
    def handle(self):
        return self._h

    @property
    def sm_count(self) -> int:
        return _L().hb_sm_count(self._h)

    @property
    def launches(self) -> int:
        return int(_L().hb_launch_count(self._h))

    def profile(self, on: bool):
        """Turns per-kernel event timing on or off (see hb_profile_enable)."""
        self.check(_L().hb_profile_enable(self._h, int(on)))

    def profile_read(self) -> dict[str, tuple[int, float]]:
        """{kernel name: (launches, total ms)} since the last read; synchronises the device."""
        from ._lib import KernelStat
        arr = (KernelStat * 64)()
        n = C.c_int(0)
        self.check(_L().hb_profile_read(self._h, arr, 64, C.byref(n)))
        return {arr[i].name.decode(): (int(arr[i].launches), float(arr[i].total_ms)) for i in range(n.value)}

    def check_device(self):
        self.check(_L().hb_check_device(self._h, _stream()))

    def close(self):
        if self._h:
            _L().hb_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_CTX: dict[int, Context] = {}


def context(device: int | None = None) -> Context:
    """The process-wide default context of a device.  HIVE_B200_FLAGS (an integer, default 0) gives its hb_config flags."""
    d = torch.cuda.current_device() if device is None else device
    if d not in _CTX:
        _CTX[d] = Context(d, flags=int(os.environ.get("HIVE_B200_FLAGS", "0")))
    return _CTX[d]


class ExpertRecLayout:
    """hive::glm::ExpertRecLayout (engine/include/hive/glm/glm_moe.h:13-22)."""

    def __init__(self, H: int, I: int):
        r = RecLayout()
        st = _L().hb_rec_layout_make(H, I, C.byref(r))
        if st != 0:
            raise HbError(st, f"bad expert shape H={H} I={I}")
        self.H, self.I = H, I
        for n, _ in RecLayout._fields_:
            setattr(self, n, int(getattr(r, n)))

    @staticmethod
    def make(H: int, I: int) -> "ExpertRecLayout":
        return ExpertRecLayout(H, I)


# ---------------------------------------------------------------------------------------------------- formats
def nvfp4_dequant(w: torch.Tensor, s: torch.Tensor, g: float, N: int, K: int, out: torch.Tensor | None = None, ctx: Context | None = None):
    ctx = ctx or context()
    out = torch.empty((N, K), dtype=torch.bfloat16, device=w.device) if out is None else out
    ctx.check(_L().hb_nvfp4_dequant(ctx.handle, _p(w), _p(s), g, N, K, _p(out), _stream()))
    return out


def nvfp4_gemv(w, s, g: float, N: int, K: int, x: torch.Tensor, y: torch.Tensor | None = None, ctx: Context | None = None):
    """y[m, n] = g·Σ_k x[m, k]·W[n, k]; x bf16 [M, K] (row stride x.stride(0)), M ≤ 16; y fp32 [M, N]."""
    ctx = ctx or context()
    M = x.shape[0]
    y = torch.empty((M, N), dtype=torch.float32, device=x.device) if y is None else y
    ctx.check(_L().hb_nvfp4_gemv(ctx.handle, _p(w), _p(s), g, N, K, _p(x), x.stride(0), M, _p(y), y.stride(0), _stream()))
    return y


def nvfp4_quantize(w: torch.Tensor, q=None, s=None, g=None, ctx: Context | None = None):
    """fp32 [N, K] → (codes u8 [N, K/2], scales u8 [N, K/16], g_mul fp32 [1]) by the reference's device rule."""
    ctx = ctx or context()
    N, K = w.shape
    q = torch.empty((N, K // 2), dtype=torch.uint8, device=w.device) if q is None else q
    s = torch.empty((N, K // 16), dtype=torch.uint8, device=w.device) if s is None else s
    g = torch.empty(1, dtype=torch.float32, device=w.device) if g is None else g
    amax = torch.empty(1, dtype=torch.float32, device=w.device)
    ctx.check(_L().hb_nvfp4_quantize(ctx.handle, _p(w), N, K, _p(q), _p(s), _p(g), _p(amax), _stream()))
    return q, s, g


def requant_nvfp4(w_fp8: torch.Tensor, row_scale: torch.Tensor, ctx: Context | None = None):
    """hive::q27::k::requant_nvfp4: FP8 (e4m3 codes u8 [N, K]) with one fp32 scale per row → (codes u8 [N, K/2], scales u8 [N, K/16],
    g_mul fp32 [1] on the device)."""
    ctx = ctx or context()
    N, K = w_fp8.shape
    q = torch.empty((N, K // 2), dtype=torch.uint8, device=w_fp8.device)
    s = torch.empty((N, K // 16), dtype=torch.uint8, device=w_fp8.device)
    g = torch.empty(1, dtype=torch.float32, device=w_fp8.device)
    amax = torch.empty(1, dtype=torch.float32, device=w_fp8.device)
    ctx.check(_L().hb_requant_nvfp4(ctx.handle, _p(w_fp8), _p(row_scale), N, K, _p(q), _p(s), _p(g), _p(amax), _stream()))
    return q, s, g


def a4_quant(x: torch.Tensor, ctx: Context | None = None):
    ctx = ctx or context()
    n, K = x.shape
    q = torch.empty((n, K // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty((n, K // 16), dtype=torch.uint8, device=x.device)
    g = torch.empty(n, dtype=torch.float32, device=x.device)
    ctx.check(_L().hb_a4_quant(ctx.handle, _p(x), x.stride(0), n, K, _p(q), _p(s), _p(g), _stream()))
    return q, s, g


# ---------------------------------------------------------------------------------------------------- routing
def router_softmax_topk(logits: torch.Tensor, k: int, renorm: bool = True, logits_bf16: bool = True, E: int | None = None, ids=None, w=None,
                        ctx: Context | None = None):
    """hive::qwen::router_softmax_topk: logits fp32 [M, ld]; returns ids int32 [M, k], w fp32 [M, k]."""
    ctx = ctx or context()
    M, ld = logits.shape[0], logits.stride(0)
    E = logits.shape[1] if E is None else E
    ids = torch.empty((M, k), dtype=torch.int32, device=logits.device) if ids is None else ids
    w = torch.empty((M, k), dtype=torch.float32, device=logits.device) if w is None else w
    ctx.check(_L().hb_route_softmax_topk(ctx.handle, _p(logits), ld, M, E, k, int(renorm), int(logits_bf16), _p(ids), _p(w), _stream()))
    return ids, w


def router_topk(logits: torch.Tensor, bias: torch.Tensor | None, k: int, scale: float = 1.0, ctx: Context | None = None, ids=None, w=None):
    """hive::glm::router_topk: sigmoid scores, selection on score + bias.  logits fp32 [M, E] dense."""
    ctx = ctx or context()
    M, E = logits.shape
    ids = torch.empty((M, k), dtype=torch.int32, device=logits.device) if ids is None else ids
    w = torch.empty((M, k), dtype=torch.float32, device=logits.device) if w is None else w
    ctx.check(_L().hb_route_sigmoid_topk(ctx.handle, _p(logits), _p(bias), M, E, k, scale, _p(ids), _p(w), _stream()))
    return ids, w


def rec_table(recs: list[torch.Tensor | None]) -> torch.Tensor:
    """Device array of record pointers (int64), 0 for a missing record."""
    dev = next(r.device for r in recs if r is not None)
    return torch.tensor([0 if r is None else r.data_ptr() for r in recs], dtype=torch.int64, device=dev)


def make_pairs(rows, recs, weights, device) -> torch.Tensor:
    """Packs (row, record pointer, weight) triples into a device array with the hb_moe_pair / hive::glm::MoePair layout."""
    n = len(rows)
    a = np.zeros(n, dtype=np.dtype([("row", "<i4"), ("pad", "<i4"), ("rec", "<u8"), ("w", "<f4"), ("pad2", "<i4")]))
    a["row"] = np.asarray(rows, np.int32)
    a["rec"] = np.asarray([0 if r is None else (r.data_ptr() if isinstance(r, torch.Tensor) else int(r)) for r in recs], np.uint64)
    a["w"] = np.asarray(weights, np.float32)
    return torch.from_numpy(a.view(np.uint8).reshape(n, 24).copy()).to(device)


def build_moe_pairs(ids, w, rec_tab, li: int, E: int, ctx: Context | None = None):
    ctx = ctx or context()
    M, K = ids.shape
    pairs = torch.empty((M * K, 24), dtype=torch.uint8, device=ids.device)
    ctx.check(_L().hb_build_moe_pairs(ctx.handle, _p(ids), _p(w), M, K, _p(rec_tab), li, E, _p(pairs), _stream()))
    return pairs


def moe_combine(routed, shared, lg=None, col: int = 0, out=None, ctx: Context | None = None):
    ctx = ctx or context()
    M, H = routed.shape
    out = torch.empty((M, H), dtype=torch.bfloat16, device=routed.device) if out is None else out
    ctx.check(_L().hb_moe_combine(ctx.handle, _p(routed), _p(shared), _p(lg), 0 if lg is None else lg.stride(0), col, M, H, _p(out), _stream()))
    return out


# ---------------------------------------------------------------------------------------------------- decode
def moe_decode_supported(H: int, I: int) -> int:
    """0 = not accepted, 1 = generic kernels, 2 = streaming tensor-core path."""
    return int(_L().hb_moe_decode_supported(H, I))


def moe_decode_ws_bytes(n_pairs: int, H: int, I: int) -> int:
    return int(_L().hb_moe_decode_ws_bytes(n_pairs, H, I))


def _ws(n_pairs, H, I, device, ws):
    if ws is None:
        ws = torch.empty(moe_decode_ws_bytes(n_pairs, H, I), dtype=torch.uint8, device=device)
    return ws


def moe_decode(pairs: torch.Tensor, x: torch.Tensor, H: int, I: int, limit: float, out: torch.Tensor, ws=None, ctx: Context | None = None):
    """hive::glm::moe_decode: out[row] += Σ_pairs w·expert(x[row]); out fp32 [M, H] accumulated in place."""
    ctx = ctx or context()
    n = pairs.shape[0]
    ws = _ws(n, H, I, x.device, ws)
    ctx.check(_L().hb_moe_decode(ctx.handle, _p(pairs), n, _p(x), H, I, limit, _p(out), _p(ws), _stream()))
    return out


def fn_moe_decode_routed(ids, w, rec_tab, li: int, E: int, x, H: int, I: int, shared=None, lg=None, col: int = 0, out=None, limit: float = 0.0,
                         ws=None, ctx: Context | None = None):
    """hive::qwen::fn_moe_decode_routed: routed sum fused with the shared-expert combine → bf16 [M, H]."""
    ctx = ctx or context()
    M, K = ids.shape
    out = torch.empty((M, H), dtype=torch.bfloat16, device=x.device) if out is None else out
    ws = _ws(M * K, H, I, x.device, ws)
    cmb = PfCombine(_p(shared), _p(lg), 0 if lg is None else lg.stride(0), col, _p(out))
    ctx.check(_L().hb_moe_decode_routed(ctx.handle, _p(ids), _p(w), M, K, _p(rec_tab), li, E, _p(x), H, I, limit, C.byref(cmb), _p(ws), _stream()))
    return out


def fn_moe_decode_routed_static(ids, w, rec_tab, li: int, E: int, x, H: int, I: int, shared=None, lg=None, col: int = 0, out=None, limit: float = 0.0,
                                ctx: Context | None = None):
    """fn_moe_decode_routed without a workspace argument, for hosts that may not allocate when they call: the scratch is the
    library's built-in 4 MiB device array.  `out` must be given by the caller if the call itself has to be allocation-free
    (this wrapper creates it with torch when it is None).  Raises HbError(-2) when M·K exceeds static_max_pairs(H, I).
    Calls sharing a device must not overlap on the GPU."""
    ctx = ctx or context()
    M, K = ids.shape
    out = torch.empty((M, H), dtype=torch.bfloat16, device=x.device) if out is None else out
    cmb = PfCombine(_p(shared), _p(lg), 0 if lg is None else lg.stride(0), col, _p(out))
    ctx.check(_L().hb_moe_decode_routed_static(ctx.handle, _p(ids), _p(w), M, K, _p(rec_tab), li, E, _p(x), H, I, limit, C.byref(cmb), _stream()))
    return out


def static_max_pairs(H: int, I: int) -> int:
    """Largest M·K hb_moe_decode_routed_static accepts at this expert shape."""
    return int(_L().hb_moe_decode_static_max_pairs(H, I))


def moe_decode_routed_f32(ids, w, rec_tab, li: int, E: int, x, H: int, I: int, out=None, limit: float = 0.0, ws=None, ctx: Context | None = None):
    """Routed sum alone: out fp32 [M, H] = Σ_k w·expert (overwritten); NULL table entries and invalid ids contribute nothing."""
    ctx = ctx or context()
    M, K = ids.shape
    out = torch.empty((M, H), dtype=torch.float32, device=x.device) if out is None else out
    ws = _ws(M * K, H, I, x.device, ws)
    ctx.check(_L().hb_moe_decode_routed_f32(ctx.handle, _p(ids), _p(w), M, K, _p(rec_tab), li, E, _p(x), H, I, limit, _p(out), _p(ws), _stream()))
    return out


def moe_layer_decode(logits, x, rec_tab, li: int, E: int, K: int, H: int, I: int, shared_rec=None, gate_col: int = -1, renorm: bool = True,
                     logits_bf16: bool = True, bias=None, sigmoid_scale: float = 0.0, limit: float = 0.0, ids=None, w=None, out=None, ws=None,
                     ctx: Context | None = None):
    """Router → routed experts → NVFP4 shared expert → combine, one call.  Returns (ids, w, out bf16 [M, H])."""
    ctx = ctx or context()
    M = x.shape[0]
    ids = torch.empty((M, K), dtype=torch.int32, device=x.device) if ids is None else ids
    w = torch.empty((M, K), dtype=torch.float32, device=x.device) if w is None else w
    out = torch.empty((M, H), dtype=torch.bfloat16, device=x.device) if out is None else out
    ws = _ws(M * (K + 1), H, I, x.device, ws)
    ctx.check(_L().hb_moe_layer_decode(ctx.handle, _p(logits), logits.stride(0), M, E, K, int(renorm), int(logits_bf16), _p(bias), sigmoid_scale,
                                       _p(rec_tab), li, _p(shared_rec), gate_col, _p(x), H, I, limit, _p(ids), _p(w), _p(out), _p(ws), _stream()))
    return ids, w, out


def moe_layer_ws_bytes(M: int, K: int, E: int, H: int, I: int) -> int:
    return int(_L().hb_moe_layer_ws_bytes(M, K, E, H, I))


def moe_layer(logits, x, rec_tab, li: int, E: int, K: int, H: int, I: int, shared_rec=None, gate_col: int = -1, renorm: bool = True,
              logits_bf16: bool = True, bias=None, sigmoid_scale: float = 0.0, limit: float = 0.0, ids=None, w=None, out=None, ws=None,
              ctx: Context | None = None):
    """hb_moe_layer: the whole layer for any number of rows — decode operators up to 64 rows, the grouped tensor-core GEMM beyond.
    Returns (ids, w, out bf16 [M, H])."""
    ctx = ctx or context()
    M = x.shape[0]
    ids = torch.empty((M, K), dtype=torch.int32, device=x.device) if ids is None else ids
    w = torch.empty((M, K), dtype=torch.float32, device=x.device) if w is None else w
    out = torch.empty((M, H), dtype=torch.bfloat16, device=x.device) if out is None else out
    ws = torch.empty(moe_layer_ws_bytes(M, K, E, H, I), dtype=torch.uint8, device=x.device) if ws is None else ws
    ctx.check(_L().hb_moe_layer(ctx.handle, _p(logits), logits.stride(0), M, E, K, int(renorm), int(logits_bf16), _p(bias), sigmoid_scale,
                                _p(rec_tab), li, _p(shared_rec), gate_col, _p(x), H, I, limit, _p(ids), _p(w), _p(out), _p(ws), _stream()))
    return ids, w, out


# ---------------------------------------------------------------------------------------------------- dense GEMV (hb_qmat)
FMT_NVFP4, FMT_LB3_G64, FMT_LB2_G64 = 0, 1, 2


class GMat:
    """hive::q27::GMat for the formats this library takes: device tensors of one [N, K] weight matrix.
    NVFP4: w u8 [N, K/2], s u8 [N, K/16], g.  LB2/LB3: w u8 codes (LB3: low plane then high plane), s / zp fp16 [N, K/64]."""

    def __init__(self, fmt: int, N: int, K: int, w, s, zp=None, g: float = 1.0):
        from ._lib import QMat
        self.fmt, self.N, self.K, self.w, self.s, self.zp, self.g = fmt, N, K, w, s, zp, g
        self.c = QMat(fmt, N, K, _p(w), _p(s), _p(zp), g)


def dense_gemv_ws_bytes(fmt: int, N: int, K: int, n_mats: int = 1) -> int:
    return int(_L().hb_dense_gemv_ws_bytes(fmt, N, K, n_mats))


def dense_gemv(W: GMat, x, out_dtype=torch.float32, y=None, ws=None, ctx: Context | None = None):
    """hive::q27::k::gemv: y[m, n] = Σ_k x[m, k]·W[n, k]; y bf16 or fp32 [M, N]."""
    ctx = ctx or context()
    M = x.shape[0]
    y = torch.empty((M, W.N), dtype=out_dtype, device=x.device) if y is None else y
    ws = torch.empty(dense_gemv_ws_bytes(W.fmt, W.N, W.K, 1), dtype=torch.uint8, device=x.device) if ws is None else ws
    yb, yf = (_p(y), None) if y.dtype == torch.bfloat16 else (None, _p(y))
    ctx.check(_L().hb_dense_gemv(ctx.handle, C.byref(W.c), _p(x), x.stride(0), M, yb, yf, y.stride(0), _p(ws), _stream()))
    return y


def dense_gemv_gu(G: GMat, U: GMat, x, act=None, ws=None, ctx: Context | None = None):
    """hive::q27::k::gemv_gu: act = bf16(bf16(silu(bf16 g)) · bf16 u), bf16 [M, N]."""
    ctx = ctx or context()
    M = x.shape[0]
    act = torch.empty((M, G.N), dtype=torch.bfloat16, device=x.device) if act is None else act
    ws = torch.empty(dense_gemv_ws_bytes(G.fmt, G.N, G.K, 2), dtype=torch.uint8, device=x.device) if ws is None else ws
    ctx.check(_L().hb_dense_gemv_gu(ctx.handle, C.byref(G.c), C.byref(U.c), _p(x), x.stride(0), M, _p(act), act.stride(0), _p(ws), _stream()))
    return act


def lb_dequant(W: GMat, out=None, ctx: Context | None = None):
    ctx = ctx or context()
    out = torch.empty((W.N, W.K), dtype=torch.bfloat16, device=W.w.device) if out is None else out
    ctx.check(_L().hb_lb_dequant(ctx.handle, C.byref(W.c), _p(out), _stream()))
    return out


def moe_decode_ep_local(ids, w, rec_tab, li: int, E: int, x, H: int, I: int, routed_out, shared_ptr: int = 0, sh_row0: int = 0, sh_rows: int = 0,
                        shared_out=None, limit: float = 0.0, ws=None, ctx: Context | None = None):
    """One rank's share of an expert-parallel decode layer (hb_moe_decode_ep_local).  ids int32 / w fp32 [M, K] and x bf16 [M, H] may be
    strided row views (e.g. columns of a gathered exchange buffer); routed_out fp32 [M, H]; shared_out bf16 [sh_rows, H]."""
    ctx = ctx or context()
    M, K = ids.shape
    assert ids.stride(1) == 1 and w.stride(1) == 1 and x.stride(1) == 1 and ids.stride(0) == w.stride(0)
    ws = _ws(M * (K + 1), H, I, x.device, ws)
    ctx.check(_L().hb_moe_decode_ep_local(ctx.handle, _p(ids), _p(w), ids.stride(0), M, K, _p(rec_tab), li, E, _p(x), x.stride(0), H, I, limit,
                                          shared_ptr or None, sh_row0, sh_rows, _p(routed_out), _p(shared_out), _p(ws), _stream()))
    return routed_out


def dispatch_plan(ids_host: np.ndarray, E: int, H: int, I: int):
    """hb_dispatch_plan on host routing ids [M, K]: dict of the plan fields plus `counts` (pairs per expert)."""
    from ._lib import Plan
    ids_host = np.ascontiguousarray(ids_host, dtype=np.int32)
    M, K = ids_host.shape
    counts = np.zeros(E, np.int32)
    p = Plan()
    st = _L().hb_dispatch_plan(ids_host.ctypes.data, M, K, E, H, I, counts.ctypes.data, C.byref(p))
    if st != 0:
        raise HbError(st, "dispatch_plan: bad arguments")
    d = {n: getattr(p, n) for n, _ in Plan._fields_}
    d["counts"] = counts
    return d


class PeerExchange:
    """hb_ep: the expert-parallel exchanges over NVLink peer memory.  `mine` is this rank's exchange memory (a zero-filled uint8
    device tensor of `layout(...)` bytes); `exchange(obj)` must return the list of every rank's `obj` (e.g. an all_gather_object):
    it carries the CUDA IPC handles, which every rank opens with its own device current."""

    @staticmethod
    def layout(world: int, B: int, H: int, K: int):
        """(offsets dict, total bytes, record bytes) of one rank's exchange memory: gather buffer, gather flags, partial buffer, partial flags."""
        rec = int(_L().hb_ep_rec_bytes(H, K))
        off, o = {}, 0
        for name, size in (("recv", world * B * rec), ("ag_flag", 256), ("rs", world * B * H * 4), ("rs_flag", 256)):
            off[name] = o
            o += (size + 255) // 256 * 256
        return off, o, rec

    def __init__(self, mine, exchange, rank: int, world: int, B: int, H: int, K: int, ctx: Context | None = None):
        self.ctx = ctx or context()
        self.mine = mine                                               # keeps the exported memory alive
        self._h = None
        self._bases = []
        off, total, self.rec_bytes = self.layout(world, B, H, K)
        assert mine.numel() >= total and mine.dtype == torch.uint8 and mine.device.index == self.ctx.device
        handle = (C.c_ubyte * 64)()
        offset = C.c_size_t(0)
        self.ctx.check(_L().hb_ep_export(self.ctx.handle, mine.data_ptr(), handle, C.byref(offset)))
        everyone = exchange((bytes(handle), int(offset.value)))
        ptrs = []
        for p in range(world):
            if p == rank:
                ptrs.append(mine.data_ptr())
                continue
            hb, ob = everyone[p]
            ptr, base = C.c_void_p(), C.c_void_p()
            self.ctx.check(_L().hb_ep_import(self.ctx.handle, (C.c_ubyte * 64).from_buffer_copy(hb), ob, C.byref(ptr), C.byref(base)))
            self._bases.append(base)
            ptrs.append(ptr.value)
        arr = lambda name: (C.c_void_p * world)(*[q + off[name] for q in ptrs])
        h = C.c_void_p()
        self.ctx.check(_L().hb_ep_create(self.ctx.handle, rank, world, B, H, K, arr("recv"), arr("ag_flag"), arr("rs"), arr("rs_flag"), C.byref(h)))
        self._h = h
        self.off = off

    def route_push(self, logits, x, ids_out, w_out, E: int, renorm: bool = True, logits_bf16: bool = True):
        self.ctx.check(_L().hb_ep_route_push(self._h, _p(logits), logits.stride(0), E, int(renorm), int(logits_bf16), _p(x), x.stride(0), _p(ids_out),
                                             _p(w_out), _stream()))

    def layer_local(self, rec_tab, li: int, E: int, I: int, shared_ptr: int, shared_out, ws, limit: float = 0.0):
        self.ctx.check(_L().hb_ep_layer_local(self._h, _p(rec_tab), li, E, I, limit, shared_ptr or None, _p(shared_out), _p(ws), _stream()))

    def push_rows(self, x, ids, w):
        self.ctx.check(_L().hb_ep_push_rows(self._h, _p(x), x.stride(0), _p(ids), _p(w), _stream()))

    def wait_rows(self):
        self.ctx.check(_L().hb_ep_wait_rows(self._h, _stream()))

    def push_partials(self, part):
        self.ctx.check(_L().hb_ep_push_partials(self._h, _p(part), _stream()))

    def combine(self, shared, lg, col: int, out):
        self.ctx.check(_L().hb_ep_combine(self._h, _p(shared), _p(lg), 0 if lg is None else lg.stride(0), col, _p(out), _stream()))

    def close(self):
        """Unmaps the peers' memory.  Call it on every rank, after a barrier, when no exchange is in flight."""
        if self._h:
            _L().hb_ep_destroy(self._h)
            self._h = None
        for b in self._bases:
            _L().hb_ep_close(self.ctx.handle, b)
        self._bases = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------------------------------- prefill (tcgen05 grouped GEMM)
def moe_prefill_supported(H: int, I: int) -> bool:
    return bool(_L().hb_moe_prefill_supported(H, I))


def moe_prefill_ws_bytes(S: int, K: int, E: int, H: int, I: int) -> int:
    return int(_L().hb_moe_prefill_ws_bytes(S, K, E, H, I))


def fn_moe_prefill(rec_tab, li: int, E: int, ids, w, x, H: int, I: int, out=None, ws=None, S: int | None = None, limit: float = 0.0,
                   shared=None, lg=None, col: int = 0, cout=None, ctx: Context | None = None):
    """hive::qwen::fn_moe_prefill (NVFP4 activations): fp32 [M, H] routed sums, or with `shared` the fused combine → bf16 [M, H]."""
    ctx = ctx or context()
    M, K = ids.shape
    S = M if S is None else S
    ws = torch.empty(moe_prefill_ws_bytes(S, K, E, H, I), dtype=torch.uint8, device=x.device) if ws is None else ws
    if shared is None:
        out = torch.empty((M, H), dtype=torch.float32, device=x.device) if out is None else out
        ctx.check(_L().hb_moe_prefill(ctx.handle, _p(rec_tab), li, E, _p(ids), _p(w), M, K, _p(x), H, I, limit, _p(out), _p(ws), S, _stream(), None))
        return out
    cout = torch.empty((M, H), dtype=torch.bfloat16, device=x.device) if cout is None else cout
    cmb = PfCombine(_p(shared), _p(lg), 0 if lg is None else lg.stride(0), col, _p(cout))
    ctx.check(_L().hb_moe_prefill(ctx.handle, _p(rec_tab), li, E, _p(ids), _p(w), M, K, _p(x), H, I, limit, None, _p(ws), S, _stream(), C.byref(cmb)))
    return cout


def nvfp4_gemm_a4(W: "GMat", xq, xs, xg, y=None, ctx: Context | None = None):
    """Dense W4A4 GEMM: y fp32 [M, N] from activations quantised by a4_quant."""
    ctx = ctx or context()
    M = xq.shape[0]
    y = torch.empty((M, W.N), dtype=torch.float32, device=xq.device) if y is None else y
    ctx.check(_L().hb_nvfp4_gemm_a4(ctx.handle, C.byref(W.c), _p(xq), _p(xs), _p(xg), M, _p(y), y.stride(0), _stream()))
    return y


def fp4_peak_probe(rounds: int = 4096, ctx: Context | None = None) -> float:
    """Dense FP4 TFLOP/s of the device's tensor pipe, measured with resident operands."""
    ctx = ctx or context()
    v = C.c_float(0.0)
    ctx.check(_L().hb_fp4_peak_probe(ctx.handle, rounds, C.byref(v)))
    return float(v.value)


# ---------------------------------------------------------------------------------------------------- prefill helpers
def expert_dequant(rec, H: int, I: int, gu=None, d=None, ctx: Context | None = None):
    """hive::glm::expert_dequant: one record → bf16 gu [2I, H] (gate rows then up rows), d [H, I]."""
    ctx = ctx or context()
    gu = torch.empty((2 * I, H), dtype=torch.bfloat16, device=rec.device) if gu is None else gu
    d = torch.empty((H, I), dtype=torch.bfloat16, device=rec.device) if d is None else d
    ctx.check(_L().hb_expert_dequant(ctx.handle, _p(rec), H, I, _p(gu), _p(d), _stream()))
    return gu, d


CSF_OK, CSF_EXC_INDEX, CSF_EXC_DELTA, CSF_EXC_VALUE, CSF_CODE = 0, 4, 5, 6, 7


def csf_decode(fixed, exc, R: int, Cc: int, out=None, status=None, ws=None, fixed_shape=None, ctx: Context | None = None):
    """hive::ckq::csf_decode on the device: compressed NVFP4 block scales (fixed u8 [R/16, 16 + 8C], exc u32-as-int32 [n]) → u8 [R, C].
    Returns (out, status int32[2] on the device: {CSF_* code, position}); raises HiveError for shapes the format rules out."""
    ctx = ctx or context()
    dev = fixed.device
    fr, fc = fixed_shape if fixed_shape is not None else tuple(fixed.shape)
    out = torch.empty((max(R, 0), max(Cc, 0)), dtype=torch.uint8, device=dev) if out is None else out
    status = torch.full((2,), -1, dtype=torch.int32, device=dev) if status is None else status
    nws = _L().hb_csf_ws_bytes(R, Cc)
    ws = torch.empty(max(nws, 256), dtype=torch.uint8, device=dev) if ws is None else ws
    n = 0 if exc is None else exc.numel()
    ctx.check(_L().hb_csf_decode(ctx.handle, _p(fixed), fr, fc, _p(exc) if n else None, n, R, Cc, _p(out), _p(status), _p(ws), ws.numel(), _stream()))
    return out, status


def record_pack_ws_bytes(H: int, I: int, n: int = 1) -> int:
    return _L().hb_record_pack_ws_bytes(H, I, n)


def _fill_proj(dst, p):
    dst.weight = _p(p["weight"])
    dst.global_ = float(p["global"])
    if p.get("scale") is not None:
        dst.scale = _p(p["scale"])
    else:
        f, e = p["csf_fixed"], p["csf_exc"]
        dst.csf_fixed = _p(f)
        dst.csf_fixed_rows, dst.csf_fixed_cols = (f.shape if f.dim() == 2 else (-1, -1))
        dst.n_exc = e.numel()
        dst.csf_exc = _p(e) if e.numel() else None


def record_pack(projs, H: int, I: int, rec=None, status=None, ws=None, ctx: Context | None = None):
    """GlmExperts::load_all for one expert on the device.  projs = (gate, up, down), each a dict with 'weight' u8 [rows, K/2], 'global'
    float and either 'scale' u8 [rows, K/16] or the compressed pair 'csf_fixed' u8 [rows/16, 16 + K/2] + 'csf_exc' (32-bit words).
    Returns (rec u8 [layout.total], status int32 [3, 2] on the device)."""
    ctx = ctx or context()
    dev = projs[0]["weight"].device
    rec = torch.zeros(int(ExpertRecLayout(H, I).total), dtype=torch.uint8, device=dev) if rec is None else rec
    status = torch.full((3, 2), -1, dtype=torch.int32, device=dev) if status is None else status
    ws = torch.empty(max(record_pack_ws_bytes(H, I), 256), dtype=torch.uint8, device=dev) if ws is None else ws
    src = (_lib.ProjSrc * 3)()
    for j, p in enumerate(projs):
        _fill_proj(src[j], p)
    ctx.check(_L().hb_record_pack(ctx.handle, src, H, I, _p(rec), _p(status), _p(ws), ws.numel(), _stream()))
    return rec, status


def record_jobs(experts, recs):
    """Device array of hb_record_job for experts = [(gate, up, down) dicts as in record_pack], recs = u8 [n, layout.total] (or a list
    of record tensors).  Keep the returned tensor and the sources alive until the packing has run."""
    n = len(experts)
    jobs = (_lib.RecordJob * n)()
    for r, projs in enumerate(experts):
        for j, p in enumerate(projs):
            _fill_proj(jobs[r].src[j], p)
        jobs[r].rec = _p(recs[r])
    host = torch.frombuffer(bytearray(bytes(jobs)), dtype=torch.uint8)
    return host.to(recs[0].device)


def record_pack_batch(jobs, n: int, H: int, I: int, status=None, ws=None, ctx: Context | None = None):
    """hb_record_pack_batch: jobs = device tensor from record_jobs.  Returns status int32 [n, 3, 2] on the device."""
    ctx = ctx or context()
    dev = jobs.device
    status = torch.full((n, 3, 2), -1, dtype=torch.int32, device=dev) if status is None else status
    ws = torch.empty(max(record_pack_ws_bytes(H, I, n), 256), dtype=torch.uint8, device=dev) if ws is None else ws
    ctx.check(_L().hb_record_pack_batch(ctx.handle, _p(jobs), n, H, I, _p(status), _p(ws), ws.numel(), _stream()))
    return status


def gather_rows(x, rows, out=None, ctx: Context | None = None):
    ctx = ctx or context()
    R, H = rows.shape[0], x.shape[1]
    out = torch.empty((R, H), dtype=torch.bfloat16, device=x.device) if out is None else out
    ctx.check(_L().hb_gather_rows(ctx.handle, _p(x), _p(rows), R, H, _p(out), _stream()))
    return out


def swiglu_rows(gu, limit: float = 0.0, ctx: Context | None = None):
    ctx = ctx or context()
    R, I = gu.shape[0], gu.shape[1] // 2
    y = torch.empty((R, I), dtype=torch.bfloat16, device=gu.device)
    ctx.check(_L().hb_swiglu_rows(ctx.handle, _p(gu), R, I, limit, _p(y), _stream()))
    return y


def scatter_add_rows(e, rows, w, out, ctx: Context | None = None):
    ctx = ctx or context()
    R, H = e.shape
    ctx.check(_L().hb_scatter_add_rows(ctx.handle, _p(e), _p(rows), _p(w), R, H, _p(out), _stream()))
    return out


def add_f32(a, b, ctx: Context | None = None):
    ctx = ctx or context()
    ctx.check(_L().hb_add_f32(ctx.handle, _p(a), _p(b), a.numel(), _stream()))
    return a
