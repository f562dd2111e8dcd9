"""TEST INFRASTRUCTURE: numpy/ctypes front end of the CPU oracle.

Two libraries sit behind this module:

* ``libhive_oracle.so`` – the plain-C restatement (``hive_oracle.c``), always available (built by ``make -C oracle``);
* ``_ref/libhive_ref.so`` – the reference engine's own CPU sources compiled in place (``ref_shim.cpp``), available
  wherever it was built before (it is a build product that travels with the working tree; the reference sources do not).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module; the shipped package
never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_u8p, _u16p, _f32p, _i32p, _u64p = (C.POINTER(t) for t in (C.c_uint8, C.c_uint16, C.c_float, C.c_int32, C.c_uint64))


def _ptr(a: np.ndarray, t):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(t)


def build(ref: bool = True) -> None:
    """Compile the C restatement and, when the reference tree is present, the reference shim."""
    subprocess.run(["make", "-s", "-C", str(HERE), str(HERE / "libhive_oracle.so")], check=True)
    root = ref_root()
    if ref and root is not None:
        subprocess.run(["make", "-s", "-C", str(HERE), "ref", f"REF={root}"], check=True, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)


def ref_root():
    """Where the reference project's sources are: $HIVE_REF, else a checkout named `reference` beside this repository; None if absent."""
    cand = os.environ.get("HIVE_REF") or str(HERE.parent.parent / "reference")
    return cand if Path(cand, "engine", "src", "cpu").is_dir() else None


def _load_c():
    so = HERE / "libhive_oracle.so"
    if not so.exists() or so.stat().st_mtime < (HERE / "hive_oracle.c").stat().st_mtime:
        build(ref=False)
    L = C.CDLL(str(so))
    L.ho_e2m1_to_f32.restype = C.c_float; L.ho_e2m1_to_f32.argtypes = [C.c_uint8]
    L.ho_e4m3_to_f32.restype = C.c_float; L.ho_e4m3_to_f32.argtypes = [C.c_uint8]
    L.ho_f32_to_e4m3.restype = C.c_uint8; L.ho_f32_to_e4m3.argtypes = [C.c_float]
    L.ho_f32_to_e2m1.restype = C.c_uint8; L.ho_f32_to_e2m1.argtypes = [C.c_float]
    L.ho_f32_to_bf16.restype = C.c_uint16; L.ho_f32_to_bf16.argtypes = [C.c_float]
    L.ho_bf16r.restype = C.c_float; L.ho_bf16r.argtypes = [C.c_float]
    L.ho_exp_portable.restype = C.c_float; L.ho_exp_portable.argtypes = [C.c_float]
    L.ho_fp16_to_f32.restype = C.c_float; L.ho_fp16_to_f32.argtypes = [C.c_uint16]
    L.ho_f32_to_fp16.restype = C.c_uint16; L.ho_f32_to_fp16.argtypes = [C.c_float]
    L.ho_lb_weight_bytes.restype = C.c_size_t; L.ho_lb_weight_bytes.argtypes = [C.c_int] * 3
    return L


_C = _load_c()


def have_ref() -> bool:
    return (HERE / "_ref" / "libhive_ref.so").exists()


_REF = None


def ref():
    """The compiled reference (ctypes handle).  Raises if it was never built."""
    global _REF
    if _REF is None:
        os.environ.setdefault("FAKE_NUMA_NODES", "1")
        R = C.CDLL(str(HERE / "_ref" / "libhive_ref.so"))
        for n in ("ref_e4m3_to_f32", "ref_e2m1_to_f32"):
            getattr(R, n).restype = C.c_float; getattr(R, n).argtypes = [C.c_uint8]
        for n in ("ref_f32_to_e4m3", "ref_f32_to_e2m1"):
            getattr(R, n).restype = C.c_uint8; getattr(R, n).argtypes = [C.c_float]
        for n in ("ref_bf16r", "ref_exp_portable", "ref_sigm_portable", "ref_silu_portable"):
            getattr(R, n).restype = C.c_float; getattr(R, n).argtypes = [C.c_float]
        R.ref_layer_create.restype = C.c_void_p
        R.ref_layer_create.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), _u64p]
        R.ref_layer_destroy.argtypes = [C.c_void_p]
        R.ref_layer_routed.argtypes = [C.c_void_p, C.c_int, C.c_int, _i32p, _f32p, _f32p, C.c_float, _f32p]
        R.ref_csf_decode.restype = C.c_int
        R.ref_csf_decode.argtypes = [_u8p, C.c_int64, C.c_int64, C.POINTER(C.c_uint32), C.c_size_t, C.c_int, C.c_int, _u8p, C.c_char_p, C.c_int]
        _REF = R
    return _REF


# ---------------------------------------------------------------------------------------------------- scalars / tables
def e4m3_table() -> np.ndarray:
    return np.array([_C.ho_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def e2m1_table() -> np.ndarray:
    return np.array([_C.ho_e2m1_to_f32(i) for i in range(16)], dtype=np.float32)


def f32_to_e4m3(x: float) -> int:
    return int(_C.ho_f32_to_e4m3(C.c_float(x)))


def f32_to_e2m1(x: float) -> int:
    return int(_C.ho_f32_to_e2m1(C.c_float(x)))


def exp_portable(x: float) -> float:
    return float(_C.ho_exp_portable(C.c_float(x)))


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 → bf16 bit patterns (RNE), vectorised restatement of ho_f32_to_bf16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    special = (u & 0x7F800000) == 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(special, (u >> 16).astype(np.uint16), r)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16r(x: np.ndarray) -> np.ndarray:
    return bf16_to_f32(bf16_bits(x))


# ---------------------------------------------------------------------------------------------------- record layout
def rec_layout(H: int, I: int) -> np.ndarray:
    off = np.zeros(8, dtype=np.uint64)
    _C.ho_rec_layout(H, I, _ptr(off, _u64p))
    return off


def pack_record(H: int, I: int, gate, up, down) -> np.ndarray:
    """gate/up/down = (q u8, s u8, g float).  Returns the record bytes (length off[7])."""
    off = rec_layout(H, I)
    rec = np.zeros(int(off[7]), dtype=np.uint8)
    for (q, s, _), a, b in ((gate, 0, 1), (up, 2, 3), (down, 4, 5)):
        rec[int(off[a]):int(off[a]) + q.size] = q.reshape(-1)
        rec[int(off[b]):int(off[b]) + s.size] = s.reshape(-1)
    rec[int(off[6]):int(off[6]) + 12] = np.array([gate[2], up[2], down[2]], dtype=np.float32).view(np.uint8)
    return rec


# ---------------------------------------------------------------------------------------------------- NVFP4
def nvfp4_quantize(w: np.ndarray, search: bool = True):
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    q = np.zeros((N, K // 2), np.uint8); s = np.zeros((N, K // 16), np.uint8); g = np.zeros(1, np.float32)
    _C.ho_nvfp4_quantize(_ptr(w, _f32p), N, K, int(search), _ptr(q, _u8p), _ptr(s, _u8p), _ptr(g, _f32p))
    return q, s, float(g[0])


def nvfp4_dequant_bf16(q, s, g: float) -> np.ndarray:
    N, K = q.shape[0], q.shape[1] * 2
    out = np.zeros((N, K), np.uint16)
    _C.ho_nvfp4_dequant_bf16(_ptr(q, _u8p), _ptr(s, _u8p), C.c_float(g), N, K, _ptr(out, _u16p))
    return out


def gemv_nvfp4(q, s, g: float, a: np.ndarray, use_ref: bool = False, scalar: bool = True) -> np.ndarray:
    """y[m, n] for activation rows a [M, K] (fp32)."""
    N, K = q.shape[0], q.shape[1] * 2
    a = np.ascontiguousarray(np.atleast_2d(a), dtype=np.float32)
    y = np.zeros((a.shape[0], N), np.float32)
    for m in range(a.shape[0]):
        args = (_ptr(q, _u8p), _ptr(s, _u8p), C.c_float(g), N, K, _ptr(a[m], _f32p), 0, N, _ptr(y[m], _f32p))
        if use_ref:
            (ref().ref_gemv_nvfp4_rows_scalar if scalar else ref().ref_gemv_nvfp4_rows)(*args)
        else:
            _C.ho_gemv_nvfp4(*args)
    return y


def expert_forward(rec: np.ndarray, H: int, I: int, a: np.ndarray, route_w: float = 1.0, limit: float = 0.0, silu_mode: int = 0,
                   use_ref: bool = False) -> np.ndarray:
    off = rec_layout(H, I)
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.zeros(H, np.float32); tmp = np.zeros(3 * I, np.float32)
    if use_ref:
        ref().ref_expert_forward_nvfp4(_ptr(rec, _u8p), _ptr(off, _u64p), H, I, _ptr(a, _f32p), C.c_float(route_w), C.c_float(limit),
                                       _ptr(out, _f32p), _ptr(tmp, _f32p))
    else:
        _C.ho_expert_forward_nvfp4(_ptr(rec, _u8p), _ptr(off, _u64p), H, I, _ptr(a, _f32p), C.c_float(route_w), C.c_float(limit),
                                   silu_mode, _ptr(out, _f32p), _ptr(tmp, _f32p))
    return out


def expert_forward_a4(rec: np.ndarray, H: int, I: int, x: np.ndarray, limit: float = 0.0) -> np.ndarray:
    """One expert on one activation row (fp32 holding bf16 values) with the prefill path's NVFP4 activations; unweighted bf16 values."""
    off = rec_layout(H, I)
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros(H, np.float32)
    _C.ho_expert_forward_a4(_ptr(rec, _u8p), _ptr(off, _u64p), H, I, _ptr(x, _f32p), C.c_float(limit), _ptr(out, _f32p))
    return out


def a4_quant(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, K = x.shape
    q = np.zeros((n, K // 2), np.uint8); s = np.zeros((n, K // 16), np.uint8); g = np.zeros(n, np.float32)
    _C.ho_a4_quant(_ptr(x, _f32p), K, n, K, _ptr(q, _u8p), _ptr(s, _u8p), _ptr(g, _f32p))
    return q, s, g


# ---------------------------------------------------------------------------------------------------- routers
def router_softmax_topk(logits: np.ndarray, k: int, renorm: bool = True, logits_bf16: bool = True, form: int = 0, E: int | None = None):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    M, ld = logits.shape
    E = ld if E is None else E
    ids = np.zeros((M, k), np.int32); w = np.zeros((M, k), np.float32)
    _C.ho_router_softmax_topk(_ptr(logits, _f32p), ld, M, E, k, int(renorm), int(logits_bf16), form, _ptr(ids, _i32p), _ptr(w, _f32p))
    return ids, w


def router_sigmoid_topk(logits: np.ndarray, bias: np.ndarray | None, k: int, scale: float = 1.0, form: int = 0):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    M, E = logits.shape
    ids = np.zeros((M, k), np.int32); w = np.zeros((M, k), np.float32)
    b = None if bias is None else _ptr(np.ascontiguousarray(bias, dtype=np.float32), _f32p)
    _C.ho_router_sigmoid_topk(_ptr(logits, _f32p), b, M, E, k, C.c_float(scale), form, _ptr(ids, _i32p), _ptr(w, _f32p))
    return ids, w


# ---------------------------------------------------------------------------------------------------- MoE operators
def _rec_ptrs(recs):
    arr = (C.c_void_p * len(recs))()
    for i, r in enumerate(recs):
        arr[i] = None if r is None else r.ctypes.data
    return arr


def moe_decode(H, I, rows, recs, pw, x, out, limit=0.0, silu_mode=0):
    """out[row] += Σ_pairs w·expert(x[row]); out fp32 [M,H] is updated in place."""
    off = rec_layout(H, I)
    rows = np.ascontiguousarray(rows, np.int32); pw = np.ascontiguousarray(pw, np.float32)
    x = np.ascontiguousarray(x, np.float32)
    _C.ho_moe_decode(_ptr(off, _u64p), _ptr(rows, _i32p), C.cast(_rec_ptrs(recs), C.POINTER(C.c_void_p)), _ptr(pw, _f32p), len(recs),
                     _ptr(x, _f32p), H, I, C.c_float(limit), silu_mode, _ptr(out, _f32p))
    return out


def moe_routed(H, I, ids, w, rec_tab, x, limit=0.0, silu_mode=0) -> np.ndarray:
    off = rec_layout(H, I)
    ids = np.ascontiguousarray(ids, np.int32); w = np.ascontiguousarray(w, np.float32); x = np.ascontiguousarray(x, np.float32)
    M, K = ids.shape
    acc = np.zeros((M, H), np.float32)
    _C.ho_moe_routed(_ptr(off, _u64p), _ptr(ids, _i32p), _ptr(w, _f32p), M, K, C.cast(_rec_ptrs(rec_tab), C.POINTER(C.c_void_p)),
                     len(rec_tab), _ptr(x, _f32p), H, I, C.c_float(limit), silu_mode, _ptr(acc, _f32p))
    return acc


def moe_combine(routed, shared, gate_logits=None, col=0, round_gate=True) -> np.ndarray:
    routed = np.ascontiguousarray(routed, np.float32); shared = np.ascontiguousarray(shared, np.float32)
    M, H = routed.shape
    out = np.zeros((M, H), np.uint16)
    if gate_logits is None:
        lg, ld = None, 0
    else:
        gate_logits = np.ascontiguousarray(gate_logits, np.float32)
        lg, ld = _ptr(gate_logits, _f32p), gate_logits.shape[1]
    _C.ho_moe_combine(_ptr(routed, _f32p), _ptr(shared, _f32p), lg, ld, col, int(round_gate), M, H, _ptr(out, _u16p))
    return out


def moe_layer(H, I, logits, x, rec_tab, k, shared_rec=None, gate_logits=None, gate_col=0, router="softmax", bias=None, scale=1.0,
              renorm=True, logits_bf16=True, limit=0.0, silu_mode=0):
    """Whole MoE layer on the CPU (engine/src/qwen/cpu/qwen_cpu_engine.cpp:655-783 order): route, routed sum in k order,
    NVFP4 shared expert (weight 1), combine.  Returns (ids, w, out bf16 bits)."""
    if router == "softmax":
        ids, w = router_softmax_topk(logits, k, renorm, logits_bf16, 0, E=len(rec_tab))
    else:
        ids, w = router_sigmoid_topk(logits[:, :len(rec_tab)], bias, k, scale, 0)
    acc = moe_routed(H, I, ids, w, rec_tab, x, limit, silu_mode)
    M = x.shape[0]
    if shared_rec is not None:
        shared = np.stack([expert_forward(shared_rec, H, I, x[m], 1.0, limit, silu_mode) for m in range(M)])
    else:
        shared = np.zeros((M, H), np.float32)
    return ids, w, moe_combine(acc, shared, gate_logits, gate_col)


def ref_layer_routed(H, I, rec_tab, ids, w, x, limit=0.0) -> np.ndarray:
    """Routed sum through the reference's own CPU backend (make_mat + matmul_multi), for pinning ho_moe_routed."""
    R = ref()
    off = rec_layout(H, I)
    h = R.ref_layer_create(H, I, len(rec_tab), C.cast(_rec_ptrs(rec_tab), C.POINTER(C.c_void_p)), _ptr(off, _u64p))
    ids = np.ascontiguousarray(ids, np.int32); w = np.ascontiguousarray(w, np.float32); x = np.ascontiguousarray(x, np.float32)
    M, K = ids.shape
    acc = np.zeros((M, H), np.float32)
    R.ref_layer_routed(h, M, K, _ptr(ids, _i32p), _ptr(w, _f32p), _ptr(x, _f32p), C.c_float(limit), _ptr(acc, _f32p))
    R.ref_layer_destroy(h)
    return acc


# ---------------------------------------------------------------------------------------------------- low-bit dense
def lb_quantize(w: np.ndarray, bits: int):
    w = np.ascontiguousarray(w, np.float32)
    N, K = w.shape
    q = np.zeros(int(_C.ho_lb_weight_bytes(bits, N, K)), np.uint8)
    s = np.zeros((N, K // 64), np.uint16); zp = np.zeros((N, K // 64), np.uint16)
    _C.ho_lb_quantize(_ptr(w, _f32p), N, K, bits, _ptr(q, _u8p), _ptr(s, _u16p), _ptr(zp, _u16p))
    return q, s, zp


def lb_dequant_bf16(q, s, zp, bits: int) -> np.ndarray:
    N, K = s.shape[0], s.shape[1] * 64
    out = np.zeros((N, K), np.uint16)
    _C.ho_lb_dequant_bf16(_ptr(q, _u8p), _ptr(s, _u16p), _ptr(zp, _u16p), bits, N, K, _ptr(out, _u16p))
    return out


def lb_gemv(q, s, zp, bits: int, a: np.ndarray) -> np.ndarray:
    N, K = s.shape[0], s.shape[1] * 64
    a = np.ascontiguousarray(np.atleast_2d(a), np.float32)
    y = np.zeros((a.shape[0], N), np.float32)
    for m in range(a.shape[0]):
        _C.ho_lb_gemv(_ptr(q, _u8p), _ptr(s, _u16p), _ptr(zp, _u16p), bits, N, K, _ptr(a[m], _f32p), 0, N, _ptr(y[m], _f32p))
    return y


def dense_act(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    g = np.ascontiguousarray(g, np.float32); u = np.ascontiguousarray(u, np.float32)
    out = np.zeros_like(g)
    _C.ho_dense_act(_ptr(g.reshape(-1), _f32p), _ptr(u.reshape(-1), _f32p), g.size, _ptr(out.reshape(-1), _f32p))
    return out


# ---------------------------------------------------------------------------------------------------- record assembly (compressed block scales)
CSF_OK, CSF_ROWS, CSF_SHAPE, CSF_TOO_MANY, CSF_EXC_INDEX, CSF_EXC_DELTA, CSF_EXC_VALUE, CSF_CODE = range(8)
_u32p = C.POINTER(C.c_uint32)


def csf_encode(scales: np.ndarray):
    """Test-side encoder written from the format description (engine/include/hive/ckpt_quant.h:5-17): base = the row's smallest code,
    entries more than 15 above it become exceptions with delta 0.  scales u8 [R, C], R % 16 == 0 → (fixed u8 [R/16, 16 + 8C], exc u32 [n])."""
    s = np.ascontiguousarray(scales, dtype=np.uint8)
    R, Cc = s.shape
    base = s.min(axis=1)
    d = s.astype(np.int32) - base[:, None]
    flat = np.flatnonzero(d.reshape(-1) > 15)
    exc = ((s.reshape(-1)[flat].astype(np.uint32) << 24) | flat.astype(np.uint32)).astype(np.uint32)
    d[d > 15] = 0
    nib = d.reshape(R // 16, 16 * Cc).astype(np.uint8)             # position n inside the group = r * C + c
    fixed = np.zeros((R // 16, 16 + 8 * Cc), dtype=np.uint8)
    fixed[:, :16] = base.reshape(R // 16, 16)
    fixed[:, 16:] = nib[:, 0::2] | (nib[:, 1::2] << 4)
    return fixed, exc


def csf_decode(fixed: np.ndarray, exc: np.ndarray, R: int, Cc: int, fixed_shape=None, use_ref: bool = False):
    """→ (status, where, scales u8 [R, C]).  use_ref: the compiled reference decoder (status 0 / -1 only, where = its message)."""
    fixed = np.ascontiguousarray(fixed, dtype=np.uint8); exc = np.ascontiguousarray(exc, dtype=np.uint32)
    fr, fc = fixed_shape if fixed_shape is not None else fixed.shape
    out = np.zeros((max(R, 0), max(Cc, 0)), dtype=np.uint8)
    ex = exc if exc.size else np.zeros(1, np.uint32)
    if use_ref:
        msg = C.create_string_buffer(256)
        ok = ref().ref_csf_decode(_ptr(fixed, _u8p), fr, fc, _ptr(ex, _u32p), exc.size, R, Cc, _ptr(out, _u8p), msg, 256)
        return (0 if ok else -1), msg.value.decode(), out
    where = C.c_int64(0)
    _C.ho_csf_decode.restype = C.c_int
    _C.ho_csf_decode.argtypes = [_u8p, C.c_int64, C.c_int64, _u32p, C.c_size_t, C.c_int, C.c_int, _u8p, C.POINTER(C.c_int64)]
    st = _C.ho_csf_decode(_ptr(fixed, _u8p), fr, fc, _ptr(ex, _u32p), exc.size, R, Cc, _ptr(out, _u8p), C.byref(where))
    return st, int(where.value), out


def record_pack(H: int, I: int, projs) -> tuple[int, np.ndarray]:
    """projs = three dicts (gate, up, down) with 'weight' u8 [rows, K/2], 'global' float and either 'scale' u8 [rows, K/16] or
    'csf_fixed' + 'csf_exc'.  → (status, record bytes)."""
    off = rec_layout(H, I)
    rec = np.zeros(int(off[7]), dtype=np.uint8)
    keep = []
    def arr(a, dt):
        a = np.ascontiguousarray(a, dtype=dt); keep.append(a); return a
    W = (C.c_void_p * 3)(); S = (C.c_void_p * 3)(); F = (C.c_void_p * 3)(); X = (C.c_void_p * 3)(); N = (C.c_size_t * 3)(); G = (C.c_float * 3)()
    for j, p in enumerate(projs):
        W[j] = arr(p["weight"], np.uint8).ctypes.data
        S[j] = arr(p["scale"], np.uint8).ctypes.data if p.get("scale") is not None else None
        if p.get("scale") is None:
            F[j] = arr(p["csf_fixed"], np.uint8).ctypes.data
            e = arr(p["csf_exc"], np.uint32)
            N[j] = e.size
            X[j] = (e if e.size else arr(np.zeros(1), np.uint32)).ctypes.data
        G[j] = float(p["global"])
    _C.ho_record_pack.restype = C.c_int
    _C.ho_record_pack.argtypes = [_u64p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, _u8p]
    st = _C.ho_record_pack(_ptr(off, _u64p), H, I, W, S, F, X, N, G, _ptr(rec, _u8p))
    return st, rec

