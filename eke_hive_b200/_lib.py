"""ctypes binding of libhive_b200.so (the C ABI declared in include/hive_b200.h).

The library is loaded from this directory; if it is missing, or a symbol the header declares is not exported, the import
fails with an error — there is no Python, PyTorch or CPU stand-in for any entry point.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

HERE = Path(__file__).resolve().parent
import os as _os

# HIVE_B200_LIB selects another build of the same library (the range-checked debug build libhive_b200_bounds.so)
LIB_PATH = Path(_os.environ["HIVE_B200_LIB"]) if _os.environ.get("HIVE_B200_LIB") else HERE / "libhive_b200.so"
HEADER = HERE.parent / "include" / "hive_b200.h"

HB_OK = 0


def _header_flags() -> dict:
    """The HB_FLAG_* context flags as include/hive_b200.h defines them (one source for the C and the Python side)."""
    import re
    return {m.group(1): int(m.group(2)) for m in re.finditer(r"^#define (HB_FLAG_\w+) (\d+)u?\b", HEADER.read_text(), re.M)}


FLAGS = _header_flags()
globals().update(FLAGS)          # HB_FLAG_NO_PDL, HB_FLAG_PREFILL_A16, HB_FLAG_DECODE_TC_GU, …


class HbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"hive_b200 status {status}: {message}")
        self.status = status


class RecLayout(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("w1", "s1", "w3", "s3", "w2", "s2", "g", "total")]


class Config(C.Structure):
    _fields_ = [("device", C.c_int), ("max_ctas", C.c_int), ("flags", C.c_int), ("wait_polls", C.c_uint)]


class MoePair(C.Structure):
    _fields_ = [("row", C.c_int32), ("rec", C.c_void_p), ("w", C.c_float)]


class PfCombine(C.Structure):
    _fields_ = [("shared", C.c_void_p), ("lg", C.c_void_p), ("ld", C.c_int), ("col", C.c_int), ("out", C.c_void_p)]


class Plan(C.Structure):
    _fields_ = [("regime", C.c_int), ("pairs", C.c_int), ("distinct_experts", C.c_int), ("max_rows", C.c_int), ("decode_groups", C.c_int),
                ("prefill_tiles", C.c_int), ("tile_fill", C.c_double), ("ws_bytes", C.c_size_t)]


class ProjSrc(C.Structure):
    _fields_ = [("weight", C.c_void_p), ("scale", C.c_void_p), ("csf_fixed", C.c_void_p), ("csf_exc", C.c_void_p), ("csf_fixed_rows", C.c_int64),
                ("csf_fixed_cols", C.c_int64), ("n_exc", C.c_uint64), ("global_", C.c_float)]


class RecordJob(C.Structure):
    _fields_ = [("src", ProjSrc * 3), ("rec", C.c_void_p)]


class KernelStat(C.Structure):
    _fields_ = [("name", C.c_char * 40), ("launches", C.c_uint32), ("total_ms", C.c_float)]


class QMat(C.Structure):
    _fields_ = [("fmt", C.c_int), ("N", C.c_int), ("K", C.c_int), ("w", C.c_void_p), ("s", C.c_void_p), ("zp", C.c_void_p), ("g", C.c_float)]


assert C.sizeof(MoePair) == 24 and MoePair.rec.offset == 8 and MoePair.w.offset == 16


def declared_symbols() -> list[str]:
    """Every function name the public header declares with HB_API."""
    text = HEADER.read_text()
    return re.findall(r"HB_API\s+[\w\s\*]+?\b(hb_\w+)\s*\(", text)


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: build it with `python eke_hive_b200/build.py` (needs nvcc); "
                          "there is no fallback implementation")
    lib = C.CDLL(str(LIB_PATH))
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    if missing:
        raise ImportError(f"{LIB_PATH} does not export {missing}; rebuild it")
    vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    sig = {
        "hb_create": (i, [C.POINTER(Config), C.POINTER(vp)]),
        "hb_destroy": (None, [vp]),
        "hb_last_error": (C.c_char_p, [vp]),
        "hb_status_string": (C.c_char_p, [i]),
        "hb_sm_count": (i, [vp]),
        "hb_check_device": (i, [vp, vp]),
        "hb_launch_count": (C.c_uint64, [vp]),
        "hb_profile_enable": (i, [vp, i]),
        "hb_profile_read": (i, [vp, C.POINTER(KernelStat), i, C.POINTER(i)]),
        "hb_rec_layout_make": (i, [i, i, C.POINTER(RecLayout)]),
        "hb_nvfp4_dequant": (i, [vp, vp, vp, f, i, i, vp, vp]),
        "hb_nvfp4_gemv": (i, [vp, vp, vp, f, i, i, vp, i, i, vp, i, vp]),
        "hb_nvfp4_quantize": (i, [vp, vp, i, i, vp, vp, vp, vp, vp]),
        "hb_requant_nvfp4": (i, [vp, vp, vp, i, i, vp, vp, vp, vp, vp]),
        "hb_a4_quant": (i, [vp, vp, i, i, i, vp, vp, vp, vp]),
        "hb_route_softmax_topk": (i, [vp, vp, i, i, i, i, i, i, vp, vp, vp]),
        "hb_route_sigmoid_topk": (i, [vp, vp, vp, i, i, i, f, vp, vp, vp]),
        "hb_build_moe_pairs": (i, [vp, vp, vp, i, i, vp, i, i, vp, vp]),
        "hb_moe_combine": (i, [vp, vp, vp, vp, i, i, i, i, vp, vp]),
        "hb_moe_decode_supported": (i, [i, i]),
        "hb_moe_decode_ws_bytes": (sz, [i, i, i]),
        "hb_moe_decode": (i, [vp, vp, i, vp, i, i, f, vp, vp, vp]),
        "hb_moe_decode_routed": (i, [vp, vp, vp, i, i, vp, i, i, vp, i, i, f, C.POINTER(PfCombine), vp, vp]),
        "hb_moe_decode_static_max_pairs": (i, [i, i]),
        "hb_moe_decode_routed_static": (i, [vp, vp, vp, i, i, vp, i, i, vp, i, i, f, C.POINTER(PfCombine), vp]),
        "hb_moe_decode_routed_f32": (i, [vp, vp, vp, i, i, vp, i, i, vp, i, i, f, vp, vp, vp]),
        "hb_moe_decode_ep_local": (i, [vp, vp, vp, i, i, i, vp, i, i, vp, i, i, i, f, vp, i, i, vp, vp, vp, vp]),
        "hb_ep_rec_bytes": (sz, [i, i]),
        "hb_ep_export": (i, [vp, vp, vp, C.POINTER(sz)]),
        "hb_ep_import": (i, [vp, vp, sz, C.POINTER(vp), C.POINTER(vp)]),
        "hb_ep_close": (i, [vp, vp]),
        "hb_ep_create": (i, [vp, i, i, i, i, i, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]),
        "hb_ep_destroy": (None, [vp]),
        "hb_ep_push_rows": (i, [vp, vp, i, vp, vp, vp]),
        "hb_ep_route_push": (i, [vp, vp, i, i, i, i, vp, i, vp, vp, vp]),
        "hb_ep_layer_local": (i, [vp, vp, i, i, i, f, vp, vp, vp, vp]),
        "hb_ep_wait_rows": (i, [vp, vp]),
        "hb_ep_push_partials": (i, [vp, vp, vp]),
        "hb_ep_combine": (i, [vp, vp, vp, i, i, vp, vp]),
        "hb_moe_layer_decode": (i, [vp, vp, i, i, i, i, i, i, vp, f, vp, i, vp, i, vp, i, i, f, vp, vp, vp, vp, vp]),
        "hb_dense_gemv_ws_bytes": (sz, [i, i, i, i]),
        "hb_dense_gemv": (i, [vp, C.POINTER(QMat), vp, i, i, vp, vp, i, vp, vp]),
        "hb_dense_gemv_gu": (i, [vp, C.POINTER(QMat), C.POINTER(QMat), vp, i, i, vp, i, vp, vp]),
        "hb_lb_dequant": (i, [vp, C.POINTER(QMat), vp, vp]),
        "hb_moe_prefill_supported": (i, [i, i]),
        "hb_moe_prefill_ws_bytes": (sz, [i, i, i, i, i]),
        "hb_moe_prefill": (i, [vp, vp, i, i, vp, vp, i, i, vp, i, i, f, vp, vp, i, vp, C.POINTER(PfCombine)]),
        "hb_nvfp4_gemm_a4": (i, [vp, C.POINTER(QMat), vp, vp, vp, i, vp, i, vp]),
        "hb_fp4_peak_probe": (i, [vp, i, C.POINTER(f)]),
        "hb_moe_layer_ws_bytes": (sz, [i, i, i, i, i]),
        "hb_moe_layer": (i, [vp, vp, i, i, i, i, i, i, vp, f, vp, i, vp, i, vp, i, i, f, vp, vp, vp, vp, vp]),
        "hb_dispatch_plan": (i, [vp, i, i, i, i, i, vp, C.POINTER(Plan)]),
        "hb_expert_dequant": (i, [vp, vp, i, i, vp, vp, vp]),
        "hb_csf_ws_bytes": (sz, [i, i]),
        "hb_csf_decode": (i, [vp, vp, C.c_int64, C.c_int64, vp, C.c_uint64, i, i, vp, vp, vp, sz, vp]),
        "hb_record_pack_ws_bytes": (sz, [i, i, i]),
        "hb_record_pack_batch": (i, [vp, vp, i, i, i, vp, vp, sz, vp]),
        "hb_record_pack": (i, [vp, C.POINTER(ProjSrc), i, i, vp, vp, vp, sz, vp]),
        "hb_gather_rows": (i, [vp, vp, vp, i, i, vp, vp]),
        "hb_swiglu_rows": (i, [vp, vp, i, i, f, vp, vp]),
        "hb_scatter_add_rows": (i, [vp, vp, vp, vp, i, i, vp, vp]),
        "hb_add_f32": (i, [vp, vp, vp, sz, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.restype = res
        fn.argtypes = args
    return lib
