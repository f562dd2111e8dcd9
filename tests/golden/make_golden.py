"""Generates tests/golden/hotpath_golden.npz from the reference engine's own CPU code.

Run where the reference tree is mounted (it compiles oracle/_ref/libhive_ref.so from the reference sources in place):

    python tests/golden/make_golden.py

Every array is the output of the compiled reference for seeded inputs that are stored beside it, so the fixtures can be
checked anywhere without the reference.  Seeds and shapes are fixed below; rerunning must reproduce the file bit for bit.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402


def main():
    O.build(ref=True)
    R = O.ref()
    rng = np.random.default_rng(20261125)
    out = {}
    # -- number formats: full decode tables, encode sweeps (reference: engine/include/hive/common.h)
    out["e4m3_decode"] = np.array([R.ref_e4m3_to_f32(i) for i in range(256)], np.float32)
    out["e2m1_decode"] = np.array([R.ref_e2m1_to_f32(i) for i in range(16)], np.float32)
    xs = np.concatenate([rng.normal(0, 1, 3000), rng.normal(0, 200, 3000), rng.normal(0, 0.01, 3000),
                         np.array([0, -0.0, 448, 449, 464, 1e9, 2.0**-10, 2.0**-9, 3 * 2.0**-10, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6, 7]),
                         out["e4m3_decode"][:127].astype(np.float64), (out["e4m3_decode"][:126] + out["e4m3_decode"][1:127]) / 2]).astype(np.float32)
    out["enc_in"] = xs
    out["e4m3_encode"] = np.array([R.ref_f32_to_e4m3(C.c_float(x)) for x in xs], np.uint8)
    out["e2m1_encode"] = np.array([R.ref_f32_to_e2m1(C.c_float(x)) for x in xs], np.uint8)
    out["bf16r"] = np.array([R.ref_bf16r(C.c_float(x)) for x in xs], np.float32)
    ex = np.concatenate([rng.normal(0, 3, 4000), rng.uniform(-90, 90, 2000), [0.0, -1e-9, 1e-9, -87.5, 88.5]]).astype(np.float32)
    out["exp_in"] = ex
    out["exp_portable"] = np.array([R.ref_exp_portable(C.c_float(x)) for x in ex], np.float32)
    # -- NVFP4 GEMV (reference: gemv_nvfp4_rows_scalar and the AVX2 gemv_nvfp4_rows)
    for tag, (N, K) in {"a": (37, 64), "b": (48, 512)}.items():
        w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
        q, s, g = O.nvfp4_quantize(w, search=True)
        a = O.bf16r(rng.normal(0, 1, (3, K)).astype(np.float32))
        out[f"gemv_{tag}_w"] = w; out[f"gemv_{tag}_q"] = q; out[f"gemv_{tag}_s"] = s; out[f"gemv_{tag}_g"] = np.float32(g)
        out[f"gemv_{tag}_x"] = a
        out[f"gemv_{tag}_y_scalar"] = O.gemv_nvfp4(q, s, g, a, use_ref=True, scalar=True)
        out[f"gemv_{tag}_y_avx2"] = O.gemv_nvfp4(q, s, g, a, use_ref=True, scalar=False)
    # a matrix with every e4m3 scale code (sign bit included, NaN codes left out) and every nibble, as the reference's own test does
    N, K = 32, 128
    q = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    s = np.resize(codes, (N, K // 16)).astype(np.uint8)
    a = O.bf16r(rng.normal(0, 1, (2, K)).astype(np.float32))
    out["gemv_c_q"] = q; out["gemv_c_s"] = s; out["gemv_c_g"] = np.float32(0.0031); out["gemv_c_x"] = a
    out["gemv_c_y_scalar"] = O.gemv_nvfp4(q, s, 0.0031, a, use_ref=True, scalar=True)
    # -- one expert and a routed layer (reference: expert_forward_nvfp4; make_mat + matmul_multi in the CPU daemon's order)
    H, I, E, M, K_ = 128, 64, 8, 4, 3
    recs = []
    for e in range(E):
        mats = [O.nvfp4_quantize(rng.normal(0, 0.02, sh).astype(np.float32)) for sh in ((I, H), (I, H), (H, I))]
        recs.append(O.pack_record(H, I, *mats))
    x = O.bf16r(rng.normal(0, 1, (M, H)).astype(np.float32))
    out["layer_recs"] = np.stack(recs); out["layer_x"] = x
    out["expert_out"] = np.stack([O.expert_forward(recs[1], H, I, x[m], 0.75, 0.0, use_ref=True) for m in range(M)])
    out["expert_out_lim"] = np.stack([O.expert_forward(recs[2], H, I, x[m] * 16, 0.5, 0.25, use_ref=True) for m in range(M)])
    ids = np.array([[0, 3, 5], [7, 1, 3], [3, 2, -1], [6, 6, 4]], np.int32)   # an invalid id and a repeated expert
    wts = rng.uniform(0.1, 0.6, (M, K_)).astype(np.float32)
    out["layer_ids"] = ids; out["layer_w"] = wts
    out["layer_routed"] = O.ref_layer_routed(H, I, recs, ids, wts, x, 0.0)
    out["layer_routed_lim"] = O.ref_layer_routed(H, I, recs, ids, wts, x * 16, 0.25)
    np.savez_compressed(Path(__file__).resolve().parent / "hotpath_golden.npz", **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
