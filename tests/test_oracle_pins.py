"""Pins the CPU oracle (oracle/hive_oracle.c) to the reference engine: against the golden vectors in tests/golden/
(outputs of the reference's compiled CPU code, see tests/golden/make_golden.py) everywhere, and against the compiled
reference itself (oracle/_ref) wherever that library was built."""
import ctypes as C

import numpy as np
import pytest


def test_format_tables(oracle, golden):
    t = oracle.e4m3_table()
    g = golden["e4m3_decode"]
    nan = np.isnan(g)
    assert nan.sum() == 2 and np.isnan(t[nan]).all()
    assert t[~nan].tobytes() == g[~nan].tobytes()
    assert oracle.e2m1_table().tobytes() == golden["e2m1_decode"].tobytes()


def test_format_encoders(oracle, golden):
    xs = golden["enc_in"]
    assert np.array_equal(np.array([oracle.f32_to_e4m3(x) for x in xs], np.uint8), golden["e4m3_encode"])
    assert np.array_equal(np.array([oracle.f32_to_e2m1(x) for x in xs], np.uint8), golden["e2m1_encode"])
    assert oracle.bf16r(xs).tobytes() == golden["bf16r"].tobytes()


def test_exp_portable(oracle, golden):
    got = np.array([oracle.exp_portable(x) for x in golden["exp_in"]], np.float32)
    assert got.tobytes() == golden["exp_portable"].tobytes()
    # and it is an exp: relative error ~1e-7 against libm inside the clamped range
    inside = np.abs(golden["exp_in"]) < 80
    ref = np.exp(golden["exp_in"].astype(np.float64))
    assert np.max(np.abs(got[inside] - ref[inside]) / ref[inside]) < 3e-7


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_gemv_against_golden(oracle, golden, tag):
    q, s, g, x = golden[f"gemv_{tag}_q"], golden[f"gemv_{tag}_s"], float(golden[f"gemv_{tag}_g"]), golden[f"gemv_{tag}_x"]
    y = oracle.gemv_nvfp4(q, s, g, x)
    ref = golden[f"gemv_{tag}_y_scalar"]
    # the reference's own bar between its scalar and AVX2 forms is rel < 1e-5 (engine/tests/test_nvfp4_cpu.cpp:26-60)
    assert np.max(np.abs(y - ref)) <= 1e-5 * np.max(np.abs(ref))
    if f"gemv_{tag}_y_avx2" in golden:
        assert np.max(np.abs(y - golden[f"gemv_{tag}_y_avx2"])) <= 1e-5 * np.max(np.abs(ref))


def test_gemv_negative_control(oracle, golden):
    """Swapping two neighbouring per-16 scales must change the result (the reference's own negative control)."""
    q, s, g, x = golden["gemv_b_q"], golden["gemv_b_s"].copy(), float(golden["gemv_b_g"]), golden["gemv_b_x"]
    y0 = oracle.gemv_nvfp4(q, s, g, x)
    n = int(np.argmax(s[:, 0] != s[:, 1]))
    s[n, 0], s[n, 1] = s[n, 1], s[n, 0]
    y1 = oracle.gemv_nvfp4(q, s, g, x)
    assert not np.array_equal(y0[:, n], y1[:, n])


def test_quantizer_roundtrip(oracle, golden):
    w = golden["gemv_a_w"]
    q, s, g = oracle.nvfp4_quantize(w, search=True)
    assert np.array_equal(q, golden["gemv_a_q"]) and np.array_equal(s, golden["gemv_a_s"])
    dq = oracle.bf16_to_f32(oracle.nvfp4_dequant_bf16(q, s, g))
    assert np.linalg.norm(dq - w) / np.linalg.norm(w) < 0.12
    # dequant is by definition bf16(E2M1[nib] * (e4m3(s) * g)) (engine/tests/test_glm_nvfp4.cu:17-57)
    E2, E4 = oracle.e2m1_table(), oracle.e4m3_table()
    nib = np.stack([q & 15, q >> 4], -1).reshape(q.shape[0], -1)
    sc = (np.repeat(E4[s], 16, axis=1) * np.float32(g)).astype(np.float32)
    assert np.array_equal(oracle.bf16_bits(E2[nib] * sc), oracle.nvfp4_dequant_bf16(q, s, g))
    # search can only lower the block error of the plain device rule
    q0, s0, g0 = oracle.nvfp4_quantize(w, search=False)
    dq0 = oracle.bf16_to_f32(oracle.nvfp4_dequant_bf16(q0, s0, g0))
    assert np.linalg.norm(dq - w) <= np.linalg.norm(dq0 - w) * 1.001


@pytest.mark.parametrize("tag", ["a", "b", "ties", "tails", "zero"])
def test_quantizer_against_reference_tool(oracle, tag):
    """The weight quantiser (factor search on) against outputs of the reference's own numpy quantiser
    (tools/q27_reencode.py nvfp4(), fixtures made by tests/golden/make_quantizer_golden.py): codes and block scales bit for bit;
    the per-tensor scale is stored there as the divisor 448*6/amax, here as its reciprocal."""
    from conftest import GOLDEN
    g = np.load(GOLDEN / "quantizer_golden.npz")
    w = g[f"{tag}_w"]
    q, s, g_mul = oracle.nvfp4_quantize(w, search=True)
    assert np.array_equal(q, g[f"{tag}_q"])
    assert np.array_equal(s, g[f"{tag}_s"])
    g_div = float(g[f"{tag}_g_div"][0])
    amax = float(np.max(np.abs(w)))
    if amax > 0:
        assert g_mul == np.float32(np.float32(amax) / np.float32(448.0 * 6.0))
        assert abs(g_mul * g_div - 1.0) < 2.0 ** -22
    else:
        assert g_mul == 1.0 and g_div == 1.0
    if tag == "ties":
        # the fixture really exercises the tie rule: some value sits exactly between two e2m1 codes for the chosen scale
        E2, E4 = oracle.e2m1_table(), oracle.e4m3_table()
        y = np.abs(w.reshape(w.shape[0], -1, 16).astype(np.float64) * g_div) / E4[s][..., None].astype(np.float64)
        mids = (E2[:7].astype(np.float64) + E2[1:8].astype(np.float64)) / 2
        assert np.isin(y, mids).sum() > 100


def test_expert_forward_golden(oracle, golden):
    recs, x = golden["layer_recs"], golden["layer_x"]
    H, I = x.shape[1], 64
    for m in range(x.shape[0]):
        o = oracle.expert_forward(recs[1], H, I, x[m], 0.75, 0.0, 0)
        ref = golden["expert_out"][m]
        assert np.max(np.abs(o - ref)) <= 2e-2 * np.sqrt(np.mean(ref ** 2))
        assert np.mean(o != ref) < 0.02          # bf16 outputs: at most a few one-ulp flips from fma contraction in the reference build
        o = oracle.expert_forward(recs[2], H, I, x[m] * 16, 0.5, 0.25, 0)
        ref = golden["expert_out_lim"][m]
        assert np.max(np.abs(o - ref)) <= 2e-2 * np.sqrt(np.mean(ref ** 2))


def test_routed_layer_golden(oracle, golden):
    recs, x, ids, w = golden["layer_recs"], golden["layer_x"], golden["layer_ids"], golden["layer_w"]
    H, I = x.shape[1], 64
    acc = oracle.moe_routed(H, I, ids, w, list(recs), x, 0.0, 1)
    ref = golden["layer_routed"]
    assert np.max(np.abs(acc - ref)) <= 5e-3 * np.sqrt(np.mean(ref ** 2))
    acc = oracle.moe_routed(H, I, ids, w, list(recs), x * 16, 0.25, 0)
    ref = golden["layer_routed_lim"]
    assert np.max(np.abs(acc - ref)) <= 5e-3 * np.sqrt(np.mean(ref ** 2))
    # the pair-list operator accumulates the same sum
    rows = np.repeat(np.arange(x.shape[0], dtype=np.int32), ids.shape[1])
    pr = [recs[i] if i >= 0 else None for i in ids.reshape(-1)]
    out = np.full_like(ref, 0.5)
    oracle.moe_decode(H, I, rows, pr, w.reshape(-1), x * 16, out, 0.25, 0)
    assert np.max(np.abs(out - 0.5 - ref)) <= 5e-3 * np.sqrt(np.mean(ref ** 2)) + 1e-6


def test_router_softmax_contract(oracle):
    """Known-answer cases of the router contract (engine/src/qwen/qwen_kernels.cu:159-206): ties go to the smaller id,
    logits are compared after rounding to bf16, renormalised weights sum to 1, both forms pick the same experts."""
    lg = np.array([[1.0, 3.0, 3.0, -2.0, 3.0, 0.5, 3.0009765625, 1.0]], np.float32)
    ids, w = oracle.router_softmax_topk(lg, 3, True, True, 0)
    assert ids.tolist() == [[1, 2, 4]]            # 3.0009765625 rounds to 3.0 in bf16 and loses the tie to smaller ids
    ids32, _ = oracle.router_softmax_topk(lg, 3, True, False, 0)
    assert ids32.tolist() == [[6, 1, 2]]
    assert abs(float(w.sum()) - 1.0) < 1e-6 and np.allclose(w, 1 / 3, atol=1e-7)
    rng = np.random.default_rng(5)
    lg = rng.normal(0, 1, (64, 512)).astype(np.float32)
    i0, w0 = oracle.router_softmax_topk(lg, 10, True, True, 0)
    i1, w1 = oracle.router_softmax_topk(lg, 10, True, True, 1)
    assert np.array_equal(i0, i1)
    assert np.max(np.abs(w0 - w1) / w1) < 4 * 2.0 ** -23 * 4
    assert np.all(np.diff(w0, axis=1) <= 0)
    i2, w2 = oracle.router_softmax_topk(lg, 10, False, True, 0)
    assert np.array_equal(i0, i2) and np.all(w2.sum(1) < 1.0)


def test_router_sigmoid_contract(oracle):
    lg = np.array([[0.0, 2.0, 2.0, -1.0, 0.1]], np.float32)
    bias = np.array([0.0, 0.0, 0.0, 5.0, 0.0], np.float32)
    ids, w = oracle.router_sigmoid_topk(lg, bias, 3, 2.5, 0)
    assert ids.tolist() == [[3, 1, 2]]            # bias selects, the unbiased score weighs; tie 1 vs 2 → smaller id
    s = 1 / (1 + np.exp(-lg[0, [3, 1, 2]].astype(np.float64)))
    assert np.allclose(w[0], s / s.sum() * 2.5, rtol=1e-6)
    rng = np.random.default_rng(6)
    lg = rng.normal(0, 1, (32, 160)).astype(np.float32); bias = rng.normal(0, 0.1, 160).astype(np.float32)
    i0, _ = oracle.router_sigmoid_topk(lg, bias, 8, 1.0, 0)
    i1, _ = oracle.router_sigmoid_topk(lg, bias, 8, 1.0, 1)
    assert np.array_equal(i0, i1)


def test_a4_quant_properties(oracle):
    rng = np.random.default_rng(7)
    x = oracle.bf16r(rng.normal(0, 1, (5, 256)).astype(np.float32))
    x[3] = 0
    q, s, g = oracle.a4_quant(x)
    assert g[3] == 1.0 and not q[3].any() and not s[3].any()
    E2, E4 = oracle.e2m1_table(), oracle.e4m3_table()
    nib = np.stack([q & 15, q >> 4], -1).reshape(5, -1)
    dq = E2[nib] * np.repeat(E4[s], 16, axis=1) * g[:, None]
    assert np.linalg.norm(dq - x) / np.linalg.norm(x) < 0.12
    assert np.all(np.abs(dq).max(1) <= np.abs(x).max(1) * 1.07)


def test_lowbit_pack_roundtrip(oracle):
    rng = np.random.default_rng(8)
    w = rng.normal(0, 0.02, (24, 256)).astype(np.float32)
    for bits, tol in ((3, 0.25), (2, 0.5)):
        q, s, zp = oracle.lb_quantize(w, bits)
        assert q.size == 24 * 256 * bits // 8
        dq = oracle.bf16_to_f32(oracle.lb_dequant_bf16(q, s, zp, bits))
        assert np.linalg.norm(dq - w) / np.linalg.norm(w) < tol
        x = oracle.bf16r(rng.normal(0, 1, (2, 256)).astype(np.float32))
        y = oracle.lb_gemv(q, s, zp, bits, x)
        ref = x.astype(np.float64) @ dq.astype(np.float64).T
        assert np.max(np.abs(y - ref)) < 2e-2 * np.sqrt(np.mean(ref ** 2))


def test_restatement_matches_compiled_reference(oracle):
    """Live comparison with the compiled reference on fresh seeds (skipped where oracle/_ref was never built)."""
    if not oracle.have_ref():
        pytest.skip("oracle/_ref/libhive_ref.so not built on this machine")
    R = oracle.ref()
    rng = np.random.default_rng(99)
    for x in rng.normal(0, 10, 2000).astype(np.float32):
        assert R.ref_f32_to_e4m3(C.c_float(x)) == oracle.f32_to_e4m3(x)
        assert R.ref_f32_to_e2m1(C.c_float(x)) == oracle.f32_to_e2m1(x)
        assert R.ref_exp_portable(C.c_float(x)) == oracle.exp_portable(x)
    H, I, E = 256, 128, 6
    recs = [oracle.pack_record(H, I, *[oracle.nvfp4_quantize(rng.normal(0, 0.02, sh).astype(np.float32), False)
                                       for sh in ((I, H), (I, H), (H, I))]) for _ in range(E)]
    x = oracle.bf16r(rng.normal(0, 1, (9, H)).astype(np.float32))     # 9 rows: one expert gets > 8 rows (the reference's GEMM path)
    ids = np.stack([rng.permutation(E)[:2] for _ in range(9)]).astype(np.int32)
    ids[:, 0] = 2
    w = rng.uniform(0.1, 0.9, ids.shape).astype(np.float32)
    acc = oracle.moe_routed(H, I, ids, w, recs, x, 0.0, 1)
    ref = oracle.ref_layer_routed(H, I, recs, ids, w, x)
    assert np.max(np.abs(acc - ref)) <= 5e-3 * np.sqrt(np.mean(ref ** 2))
    o = oracle.expert_forward(recs[0], H, I, x[0], 0.3, 0.0, 0)
    r = oracle.expert_forward(recs[0], H, I, x[0], 0.3, 0.0, 0, use_ref=True)
    assert np.max(np.abs(o - r)) <= 5e-3 * np.sqrt(np.mean(r ** 2))
