"""GPU parity, routed-expert decode: the three decode entry points against the CPU oracle on identical seeded inputs, on
the streaming tensor-core path (H, I multiples of 256) and on the generic path (any multiple of 32), plus golden fixtures
produced by the reference's own CPU code.  Tolerance: max-abs-error ≤ 2e-2 × per-row RMS of the reference output."""
import numpy as np
import pytest

from util import bf16_bits_of, bf16_tensor, make_records, random_records, rel_rms_err, upload

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def E():
    import eke_hive_b200 as E
    return E


@pytest.fixture(params=[8, 64, 192], ids=["mma_sync", "tensor_memory_gate_up", "tensor_memory_both"])
def eng(request, E):
    """A context pinned to one of the decode engines of the routed operators (HB_FLAG_DECODE_MMA_SYNC: the streaming kernels throughout;
    HB_FLAG_DECODE_TC_GU: gate/up on the tensor-memory kernel between the streaming path's grouping and down kernels)."""
    c = E.Context(flags=request.param)
    yield c
    c.close()


def _routing(rng, M, Ex, K):
    ids = np.stack([rng.permutation(Ex)[:K] for _ in range(M)]).astype(np.int32)
    w = rng.uniform(0.05, 0.5, (M, K)).astype(np.float32)
    return ids, w


def test_golden_routed_layer_generic_path(E, oracle, golden):
    """Inputs and expected output come from the reference's CPU backend (tests/golden): H=128, I=64 → generic kernels."""
    import torch
    recs, x, ids, w = golden["layer_recs"], golden["layer_x"], golden["layer_ids"], golden["layer_w"]
    H, I = 128, 64
    assert E.moe_decode_supported(H, I) == 1
    drecs = upload(list(recs))
    tab = E.rec_table(drecs)
    for scale, limit, key in ((1.0, 0.0, "layer_routed"), (16.0, 0.25, "layer_routed_lim")):
        pairs = E.build_moe_pairs(torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), tab, 0, len(recs))
        out = torch.zeros((4, H), dtype=torch.float32, device="cuda")
        E.moe_decode(pairs, bf16_tensor(x * scale), H, I, limit, out)
        assert rel_rms_err(out.cpu().numpy(), golden[key]) <= TOL


@pytest.mark.parametrize("H,I,Ex,K,M", [(256, 256, 8, 2, 3), (2048, 512, 64, 8, 1), (2048, 512, 16, 4, 16), (1024, 768, 12, 3, 9),
                                          (512, 1536, 6, 2, 5), (4096, 256, 4, 2, 2), (768, 3072, 4, 2, 3),
                                          (256, 256, 24, 17, 3)])          # last: more than 16 experts per row (the sums run over every k)
def test_routed_fast_path_vs_oracle(E, oracle, H, I, Ex, K, M):
    import torch
    assert E.moe_decode_supported(H, I) == 2
    rng = np.random.default_rng(H + I + M)
    recs = make_records(oracle, H, I, Ex, seed=H * 3 + I) if H * I <= 2048 * 512 and Ex <= 16 else random_records(oracle, H, I, Ex, seed=H + I)
    x = oracle.bf16r(rng.normal(0, 1, (M, H)).astype(np.float32))
    ids, w = _routing(rng, M, Ex, K)
    if M >= 9:
        ids[:, 0] = 1                                            # one expert gets every row: more than one group of 8
        for m in range(M):
            if (ids[m, 1:] == 1).any():
                ids[m, 1:][ids[m, 1:] == 1] = (0 if 0 not in ids[m] else 2)
    if M >= 3:
        ids[1, -1] = -1                                          # invalid id: contributes nothing
    shared = oracle.bf16r(rng.normal(0, 0.1, (M, H)).astype(np.float32))
    lg = rng.normal(0, 1, (M, 3)).astype(np.float32)
    drecs = upload(recs)
    out = E.fn_moe_decode_routed(torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), E.rec_table(drecs), 0, Ex, bf16_tensor(x), H, I,
                                 shared=bf16_tensor(shared), lg=torch.from_numpy(lg).cuda(), col=1)
    acc = oracle.moe_routed(H, I, ids, w, recs, x, 0.0, 0)
    ref = oracle.bf16_to_f32(oracle.moe_combine(acc, shared, lg, 1, True))
    got = out.float().cpu().numpy()
    assert rel_rms_err(got, ref) <= TOL
    E.context().check_device()
    # run-to-run determinism, bit for bit
    out2 = E.fn_moe_decode_routed(torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), E.rec_table(drecs), 0, Ex, bf16_tensor(x), H, I,
                                  shared=bf16_tensor(shared), lg=torch.from_numpy(lg).cuda(), col=1)
    assert torch.equal(out, out2)
    # the register-dequantisation kernels forced (HB_FLAG_DECODE_MMA_SYNC = 8) and their single persistent kernel form
    # (HB_FLAG_FUSED = 2), which performs the same arithmetic in the same order: bit-identical to the three-kernel form
    outs = []
    for flags in (8, 2):
        c = E.Context(flags=flags)
        o = E.fn_moe_decode_routed(torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), E.rec_table(drecs), 0, Ex, bf16_tensor(x), H, I,
                                   shared=bf16_tensor(shared), lg=torch.from_numpy(lg).cuda(), col=1, ctx=c)
        torch.cuda.synchronize()
        c.check_device()
        outs.append(o)
        c.close()
    assert rel_rms_err(outs[0].float().cpu().numpy(), ref) <= TOL
    assert torch.equal(outs[0], outs[1])
    # gate/up on the tensor-memory kernel, the rest on the streaming kernels (HB_FLAG_DECODE_TC_GU = 64): tolerance, and bit-identical
    # run to run
    o64 = []
    for _ in range(2):
        c = E.Context(flags=64)
        o64.append(E.fn_moe_decode_routed(torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), E.rec_table(drecs), 0, Ex, bf16_tensor(x), H, I,
                                          shared=bf16_tensor(shared), lg=torch.from_numpy(lg).cuda(), col=1, ctx=c))
        torch.cuda.synchronize()
        c.check_device()
        c.close()
    assert rel_rms_err(o64[0].float().cpu().numpy(), ref) <= TOL
    assert torch.equal(o64[0], o64[1])


def test_pair_list_accumulates_in_pair_order(E, oracle):
    """hb_moe_decode: shuffled pair order, a repeated (row, expert), a null record, out pre-filled (the operator accumulates)."""
    import torch
    H, I, Ex = 512, 256, 6
    rng = np.random.default_rng(21)
    recs = make_records(oracle, H, I, Ex, seed=77)
    drecs = upload(recs)
    x = oracle.bf16r(rng.normal(0, 1, (5, H)).astype(np.float32))
    rows = np.array([3, 0, 4, 3, 1, 0, 2, 3, 4, 0, 3], np.int32)
    eids = np.array([1, 2, 0, 1, 5, 2, 3, 4, 4, 1, -1], np.int32)
    w = rng.uniform(0.1, 0.9, rows.size).astype(np.float32)
    pr = [None if e < 0 else recs[e] for e in eids]
    dpr = [None if e < 0 else drecs[e] for e in eids]
    pairs = E.make_pairs(rows, dpr, w, "cuda")
    out0 = rng.normal(0, 0.01, (5, H)).astype(np.float32)
    out = torch.from_numpy(out0.copy()).cuda()
    E.moe_decode(pairs, bf16_tensor(x), H, I, 0.0, out)
    ref = out0.copy()
    oracle.moe_decode(H, I, rows, pr, w, x, ref, 0.0, 0)
    assert rel_rms_err(out.cpu().numpy() - out0, ref - out0) <= TOL
    # with a clamp
    out = torch.zeros((5, H), dtype=torch.float32, device="cuda")
    E.moe_decode(pairs, bf16_tensor(x * 8), H, I, 0.5, out)
    ref = np.zeros((5, H), np.float32)
    oracle.moe_decode(H, I, rows, pr, w, x * 8, ref, 0.5, 0)
    assert rel_rms_err(out.cpu().numpy(), ref) <= TOL


def test_outlier_activations_stay_finite(E, oracle):
    """Activations far outside the f16 range (±3e5, the reference's own case in engine/tests/test_glm_moe.cu): the streaming path
    rescales each row slice by a power of two, so results stay finite and within tolerance."""
    import torch
    H, I, Ex = 1024, 256, 4
    rng = np.random.default_rng(31)
    recs = make_records(oracle, H, I, Ex, seed=5)
    x = oracle.bf16r(rng.normal(0, 1, (3, H)).astype(np.float32))
    x[0, 17] = 3.0e5; x[1, 900] = -3.0e5; x[2] *= 1e-6
    x = oracle.bf16r(x)
    ids = np.array([[0, 1], [2, 1], [3, 0]], np.int32)
    w = np.full((3, 2), 0.5, np.float32)
    acc = oracle.moe_routed(H, I, ids, w, recs, x, 0.0, 0)
    out = torch.zeros((3, H), dtype=torch.float32, device="cuda")
    drecs = upload(recs)
    pairs = E.build_moe_pairs(torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), E.rec_table(drecs), 0, Ex)
    E.moe_decode(pairs, bf16_tensor(x), H, I, 0.0, out)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_rms_err(got, acc) <= TOL


@pytest.mark.parametrize("router", ["softmax", "sigmoid"])
def test_whole_layer_with_shared_expert(E, oracle, router, eng):
    """hb_moe_layer_decode against the oracle's layer (config-1 style: H 2048, I 512, 64 experts, top-8, NVFP4 shared expert)."""
    import torch
    H, I, Ex, K, M = 2048, 512, 64, 8, 4
    rng = np.random.default_rng(41)
    recs = random_records(oracle, H, I, Ex + 1, seed=9)
    # scale the random records' globals so outputs are O(1)
    x = oracle.bf16r(rng.normal(0, 1, (M, H)).astype(np.float32))
    logits = rng.normal(0, 1, (M, Ex + 1)).astype(np.float32)        # column Ex = the shared-expert gate logit
    drecs = upload(recs)
    tab = E.rec_table(drecs[:Ex])
    if router == "softmax":
        ids, w, out = E.moe_layer_decode(torch.from_numpy(logits).cuda(), bf16_tensor(x), tab, 0, Ex, K, H, I, shared_rec=drecs[Ex], gate_col=Ex, ctx=eng)
        rids, rw, rout = oracle.moe_layer(H, I, logits, x, recs[:Ex], K, shared_rec=recs[Ex], gate_logits=logits, gate_col=Ex)
    else:
        bias = rng.normal(0, 0.2, Ex).astype(np.float32)
        lg = np.ascontiguousarray(logits[:, :Ex])
        ids, w, out = E.moe_layer_decode(torch.from_numpy(lg).cuda(), bf16_tensor(x), tab, 0, Ex, K, H, I, shared_rec=drecs[Ex], gate_col=-1,
                                         bias=torch.from_numpy(bias).cuda(), sigmoid_scale=2.5, limit=10.0, ctx=eng)
        rids, rw, rout = oracle.moe_layer(H, I, lg, x, recs[:Ex], K, shared_rec=recs[Ex], router="sigmoid", bias=bias, scale=2.5, limit=10.0)
    assert np.array_equal(ids.cpu().numpy(), rids)                   # routing indices bit-exact
    assert w.cpu().numpy().tobytes() == rw.tobytes()
    assert rel_rms_err(out.float().cpu().numpy(), oracle.bf16_to_f32(rout)) <= TOL
    torch.cuda.synchronize()
    eng.check_device()


def test_batch_invariance_and_weight_linearity(E, oracle):
    """Size-independent properties at the full config-2 expert shape with many experts: a row's result does not depend on which
    other rows share the batch (bit-exact), and doubling every routing weight doubles the fp32 routed sum exactly."""
    import torch
    H, I, Ex, K, M = 2048, 512, 96, 10, 16
    rng = np.random.default_rng(51)
    recs = random_records(oracle, H, I, 8, seed=3)
    drecs = upload(recs)
    drecs = [drecs[i % 8].clone() for i in range(Ex)]                # distinct device copies: 96 records, 170 MB
    tab = E.rec_table(drecs)
    x = bf16_tensor(oracle.bf16r(rng.normal(0, 1, (M, H)).astype(np.float32)))
    ids_np, w_np = _routing(rng, M, Ex, K)
    ids = torch.from_numpy(ids_np).cuda(); w = torch.from_numpy(w_np).cuda()
    pairs = E.build_moe_pairs(ids, w, tab, 0, Ex)
    full = torch.zeros((M, H), dtype=torch.float32, device="cuda")
    E.moe_decode(pairs, x, H, I, 0.0, full)
    for m in (0, 7, 15):
        one = torch.zeros((1, H), dtype=torch.float32, device="cuda")
        p1 = E.build_moe_pairs(ids[m:m + 1].contiguous(), w[m:m + 1].contiguous(), tab, 0, Ex)
        E.moe_decode(p1, x[m:m + 1].contiguous(), H, I, 0.0, one)
        assert torch.equal(one[0], full[m])
    dbl = torch.zeros((M, H), dtype=torch.float32, device="cuda")
    E.moe_decode(E.build_moe_pairs(ids, (w * 2).contiguous(), tab, 0, Ex), x, H, I, 0.0, dbl)
    assert torch.equal(dbl, full * 2)
    # spot-check two rows against the oracle
    host = [r.cpu().numpy() for r in drecs]
    acc = oracle.moe_routed(H, I, ids_np[[0, 15]], w_np[[0, 15]], host, x[[0, 15]].float().cpu().numpy(), 0.0, 0)
    assert rel_rms_err(full[[0, 15]].cpu().numpy(), acc) <= TOL
    E.context().check_device()


def test_routed_rows_do_not_depend_on_the_batch(E, oracle, eng):
    """Routed form, every engine: a row run alone gives the bits it gives inside a batch of 12 (its expert groups then hold other rows
    too), and a second run of the batch repeats the first bit for bit."""
    import torch
    H, I, Ex, K, M = 2048, 512, 24, 6, 12
    rng = np.random.default_rng(77)
    recs = random_records(oracle, H, I, 6, seed=9)
    drecs = upload(recs)
    drecs = [drecs[i % 6].clone() for i in range(Ex)]
    tab = E.rec_table(drecs)
    x = bf16_tensor(oracle.bf16r((rng.normal(0, 1, (M, H)) * np.exp(rng.normal(0, 1, (M, 1)))).astype(np.float32)))
    ids_np, w_np = _routing(rng, M, Ex, K)
    ids = torch.from_numpy(ids_np).cuda(); w = torch.from_numpy(w_np).cuda()
    full = E.moe_decode_routed_f32(ids, w, tab, 0, Ex, x, H, I, ctx=eng)
    again = E.moe_decode_routed_f32(ids, w, tab, 0, Ex, x, H, I, ctx=eng)
    assert torch.equal(full, again)
    for m in (0, 5, 11):
        one = E.moe_decode_routed_f32(ids[m:m + 1].contiguous(), w[m:m + 1].contiguous(), tab, 0, Ex, x[m:m + 1].contiguous(), H, I, ctx=eng)
        assert torch.equal(one[0], full[m]), m
    torch.cuda.synchronize()
    eng.check_device()


def test_decode_argument_errors(E):
    import torch
    x = torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((1, 256), dtype=torch.float32, device="cuda")
    pairs = torch.zeros((1, 24), dtype=torch.uint8, device="cuda")
    with pytest.raises(E.HbError) as ei:
        E.moe_decode(pairs, x, 250, 256, 0.0, out)                   # H not a multiple of 32
    assert ei.value.status == -2
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    with pytest.raises(E.HbError) as ei:
        E.moe_decode(pairs, x, 256, 256, 0.0, out, ws=ws[1:])        # misaligned workspace
    assert ei.value.status == -5
    # an all-null pair list is a no-op, not an error
    E.moe_decode(pairs, x, 256, 256, 0.0, out)
    assert float(out.abs().sum()) == 0.0


def test_ep_local_matches_separate_operators(E, oracle, eng):
    """hb_moe_decode_ep_local on strided views of a packed exchange buffer (with NULL table entries for experts held elsewhere)
    equals the routed fp32 operator on contiguous copies bit for bit, and its shared-expert rows equal a separate pass."""
    import torch
    H, I, Ex, K, G, B = 2048, 512, 16, 4, 2, 8
    M = G * B
    rng = np.random.default_rng(5)
    recs = random_records(oracle, H, I, Ex + 1, 31)
    drecs = upload(recs)
    local = [drecs[e] if e < Ex // 2 else None for e in range(Ex)]              # rank 0 of 2 holds the first half
    tab = E.rec_table(local)
    rec_bytes = (H * 2 + K * 8 + 15) // 16 * 16
    buf = torch.zeros((M, rec_bytes), dtype=torch.uint8, device="cuda")
    x = bf16_tensor(rng.standard_normal((M, H)).astype(np.float32))
    ids = torch.from_numpy(np.stack([rng.permutation(Ex)[:K] for _ in range(M)]).astype(np.int32)).cuda()
    w = torch.from_numpy(rng.random((M, K), dtype=np.float32)).cuda()
    buf[:, :H * 2] = x.view(torch.uint8).view(M, H * 2)
    buf[:, H * 2:H * 2 + K * 4] = ids.view(torch.uint8).view(M, K * 4)
    buf[:, H * 2 + K * 4:H * 2 + K * 8] = w.view(torch.uint8).view(M, K * 4)
    xv, iv, wv = buf[:, :H * 2].view(torch.bfloat16), buf[:, H * 2:H * 2 + K * 4].view(torch.int32), buf[:, H * 2 + K * 4:H * 2 + K * 8].view(torch.float32)
    routed = torch.empty((M, H), dtype=torch.float32, device="cuda")
    shared = torch.empty((B, H), dtype=torch.bfloat16, device="cuda")
    E.moe_decode_ep_local(iv, wv, tab, 0, Ex, xv, H, I, routed, shared_ptr=drecs[Ex].data_ptr(), sh_row0=B, sh_rows=B, shared_out=shared, ctx=eng)
    ref = torch.empty_like(routed)
    E.moe_decode_routed_f32(ids, w, tab, 0, Ex, x, H, I, out=ref, ctx=eng)
    one_tab = E.rec_table([drecs[Ex]])
    sh_ref = torch.empty((B, H), dtype=torch.float32, device="cuda")
    E.moe_decode_routed_f32(torch.zeros((B, 1), dtype=torch.int32, device="cuda"), torch.ones((B, 1), dtype=torch.float32, device="cuda"), one_tab, 0, 1,
                            x[B:2 * B].contiguous(), H, I, out=sh_ref, ctx=eng)
    torch.cuda.synchronize()
    eng.check_device()
    assert torch.equal(routed, ref)
    assert torch.equal(shared.float(), sh_ref)


def test_glm_shaped_layer_with_zipf_bias(E, oracle, eng):
    """The GLM-style configuration at its full shape: hidden 4096, intermediate 1536, 160 routed experts, top-8 + shared expert,
    8 tokens, sigmoid router with a Zipf(1.1) log-weight bias over a seeded permutation of the experts, SwiGLU clamp 10."""
    import torch
    H, I, Ex, K, M = 4096, 1536, 160, 8, 8
    rng = np.random.default_rng(160)
    recs = random_records(oracle, H, I, Ex + 1, seed=160)
    x = oracle.bf16r(rng.normal(0, 1, (M, H)).astype(np.float32))
    lg = rng.normal(0, 1, (M, Ex)).astype(np.float32)
    zipf = 1.0 / np.arange(1, Ex + 1) ** 1.1
    bias = np.log(zipf / zipf.sum())[rng.permutation(Ex)].astype(np.float32)
    drecs = upload(recs)
    tab = E.rec_table(drecs[:Ex])
    ids, w, out = E.moe_layer_decode(torch.from_numpy(lg).cuda(), bf16_tensor(x), tab, 0, Ex, K, H, I, shared_rec=drecs[Ex], gate_col=-1,
                                     bias=torch.from_numpy(bias).cuda(), sigmoid_scale=2.5, limit=10.0, ctx=eng)
    rids, rw, rout = oracle.moe_layer(H, I, lg, x, recs[:Ex], K, shared_rec=recs[Ex], router="sigmoid", bias=bias, scale=2.5, limit=10.0)
    assert np.array_equal(ids.cpu().numpy(), rids)
    assert w.cpu().numpy().tobytes() == rw.tobytes()
    assert rel_rms_err(out.float().cpu().numpy(), oracle.bf16_to_f32(rout)) <= TOL
    hot = np.bincount(rids.ravel(), minlength=Ex)
    assert hot.max() >= 4                                            # the bias does skew the routing: some expert takes several of the 8 rows
    torch.cuda.synchronize()
    eng.check_device()
