"""GPU parity of the prefill path: the block-scaled FP4 GEMM against an fp64 evaluation of the same quantised operands, and
hb_moe_prefill against the CPU oracle's W4A4 expert (activations quantised by the reference's a4 rule, fn_moe_pf.cu:456-502)."""
import numpy as np
import pytest
import torch

from util import random_records, upload

pytestmark = pytest.mark.gpu

E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def _lut_e2m1(dev):
    return torch.tensor(E2M1 + [-v for v in E2M1], dtype=torch.float64, device=dev)


def _lut_e4m3(dev):
    v = np.zeros(256)
    for b in range(256):
        e, m = (b >> 3) & 15, b & 7
        mag = m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
        v[b] = -mag if b & 0x80 else mag
    return torch.tensor(v, dtype=torch.float64, device=dev)


def dequant64(q, s):
    """codes u8 [R, K/2] + e4m3 scales u8 [R, K/16] → fp64 [R, K] (no global)."""
    dev = q.device
    lo, hi = (q & 0xF).long(), (q >> 4).long()
    codes = torch.stack([lo, hi], dim=-1).reshape(q.shape[0], -1)
    vals = _lut_e2m1(dev)[codes]
    sc = _lut_e4m3(dev)[s.long()].repeat_interleave(16, dim=1)
    return vals * sc


@pytest.fixture(scope="module")
def E():
    import eke_hive_b200 as E
    return E


def test_fp4_peak_probe_runs(E):
    tf = E.fp4_peak_probe(512)
    assert 100.0 < tf < 20000.0, tf


@pytest.mark.parametrize("M,N,K", [(128, 256, 256), (100, 256, 512), (300, 512, 2048), (1024, 1024, 7168)])
def test_gemm_a4_matches_fp64(E, M, N, K):
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N + K)
    x = (torch.randn((M, K), generator=g) * torch.exp(torch.randn((M, 1), generator=g))).to(torch.bfloat16).to(dev)
    wq = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g).to(dev)
    ws = torch.randint(0x20, 0x48, (N, K // 16), dtype=torch.uint8, generator=g).to(dev)
    xq, xs, xg = E.a4_quant(x)
    W = E.GMat(E.FMT_NVFP4, N, K, wq, ws, None, 0.0123)
    y = E.nvfp4_gemm_a4(W, xq, xs, xg)
    torch.cuda.synchronize()
    E.context().check_device()
    A, B = dequant64(xq, xs), dequant64(wq, ws)
    ref = (A @ B.T) * xg.double()[:, None] * 0.0123
    bound = (A.abs() @ B.abs().T) * xg.double()[:, None] * 0.0123
    err = (y.double() - ref).abs()
    assert torch.all(err <= 2e-6 * bound + 1e-30), float((err / (bound + 1e-30)).max())


def _oracle_prefill(oracle, recs, H, I, ids, w, x_f32, limit=0.0):
    """Σ_k w·bf16(expert(x)) per row with the W4A4 rounding points, on the CPU."""
    M, K = ids.shape
    out = np.zeros((M, H), dtype=np.float32)
    for m in range(M):
        for k in range(K):
            e = int(ids[m, k])
            if e < 0 or e >= len(recs) or recs[e] is None:
                continue
            out[m] += oracle.expert_forward_a4(recs[e], H, I, x_f32[m], limit) * np.float32(w[m, k])
    return out


@pytest.mark.parametrize("H,I,E_,K,M,S", [(256, 256, 4, 2, 70, 70), (512, 256, 8, 2, 300, 128), (2048, 512, 16, 4, 200, 200),
                                            (7168, 2048, 3, 2, 40, 40)])          # last: the DeepSeek-shaped expert at full size
def test_moe_prefill_vs_oracle(E, oracle, H, I, E_, K, M, S):
    dev = torch.device("cuda")
    rng = np.random.default_rng(H + I + M)
    recs = random_records(oracle, H, I, E_, H + M)
    keep = upload(recs, dev)
    tab = E.rec_table(keep)
    ids = np.stack([rng.permutation(E_)[:K] for _ in range(M)]).astype(np.int32)
    ids[3, 0] = -1
    ids[5, 1] = E_ + 3
    w = rng.random((M, K), dtype=np.float32)
    x = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16)
    out = E.fn_moe_prefill(tab, 0, E_, torch.tensor(ids, device=dev), torch.tensor(w, device=dev), x.to(dev), H, I, S=S)
    torch.cuda.synchronize()
    E.context().check_device()
    ref = _oracle_prefill(oracle, recs, H, I, ids, w, x.float().numpy())
    got = out.cpu().numpy()
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-12
    assert np.max(np.abs(got - ref) / rms) <= 2e-2          # tolerance of the expert-output gate: 2e-2 × row RMS


def test_moe_prefill_combine_matches_separate(E, oracle):
    dev = torch.device("cuda")
    H, I, E_, K, M = 512, 256, 8, 2, 150
    rng = np.random.default_rng(11)
    recs = random_records(oracle, H, I, E_, 11)
    keep = upload(recs, dev)
    tab = E.rec_table(keep)
    ids = torch.tensor(np.stack([rng.permutation(E_)[:K] for _ in range(M)]).astype(np.int32), device=dev)
    w = torch.tensor(rng.random((M, K), dtype=np.float32), device=dev)
    x = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
    shared = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
    lg = torch.tensor(rng.standard_normal((M, 3)).astype(np.float32), device=dev)
    routed = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I)
    fused = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, shared=shared, lg=lg, col=1)
    sep = E.moe_combine(routed, shared, lg, 1)
    torch.cuda.synchronize()
    assert torch.equal(fused.view(torch.int16), sep.view(torch.int16))


def test_moe_prefill_bf16_activations_equals_decode_operator(E, oracle):
    """HB_FLAG_PREFILL_A16 | HB_FLAG_PREFILL_A16_ROWS: hb_moe_prefill with bf16 activations as the decode arithmetic on sub-chunks of
    rows — bit-identical to hb_moe_decode_routed_f32 on the same rows, and within the expert-output gate of the W4A16 oracle."""
    dev = torch.device("cuda")
    H, I, E_, K, M = 512, 256, 8, 2, 150
    rng = np.random.default_rng(21)
    recs = random_records(oracle, H, I, E_, 21)
    keep = upload(recs, dev)
    tab = E.rec_table(keep)
    ids_np = np.stack([rng.permutation(E_)[:K] for _ in range(M)]).astype(np.int32)
    w_np = rng.random((M, K), dtype=np.float32)
    ids, w = torch.tensor(ids_np, device=dev), torch.tensor(w_np, device=dev)
    x = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
    ctx16 = E.Context(flags=4 | 256)
    out = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, S=64, ctx=ctx16)
    ref = E.moe_decode_routed_f32(ids, w, tab, 0, E_, x, H, I)
    torch.cuda.synchronize()
    ctx16.check_device()
    assert torch.equal(out, ref)
    xs = x.float().cpu().numpy()
    orc = oracle.moe_routed(H, I, ids_np, w_np, recs, xs, 0.0, 0)
    rms = np.sqrt((orc.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-12
    assert np.max(np.abs(out.cpu().numpy() - orc) / rms) <= 2e-2


@pytest.mark.parametrize("H,I,E_,K,M,S,limit", [(512, 256, 8, 2, 150, 150, 0.0), (256, 256, 4, 2, 700, 700, 0.0), (2048, 512, 16, 4, 300, 128, 7.0),
                                                  (7168, 2048, 3, 2, 70, 70, 0.0)])
def test_moe_prefill_bf16_activations_on_tensor_cores(E, oracle, H, I, E_, K, M, S, limit):
    """HB_FLAG_PREFILL_A16 with more than 64 rows: the kind::f16 grouped GEMM over exactly dequantised weight tiles.  Same products and
    rounding points as the decode operators, fp32 sums in another order: within the expert-output gate of the W4A16 oracle
    (2e-2 × row RMS), and much closer than that to the decode operators; the same bits on a second run."""
    dev = torch.device("cuda")
    rng = np.random.default_rng(H + I + M + 5)
    recs = random_records(oracle, H, I, E_, H + M + 5)
    keep = upload(recs, dev)
    tab = E.rec_table(keep)
    ids_np = np.stack([rng.permutation(E_)[:K] for _ in range(M)]).astype(np.int32)
    ids_np[3, 0] = -1
    ids_np[5, 1] = E_ + 3
    w_np = rng.random((M, K), dtype=np.float32)
    ids, w = torch.tensor(ids_np, device=dev), torch.tensor(w_np, device=dev)
    x = torch.tensor((rng.standard_normal((M, H)) * np.exp(rng.standard_normal((M, 1)))).astype(np.float32)).to(torch.bfloat16).to(dev)
    ctx16 = E.Context(flags=4)
    out = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, S=S, limit=limit, ctx=ctx16)
    again = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, S=S, limit=limit, ctx=ctx16)
    torch.cuda.synchronize()
    ctx16.check_device()
    assert torch.equal(out, again)
    dec = torch.cat([E.moe_decode_routed_f32(ids[m0:m0 + 64], w[m0:m0 + 64], tab, 0, E_, x[m0:m0 + 64], H, I, limit=limit) for m0 in range(0, M, 64)])
    rms_d = dec.double().pow(2).mean(1, keepdim=True).sqrt() + 1e-12
    dd = (out.double() - dec.double()).abs() / rms_d
    assert float(dd.max()) <= 3e-2                            # bf16 rounding flips of g, u, y and the down rows (one bf16 step of an element of several row RMS)
    # the reference's own comparison of its W4A16 GEMM path with its decode path (engine/tests/test_fn_moe_pf.cu:172-181): per-row cosine
    # above 0.99999 and no more than M outputs further than 1e-2 × RMS apart — its case sums 10 terms per output, so one term's bf16 flip
    # stays below 1e-2 × RMS; with the 2 terms of these cases a flip of a large element does not, hence the rate beside the count
    cos = (out.double() * dec.double()).sum(1) / (out.double().norm(dim=1) * dec.double().norm(dim=1) + 1e-30)
    live = dec.double().norm(dim=1) > 0
    assert float(cos[live].min()) > 0.99999, float(cos[live].min())
    assert int((dd > 1e-2).sum()) <= max(M, int(1e-3 * M * H)), int((dd > 1e-2).sum())
    rows = list(range(0, M, max(1, M // 24)))                                            # the oracle on a sample of rows
    orc = oracle.moe_routed(H, I, ids_np[rows], w_np[rows], recs, x.float().cpu().numpy()[rows], limit, 0)
    rms = np.sqrt((orc.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-12
    # the expert-output gate, plus one bf16 step of the value itself: the per-pair down rows are rounded to bf16 before they are summed,
    # and with fp32 sums in another order an element of several row RMS lands one step away (2^-8 of its size, more than 2e-2 RMS)
    assert np.all(np.abs(out.cpu().numpy()[rows] - orc) <= 2e-2 * rms + 2.0 ** -7 * np.abs(orc))
    assert np.max(np.abs(out.cpu().numpy()[rows] - orc) / rms) <= 4e-2
    ctx16.close()


def test_moe_prefill_bf16_activations_combine(E, oracle):
    """The fused shared-expert combine behind the bf16-activation GEMM equals hb_moe_combine on its routed sums."""
    dev = torch.device("cuda")
    H, I, E_, K, M = 512, 256, 8, 2, 200
    rng = np.random.default_rng(31)
    recs = random_records(oracle, H, I, E_, 31)
    keep = upload(recs, dev)
    tab = E.rec_table(keep)
    ids = torch.tensor(np.stack([rng.permutation(E_)[:K] for _ in range(M)]).astype(np.int32), device=dev)
    w = torch.tensor(rng.random((M, K), dtype=np.float32), device=dev)
    x = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
    shared = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
    lg = torch.tensor(rng.standard_normal((M, 3)).astype(np.float32), device=dev)
    ctx16 = E.Context(flags=4)
    routed = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, ctx=ctx16)
    fused = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, shared=shared, lg=lg, col=1, ctx=ctx16)
    sep = E.moe_combine(routed, shared, lg, 1)
    torch.cuda.synchronize()
    ctx16.check_device()
    assert torch.equal(fused.view(torch.int16), sep.view(torch.int16))
    ctx16.close()


def test_w4a4_distance_from_w4a16(E, oracle):
    """How far the grouped GEMM's arithmetic (NVFP4 activations, W4A4) is from the reference's default (bf16 activations, W4A16) on
    the same rows, at the DeepSeek-shaped expert size: the reference's own gate for its W4A4 option is cosine > 0.98 per row
    (engine/tests/test_fn_moe_pf.cu:419).  The W4A16 side is both this library's decode operator and the CPU oracle."""
    dev = torch.device("cuda")
    H, I, E_, K, M = 7168, 2048, 4, 2, 96
    rng = np.random.default_rng(419)
    recs = random_records(oracle, H, I, E_, 419)
    keep = upload(recs, dev)
    tab = E.rec_table(keep)
    ids_np = np.stack([rng.permutation(E_)[:K] for _ in range(M)]).astype(np.int32)
    w_np = rng.random((M, K), dtype=np.float32)
    ids, w = torch.tensor(ids_np, device=dev), torch.tensor(w_np, device=dev)
    x = torch.tensor((rng.standard_normal((M, H)) * np.exp(rng.standard_normal((M, 1)))).astype(np.float32)).to(torch.bfloat16).to(dev)
    a4 = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I).double()
    a16 = torch.cat([E.moe_decode_routed_f32(ids[m0:m0 + 64], w[m0:m0 + 64], tab, 0, E_, x[m0:m0 + 64], H, I) for m0 in range(0, M, 64)]).double()
    torch.cuda.synchronize()
    E.context().check_device()
    cos = (a4 * a16).sum(1) / (a4.norm(dim=1) * a16.norm(dim=1) + 1e-30)
    rel = (a4 - a16).abs().max(1).values / (a16.pow(2).mean(1).sqrt() + 1e-30)
    print(f"W4A4 vs W4A16 over {M} rows: cosine min {float(cos.min()):.5f} mean {float(cos.mean()):.5f}; max |diff| / row RMS {float(rel.max()):.3f}")
    assert float(cos.min()) > 0.98
    # the oracle's W4A16 expert on two of the rows says the same about the W4A4 results
    for m in (0, M - 1):
        ref = sum(np.float64(w_np[m, k]) * oracle.expert_forward(recs[ids_np[m, k]], H, I, x[m].float().cpu().numpy(), 1.0, 0.0).astype(np.float64) for k in range(K))
        g = a4[m].cpu().numpy()
        assert float((g * ref).sum() / (np.linalg.norm(g) * np.linalg.norm(ref))) > 0.98


def test_moe_layer_dispatches_by_row_count(E, oracle):
    """hb_moe_layer: without HB_FLAG_LAYER_A4 every row count is the decode layer bit for bit (W4A16, rows independent of the batch);
    with the flag, more than 64 rows equal router → shared expert through the W4A4 grouped GEMM → routed experts with the fused
    combine, composed by hand from the same operators, and ≤ 64 rows are still the decode layer."""
    dev = torch.device("cuda")
    H, I, E_, K = 512, 256, 8, 2
    rng = np.random.default_rng(31)
    recs = random_records(oracle, H, I, E_ + 1, 31)
    keep = upload(recs, dev)
    tab = E.rec_table(keep[:E_])
    ctx_a4 = E.Context(flags=32)                                        # HB_FLAG_LAYER_A4
    try:
        for M in (20, 150):
            x = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
            lg = torch.tensor(rng.standard_normal((M, E_ + 1)).astype(np.float32), device=dev)
            # default context: the decode operators at every row count — each row equals the row run alone in a 64-row slice
            ids, w, out = E.moe_layer(lg, x, tab, 0, E_, K, H, I, shared_rec=keep[E_], gate_col=E_)
            for m0 in range(0, M, 64):
                sl = slice(m0, min(M, m0 + 64))
                ids2, w2, out2 = E.moe_layer_decode(lg[sl], x[sl], tab, 0, E_, K, H, I, shared_rec=keep[E_], gate_col=E_)
                assert torch.equal(ids[sl], ids2) and torch.equal(w[sl], w2), M
                assert torch.equal(out[sl].view(torch.int16), out2.view(torch.int16)), M
            # opt-in context
            ids, w, out = E.moe_layer(lg, x, tab, 0, E_, K, H, I, shared_rec=keep[E_], gate_col=E_, ctx=ctx_a4)
            if M <= 64:
                ids2, w2, out2 = E.moe_layer_decode(lg, x, tab, 0, E_, K, H, I, shared_rec=keep[E_], gate_col=E_)
            else:
                ids2, w2 = E.router_softmax_topk(lg, K, True, True, E=E_)
                sh = E.fn_moe_prefill(E.rec_table([keep[E_]]), 0, 1, torch.zeros((M, 1), dtype=torch.int32, device=dev),
                                      torch.ones((M, 1), dtype=torch.float32, device=dev), x, H, I)
                out2 = E.fn_moe_prefill(tab, 0, E_, ids2, w2, x, H, I, shared=sh.to(torch.bfloat16), lg=lg, col=E_)
            torch.cuda.synchronize()
            E.context().check_device(); ctx_a4.check_device()
            assert torch.equal(ids, ids2) and torch.equal(w, w2), M
            assert torch.equal(out.view(torch.int16), out2.view(torch.int16)), M
    finally:
        torch.cuda.synchronize()
        ctx_a4.close()


def test_moe_prefill_bf16_activations_nothing_routed(E, oracle):
    """More than 64 rows none of which has a usable expert: the bf16-activation GEMM runs over an empty tile list and the sums are zero."""
    dev = torch.device("cuda")
    H, I, E_, K, M = 256, 256, 4, 2, 100
    recs = random_records(oracle, H, I, E_, 5)
    keep = upload(recs, dev)
    tab = E.rec_table(keep)
    ids = torch.full((M, K), -1, dtype=torch.int32, device=dev)
    ids[::3, 1] = E_ + 2
    w = torch.ones((M, K), dtype=torch.float32, device=dev)
    x = torch.randn((M, H), device=dev).to(torch.bfloat16)
    ctx16 = E.Context(flags=4)
    out = E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, ctx=ctx16)
    torch.cuda.synchronize()
    ctx16.check_device()
    assert float(out.abs().max()) == 0.0
    ctx16.close()


def test_moe_layer_with_bf16_activation_gemm(E, oracle):
    """hb_moe_layer on a context with HB_FLAG_PREFILL_A16: more than 64 rows go router → shared expert → routed experts through the
    bf16-activation grouped GEMM.  Routing is the decode layer's bit for bit; the outputs are the decode layer's up to the order of
    the fp32 sums (a bf16 step of the output here and there), and within the gate of the oracle's layer."""
    dev = torch.device("cuda")
    H, I, E_, K, M = 512, 256, 8, 2, 150
    rng = np.random.default_rng(41)
    recs = random_records(oracle, H, I, E_ + 1, 41)
    keep = upload(recs, dev)
    tab = E.rec_table(keep[:E_])
    x = torch.tensor(rng.standard_normal((M, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
    lg = torch.tensor(rng.standard_normal((M, E_ + 1)).astype(np.float32), device=dev)
    ctx16 = E.Context(flags=4)
    try:
        ids, w, out = E.moe_layer(lg, x, tab, 0, E_, K, H, I, shared_rec=keep[E_], gate_col=E_, ctx=ctx16)
        ids2, w2, out2 = E.moe_layer(lg, x, tab, 0, E_, K, H, I, shared_rec=keep[E_], gate_col=E_)          # decode operators
        torch.cuda.synchronize()
        ctx16.check_device(); E.context().check_device()
        assert torch.equal(ids, ids2) and torch.equal(w, w2)
        d = (out.double() - out2.double()).abs()
        rms = out2.double().pow(2).mean(1, keepdim=True).sqrt() + 1e-12
        assert float((d / rms).max()) <= 3e-2
        assert float((d > 0).double().mean()) < 0.2                        # most elements are the same bits
    finally:
        torch.cuda.synchronize()
        ctx16.close()


def test_moe_prefill_degenerate_inputs(E, oracle):
    """Nothing to do is not an error: zero rows, and rows whose every id is invalid or points at an absent record (output zeros)."""
    dev = torch.device("cuda")
    H, I, E_, K, M = 256, 256, 4, 2, 9
    recs = random_records(oracle, H, I, E_, 3)
    keep = upload(recs, dev)
    tab = E.rec_table([keep[0], None, keep[2], None])
    x = torch.randn((M, H), device=dev).to(torch.bfloat16)
    ids = torch.tensor([[1, 3]] * M, dtype=torch.int32, device=dev)
    ids[0, 0] = -7; ids[1, 1] = 99
    w = torch.ones((M, K), dtype=torch.float32, device=dev)
    out = torch.full((M, H), 5.0, dtype=torch.float32, device=dev)
    E.fn_moe_prefill(tab, 0, E_, ids, w, x, H, I, out=out)
    torch.cuda.synchronize()
    E.context().check_device()
    assert float(out.abs().max()) == 0.0
    ctx = E.context()
    ws = torch.empty(E.moe_prefill_ws_bytes(8, K, E_, H, I), dtype=torch.uint8, device=dev)
    import ctypes as C
    from eke_hive_b200 import _lib
    assert _lib.load().hb_moe_prefill(ctx.handle, tab.data_ptr(), 0, E_, ids.data_ptr(), w.data_ptr(), 0, K, x.data_ptr(), H, I, 0.0, out.data_ptr(),
                                      ws.data_ptr(), 8, None, None) == 0

