"""GPU parity, dense decode GEMV (the 27B-style MLP): NVFP4 against the oracle of the reference's GEMV, and the 3-/2-bit group-64
formats against this project's own CPU restatement of the format (the reference ships no low-bit layout: parity unpinned there).
Dequantised values bit-exact; GEMV outputs within 2e-2 x RMS (observed ~1e-3: fp32 reassociation plus the 1024-offset removal)."""
import numpy as np
import pytest

from util import bf16_bits_of, bf16_tensor, rel_rms_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def E():
    import eke_hive_b200 as E
    return E


def _lb_mat(E, oracle, N, K, bits, seed):
    import torch
    rng = np.random.default_rng(seed)
    w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    q, s, zp = oracle.lb_quantize(w, bits)
    fmt = E.FMT_LB3_G64 if bits == 3 else E.FMT_LB2_G64
    G = E.GMat(fmt, N, K, torch.from_numpy(q).cuda(), torch.from_numpy(s.view(np.int16)).cuda(), torch.from_numpy(zp.view(np.int16)).cuda())
    return G, (q, s, zp)


@pytest.mark.parametrize("bits", [2, 3])
def test_lowbit_dequant_bit_exact(E, oracle, bits):
    G, (q, s, zp) = _lb_mat(E, oracle, 96, 512, bits, 1)
    out = E.lb_dequant(G)
    assert np.array_equal(bf16_bits_of(out), oracle.lb_dequant_bf16(q, s, zp, bits))


@pytest.mark.parametrize("bits,N,K,M", [(2, 128, 256, 1), (2, 200, 1024, 8), (3, 128, 512, 3), (3, 304, 2560, 8), (2, 256, 5120, 16), (3, 136, 4352, 5)])
def test_lowbit_gemv_vs_oracle(E, oracle, bits, N, K, M):
    G, (q, s, zp) = _lb_mat(E, oracle, N, K, bits, N + K + M)
    rng = np.random.default_rng(K + M)
    x = oracle.bf16r(rng.normal(0, 1, (M, K)).astype(np.float32))
    if M >= 3:
        x[1, 7] = 3.0e5; x[2] *= 1e-4                                   # outlier row, tiny row
        x = oracle.bf16r(x)
    import torch
    y = E.dense_gemv(G, bf16_tensor(x)).cpu().numpy()
    ref = oracle.lb_gemv(q, s, zp, bits, x)
    assert np.isfinite(y).all()
    assert rel_rms_err(y, ref) <= 2e-2
    yb = E.dense_gemv(G, bf16_tensor(x), out_dtype=torch.bfloat16)
    assert np.array_equal(bf16_bits_of(yb), oracle.bf16_bits(y))        # the bf16 form is the rounded fp32 form
    y2 = E.dense_gemv(G, bf16_tensor(x)).cpu().numpy()
    assert y.tobytes() == y2.tobytes()                                  # deterministic
    # batch invariance: a row alone gives the same bits as inside the batch
    y0 = E.dense_gemv(G, bf16_tensor(x[:1])).cpu().numpy()
    assert y0.tobytes() == y[:1].tobytes()


@pytest.mark.parametrize("N,K,M", [(128, 256, 1), (272, 2048, 8), (128, 5120, 4)])
def test_nvfp4_dense_gemv_vs_oracle(E, oracle, N, K, M):
    import torch
    rng = np.random.default_rng(N + K)
    w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    q, s, g = oracle.nvfp4_quantize(w, search=False)
    x = oracle.bf16r(rng.normal(0, 1, (M, K)).astype(np.float32))
    G = E.GMat(E.FMT_NVFP4, N, K, torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), None, g)
    y = E.dense_gemv(G, bf16_tensor(x)).cpu().numpy()
    ref = oracle.gemv_nvfp4(q, s, g, x)
    assert rel_rms_err(y, ref) <= 2e-2
    assert np.max(np.abs(y - ref)) <= 1e-4 * np.max(np.abs(ref))       # products are exact in f16, sums in fp32: only the order differs


@pytest.mark.parametrize("fmt", ["nvfp4", "lb3", "lb2"])
@pytest.mark.parametrize("N,K", [(17408, 5120), (5120, 17408)])
def test_dense_gemv_full_shapes(E, oracle, fmt, N, K):
    """The shapes the dense workload is measured on — 17408 × 5120 (gate, up) and 5120 × 17408 (down: the longest K, nine K splits) — at
    1 and 8 rows, every output row against the CPU oracle (NVFP4: the reference GEMV's restatement; 3-/2-bit: this project's own)."""
    import torch
    rng = np.random.default_rng(N // 7 + K)
    w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    x = oracle.bf16r(rng.normal(0, 1, (8, K)).astype(np.float32))
    if fmt == "nvfp4":
        q, s, g = oracle.nvfp4_quantize(w, search=False)
        G = E.GMat(E.FMT_NVFP4, N, K, torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), None, g)
        ref = oracle.gemv_nvfp4(q, s, g, x)
    else:
        bits = 3 if fmt == "lb3" else 2
        q, s, zp = oracle.lb_quantize(w, bits)
        G = E.GMat(E.FMT_LB3_G64 if bits == 3 else E.FMT_LB2_G64, N, K, torch.from_numpy(q).cuda(), torch.from_numpy(s.view(np.int16)).cuda(),
                   torch.from_numpy(zp.view(np.int16)).cuda())
        ref = oracle.lb_gemv(q, s, zp, bits, x)
    y8 = E.dense_gemv(G, bf16_tensor(x)).cpu().numpy()
    y1 = E.dense_gemv(G, bf16_tensor(x[:1])).cpu().numpy()
    E.context().check_device()
    assert np.isfinite(y8).all()
    assert rel_rms_err(y8, ref) <= 2e-2
    assert y1.tobytes() == y8[:1].tobytes()                              # a row alone = the row inside the batch


@pytest.mark.parametrize("bits", [2, 3])
def test_gate_up_fused_activation(E, oracle, bits):
    N, K, M = 256, 1024, 8
    Gm, (qg, sg, zg) = _lb_mat(E, oracle, N, K, bits, 11)
    Um, (qu, su, zu) = _lb_mat(E, oracle, N, K, bits, 12)
    rng = np.random.default_rng(13)
    x = oracle.bf16r(rng.normal(0, 1, (M, K)).astype(np.float32))
    act = E.dense_gemv_gu(Gm, Um, bf16_tensor(x)).float().cpu().numpy()
    ref = oracle.dense_act(oracle.lb_gemv(qg, sg, zg, bits, x), oracle.lb_gemv(qu, su, zu, bits, x))
    # act passes three bf16 roundings (g, silu(g), the product): a last-bit difference in g moves the result by one bf16 ulp of
    # its own magnitude, so the bound is 1.5 bf16 ulp of |ref| (2^-7 relative) plus 5e-3 x RMS for values near zero
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert np.all(np.abs(act - ref) <= 1.5 * 2.0 ** -7 * np.abs(ref) + 5e-3 * rms)


def test_dense_argument_errors(E):
    import torch
    w = torch.zeros(128 * 64, dtype=torch.uint8, device="cuda"); s = torch.zeros((128, 4), dtype=torch.int16, device="cuda")
    G = E.GMat(E.FMT_LB2_G64, 128, 200, w, s, s)                       # K not a multiple of 256
    with pytest.raises(E.HbError) as ei:
        E.dense_gemv(G, torch.zeros((1, 200), dtype=torch.bfloat16, device="cuda"), ws=torch.zeros(4096, dtype=torch.uint8, device="cuda"))
    assert ei.value.status == -2
