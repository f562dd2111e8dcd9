"""GPU parity, formats and single-matrix kernels: dequantised values bit-exact, quantisers bit-exact, GEMV within fp32 noise.
All calls go through the C ABI (eke_hive_b200 → libhive_b200.so)."""
import numpy as np
import pytest

from util import bf16_bits_of, bf16_tensor

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def E():
    import eke_hive_b200 as E
    return E


def test_dequant_bit_exact_all_codes(E, oracle, golden):
    import torch
    # every nibble and every non-NaN scale code, plus the reference-generated fixture matrix
    for q, s, g in ((golden["gemv_c_q"], golden["gemv_c_s"], float(golden["gemv_c_g"])),
                    (golden["gemv_b_q"], golden["gemv_b_s"], float(golden["gemv_b_g"]))):
        N, K = q.shape[0], q.shape[1] * 2
        out = E.nvfp4_dequant(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), g, N, K)
        assert np.array_equal(bf16_bits_of(out), oracle.nvfp4_dequant_bf16(q, s, g))


def test_dequant_large_bit_exact(E, oracle):
    import torch
    rng = np.random.default_rng(3)
    N, K = 512, 2048
    q = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    s = rng.integers(0, 0x7F, (N, K // 16), dtype=np.uint8)
    out = E.nvfp4_dequant(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), 0.0042, N, K)
    assert np.array_equal(bf16_bits_of(out), oracle.nvfp4_dequant_bf16(q, s, 0.0042))


def test_quantize_matches_device_rule(E, oracle):
    import torch
    rng = np.random.default_rng(4)
    w = rng.normal(0, 0.02, (96, 512)).astype(np.float32)
    w[5, 32:48] = 0                                             # an all-zero block: scale 0, codes 0
    q, s, g = E.nvfp4_quantize(torch.from_numpy(w).cuda())
    q0, s0, g0 = oracle.nvfp4_quantize(w, search=False)
    assert np.array_equal(q.cpu().numpy(), q0) and np.array_equal(s.cpu().numpy(), s0)
    assert np.float32(g.item()).tobytes() == np.float32(g0).tobytes()
    # round trip through the GPU dequantiser stays within NVFP4's error on Gaussian weights
    dq = E.nvfp4_dequant(q, s, float(g.item()), 96, 512).float().cpu().numpy()
    assert np.linalg.norm(dq - w) / np.linalg.norm(w) < 0.12


def test_requant_fp8_rows_to_nvfp4(E, oracle):
    """hb_requant_nvfp4 (FP8 codes with one fp32 scale per row → NVFP4): the same bits as the quantisation rule applied to the fp32
    values the FP8 matrix stands for (code value × row scale, one fp32 multiply), including an all-zero block, a zero row scale
    and the largest finite e4m3 codes."""
    import torch
    rng = np.random.default_rng(27)
    N, K = 80, 768
    w8 = rng.integers(0, 256, (N, K), dtype=np.uint8)
    w8[(w8 & 0x7F) == 0x7F] = 0x3A                              # no NaN codes in weights
    w8[3, 64:80] = 0                                            # an all-zero block
    w8[9, :16] = 0x7E                                           # 448, the largest e4m3 value
    sr = rng.uniform(0.5e-3, 4e-3, N).astype(np.float32)
    sr[11] = 0.0                                                # a row scaled to nothing
    sr[12] = -sr[12]                                            # a negative row scale flips the signs
    f = (oracle.e4m3_table()[w8].astype(np.float32) * sr[:, None]).astype(np.float32)
    q, s, g = E.requant_nvfp4(torch.from_numpy(w8).cuda(), torch.from_numpy(sr).cuda())
    q0, s0, g0 = oracle.nvfp4_quantize(f, search=False)

    def no_signed_zero(codes):
        """nibble 8 (-0) → 0: an FP8 code of -0, or +0 under a negative row scale, is -0.0 in fp32; the hardware converter keeps that
        sign, the reference's numpy rule (sign = x < 0) drops it.  Both decode to zero."""
        lo, hi = codes & 0xF, codes >> 4
        return np.where(lo == 8, 0, lo) | (np.where(hi == 8, 0, hi) << 4)
    assert np.array_equal(no_signed_zero(q.cpu().numpy()), no_signed_zero(q0)) and np.array_equal(s.cpu().numpy(), s0)
    assert np.float32(g.item()).tobytes() == np.float32(g0).tobytes()
    E.context().check_device()


def test_a4_quant_bit_exact(E, oracle):
    rng = np.random.default_rng(5)
    x = oracle.bf16r(rng.normal(0, 1, (9, 512)).astype(np.float32))
    x[4] = 0
    x[7, 100] = 3.0e5
    x = oracle.bf16r(x)
    q, s, g = E.a4_quant(bf16_tensor(x))
    q0, s0, g0 = oracle.a4_quant(x)
    assert np.array_equal(q.cpu().numpy(), q0) and np.array_equal(s.cpu().numpy(), s0)
    assert g.cpu().numpy().tobytes() == g0.tobytes()


@pytest.mark.parametrize("N,K,M", [(37, 64, 1), (37, 64, 3), (48, 512, 8), (256, 2048, 16), (512, 4096, 5)])
def test_gemv_vs_oracle(E, oracle, N, K, M):
    import torch
    rng = np.random.default_rng(N * 7 + K + M)
    w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    q, s, g = oracle.nvfp4_quantize(w, search=False)
    x = oracle.bf16r(rng.normal(0, 1, (M, K)).astype(np.float32))
    y = E.nvfp4_gemv(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), g, N, K, bf16_tensor(x)).cpu().numpy()
    ref = oracle.gemv_nvfp4(q, s, g, x)
    # the reference's own bar between two of its fp32 summation orders: rel < 1e-5 (engine/tests/test_nvfp4_cpu.cpp:26-60)
    assert np.max(np.abs(y - ref)) <= 2e-5 * np.max(np.abs(ref))


def test_gemv_golden_and_strided(E, oracle, golden):
    import torch
    q, s, g, x = golden["gemv_b_q"], golden["gemv_b_s"], float(golden["gemv_b_g"]), golden["gemv_b_x"]
    N, K = q.shape[0], q.shape[1] * 2
    xb = torch.zeros((3, K + 64), dtype=torch.bfloat16, device="cuda")
    xb[:, :K] = bf16_tensor(x)
    ybuf = torch.full((3, N + 5), -7.0, dtype=torch.float32, device="cuda")
    E.nvfp4_gemv(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), g, N, K, xb[:, :K], ybuf[:, :N])
    y = ybuf.cpu().numpy()
    assert np.max(np.abs(y[:, :N] - golden["gemv_b_y_scalar"])) <= 2e-5 * np.max(np.abs(golden["gemv_b_y_scalar"]))
    assert np.all(y[:, N:] == -7.0)                              # row stride respected, nothing written past N


def test_argument_errors_are_codes_not_aborts(E):
    import torch
    x = torch.zeros((17, 64), dtype=torch.bfloat16, device="cuda")
    q = torch.zeros((8, 32), dtype=torch.uint8, device="cuda"); s = torch.zeros((8, 4), dtype=torch.uint8, device="cuda")
    with pytest.raises(E.HbError) as ei:
        E.nvfp4_gemv(q, s, 1.0, 8, 64, x)                        # M = 17
    assert ei.value.status == -2
    with pytest.raises(E.HbError) as ei:
        E.nvfp4_gemv(q, s, 1.0, 8, 48, x[:1, :48].contiguous())  # K % 32
    assert ei.value.status == -2
    with pytest.raises(E.HbError):
        E.ExpertRecLayout.make(100, 64)


def test_expert_dequant_bit_exact(E, oracle):
    """hive::glm::expert_dequant: the three matrices of a record, values bit-exact against the oracle's dequantiser."""
    import torch
    from util import random_records
    H, I = 256, 128
    rec = random_records(oracle, H, I, 1, 5)[0]
    off = oracle.rec_layout(H, I)
    gu, d = E.expert_dequant(torch.from_numpy(rec).cuda(), H, I)
    g = rec[int(off[6]):int(off[6]) + 12].view(np.float32)
    for name, got, (a, b), gi, (N, K) in (("w1", gu[:I], (0, 1), 0, (I, H)), ("w3", gu[I:], (2, 3), 1, (I, H)), ("w2", d, (4, 5), 2, (H, I))):
        q = rec[int(off[a]):int(off[a]) + N * K // 2].reshape(N, K // 2)
        s = rec[int(off[b]):int(off[b]) + N * K // 16].reshape(N, K // 16)
        ref = oracle.nvfp4_dequant_bf16(q, s, float(g[gi]))
        assert np.array_equal(bf16_bits_of(got), ref), name

