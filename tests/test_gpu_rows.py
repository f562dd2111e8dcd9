"""GPU parity of the row helpers kept for callers that compose an expert pass themselves (gather_rows, swiglu_rows,
scatter_add_rows, add_f32, expert_dequant — the reference's engine/include/hive/glm/glm_moe.h:32-41), each against a numpy
statement of its definition, and one composition of all of them in the order of the reference's per-expert prefill
(engine/src/glm/glm_experts.cpp:815-823) against the oracle's expert."""
import numpy as np
import pytest

from util import bf16_tensor, make_records, rel_rms_err, upload

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def E():
    import eke_hive_b200 as E
    return E


def _silu_portable(oracle, g):
    e = np.array([oracle.exp_portable(-float(v)) for v in g.ravel()], np.float32).reshape(g.shape)
    return (g / (np.float32(1.0) + e)).astype(np.float32)


def test_gather_rows_is_a_row_copy(E):
    import torch
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.normal(0, 1, (9, 264)).astype(np.float32)).cuda().to(torch.bfloat16)
    rows = torch.tensor([8, 0, 3, 3, 7], dtype=torch.int32, device="cuda")
    out = E.gather_rows(x, rows)
    assert torch.equal(out, x[rows.long()])
    assert E.gather_rows(x, rows[:0]).shape[0] == 0                    # empty row list: a no-op


@pytest.mark.parametrize("limit", [0.0, 0.75])
def test_swiglu_rows_bit_exact(E, oracle, limit):
    """y = bf16(silu(g)·u) on [R, 2I] rows (gate half, then up half), clamp first when limit > 0 (u to [-L, L], g to (-inf, L]);
    the kernel's SiLU is x / (1 + exp(-x)) with the portable exp, so the expected bits follow from the oracle's exp."""
    import torch
    rng = np.random.default_rng(2)
    R, I = 5, 96
    gu = oracle.bf16r(rng.normal(0, 1.5, (R, 2 * I)).astype(np.float32))
    gu[0, :4] = [0.0, -0.0, 30.0, -30.0]
    gu = oracle.bf16r(gu)
    g, u = gu[:, :I].copy(), gu[:, I:].copy()
    if limit > 0:
        u = np.clip(u, -limit, limit); g = np.minimum(g, np.float32(limit))
    want = oracle.bf16_bits((_silu_portable(oracle, g) * u).astype(np.float32))
    y = E.swiglu_rows(bf16_tensor(gu), limit)
    got = y.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, want)
    # against libm's exp (the reference CPU's silu_lim_act, engine/src/glm/cpu/glm_cpu_engine.cpp:50-53): at most one bf16 ulp
    lib = oracle.bf16_bits((g / (1 + np.exp(-g.astype(np.float64))) * u).astype(np.float32))
    assert np.max(np.abs(got.astype(np.int32) - lib.astype(np.int32))) <= 1


def test_scatter_add_rows_and_add_f32(E, oracle):
    """out[rows[r]] += w[r]·e[r] with one multiply and one add per element (rows unique per call); a += b."""
    import torch
    rng = np.random.default_rng(3)
    R, H, M = 4, 200, 7
    e = oracle.bf16r(rng.normal(0, 1, (R, H)).astype(np.float32))
    rows = np.array([5, 0, 6, 2], np.int32)
    w = rng.uniform(0.1, 0.9, R).astype(np.float32)
    out0 = rng.normal(0, 1, (M, H)).astype(np.float32)
    out = torch.from_numpy(out0.copy()).cuda()
    E.scatter_add_rows(bf16_tensor(e), torch.from_numpy(rows).cuda(), torch.from_numpy(w).cuda(), out)
    want = out0.copy()
    want[rows] = out0[rows] + (w[:, None] * e).astype(np.float32)
    assert out.cpu().numpy().tobytes() == want.tobytes()
    b = rng.normal(0, 1, (M, H)).astype(np.float32)
    E.add_f32(out, torch.from_numpy(b).cuda())
    assert out.cpu().numpy().tobytes() == (want + b).astype(np.float32).tobytes()


def test_composed_expert_pass_matches_oracle(E, oracle):
    """expert_dequant → gather → GEMM → swiglu_rows → GEMM → scatter_add_rows, the reference's per-expert prefill sequence with a
    plain fp32 matrix product standing in for the vendor GEMM, against the oracle's expert on the same rows."""
    import torch
    H, I, M = 256, 128, 6
    rng = np.random.default_rng(4)
    rec = make_records(oracle, H, I, 1, seed=11)[0]
    drec = upload([rec])[0]
    x = oracle.bf16r(rng.normal(0, 1, (M, H)).astype(np.float32))
    rows = np.array([4, 1, 5], np.int32)
    w = np.array([0.5, 0.25, 0.125], np.float32)
    gu_w, d_w = E.expert_dequant(drec, H, I)                           # bf16 [2I, H], [H, I]
    xr = E.gather_rows(bf16_tensor(x), torch.from_numpy(rows).cuda())
    gu = (xr.float() @ gu_w.float().view(2 * I, H).T).to(torch.bfloat16)
    y = E.swiglu_rows(gu.contiguous(), 0.0)
    e = (y.float() @ d_w.float().view(H, I).T).to(torch.bfloat16)
    out = torch.zeros((M, H), dtype=torch.float32, device="cuda")
    E.scatter_add_rows(e.contiguous(), torch.from_numpy(rows).cuda(), torch.from_numpy(w).cuda(), out)
    got = out.cpu().numpy()
    want = np.zeros((M, H), np.float32)
    for r, wt in zip(rows, w):
        want[r] = oracle.expert_forward(rec, H, I, x[r], float(wt), 0.0, 1)
    # The composed pass rounds the weights to bf16 (the oracle multiplies exact e2m1·e4m3 products and applies the global scale after
    # the sum) and rounds gate, up and y to bf16 from slightly different sums: a y value that lands on the neighbouring bf16 value
    # is spread over the whole output row by the down product, and a result can itself land a bf16 value or two away — two bf16
    # steps of the element (2^-6 relative) on top of 3e-2 × row RMS, and the rows must point the same way.
    g64, w64 = got[rows].astype(np.float64), want[rows].astype(np.float64)
    rms = np.sqrt((w64 ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(g64 - w64) <= 2.0 ** -6 * np.abs(w64) + 3e-2 * rms), float((np.abs(g64 - w64) / rms).max())
    cos = (g64 * w64).sum(1) / (np.linalg.norm(g64, axis=1) * np.linalg.norm(w64, axis=1))
    assert cos.min() > 0.9999
    assert not got[[0, 2, 3]].any()
    E.context().check_device()
