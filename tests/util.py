"""Helpers shared by the GPU parity tests: seeded synthetic experts packed into reference-layout records, uploads, tolerances."""
from __future__ import annotations

import numpy as np


def make_records(O, H, I, E, seed, search=False, sigma=0.02):
    """E expert records (numpy uint8 arrays) quantized from fp32 ~N(0, sigma) with the oracle's quantizer."""
    rng = np.random.default_rng(seed)
    recs = []
    for _ in range(E):
        mats = [O.nvfp4_quantize(rng.normal(0, sigma, sh).astype(np.float32), search) for sh in ((I, H), (I, H), (H, I))]
        recs.append(O.pack_record(H, I, *mats))
    return recs


def random_records(O, H, I, E, seed):
    """Records with random nibbles and scale codes 0x28..0x47 and the globals the reference's GPU test uses
    (engine/tests/test_glm_moe.cu:61-69) — cheap to make at any size."""
    rng = np.random.default_rng(seed)
    off = O.rec_layout(H, I)
    recs = []
    for _ in range(E):
        rec = np.zeros(int(off[7]), np.uint8)
        for a, b, n in ((0, 1, I * H), (2, 3, I * H), (4, 5, H * I)):
            rec[int(off[a]):int(off[a]) + n // 2] = rng.integers(0, 256, n // 2, dtype=np.uint8)
            rec[int(off[b]):int(off[b]) + n // 16] = rng.integers(0x28, 0x48, n // 16, dtype=np.uint8)
        rec[int(off[6]):int(off[6]) + 12] = np.array([0.0031, 0.0027, 0.0042], np.float32).view(np.uint8)
        recs.append(rec)
    return recs


def upload(recs, device="cuda"):
    import torch
    return [None if r is None else torch.from_numpy(r).to(device) for r in recs]


def bf16_tensor(x_f32, device="cuda"):
    """fp32 numpy array of bf16-representable values → torch bf16 tensor with the same values."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(x_f32, np.float32)).to(device).to(torch.bfloat16)


def bf16_bits_of(t):
    """torch bf16 tensor → numpy uint16 bit patterns."""
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rel_rms_err(got, ref):
    """max-abs-error divided by the RMS of the reference, per row (the tolerance form the spec uses)."""
    got = np.asarray(got, np.float64); ref = np.asarray(ref, np.float64)
    rms = np.sqrt(np.mean(ref ** 2, axis=-1)) + 1e-30
    return float(np.max(np.max(np.abs(got - ref), axis=-1) / rms))


# ---- compressed block scales: inputs of the record-assembly tests and of tests/golden/make_csf_golden.py
CSF_SHAPES = [(640, 160), (2560, 40), (16, 1), (32, 3)]


def csf_scale_matrix(rng, R, C):
    """codes around one level per matrix with a 2 % tail of outliers, all ≤ 0x7E (the distribution the reference's test draws)"""
    s = 40 + rng.integers(0, 12, (R, C)) + np.where(rng.integers(0, 50, (R, C)) == 0, rng.integers(0, 70, (R, C)), 0)
    return np.minimum(s, 0x7E).astype(np.uint8)


def csf_damaged(fx, ex, R, C):
    """the reference test's negative controls: name → (fixed, exceptions, fixed_shape)"""
    out = {}
    out["index"] = (fx, np.append(ex, np.uint32((60 << 24) | (R * C))), fx.shape)
    if ex.size:
        i = int(ex[0] & 0xFFFFFF); n = (i // C % 16) * C + i % C
        f2 = fx.copy(); f2[i // C // 16, 16 + (n >> 1)] |= 1 << ((n & 1) * 4)
        out["delta"] = (f2, ex, fx.shape)
        e2 = ex.copy(); e2[0] = (0x7F << 24) | (e2[0] & 0xFFFFFF)
        out["value"] = (fx, e2, fx.shape)
    if not np.any((ex & 0xFFFFFF) == 0):
        f2 = fx.copy(); f2[0, 0] = 0x7E; f2[0, 16] |= 0x0F
        out["code"] = (f2, ex, fx.shape)
    out["shape"] = (fx, ex, (fx.shape[0], fx.shape[1] + 1))
    return out
