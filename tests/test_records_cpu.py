"""Pins the oracle's record assembly (compressed NVFP4 block scales, oracle/hive_oracle.c ho_csf_decode / ho_record_pack) to the
reference: against tests/golden/csf_golden.npz (outputs and verdicts of the reference's compiled hive::ckq::csf_decode,
engine/src/ckpt_quant.cpp:34-73) everywhere, and against the compiled reference itself where oracle/_ref exists.  Cases follow
the reference's engine/tests/test_ckpt_quant_cpu.cpp: round trip on four shapes, five damaged variants each."""
import numpy as np
import pytest

from conftest import GOLDEN
from util import CSF_SHAPES, csf_damaged, csf_scale_matrix

EXPECT = {"index": 4, "delta": 5, "value": 6, "code": 7, "shape": 2}


@pytest.fixture(scope="module")
def csf_golden():
    return np.load(GOLDEN / "csf_golden.npz")


@pytest.mark.parametrize("k", range(len(CSF_SHAPES)))
def test_csf_decode_matches_reference_output(oracle, csf_golden, k):
    R, C = CSF_SHAPES[k]
    fx, ex = csf_golden[f"c{k}_fixed"], csf_golden[f"c{k}_exc"]
    st, _, out = oracle.csf_decode(fx, ex, R, C)
    assert st == 0 and np.array_equal(out, csf_golden[f"c{k}_decoded"])
    fx2, ex2 = oracle.csf_encode(out)                                   # the test-side encoder reproduces the stored tensors
    assert np.array_equal(fx2, fx) and np.array_equal(ex2, ex)


@pytest.mark.parametrize("k", range(len(CSF_SHAPES)))
def test_csf_damaged_tensors_refused_like_the_reference(oracle, csf_golden, k):
    R, C = CSF_SHAPES[k]
    fx, ex = csf_golden[f"c{k}_fixed"], csf_golden[f"c{k}_exc"]
    for name, (f2, e2, shp) in csf_damaged(fx, ex, R, C).items():
        st, where, _ = oracle.csf_decode(f2, e2, R, C, fixed_shape=shp)
        assert st == EXPECT[name], (name, st, where)
        assert int(csf_golden[f"c{k}_bad_{name}"][0]) == 0               # the reference refused it too
        if name == "index":
            assert where == ex.size                                       # the appended word
        if name in ("delta", "value"):
            assert where == 0                                             # the first exception word was damaged
        if name == "code":
            assert where == 0                                             # scale (0, 0)


def test_csf_repeated_exception_last_wins(oracle, csf_golden):
    fx, ex = csf_golden["dup_fixed"], csf_golden["dup_exc"]
    st, _, out = oracle.csf_decode(fx, ex, 32, 8)
    assert st == 0 and np.array_equal(out, csf_golden["dup_decoded"])


def test_csf_shape_rules(oracle):
    fx = np.zeros((1, 24), np.uint8)
    assert oracle.csf_decode(fx, np.zeros(0, np.uint32), 8, 1)[0] == 1             # rows not a multiple of 16
    assert oracle.csf_decode(fx, np.zeros(0, np.uint32), 16, 0)[0] == 1
    big = np.zeros((1, 16), np.uint8)
    assert oracle.csf_decode(big, np.zeros(0, np.uint32), 1 << 20, 32, fixed_shape=((1 << 20) // 16, 16 + 8 * 32))[0] == 3   # > 2^24 scales


def test_csf_against_compiled_reference(oracle):
    if not oracle.have_ref():
        pytest.skip("compiled reference not present")
    rng = np.random.default_rng(7)
    for R, C in [(16, 1), (48, 5), (128, 16), (640, 160)]:
        s = csf_scale_matrix(rng, R, C)
        fx, ex = oracle.csf_encode(s)
        a = oracle.csf_decode(fx, ex, R, C)
        b = oracle.csf_decode(fx, ex, R, C, use_ref=True)
        assert a[0] == 0 and b[0] == 0 and np.array_equal(a[2], b[2]) and np.array_equal(a[2], s)
        for name, (f2, e2, shp) in csf_damaged(fx, ex, R, C).items():
            assert oracle.csf_decode(f2, e2, R, C, fixed_shape=shp)[0] == EXPECT[name]
            assert oracle.csf_decode(f2, e2, R, C, fixed_shape=shp, use_ref=True)[0] == -1


def test_record_pack_equals_layout_copy(oracle):
    """plain scales: the packed record is the byte-for-byte concatenation the kernels read; compressed scales give the same record"""
    H, I = 256, 128
    rng = np.random.default_rng(3)
    projs, plain = [], []
    for rows, K in ((I, H), (I, H), (H, I)):
        q = rng.integers(0, 256, (rows, K // 2), dtype=np.uint8)
        s = csf_scale_matrix(rng, rows, K // 16)
        g = float(rng.random() * 1e-3)
        plain.append((q, s, g))
        fx, ex = oracle.csf_encode(s)
        projs.append({"weight": q, "csf_fixed": fx, "csf_exc": ex, "global": g})
    want = oracle.pack_record(H, I, *plain)
    st, rec = oracle.record_pack(H, I, [{"weight": q, "scale": s, "global": g} for q, s, g in plain])
    assert st == 0 and np.array_equal(rec, want)
    st, rec = oracle.record_pack(H, I, projs)
    assert st == 0 and np.array_equal(rec, want)
    projs[2]["csf_exc"] = np.append(projs[2]["csf_exc"], np.uint32(H * I // 16)).astype(np.uint32)
    assert oracle.record_pack(H, I, projs)[0] == 34                                 # third projection, exception index out of range
