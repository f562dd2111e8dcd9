"""GPU parity of record assembly (hb_csf_decode, hb_record_pack) against the CPU oracle and the reference's decoded fixtures:
bit-exact scales, the same verdict and position for every damaged tensor, and a packed record the decode operator can run on."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN
from util import CSF_SHAPES, csf_damaged, csf_scale_matrix

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def E():
    import eke_hive_b200 as E
    return E


def _dev(a, dev="cuda"):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(a).to(dev) if a.size else torch.zeros(0, dtype=torch.int32 if a.dtype == np.int32 else torch.uint8, device=dev)


@pytest.mark.parametrize("k", range(len(CSF_SHAPES)))
def test_csf_decode_golden_and_damaged(E, oracle, k):
    g = np.load(GOLDEN / "csf_golden.npz")
    R, C = CSF_SHAPES[k]
    fx, ex = g[f"c{k}_fixed"], g[f"c{k}_exc"]
    out, st = E.csf_decode(_dev(fx), _dev(ex), R, C)
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0]
    assert np.array_equal(out.cpu().numpy(), g[f"c{k}_decoded"])
    for name, (f2, e2, shp) in csf_damaged(fx, ex, R, C).items():
        want, where, _ = oracle.csf_decode(f2, e2, R, C, fixed_shape=shp)
        if name == "shape":
            with pytest.raises(E.HbError):
                E.csf_decode(_dev(f2), _dev(e2), R, C, fixed_shape=shp)
            continue
        _, st = E.csf_decode(_dev(f2), _dev(e2), R, C, fixed_shape=shp)
        assert st.tolist() == [want, where], name


def test_csf_repeated_exception_and_many_shapes(E, oracle):
    g = np.load(GOLDEN / "csf_golden.npz")
    out, st = E.csf_decode(_dev(g["dup_fixed"]), _dev(g["dup_exc"]), 32, 8)
    assert st.tolist() == [0, 0] and np.array_equal(out.cpu().numpy(), g["dup_decoded"])
    rng = np.random.default_rng(17)
    for R, C in [(16, 1), (16, 7), (48, 5), (128, 16), (2048, 128), (7168, 128), (4096, 448), (65536, 256)]:   # last: 2^24 scales, the format's limit
        s = csf_scale_matrix(rng, R, C)
        fx, ex = oracle.csf_encode(s)
        out, st = E.csf_decode(_dev(fx), _dev(ex), R, C)
        assert st.tolist() == [0, 0], (R, C)
        assert torch.equal(out.cpu(), torch.from_numpy(s)), (R, C)
    # every violation at once: the first exception word that fails decides, then the first bad scale
    R, C = 64, 12
    s = csf_scale_matrix(rng, R, C); s[5, 3] = 0x7E; s[5, 4] = 0x50
    fx, ex = oracle.csf_encode(s)
    ex = np.concatenate([ex, np.array([(0x7F << 24) | 9, (0x20 << 24) | (R * C + 5)], np.uint32)]).astype(np.uint32)
    want = oracle.csf_decode(fx, ex, R, C)
    _, st = E.csf_decode(_dev(fx), _dev(ex), R, C)
    assert want[0] != 0 and st.tolist() == [want[0], want[1]]
    with pytest.raises(E.HbError):
        E.csf_decode(_dev(np.zeros((1, 24), np.uint8)), None, 8, 1)                # rows not a multiple of 16


@pytest.mark.parametrize("H,I", [(256, 128), (2048, 512)])
def test_record_pack_matches_oracle_and_runs(E, oracle, H, I):
    dev = torch.device("cuda")
    rng = np.random.default_rng(H + I)
    plain, csf_np, csf_dev, mixed_dev = [], [], [], []
    for j, (rows, K) in enumerate(((I, H), (I, H), (H, I))):
        q = rng.integers(0, 256, (rows, K // 2), dtype=np.uint8)
        s = np.minimum(csf_scale_matrix(rng, rows, K // 16), 0x48).astype(np.uint8)
        gl = float(1e-4 * (1 + rng.random()))
        plain.append((q, s, gl))
        fx, ex = oracle.csf_encode(s)
        csf_np.append({"weight": q, "csf_fixed": fx, "csf_exc": ex, "global": gl})
        csf_dev.append({"weight": _dev(q), "csf_fixed": _dev(fx), "csf_exc": _dev(ex), "global": gl})
        mixed_dev.append(csf_dev[-1] if j != 1 else {"weight": _dev(q), "scale": _dev(s), "global": gl})
    st0, want = oracle.record_pack(H, I, csf_np)
    assert st0 == 0 and np.array_equal(want, oracle.pack_record(H, I, *plain))
    used = int(E.ExpertRecLayout(H, I).g) + 12
    for projs in (csf_dev, mixed_dev):
        rec, st = E.record_pack(projs, H, I)
        torch.cuda.synchronize()
        E.context().check_device()
        assert st.tolist() == [[0, 0]] * 3
        assert np.array_equal(rec.cpu().numpy()[:used], want[:used])
    # the packed record through the decode operator equals the oracle's expert on the same bytes
    x = torch.tensor(rng.standard_normal((3, H)).astype(np.float32)).to(torch.bfloat16).to(dev)
    ids = torch.zeros((3, 1), dtype=torch.int32, device=dev); w = torch.ones((3, 1), dtype=torch.float32, device=dev)
    out = E.moe_decode_routed_f32(ids, w, E.rec_table([rec]), 0, 1, x, H, I)
    torch.cuda.synchronize()
    ref = np.stack([oracle.expert_forward(want, H, I, x[m].float().cpu().numpy()) for m in range(3)])
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True)) + 1e-12
    assert np.max(np.abs(out.cpu().numpy() - ref) / rms) <= 2e-2
    # a damaged down projection is reported in its slot, the others stay clear
    bad = list(csf_dev)
    e2 = np.append(csf_np[2]["csf_exc"], np.uint32(H * I // 16)).astype(np.uint32)
    bad[2] = dict(bad[2], csf_exc=_dev(e2))
    _, st = E.record_pack(bad, H, I)
    assert st.tolist() == [[0, 0], [0, 0], [4, e2.size - 1]]


@pytest.mark.parametrize("H,I,n", [(512, 256, 7), (256, 128, 60)])     # 21 tensors: one kernel per phase; 180: one block per tensor
def test_record_pack_batch_matches_oracle(E, oracle, H, I, n):
    """a batch of experts in one call: compressed, plain and mixed projections, one expert damaged, one with a repeated exception
    index — every record equals the oracle's, the damaged projection is reported in its own slot and nothing else is disturbed"""
    dev = torch.device("cuda")
    rng = np.random.default_rng(99)
    L = E.ExpertRecLayout(H, I)
    used = int(L.g) + 12
    recs = torch.zeros((n, int(L.total)), dtype=torch.uint8, device=dev)
    experts, want, keep = [], [], []
    for r in range(n):
        projs_np, projs_dev = [], []
        for j, (rows, K) in enumerate(((I, H), (I, H), (H, I))):
            q = rng.integers(0, 256, (rows, K // 2), dtype=np.uint8)
            s = csf_scale_matrix(rng, rows, K // 16)
            gl = float(1e-4 * (1 + rng.random()))
            fx, ex = oracle.csf_encode(s)
            if (r + j) % 3 == 0:
                projs_np.append({"weight": q, "scale": s, "global": gl}); projs_dev.append({"weight": _dev(q), "scale": _dev(s), "global": gl})
            else:
                if r == 2 and j == 2:                                   # entry 9 named twice with different values: the later word wins
                    fx = fx.copy(); fx[0, 16 + 4] &= 0x0F
                    ex = np.concatenate([ex, np.array([(0x31 << 24) | 9, (0x42 << 24) | 9], np.uint32)]).astype(np.uint32)
                if r == 4 and j == 1:
                    ex = np.append(ex, np.uint32((0x7F << 24) | 3)).astype(np.uint32); fx = fx.copy(); fx[0, 17] &= 0x0F   # delta of entry 3 cleared, value NaN
                projs_np.append({"weight": q, "csf_fixed": fx, "csf_exc": ex, "global": gl})
                projs_dev.append({"weight": _dev(q), "csf_fixed": _dev(fx), "csf_exc": _dev(ex), "global": gl})
        experts.append(projs_dev); keep.append(projs_np)
        want.append(oracle.record_pack(H, I, projs_np))
    jobs = E.record_jobs(experts, recs)
    st = E.record_pack_batch(jobs, n, H, I)
    torch.cuda.synchronize()
    E.context().check_device()
    st = st.cpu().numpy()
    got = recs.cpu().numpy()
    for r in range(n):
        code, rec = want[r]
        if r == 4:
            assert code == 20 + 6 and st[r].tolist() == [[0, 0], [6, keep[r][1]["csf_exc"].size - 1], [0, 0]]
            o = oracle.rec_layout(H, I)
            for a, b in ((0, int(o[3])), (int(o[4]), used)):                       # everything but the refused projection's scales
                assert np.array_equal(got[r, a:b], _expected_without_up_scales(oracle, H, I, keep[r])[a:b])
            continue
        assert code == 0 and st[r].tolist() == [[0, 0]] * 3, r
        assert np.array_equal(got[r, :used], rec[:used]), r


def _expected_without_up_scales(oracle, H, I, projs):
    good = [dict(p) for p in projs]
    good[1] = {"weight": projs[1]["weight"], "scale": np.zeros((I, H // 16), np.uint8), "global": projs[1]["global"]}
    code, rec = oracle.record_pack(H, I, good)
    assert code == 0
    return rec
