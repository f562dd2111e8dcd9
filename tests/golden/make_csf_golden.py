"""Generates tests/golden/csf_golden.npz: compressed NVFP4 block-scale tensors ("CSF") and what the reference engine's own decoder
(hive::ckq::csf_decode, compiled into oracle/_ref from the reference sources in place) makes of them.

    python tests/golden/make_csf_golden.py        (where the reference tree is mounted)

Inputs are seeded; the encoder is the test-side one in oracle/oracle.py (written from the format description).  Stored per case:
the compressed pair, the decoded matrix the reference returned, and for the damaged variants the reference's verdict (0 = refused).
The shapes are those of the reference's own test (640 x 160 and 2560 x 40 are the checkpoint's projections, 16 x 1 and 32 x 3 the
ragged small ones); rerunning must reproduce the file bit for bit.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
from oracle import oracle as O  # noqa: E402
from util import csf_damaged as damaged, csf_scale_matrix as scale_matrix, CSF_SHAPES as SHAPES  # noqa: E402


def main():
    O.build(ref=True)
    rng = np.random.default_rng(20261031)
    out = {}
    for k, (R, C) in enumerate(SHAPES):
        s = scale_matrix(rng, R, C)
        fx, ex = O.csf_encode(s)
        st, _, dec = O.csf_decode(fx, ex, R, C, use_ref=True)
        assert st == 0 and np.array_equal(dec, s)
        out[f"c{k}_fixed"], out[f"c{k}_exc"], out[f"c{k}_decoded"] = fx, ex, dec
        for name, (f2, e2, shp) in damaged(fx, ex, R, C).items():
            st, msg, _ = O.csf_decode(f2, e2, R, C, fixed_shape=shp, use_ref=True)
            out[f"c{k}_bad_{name}"] = np.array([st == 0], np.uint8)
            print(R, C, name, st, msg)
    # a repeated exception index: the later word wins in the reference's sequential loop
    R, C = 32, 8
    s = scale_matrix(rng, R, C)
    fx, ex = O.csf_encode(s)
    i = 5 if not ex.size else int(ex[0] & 0xFFFFFF)
    n = (i // C % 16) * C + i % C
    fx[i // C // 16, 16 + (n >> 1)] &= np.uint8(~(15 << ((n & 1) * 4)) & 0xFF)
    ex = np.concatenate([ex, np.array([(0x33 << 24) | i, (0x44 << 24) | i], np.uint32)]).astype(np.uint32)
    st, _, dec = O.csf_decode(fx, ex, R, C, use_ref=True)
    assert st == 0 and dec.reshape(-1)[i] == 0x44
    out["dup_fixed"], out["dup_exc"], out["dup_decoded"] = fx, ex, dec
    np.savez_compressed(Path(__file__).resolve().parent / "csf_golden.npz", **out)
    print("wrote csf_golden.npz", sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
