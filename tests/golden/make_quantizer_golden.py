"""Generates tests/golden/quantizer_golden.npz with the reference's own NVFP4 weight quantiser.

The reference rule lives in a numpy-only tool of the reference project (tools/q27_reencode.py, function nvfp4():
global scale 448*6/amax, per-16 e4m3 scale searched over five factors, e2m1 codes by round-to-nearest with ties to the
even code).  This script imports that function, runs it on seeded matrices and stores inputs and outputs, so that the
oracle's restatement (ho_nvfp4_quantize, search on) can be held to it bit for bit anywhere:

    python tests/golden/make_quantizer_golden.py <path of the reference checkout>
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np


def cases():
    rng = np.random.default_rng(20261126)
    out = {}
    out["a"] = rng.normal(0, 0.02, (37, 64)).astype(np.float32)
    out["b"] = rng.normal(0, 0.02, (48, 512)).astype(np.float32)
    # quarter-integers: many values sit exactly between two e2m1 codes for several of the searched scales (ties to the even code),
    # and many blocks give the same error for two factors (the first factor wins)
    out["ties"] = (rng.integers(-12, 13, (64, 256)) * 0.25).astype(np.float32)
    # heavy tails: a few blocks get subnormal e4m3 scales, one block is all zero
    w = (rng.standard_t(2, (24, 1024)) * 0.02).astype(np.float32)
    w[3, 32:48] = 0.0
    w[5, :16] *= 1e-4
    out["tails"] = w
    out["zero"] = np.zeros((4, 32), np.float32)
    return out


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    spec = importlib.util.spec_from_file_location("q27_reencode", Path(sys.argv[1]) / "tools" / "q27_reencode.py")
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {}
    for tag, w in cases().items():
        q, s, g = ref.nvfp4(w)
        out[f"{tag}_w"] = w
        out[f"{tag}_q"] = q
        out[f"{tag}_s"] = s
        out[f"{tag}_g_div"] = g            # divide convention: w ≈ e2m1·e4m3 / g
    np.savez_compressed(Path(__file__).resolve().parent / "quantizer_golden.npz", **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
