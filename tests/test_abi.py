"""CPU-side checks of the boundary: the shared library loads, exports every symbol the public header declares, lays records out
exactly like the reference, and sizes workspaces sanely.  No compute call is made (no GPU here)."""
import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def lib():
    from eke_hive_b200 import _lib
    return _lib


def test_library_exports_every_declared_symbol(lib):
    names = lib.declared_symbols()
    assert len(names) >= 25 and len(set(names)) == len(names)
    L = lib.load()
    for n in names:
        assert hasattr(L, n), n


def test_debug_library_exports_the_same_symbols(lib):
    """The range-checked debug build (-DHB_BOUNDS, `python eke_hive_b200/build.py --bounds`) is the same library: when it has been
    built it exports every declared symbol too."""
    from pathlib import Path
    p = Path(lib.__file__).resolve().parent / "libhive_b200_bounds.so"
    if not p.exists():
        pytest.skip("debug library not built")
    L = C.CDLL(str(p))
    for n in lib.declared_symbols():
        assert hasattr(L, n), n


def test_context_flags_are_the_headers(lib):
    """The Python mirror takes the HB_FLAG_* values from the header; they are distinct bits, and the ones the tests and the benchmark
    pass as numbers have the values used there."""
    import eke_hive_b200 as E
    vals = list(E.FLAGS.values())
    assert len(vals) >= 9 and all(v > 0 and v & (v - 1) == 0 for v in vals) and len(set(vals)) == len(vals)
    assert (E.HB_FLAG_PREFILL_A16, E.HB_FLAG_PREFILL_A16_ROWS, E.HB_FLAG_LAYER_A4) == (4, 256, 32)
    assert (E.HB_FLAG_DECODE_MMA_SYNC, E.HB_FLAG_DECODE_TC_GU, E.HB_FLAG_DECODE_TC_DOWN, E.HB_FLAG_FUSED, E.HB_FLAG_NO_PDL) == (8, 64, 128, 2, 1)


def test_pair_struct_matches_reference_abi(lib):
    # hive::glm::MoePair {int row; const uint8_t* rec; float w;} on LP64: 24 bytes, rec at 8, w at 16
    assert C.sizeof(lib.MoePair) == 24 and lib.MoePair.rec.offset == 8 and lib.MoePair.w.offset == 16


@pytest.mark.parametrize("H,I", [(2048, 512), (4096, 1536), (7168, 2048), (128, 64)])
def test_record_layout_matches_reference_and_oracle(lib, oracle, H, I):
    L = lib.load()
    r = lib.RecLayout()
    assert L.hb_rec_layout_make(H, I, C.byref(r)) == 0
    off = oracle.rec_layout(H, I)
    got = [r.w1, r.s1, r.w3, r.s3, r.w2, r.s2, r.g, r.total]
    assert got == [int(v) for v in off]
    assert r.total % 4096 == 0 and r.total - r.g >= 12 and r.g == 3 * H * I * 9 // 16


def test_layout_rejects_bad_shapes(lib):
    L = lib.load()
    r = lib.RecLayout()
    assert L.hb_rec_layout_make(100, 64, C.byref(r)) < 0
    assert L.hb_rec_layout_make(0, 64, C.byref(r)) < 0
    assert L.hb_rec_layout_make(128, 64, None) < 0


def test_workspace_and_support_queries(lib):
    L = lib.load()
    assert L.hb_moe_decode_supported(2048, 512) == 2      # streaming path
    assert L.hb_moe_decode_supported(4096, 1536) == 2
    assert L.hb_moe_decode_supported(128, 64) == 1        # generic kernels
    assert L.hb_moe_decode_supported(7168, 2048) == 1
    assert L.hb_moe_decode_supported(100, 64) == 0
    a, b = L.hb_moe_decode_ws_bytes(176, 2048, 512), L.hb_moe_decode_ws_bytes(352, 2048, 512)
    assert a % 256 == 0 and a >= 176 * (2048 + 512) * 2 and a < b < 2 * a + 4096


def test_status_strings_and_null_context(lib):
    L = lib.load()
    assert L.hb_status_string(0) == b"ok" and b"unsupported" in L.hb_status_string(-2)
    assert L.hb_sm_count(None) == 0 and L.hb_launch_count(None) == 0
    assert L.hb_moe_decode(None, None, 1, None, 256, 256, 0.0, None, None, None) == -1     # null context: a code, not a crash


def test_no_cpu_fallback_without_device(lib):
    """On a machine without a GPU the context cannot be created: the product path fails loudly instead of computing on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = lib.load()
    h = C.c_void_p()
    cfg = lib.Config(0, 0, 0)
    assert L.hb_create(C.byref(cfg), C.byref(h)) == -4 and not h.value
    import eke_hive_b200 as E
    with pytest.raises(E.HbError):
        E.Context()


def test_dispatch_plan_host_logic(lib):
    """hb_dispatch_plan is pure host code: counts, group / tile numbers and the rows ≤ 64 → decode, more → grouped GEMM switch."""
    L = lib
    lib = L.load()
    rng = np.random.default_rng(3)
    for M, K, E, H, I in ((16, 10, 512, 2048, 512), (8192, 8, 256, 7168, 2048), (100, 4, 16, 2048 + 32, 512), (64, 8, 160, 4096, 1536)):
        ids = np.stack([rng.permutation(E)[:K] for _ in range(M)]).astype(np.int32)
        ids[0, 0] = -1
        ids[M - 1, K - 1] = E + 5
        counts = np.zeros(E, np.int32)
        p = L.Plan()
        assert lib.hb_dispatch_plan(ids.ctypes.data, M, K, E, H, I, counts.ctypes.data, C.byref(p)) == 0
        ref = np.bincount(ids[(ids >= 0) & (ids < E)], minlength=E)
        assert np.array_equal(counts, ref)
        assert p.pairs == int(ref.sum()) and p.distinct_experts == int((ref > 0).sum()) and p.max_rows == int(ref.max())
        assert p.decode_groups == int(((ref + 7) // 8).sum()) and p.prefill_tiles == int(((ref + 127) // 128).sum())
        want = 1 if (M > 64 and H % 256 == 0 and I % 256 == 0) else 0
        assert p.regime == want
        assert abs(p.tile_fill - ref.sum() / (128.0 * p.prefill_tiles)) < 1e-12
        if want == 1:
            assert p.ws_bytes == lib.hb_moe_prefill_ws_bytes(M, K, E, H, I) > 0


def test_cxx_drop_in_header_compiles_and_links(tmp_path):
    """The C++ surface with the reference's namespaces and signatures (csrc/hive_compat.hpp) compiles as host C++ against the public
    header and links against the shared library — a maintainer's call sites keep compiling.  Nothing is run (no GPU here)."""
    import shutil
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cxx = shutil.which("g++", path="/usr/bin") or shutil.which("g++")
    if cxx is None or not Path("/usr/local/cuda/include/cuda_runtime.h").exists():
        pytest.skip("no host C++ compiler or CUDA headers")
    src = tmp_path / "callsites.cpp"
    src.write_text(r'''
#include "hive_compat.hpp"
// the reference's own call shapes (glm_experts.cpp:630, qwen_engine.cpp:842-878, fn_moe.h, q27_kernels.h)
void decode_site(const hive::glm::ExpertRecLayout& L, const hive::glm::MoePair* pairs, int n, const __nv_bfloat16* x, float* out, void* ws, cudaStream_t st) {
  hive::glm::moe_decode(L, pairs, n, x, 4096, 1536, 10.f, out, ws, st);
}
void routed_site(const hive::glm::ExpertRecLayout& L, const int32_t* ids, const float* w, const uint8_t* const* tab, const __nv_bfloat16* x,
                 const __nv_bfloat16* shared, const float* lg, __nv_bfloat16* out, void* ws, cudaStream_t st) {
  hive::qwen::fn_moe_decode_routed(L, ids, w, 16, 10, tab, 3, 512, x, 2048, 512, shared, lg, 513, 512, out, ws, st);
  hive::qwen::FnPfCombine c{shared, lg, 513, 512, out};
  hive::qwen::fn_moe_prefill(L, tab, 3, 512, ids, w, 8192, 10, x, 2048, 512, nullptr, ws, 8192, st, &c);
}
size_t sizes() { return hive::glm::moe_decode_ws_bytes(176, 2048, 512) + hive::qwen::fn_moe_prefill_ws_bytes(8192, 8, 256, 7168, 2048); }
int main() { return sizes() > 0 ? 0 : 1; }
''')
    exe = tmp_path / "callsites"
    cmd = [cxx, "-std=c++17", "-I", str(root / "include"), "-I", str(root / "eke_hive_b200" / "csrc"), "-I", "/usr/local/cuda/include", str(src),
           "-L", str(root / "eke_hive_b200"), "-lhive_b200", "-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + str(root / "eke_hive_b200"),
           "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]


def test_python_signatures_have_the_headers_argument_counts(lib):
    """every prototype of include/hive_b200.h that the ctypes mirror binds is bound with the same number of arguments (a missing
    argtype shifts every later argument: a host crash, not an error code)"""
    import re
    from pathlib import Path
    text = (Path(__file__).resolve().parent.parent / "include" / "hive_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    protos = dict()
    for m in re.finditer(r"HB_API\s+[\w\s\*]+?\b(hb_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        protos[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    assert len(protos) > 40
    bound = 0
    dll = lib.load()
    for name, n in protos.items():
        fn = getattr(dll, name)
        if fn.argtypes is None:
            continue
        bound += 1
        assert len(fn.argtypes) == n, f"{name}: header has {n} arguments, the Python mirror binds {len(fn.argtypes)}"
    assert bound > 40
