// Routed-expert prefill (rows > 64): one grouped W4A4 GEMM pass over every expert that received rows, on the 5th-generation tensor
// cores.  Mirrors hive::qwen::fn_moe_prefill with its NVFP4-activation switch on (engine/src/qwen/fn_moe_pf.cu:439-446, :858-941):
//
//   plan                  the (row, k) pairs sorted by expert (the order inside an expert is irrelevant: a pair's result depends only
//                         on its own row) and a list of 128-pair tiles — one launch of a few CTAs that meet once (pf_plan_kernel)
//   quantise x            per-row dynamic NVFP4 (hb_a4_quant's rule); a row is quantised once and written straight into the slots of
//                         its pairs, so the GEMM's activation tiles are contiguous
//   gate|up GEMM          tile = 128 pairs × (128 gate + 128 up rows of I); block-scaled FP4 MMA, fp32 accumulators in tensor memory;
//                         epilogue g = bf16(acc·gx·g1), u = bf16(acc·gx·g3), y = bf16(silu(g)·u)
//   quantise y            per pair
//   down GEMM             tile = 128 pairs × 256 rows of H; part[pair] = bf16(acc·(gy·g2))
//   sum                   out[row] = Σ_k part·w in k order (or the fused shared-expert combine)
//
// GEMM kernel: persistent CTAs of 15 warps.  One warp moves the e2m1 codes of both operands with TMA (`cp.async.bulk.tensor`, 128-byte
// swizzle: the K-major layout the MMA reads).  The activation rows of a tile are contiguous because the quantised rows are first
// copied into expert order; the weight matrices sit inside expert records at arbitrary addresses, so a small kernel stamps each
// record's addresses into tensor maps on the device (`tensormap.replace`).  The e4m3 block scales are fetched by the scale warps with
// plain 16-byte loads (one row of a stage each) and put into the chunk order tensor memory wants.  One warp issues
// `tcgen05.mma kind::mxf4nvf4` (block 16, ue4m3 scales: both operands' block scales are applied by the tensor core) and commits to
// the stage's mbarrier.  Four warps read the accumulators back with `tcgen05.ld` and run the epilogue.  Every wait is bounded; on a
// timeout the kernel records a site code in the context's error word, drains its copies, frees its tensor memory and returns.
//
// With bf16 activations (HB_FLAG_PREFILL_A16, the reference's default prefill arithmetic, fn_moe_pf.cu:118-437) the same plan feeds
// another pair of GEMMs: tcgen05 kind::f16 over weight tiles dequantised exactly to bf16, the pairs as the B operand (pf_a16.cuh);
// no quantisation passes, a slot-ordered copy of the activation rows instead.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "hb_common.cuh"
#include "hb_kernels.h"
#include "tc_common.cuh"

namespace hb {

constexpr int PF_BM = 128;              // pairs per tile (MMA M)
constexpr int PF_BN = 256;              // weight rows per tile (MMA N)
constexpr int PF_BK = 256;              // k values per stage = one 128-byte swizzle row of e2m1 codes
constexpr int PF_ST = 3;                // stages
constexpr int PF_A_BYTES = PF_BM * 128, PF_B_BYTES = PF_BN * 128;
constexpr int PF_SFA_BYTES = 4 * 512;   // 4 MMA k-steps × one 128-row chunk
constexpr int PF_SFB_BYTES = 8 * 512;   // two 128-row blocks × 4 k-steps
constexpr int PF_STAGE = PF_A_BYTES + PF_B_BYTES + PF_SFA_BYTES + PF_SFB_BYTES;
constexpr int PF_STG_PITCH = 144;        // epilogue staging: 32 rows × 128 bytes per warp, rows padded to 144 bytes (conflict-free 16-byte accesses)
constexpr int PF_STG_BYTES = 32 * PF_STG_PITCH;
constexpr int PF_SMEM = PF_ST * PF_STAGE + 1024 + 512 + 8 * PF_STG_BYTES;
constexpr int PF_THREADS = 14 * 32;     // warps 0-3 and 10-13 epilogue, 4 MMA issue, 5 TMA, 6-9 scales (global → tensor memory)
constexpr int PF_TMEM_COLS = 512;
constexpr int PF_SF_COL0 = 256;         // accumulator: columns [0, 256); scales of stage s: [256 + 48 s, 256 + 48 s + 48)
static_assert(PF_SF_COL0 + 48 * PF_ST <= PF_TMEM_COLS, "tensor memory");
static_assert(PF_STAGE % 1024 == 0, "stage buffers must keep the 1024-byte alignment of the swizzle atom");
static_assert(PF_SMEM <= 227 * 1024, "shared memory");

struct TileRef { int slot0, rows, expert; };   // 128 consecutive slots (or fewer) of one expert's run of the sorted pairs (256 for the bf16-activation GEMM)
}  // namespace hb
#include "pf_a16.cuh"
namespace hb {

enum { PF_PLAIN = 0, PF_GU = 1, PF_DOWN = 2 };

struct PfGemmArgs {
  // work list
  const TileRef* tiles; const int* n_tiles;     // n_tiles == nullptr: one implicit tile list of ceil(M / 128) tiles over rows [0, M)
  int M;                                       // PLAIN only
  const int* perm;                             // pair of a sorted slot (DOWN scatters its rows by it)
  // A operand (quantised activations, tile rows contiguous): codes come through the kernel's tensor-map parameter
  const uint8_t* as; const float* ag; int Kd;  // scales [rows, Kd/16] and per-row global (codes: tensor-map parameter)
  // B operand
  const uint8_t* const* tab; hb_rec_layout L;  // GU / DOWN: expert records
  const CUtensorMap* tmB;                      // GU / DOWN: [expert][6] tensor maps of w1, w3, w2, s1, s3, s2 (written by pf_tmaps_kernel)
  const uint8_t* bs; float bg;                 // PLAIN: scales and global of the one matrix [N, Kd] (codes: tensor-map parameter)
  int N;                                       // output columns in all (I for GU, H for DOWN, N for PLAIN)
  float limit;
  void* out; int ldo;                          // GU: y bf16 [slots, I]; DOWN: part bf16 [pairs, H]; PLAIN: fp32 [M, ldo]
  uint32_t* err;
};

// Instruction descriptor, kind::mxf4nvf4: A and B e2m1 (format 1, bits 7-9 and 10-12), both K-major, N / 8 at bit 17, ue4m3 scales
// (bit 23 = 0), M / 16 at bit 24, K = 64 per instruction (bit 31 = 0).
constexpr uint32_t PF_IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(PF_BN >> 3) << 17) | ((uint32_t)(PF_BM >> 4) << 24);

// ---- the grouped GEMM ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ TileRef pf_tile(const PfGemmArgs& a, int ti) {
  if (a.tiles) return a.tiles[ti];
  TileRef t; t.expert = 0; t.slot0 = ti * PF_BM; t.rows = min(PF_BM, a.M - ti * PF_BM);
  return t;
}
__device__ __forceinline__ uint4 pf_pack8(const float* v) {
  const __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
  const __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
  return make_uint4(*reinterpret_cast<const uint32_t*>(&p0), *reinterpret_cast<const uint32_t*>(&p1), *reinterpret_cast<const uint32_t*>(&p2),
                    *reinterpret_cast<const uint32_t*>(&p3));
}

// Epilogue staging → global: the warp's 32 rows × 128 bytes leave as 8 stores of 4 rows × 128 contiguous bytes (a thread owns a row
// when it reads tensor memory, which would make every store instruction touch 32 different rows).  gptr: this lane's row in
// global memory (nullptr = row past the tile's end), already offset to the first of the 128 bytes.
__device__ __forceinline__ void pf_epi_flush(const uint8_t* stg, uint8_t* gptr, int lane) {
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    uint8_t* p = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(gptr), r));
    const uint4 v = *reinterpret_cast<const uint4*>(stg + r * PF_STG_PITCH + (lane & 7) * 16);
    if (p) *reinterpret_cast<uint4*>(p + (lane & 7) * 16) = v;
  }
  __syncwarp();
}

template <int MODE>
__global__ void __launch_bounds__(PF_THREADS, 1) pf_gemm_kernel(const PfGemmArgs a, const __grid_constant__ CUtensorMap tmA,
                                                                const __grid_constant__ CUtensorMap tmB0) {
  extern __shared__ uint8_t pf_raw[];
  const uint32_t raw = smem_u32(pf_raw), base = (raw + 1023u) & ~1023u;     // swizzle atoms want 1024-byte alignment
  uint8_t* sm = pf_raw + (base - raw);
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + PF_ST * PF_STAGE);       // [ST] operands of the stage have landed
  uint64_t* empty = full + PF_ST;                                            // [ST] the MMAs that read the stage are done
  uint64_t* acc_full = empty + PF_ST;                                        // the tile's accumulators are complete
  uint64_t* acc_empty = acc_full + 1;                                        // the epilogue has read them
  uint64_t* mma_done = acc_empty + 1;                                        // the issuing thread's last operation has retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < PF_ST; ++s) { mbar_init(&full[s], 128 + 1); mbar_init(&empty[s], 1); }   // full: 128 scale threads (scales are in tensor memory) + the TMA thread
    mbar_init(acc_full, 1); mbar_init(acc_empty, 256); mbar_init(mma_done, 1);
    mbar_fence_init();
  }
  if (warp == 4) { tmem_alloc(tmem_slot, PF_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  griddep_wait();
  griddep_launch();
  const int n_tiles = a.tiles ? *a.n_tiles : (a.M + PF_BM - 1) / PF_BM;
  constexpr int NW = MODE == PF_GU ? 128 : 256;                              // output columns per tile
  const int n_nt = a.N / NW, nkb = a.Kd / PF_BK;
  const long long work = (long long)n_tiles * n_nt;                          // tile-major: the CTAs of a wave share activation tiles and expert rows in L2

  if (warp == 5) {
    // ------------------------------------------------------------------------------------------------ TMA: codes of both operands, one thread
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long w = blockIdx.x; w < work && ok; w += gridDim.x) {
        const int ti = (int)(w / n_nt), nt = (int)(w - (long long)ti * n_nt);
        const TileRef tl = pf_tile(a, ti);
        const CUtensorMap *m0 = &tmB0, *m1 = &tmB0;
        int r0 = nt * 256, r1 = nt * 256 + 128;                               // B rows of the tile's two 128-row boxes
        if (MODE == PF_GU) { m0 = a.tmB + (size_t)tl.expert * 6; m1 = m0 + 1; r0 = r1 = nt * 128; }
        if (MODE == PF_DOWN) m0 = m1 = a.tmB + (size_t)tl.expert * 6 + 2;
        if (MODE != PF_PLAIN) { tmap_acquire(m0); if (m1 != m0) tmap_acquire(m1); }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t stage = it % PF_ST;
          if (!(ok = mbar_wait(&empty[stage], ((it / PF_ST) & 1) ^ 1, a.err, 0x100u))) break;
          const uint32_t sb = base + stage * PF_STAGE;
          mbar_expect_tx(&full[stage], PF_A_BYTES + PF_B_BYTES);
          tma_load_2d(sb, &tmA, kb * 128, tl.slot0, &full[stage]);
          tma_load_2d(sb + PF_A_BYTES, m0, kb * 128, r0, &full[stage]);
          tma_load_2d(sb + PF_A_BYTES + 128 * 128, m1, kb * 128, r1, &full[stage]);
        }
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // ------------------------------------------------------------------------------------------------ scales: thread lt owns row lt of each 128-row block
    // A row's 16 scale bytes of a stage = 4 MMA k-steps × 4 scales (one 32-bit word per k-step).  The tensor core reads the scales
    // from tensor memory: for the A rows of lane quarter q, word j of row 32 q + l from lane l, column 4 j + q; for the B rows, word j
    // of row 32 c + l (c = 0..7) from lane l, column 16 + 8 j + c, of EVERY quarter.  Each thread fetches its three rows (A block, two
    // B blocks) two stages ahead into registers, drops them row-major into the stage's shared-memory slab (consecutive threads,
    // consecutive 16 bytes: no bank conflicts), and after a barrier among the four warps picks up the eight B rows its own lane needs and
    // stores everything into its own lane of tensor memory with two tcgen05.st — no tcgen05.cp on the MMA pipe, no transposition.
    const int q = warp & 3, l = lane, lt = 32 * q + l;                      // a warp reaches the tensor-memory lanes of quarter (warp index mod 4): its rows are those
    const uint32_t sf_lane = tmem + ((uint32_t)(q * 32) << 16);
    const size_t rows = (size_t)a.Kd / 16;
    uint32_t it = 0;
    bool ok = true;
    struct Rows { const uint8_t *pa, *pb, *pc; };
    auto rows_of = [&](long long w) {                                       // this thread's three scale rows of work item w
      Rows r = {nullptr, nullptr, nullptr};
      if (w >= work) return r;
      const int ti = (int)(w / n_nt), nt = (int)(w - (long long)ti * n_nt);
      const TileRef tl = pf_tile(a, ti);
      r.pa = a.as + (size_t)(tl.slot0 + min(lt, tl.rows - 1)) * rows;          // rows past the tile's end repeat its last row (never stored)
      if (MODE == PF_PLAIN) { r.pb = a.bs + (size_t)(nt * 256 + lt) * rows; r.pc = r.pb + 128 * rows; }
      else {
        const uint8_t* rec = a.tab[tl.expert];
        if (MODE == PF_GU) { r.pb = rec + a.L.s1 + (size_t)(nt * 128 + lt) * rows; r.pc = rec + a.L.s3 + (size_t)(nt * 128 + lt) * rows; }
        else { r.pb = rec + a.L.s2 + (size_t)(nt * 256 + lt) * rows; r.pc = r.pb + 128 * rows; }
      }
      return r;
    };
    // the loads run two stages ahead of the stores, across work items: a cursor of their own
    long long pw = blockIdx.x;
    int pkb = 0;
    Rows pr = rows_of(pw);
    auto fetch = [&](uint4& x0, uint4& x1, uint4& x2) {
      if (pr.pa) {
        x0 = __ldg(reinterpret_cast<const uint4*>(pr.pa) + pkb); x1 = __ldg(reinterpret_cast<const uint4*>(pr.pb) + pkb); x2 = __ldg(reinterpret_cast<const uint4*>(pr.pc) + pkb);
      }
      if (++pkb == nkb) { pkb = 0; pw += gridDim.x; pr = rows_of(pw); }
    };
    uint4 va = make_uint4(0, 0, 0, 0), vb = va, vc = va, na = va, nb = va, nc = va;
    fetch(va, vb, vc);
    fetch(na, nb, nc);
    for (long long w = blockIdx.x; w < work && ok; w += gridDim.x) {
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const uint32_t stage = it % PF_ST;
        uint4 fa = make_uint4(0, 0, 0, 0), fb = fa, fc = fa;
        fetch(fa, fb, fc);                                                   // the latency of these loads is never waited for
        if (!(ok = mbar_wait(&empty[stage], ((it / PF_ST) & 1) ^ 1, a.err, 0x4000u))) break;   // the MMAs that read the stage's slab and scale columns are done
        tc_fence_after();
        uint4* slab = reinterpret_cast<uint4*>(sm + stage * PF_STAGE + PF_A_BYTES + PF_B_BYTES + PF_SFA_BYTES);   // B scales, row-major: [256][16 bytes]
        slab[lt] = vb; slab[128 + lt] = vc;
        named_bar_sync(5, 128);
        uint32_t wa[16], wb[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) wa[i] = 0u;
        const uint32_t va4[4] = {va.x, va.y, va.z, va.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) if (qq == q) wa[4 * j + qq] = va4[j];
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 r4 = slab[32 * c + l];
          wb[c] = r4.x; wb[8 + c] = r4.y; wb[16 + c] = r4.z; wb[24 + c] = r4.w;
        }
        const uint32_t sfc = sf_lane + PF_SF_COL0 + stage * 48;
        tc_st16(sfc, wa);
        tc_st32(sfc + 16, wb);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&full[stage]);                                           // (the slab is not written again before every thread has arrived here: the MMAs wait for all)
        va = na; vb = nb; vc = nc; na = fa; nb = fb; nc = fc;
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------------------------------------ MMA issue: one thread
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (long long w = blockIdx.x; w < work && ok; w += gridDim.x, ++tcount) {
        if (tcount > 0 && !(ok = mbar_wait(acc_empty, (tcount - 1) & 1, a.err, 0x200u))) break;
        tc_fence_after();
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t stage = it % PF_ST;
          if (!(ok = mbar_wait(&full[stage], (it / PF_ST) & 1, a.err, 0x400u))) break;
          tc_fence_after();
          const uint32_t sb = base + stage * PF_STAGE, sfc = tmem + PF_SF_COL0 + stage * 48;
          const uint64_t ad = tc_desc_sw128(sb), bd = tc_desc_sw128(sb + PF_A_BYTES);
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j)                                   // 64 k values = 32 bytes further along the swizzled row
            tc_mma_nvf4(tmem, ad + 2 * j, bd + 2 * j, PF_IDESC, sfc + 4 * j, sfc + 16 + 8 * j, (kb | (int)j) != 0 ? 1u : 0u);
          tc_commit(&empty[stage]);
        }
        if (ok) tc_commit(acc_full);
      }
      tc_commit(mma_done);                                                   // nothing of this thread's is in flight when tensor memory is freed
      mbar_wait(mma_done, 0, a.err, 0x800u);
    }
  } else if (warp < 4 || (warp >= 10 && warp < 14)) {
    // ------------------------------------------------------------------------------------------------ epilogue: a warp reads the 32 lanes of its quarter (warp index mod 4);
    // warps 0-3 take the first half of the tile's columns, warps 10-13 the second
    const int qtr = warp & 3, half = warp >= 10 ? 1 : 0;
    const int m = qtr * 32 + lane;
    const uint32_t trow = tmem + ((uint32_t)(qtr * 32) << 16);
    uint8_t* stg = sm + PF_ST * PF_STAGE + 512 + (size_t)(half * 4 + qtr) * PF_STG_BYTES;
    uint32_t tcount = 0;
    bool ok = true;
    for (long long w = blockIdx.x; w < work && ok; w += gridDim.x, ++tcount) {
      const int ti = (int)(w / n_nt), nt = (int)(w - (long long)ti * n_nt);
      const TileRef tl = pf_tile(a, ti);
      const bool valid = m < tl.rows;
      const int slot = tl.slot0 + min(m, tl.rows - 1);
      float f0 = 0.f, f1 = 0.f, f2 = 0.f;
      size_t orow = 0;
      if (MODE == PF_PLAIN) { f0 = a.ag[slot] * a.bg; orow = (size_t)slot; }
      else {
        const float* g = reinterpret_cast<const float*>(a.tab[tl.expert] + a.L.g);
        if (MODE == PF_GU) { f0 = a.ag[slot]; f1 = g[0]; f2 = g[1]; orow = (size_t)slot; }
        else { f0 = a.ag[slot] * g[2]; orow = (size_t)a.perm[slot]; }
        (void)HB_BOUND(a.err, tl.expert >= 0 && tl.rows >= 1 && tl.rows <= PF_BM && tl.slot0 >= 0, 0x202u, tl.slot0);
      }
      if (!(ok = mbar_wait(acc_full, tcount & 1, a.err, 0x1000u))) break;
      tc_fence_after();
      uint8_t* mine = stg + lane * PF_STG_PITCH;
      if (MODE == PF_GU) {
        uint8_t* gp = valid ? reinterpret_cast<uint8_t*>(reinterpret_cast<__nv_bfloat16*>(a.out) + orow * a.ldo + (size_t)nt * 128 + 64 * half) : nullptr;
#pragma unroll 1
        for (int c2 = 0; c2 < 2; ++c2) {
          const int c = 2 * half + c2;
          uint32_t rg[32], ru[32];
          tc_ld32(trow + 32 * c, rg);
          tc_ld32(trow + 128 + 32 * c, ru);
          tc_wait_ld();
          if (c2 == 1) { tc_fence_before(); mbar_arrive(acc_empty); }       // the accumulators are read: the next tile may start
          float y[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float gv = bf16r(__uint_as_float(rg[i]) * f0 * f1), uv = bf16r(__uint_as_float(ru[i]) * f0 * f2);
            if (a.limit > 0.f) { gv = fminf(gv, a.limit); uv = fminf(fmaxf(uv, -a.limit), a.limit); }
            y[i] = gv / (1.f + __expf(-gv)) * uv;
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(mine + c2 * 64 + q * 16) = pf_pack8(y + 8 * q);
        }
        pf_epi_flush(stg, gp, lane);
      } else if (MODE == PF_DOWN) {
#pragma unroll 1
        for (int p2 = 0; p2 < 2; ++p2) {
          uint8_t* gp = valid ? reinterpret_cast<uint8_t*>(reinterpret_cast<__nv_bfloat16*>(a.out) + orow * a.ldo + (size_t)nt * 256 + 128 * half + 64 * p2) : nullptr;
#pragma unroll 1
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t r[32];
            tc_ld32(trow + 128 * half + 64 * p2 + 32 * c2, r);
            tc_wait_ld();
            if (p2 == 1 && c2 == 1) { tc_fence_before(); mbar_arrive(acc_empty); }
            float y[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(r[i]) * f0;
#pragma unroll
            for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(mine + c2 * 64 + q * 16) = pf_pack8(y + 8 * q);
          }
          pf_epi_flush(stg, gp, lane);
        }
      } else {
#pragma unroll 1
        for (int c = 4 * half; c < 4 * half + 4; ++c) {
          uint8_t* gp = valid ? reinterpret_cast<uint8_t*>(reinterpret_cast<float*>(a.out) + orow * a.ldo + (size_t)nt * 256 + 32 * c) : nullptr;
          uint32_t r[32];
          tc_ld32(trow + 32 * c, r);
          tc_wait_ld();
          if (c == 4 * half + 3) { tc_fence_before(); mbar_arrive(acc_empty); }
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(mine + q * 16) = make_float4(__uint_as_float(r[4 * q]) * f0, __uint_as_float(r[4 * q + 1]) * f0,
                                                                    __uint_as_float(r[4 * q + 2]) * f0, __uint_as_float(r[4 * q + 3]) * f0);
          pf_epi_flush(stg, gp, lane);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, PF_TMEM_COLS); }
}

// Tensor-pipe ceiling: the same MMA issued back to back on operands that sit in shared memory (arbitrary bytes), no loads, no epilogue.
__global__ void __launch_bounds__(128, 1) pf_peak_kernel(int n_rounds, uint32_t* err) {
  extern __shared__ uint8_t pf_raw[];
  const uint32_t raw = smem_u32(pf_raw), base = (raw + 1023u) & ~1023u;
  uint8_t* sm = pf_raw + (base - raw);
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + PF_STAGE);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < PF_STAGE / 4; i += blockDim.x) {            // e2m1 codes: any bytes; scales: 0x38 = 1.0
    uint32_t v = (uint32_t)i * 2654435761u + 0x9E3779B9u * (blockIdx.x + 1);
    reinterpret_cast<uint32_t*>(sm)[i] = i * 4 < PF_A_BYTES + PF_B_BYTES ? v : 0x38383838u;
  }
  if (threadIdx.x == 0) { mbar_init(bar, 1); mbar_fence_init(); }
  fence_proxy_async_smem();
  if (warp == 0) { tmem_alloc(tmem_slot, PF_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t sfc = tmem + PF_SF_COL0;
    for (uint32_t j = 0; j < 4; ++j) {
      tc_cp_sf(sfc + 4 * j, tc_desc_sf(base + PF_A_BYTES + PF_B_BYTES + j * 512));
      tc_cp_sf(sfc + 16 + 8 * j, tc_desc_sf(base + PF_A_BYTES + PF_B_BYTES + PF_SFA_BYTES + (2 * j) * 512));
      tc_cp_sf(sfc + 16 + 8 * j + 4, tc_desc_sf(base + PF_A_BYTES + PF_B_BYTES + PF_SFA_BYTES + (2 * j + 1) * 512));
    }
    const uint64_t ad = tc_desc_sw128(base), bd = tc_desc_sw128(base + PF_A_BYTES);
    for (int r = 0; r < n_rounds; ++r)
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) tc_mma_nvf4(tmem, ad + 2 * j, bd + 2 * j, PF_IDESC, sfc + 4 * j, sfc + 16 + 8 * j, (r | (int)j) != 0 ? 1u : 0u);
    tc_commit(bar);
    mbar_wait(bar, 0, err, 0x2000u);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, PF_TMEM_COLS); }
}

// ---- the plan of a call: pairs sorted by expert, and the tile list ---------------------------------------------------------------
// One launch of up to 64 CTAs that meet once in the middle (all are resident: the grid is smaller than the machine).  A CTA owns a
// contiguous slice of the pairs.  First half: a histogram of its slice over the experts in shared memory, stored as row `cta` of a
// [CTAs][E] table.  After the meeting every CTA adds up the table's columns for itself — the column total gives the expert's run
// (an exclusive scan over the experts, done redundantly by every CTA), the rows above its own give where its slice's share of the run
// starts — and places its pairs with shared-memory cursors.  No global atomics on the data, no separate scan launch, and a pair's
// slot depends only on which CTA holds it and on the order inside that CTA (any order inside an expert's run gives the same
// results: a pair's output depends on its own row alone).  CTA 0 also writes the tile list.  pos_of[p] = slot of pair p, or -1 for
// a pair that contributes nothing (id outside [0, E), or no record for the expert on this GPU).
constexpr int PLAN_THREADS = 1024, PLAN_MAX_CTAS = 64;
struct PlanArgs {
  const int32_t* ids; int P, E; const uint8_t* const* tab;
  int bm;                          // pairs per tile, at most
  int even;                        // 1: an expert's run is cut into its ceil(run / bm) tiles of equal size instead of full tiles and a rest
  int* hist;                       // [CTAs][E]
  int* perm; int* pos_of; TileRef* tiles; int* n_tiles; int* n_slots;
  unsigned int* meet;              // two context-owned counters, zero between launches
  uint32_t* err;
};
__global__ void __launch_bounds__(PLAN_THREADS) pf_plan_kernel(const PlanArgs a) {
  __shared__ int cur[1024];
  __shared__ int wsum[2][32];
  const int G = gridDim.x, cta = blockIdx.x, t = threadIdx.x, lane = t & 31, wp = t >> 5;
  const int per = (a.P + G - 1) / G, p0 = min(a.P, cta * per), p1 = min(a.P, p0 + per);
  auto expert_of = [&](int p) -> int { const int e = a.ids[p]; return (e >= 0 && e < a.E && a.tab[e] != nullptr) ? e : -1; };
  cur[t] = 0;
  __syncthreads();
  for (int p = p0 + t; p < p1; p += PLAN_THREADS) { const int e = expert_of(p); if (e >= 0) atomicAdd(&cur[e], 1); }
  __syncthreads();
  if (t < a.E) a.hist[(size_t)cta * a.E + t] = cur[t];
  // ---- the meeting
  __threadfence();
  __syncthreads();
  if (t == 0) {
    atomicAdd(a.meet, 1u);
    uint32_t spins = 0;
    while (*reinterpret_cast<volatile unsigned int*>(a.meet) < (unsigned)G) {
      if (++spins > (1u << 24)) { atomicOr(a.err, 0x4000u); break; }
      __nanosleep(64);
    }
    __threadfence();
    if (atomicAdd(a.meet + 1, 1u) == (unsigned)G - 1) { a.meet[0] = 0u; a.meet[1] = 0u; }   // the last one through clears both for the next launch
  }
  __syncthreads();
  // ---- column sums, the scan over the experts, this CTA's cursors
  int tot = 0, above = 0;
  if (t < a.E) {
    for (int g = 0; g < G; ++g) { const int h = __ldcg(a.hist + (size_t)g * a.E + t); if (g < cta) above += h; tot += h; }
  }
  const int nt = (tot + a.bm - 1) / a.bm;
  int ic = tot, it = nt;
  for (int o = 1; o < 32; o <<= 1) {
    const int uc = __shfl_up_sync(0xffffffffu, ic, o), ut = __shfl_up_sync(0xffffffffu, it, o);
    if (lane >= o) { ic += uc; it += ut; }
  }
  if (lane == 31) { wsum[0][wp] = ic; wsum[1][wp] = it; }
  __syncthreads();
  if (wp == 0) {
    int vc = wsum[0][lane], vt = wsum[1][lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int uc = __shfl_up_sync(0xffffffffu, vc, o), ut = __shfl_up_sync(0xffffffffu, vt, o);
      if (lane >= o) { vc += uc; vt += ut; }
    }
    wsum[0][lane] = vc; wsum[1][lane] = vt;
  }
  __syncthreads();
  const int run0 = ic - tot + (wp ? wsum[0][wp - 1] : 0), tile0 = it - nt + (wp ? wsum[1][wp - 1] : 0);
  cur[t] = run0 + above;
  if (cta == 0) {
    const int tper = a.even && nt > 0 ? (tot + nt - 1) / nt : a.bm;
    for (int i = 0; i < nt; ++i) { TileRef tl; tl.expert = t; tl.slot0 = run0 + i * tper; tl.rows = min(tper, tot - i * tper); a.tiles[tile0 + i] = tl; }
    if (t == PLAN_THREADS - 1) { *a.n_tiles = wsum[1][31]; *a.n_slots = wsum[0][31]; }
  }
  __syncthreads();
  for (int p = p0 + t; p < p1; p += PLAN_THREADS) {
    const int e = expert_of(p);
    int pos = -1;
    if (e >= 0) { pos = atomicAdd(&cur[e], 1); if (HB_BOUND(a.err, pos >= 0 && pos < a.P, 0x201u, pos)) a.perm[pos] = p; }
    a.pos_of[p] = pos;
  }
}

// Tensor maps of every resident expert's three matrices: the host encodes one map per matrix shape (on any valid address), this
// kernel copies it and stamps in the address of the matrix inside the expert's record.
struct PfMapSet { CUtensorMap gu, dn, gu_s, dn_s; };    // codes [I × H/2] (w1, w3), [H × I/2] (w2); scales [I × H/16] (s1, s3), [H × I/16] (s2)
__global__ void pf_tmaps_kernel(const __grid_constant__ PfMapSet tpl, const uint8_t* const* __restrict__ tab, int E, hb_rec_layout L,
                                CUtensorMap* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= E * 6) return;
  const int e = i / 6, mat = i - e * 6;                                      // w1, w3, w2, s1, s3, s2
  const uint8_t* rec = tab[e];
  if (!rec) return;
  const CUtensorMap* t = mat < 2 ? &tpl.gu : mat == 2 ? &tpl.dn : mat < 5 ? &tpl.gu_s : &tpl.dn_s;
  const uint64_t offs[6] = {L.w1, L.w3, L.w2, L.s1, L.s3, L.s2};
  const uint4* src = reinterpret_cast<const uint4*>(t);
  uint4* dst = reinterpret_cast<uint4*>(out + i);
#pragma unroll
  for (int j = 0; j < 8; ++j) dst[j] = src[j];
  const uint64_t addr = reinterpret_cast<uint64_t>(rec + offs[mat]);
  asm volatile("tensormap.replace.tile.global_address.global.b1024.b64 [%0], %1;" ::"l"(dst), "l"(addr) : "memory");
  asm volatile("fence.proxy.tensormap::generic.release.gpu;" ::: "memory");
}

// ---- the sum over a row's pairs -----------------------------------------------------------------------------------------------------
// out[row] = Σ_k part[row·K + k]·w[row, k], fp32 in k order, overwritten — or the shared-expert combine on top of it:
// out = bf16(bf16(Σ) + bf16(bf16(sigmoid(bf16 gate logit))·shared)); lg == NULL: no gate.  A CTA takes whole rows: the row's weights
// and which of its pairs contributed (pos_of ≥ 0) are looked up once per row, then every thread streams 8 columns at a time.
constexpr int SUM_ROWS = 4;              // rows a CTA of pf_sum_pairs_kernel works on at once
__global__ void __launch_bounds__(256) pf_sum_pairs_kernel(const __nv_bfloat16* __restrict__ part, const int* __restrict__ pos_of, const float* __restrict__ w, int M,
                                                           int K, int H, float* __restrict__ out, const __nv_bfloat16* __restrict__ shared,
                                                           const float* __restrict__ lg, int ld, int col, __nv_bfloat16* __restrict__ cout) {
  __shared__ float wk[SUM_ROWS][32];
  __shared__ uint32_t live[SUM_ROWS];
  __shared__ float gate_s[SUM_ROWS];
  const int chunks = H / 8;                                                   // 8 columns (16 bytes of bf16) per step of a thread
  for (int m0 = blockIdx.x * SUM_ROWS; m0 < M; m0 += gridDim.x * SUM_ROWS) {
    const int nr = min(SUM_ROWS, M - m0);
    if ((int)threadIdx.x < nr * 32) {
      const int r = threadIdx.x >> 5, k = threadIdx.x & 31;
      const bool on = k < K && pos_of[(size_t)(m0 + r) * K + k] >= 0;
      wk[r][k] = k < K ? w[(size_t)(m0 + r) * K + k] : 0.f;
      const uint32_t mask = __ballot_sync(0xffffffffu, on);
      if (k == 0) {
        live[r] = mask;
        gate_s[r] = cout && lg ? bf16r(1.f / (1.f + expf(-bf16r(lg[(size_t)(m0 + r) * ld + col])))) : 1.f;
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nr * chunks; i += 256) {
      const int r = i / chunks, n = (i - r * chunks) * 8, m = m0 + r;
      const uint32_t lv = live[r];
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k0 = 0; k0 < K; k0 += 4) {                                     // four pairs' pieces are fetched together, then added in k order
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (k0 + j < K && ((lv >> (k0 + j)) & 1u)) v[j] = __ldcs(reinterpret_cast<const uint4*>(part + ((size_t)m * K + k0 + j) * H + n));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (k0 + j >= K || !((lv >> (k0 + j)) & 1u)) continue;
          const uint32_t u[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
          const float wv = wk[r][k0 + j];
#pragma unroll
          for (int c = 0; c < 4; ++c) { acc[2 * c] += __uint_as_float(u[c] << 16) * wv; acc[2 * c + 1] += __uint_as_float(u[c] & 0xffff0000u) * wv; }
        }
      }
      const size_t o = (size_t)m * H + n;
      if (!cout) {
        *reinterpret_cast<float4*>(out + o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(out + o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      } else {
        const float gate = gate_s[r];
        const uint4 sv = *reinterpret_cast<const uint4*>(shared + o);
        const uint32_t su[4] = {sv.x, sv.y, sv.z, sv.w};
        float rr[8];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          rr[2 * c] = bf16r(acc[2 * c]) + bf16r(gate * __uint_as_float(su[c] << 16));
          rr[2 * c + 1] = bf16r(acc[2 * c + 1]) + bf16r(gate * __uint_as_float(su[c] & 0xffff0000u));
        }
        *reinterpret_cast<uint4*>(cout + o) = pf_pack8(rr);
      }
    }
    __syncthreads();
  }
}

}  // namespace hb

using namespace hb;

namespace {
struct PfWs {
  int* hist; int* n_slots; int* n_tiles; TileRef* tiles; int* perm; int* pos_of; CUtensorMap* tmB; __nv_bfloat16* y; __nv_bfloat16* part;
  uint8_t *yq, *ys, *xq_s, *xs_s; float *yg, *xg_s;
};
size_t pf_carve(void* ws, int S, int K, int E, int H, int I, PfWs* w) {
  size_t off = 0;
  auto take = [&](size_t b) { void* r = ws ? static_cast<char*>(ws) + off : nullptr; off += hb_align256(b); return r; };
  const size_t P = (size_t)S * K;
  PfWs t;
  t.hist = (int*)take((size_t)PLAN_MAX_CTAS * E * 4); t.n_slots = (int*)take(4); t.n_tiles = (int*)take(4);
  t.tiles = (TileRef*)take((P / PF_BM + E) * sizeof(TileRef)); t.perm = (int*)take(P * 4); t.pos_of = (int*)take(P * 4);
  t.tmB = (CUtensorMap*)take((size_t)E * 6 * sizeof(CUtensorMap));
  t.y = (__nv_bfloat16*)take(P * I * 2); t.part = (__nv_bfloat16*)take(P * H * 2);
  t.xq_s = (uint8_t*)take(P * H / 2); t.xs_s = (uint8_t*)take(P * H / 16); t.xg_s = (float*)take(P * 4);
  t.yq = (uint8_t*)take(P * I / 2); t.ys = (uint8_t*)take(P * I / 16); t.yg = (float*)take(P * 4);
  if (w) *w = t;
  return off;
}

// map of a byte matrix [n_rows][row_bytes] with boxes of 128 rows: e2m1 codes (two per byte) in boxes 128 bytes wide under the
// 128-byte swizzle, or e4m3 block scales in boxes 16 bytes wide, unswizzled
int pf_make_map(hb_ctx* ctx, CUtensorMap* m, const void* base, size_t row_bytes, size_t n_rows, bool scales = false) {
  TcEncodeFn fn = tc_encode_fn();
  HB_REQUIRE(ctx, fn, HB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n_rows}, strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {scales ? 16u : 128u, 128}, estr[2] = {1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        scales ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HB_REQUIRE(ctx, r == CUDA_SUCCESS, HB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for %zu rows of %zu bytes at %p", (int)r, n_rows, row_bytes, base);
  return HB_OK;
}
template <int MODE>
int pf_launch(hb_ctx* ctx, const char* name, const PfGemmArgs& a, const CUtensorMap& tmA, const CUtensorMap& tmB0, cudaStream_t st) {
  const int grid = ctx->max_ctas > 0 && ctx->max_ctas < ctx->sm_count ? ctx->max_ctas : ctx->sm_count;
  return hb_launch(ctx, name, false, pf_gemm_kernel<MODE>, dim3(grid), dim3(PF_THREADS), (size_t)PF_SMEM, st, a, tmA, tmB0);
}
}  // namespace

namespace {
// map of a bf16 matrix [n_rows][row_len] with boxes of 64 values × 64 rows under the 128-byte swizzle
int a16_make_map(hb_ctx* ctx, CUtensorMap* m, const void* base, size_t row_len, size_t n_rows) {
  TcEncodeFn fn = tc_encode_fn();
  HB_REQUIRE(ctx, fn, HB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)row_len, (cuuint64_t)n_rows}, strides[1] = {(cuuint64_t)row_len * 2};
  const cuuint32_t box[2] = {64u, 64u}, estr[2] = {1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HB_REQUIRE(ctx, r == CUDA_SUCCESS, HB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for %zu rows of %zu bf16 at %p", (int)r, n_rows, row_len, base);
  return HB_OK;
}

// bf16 activations on the tensor cores: plan (tiles of ≤ 256 pairs) → slot-ordered copy of the rows → gate/up GEMM → down GEMM → sums.
// The copy of the rows lives in the buffer of the per-pair down rows: the gate/up GEMM has read it before the down GEMM writes there.
int pf_a16_run(hb_ctx* ctx, const uint8_t* const* lt, int E, const int32_t* ids, const float* w, int M, int K, const __nv_bfloat16* x, int H, int I, float limit,
               float* out, const PfWs& W, int S, cudaStream_t st, const hb_pf_combine* cmb) {
  hb_rec_layout L;
  hb_rec_layout_make(H, I, &L);
  int r = hbk_moe_dtc_maps(ctx, lt, E, nullptr, H, I, st);
  if (r) return r;
  const size_t Pcap = (size_t)S * K;
  CUtensorMap tm_x, tm_y;
  if ((r = a16_make_map(ctx, &tm_x, W.part, (size_t)H, Pcap))) return r;
  if ((r = a16_make_map(ctx, &tm_y, W.y, (size_t)I, Pcap))) return r;
  const int grid = ctx->max_ctas > 0 && ctx->max_ctas < ctx->sm_count ? ctx->max_ctas : ctx->sm_count;
  auto common = [&](int kind, A16Args* a) {
    const void* maps; const unsigned long long* anchor;
    hbk_moe_dtc_map_set(ctx, kind, &maps, &anchor);
    const int Kd = kind ? I : H;
    a->tiles = W.tiles; a->n_tiles = W.n_tiles; a->perm = W.perm; a->tab = lt; a->down = kind; a->K = Kd; a->n_out = kind ? H : I;
    a->maps = reinterpret_cast<const CUtensorMap*>(maps); a->anchor = anchor; a->vmax = hbk_moe_dtc_vmax();
    a->pitch = Kd / 2;
    int g = a->pitch, b = 4096;
    while (b) { const int t2 = g % b; g = b; b = t2; }
    a->gstep = g; a->pshift = -1;
    for (int sft = 7; sft <= 12; ++sft) if (a->pitch == (1 << sft)) a->pshift = sft;
    a->off_g = (uint32_t)L.g; a->limit = limit; a->err = ctx->dev_err;
  };
  for (int s0 = 0; s0 < M; s0 += S) {
    const int n = M - s0 < S ? M - s0 : S, P = n * K;
    PlanArgs pl{ids + (size_t)s0 * K, P, E, lt, A16_BN, 1, W.hist, W.perm, W.pos_of, W.tiles, W.n_tiles, W.n_slots,
                reinterpret_cast<unsigned int*>(ctx->dev_err) + kErrPlanMeet, ctx->dev_err};
    int plan_ctas = (P + 2047) / 2048;
    if (plan_ctas > PLAN_MAX_CTAS) plan_ctas = PLAN_MAX_CTAS;
    if (plan_ctas > ctx->sm_count) plan_ctas = ctx->sm_count;
    if ((r = hb_launch(ctx, "pf_plan", false, pf_plan_kernel, dim3(plan_ctas), dim3(PLAN_THREADS), 0, st, pl))) return r;
    if ((r = hb_launch(ctx, "a16_gather", false, a16_gather_kernel, dim3(P < ctx->sm_count * 16 ? P : ctx->sm_count * 16), dim3(256), 0, st, x + (size_t)s0 * H,
                       (const int*)W.perm, (const int*)W.n_slots, K, H, W.part)))
      return r;
    A16Args a{};
    common(0, &a);
    a.off_w = (uint32_t)L.w1; a.off_s0 = (uint32_t)L.s1; a.off_s1 = (uint32_t)L.s3; a.row2 = (int)((L.w3 - L.w1) / (size_t)(H / 2)); a.out = W.y;
    if ((r = hb_launch(ctx, "a16_gemm_gu", false, a16_gemm_kernel, dim3(grid), dim3(A16_THREADS), (size_t)A16_SMEM, st, a, tm_x))) return r;
    A16Args d{};
    common(1, &d);
    d.off_w = (uint32_t)L.w2; d.off_s0 = (uint32_t)L.s2; d.off_s1 = (uint32_t)L.s2; d.row2 = 64; d.out = W.part;
    if ((r = hb_launch(ctx, "a16_gemm_down", false, a16_gemm_kernel, dim3(grid), dim3(A16_THREADS), (size_t)A16_SMEM, st, d, tm_y))) return r;
    const __nv_bfloat16* sh = cmb ? reinterpret_cast<const __nv_bfloat16*>(cmb->shared) + (size_t)s0 * H : nullptr;
    if ((r = hb_launch(ctx, "pf_sum_pairs", false, pf_sum_pairs_kernel, dim3((unsigned)((n + SUM_ROWS - 1) / SUM_ROWS < ctx->sm_count * 8 ? (n + SUM_ROWS - 1) / SUM_ROWS : ctx->sm_count * 8)), dim3(256), 0, st,
                       (const __nv_bfloat16*)W.part, (const int*)W.pos_of, w + (size_t)s0 * K, n, K, H, cmb ? (float*)nullptr : out + (size_t)s0 * H, sh,
                       cmb && cmb->lg ? cmb->lg + (size_t)s0 * cmb->ld : (const float*)nullptr, cmb ? cmb->ld : 0, cmb ? cmb->col : 0,
                       cmb ? reinterpret_cast<__nv_bfloat16*>(cmb->out) + (size_t)s0 * H : (__nv_bfloat16*)nullptr)))
      return r;
  }
  return HB_OK;
}
}  // namespace

#ifdef HB_A16_TRACE
extern "C" __attribute__((visibility("default"))) int hb_a16_trace_read(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_a16_trace, (size_t)n * 8);
}
#endif

int hbk_moe_prefill_setup(hb_ctx* ctx) {
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(pf_gemm_kernel<PF_PLAIN>), cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(pf_gemm_kernel<PF_GU>), cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(pf_gemm_kernel<PF_DOWN>), cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(pf_peak_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, PF_STAGE + 2048));
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(a16_gemm_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, A16_SMEM));
  return HB_OK;
}

extern "C" {

int hb_moe_prefill_supported(int H, int I) { return H > 0 && I > 0 && H % 256 == 0 && I % 256 == 0; }

size_t hb_moe_prefill_ws_bytes(int S, int K, int E, int H, int I) {
  if (S < 1 || K < 1 || E < 1 || !hb_moe_prefill_supported(H, I)) return 0;
  return pf_carve(nullptr, S, K, E, H, I, nullptr);
}

int hb_moe_prefill(hb_ctx* ctx, const uint8_t* const* rec_tab, int li, int E, const int32_t* ids, const float* w, int M, int K, const void* x_bf16,
                   int H, int I, float limit, float* out, void* ws, int S, void* stream, const hb_pf_combine* cmb) {
  if (!ctx) return HB_ERR_INVALID;
  if (M <= 0) return HB_OK;
  HB_REQUIRE(ctx, rec_tab && ids && w && x_bf16 && (out || cmb), HB_ERR_INVALID, "moe_prefill: NULL argument");
  HB_REQUIRE(ctx, !cmb || (cmb->shared && cmb->out), HB_ERR_INVALID, "moe_prefill: combine without shared rows or output");
  HB_REQUIRE(ctx, hb_moe_prefill_supported(H, I) && S >= 1 && K >= 1 && K <= 32 && E >= 1 && E <= 1024 && li >= 0, HB_ERR_UNSUPPORTED,
             "moe_prefill: H=%d I=%d (multiples of 256) E=%d (≤ 1024) K=%d (≤ 32) S=%d", H, I, E, K, S);
  HB_REQUIRE(ctx, (long long)S * K < (1ll << 30), HB_ERR_UNSUPPORTED, "moe_prefill: S·K too large");
  HB_REQUIRE(ctx, ws && hb_aligned(ws, 256), HB_ERR_WORKSPACE, "moe_prefill: ws NULL or not 256-byte aligned");
  HB_REQUIRE(ctx, hb_aligned(x_bf16, 16) && hb_aligned(out, 16) && (!cmb || (hb_aligned(cmb->shared, 16) && hb_aligned(cmb->out, 16))), HB_ERR_INVALID,
             "moe_prefill: x, out, shared rows and combined output must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if ((ctx->flags & HB_FLAG_PREFILL_A16) && M > 64 && !(ctx->flags & HB_FLAG_PREFILL_A16_ROWS) && hbk_moe_dtc_supported(H, I)) {
    // bf16 activations, more rows than a decode batch: the kind::f16 grouped GEMM over dequantised weight tiles
    PfWs W;
    pf_carve(ws, S, K, E, H, I, &W);
    return pf_a16_run(ctx, rec_tab + (size_t)li * E, E, ids, w, M, K, reinterpret_cast<const __nv_bfloat16*>(x_bf16), H, I, limit, out, W, S, st, cmb);
  }
  if (ctx->flags & HB_FLAG_PREFILL_A16) {
    // bf16 activations, few rows (or HB_FLAG_PREFILL_A16_ROWS): the decode operators over sub-chunks of rows (their scratch fits inside
    // this operator's workspace)
    int rows = HB_MAX_PAIRS / K < S ? HB_MAX_PAIRS / K : S;
    HB_REQUIRE(ctx, rows >= 1 && hb_moe_decode_supported(H, I) > 0, HB_ERR_UNSUPPORTED, "moe_prefill (bf16 activations): K=%d H=%d I=%d", K, H, I);
    while (rows > 1 && hbk_moe_decode_ws_bytes(rows * K, H, I) > hb_moe_prefill_ws_bytes(S, K, E, H, I)) rows /= 2;
    for (int m0 = 0; m0 < M; m0 += rows) {
      const int n = M - m0 < rows ? M - m0 : rows;
      hbk_pair_src src; src.ids = ids + (size_t)m0 * K; src.w = w + (size_t)m0 * K; src.M = n; src.K = K; src.tab = rec_tab; src.li = li; src.E = E;
      src.pairs_hint = M * K;                                               // every sub-chunk runs on the engine the whole call would get
      hbk_reduce red;
      if (cmb) {
        red.shared = reinterpret_cast<const __nv_bfloat16*>(cmb->shared) + (size_t)m0 * H; red.lg = cmb->lg ? cmb->lg + (size_t)m0 * cmb->ld : nullptr;
        red.ld = cmb->ld; red.col = cmb->col; red.out_bf16 = reinterpret_cast<__nv_bfloat16*>(cmb->out) + (size_t)m0 * H;
      } else red.out_f32 = out + (size_t)m0 * H;
      const int r2 = hbk_moe_decode_run(ctx, src, reinterpret_cast<const __nv_bfloat16*>(x_bf16) + (size_t)m0 * H, H, I, limit, red, ws, st);
      if (r2) return r2;
    }
    return HB_OK;
  }
  PfWs W;
  pf_carve(ws, S, K, E, H, I, &W);
  hb_rec_layout L;
  hb_rec_layout_make(H, I, &L);
  const uint8_t* const* lt = rec_tab + (size_t)li * E;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(x_bf16);
  int r;
  const size_t Pcap = (size_t)S * K;
  CUtensorMap tm_x, tm_y;
  PfMapSet tpl;
  if ((r = pf_make_map(ctx, &tm_x, W.xq_s, (size_t)H / 2, Pcap))) return r;
  if ((r = pf_make_map(ctx, &tm_y, W.yq, (size_t)I / 2, Pcap))) return r;
  if ((r = pf_make_map(ctx, &tpl.gu, W.xq_s, (size_t)H / 2, (size_t)I))) return r;          // addresses are stamped per expert on the device
  if ((r = pf_make_map(ctx, &tpl.dn, W.xq_s, (size_t)I / 2, (size_t)H))) return r;
  if ((r = pf_make_map(ctx, &tpl.gu_s, W.xq_s, (size_t)H / 16, (size_t)I, true))) return r;
  if ((r = pf_make_map(ctx, &tpl.dn_s, W.xq_s, (size_t)I / 16, (size_t)H, true))) return r;
  if ((r = hb_launch(ctx, "pf_tmaps", false, pf_tmaps_kernel, dim3((E * 6 + 127) / 128), dim3(128), 0, st, tpl, lt, E, L, W.tmB))) return r;
  for (int s0 = 0; s0 < M; s0 += S) {
    const int n = M - s0 < S ? M - s0 : S, P = n * K;
    const int32_t* sid = ids + (size_t)s0 * K;
    PlanArgs pl{sid, P, E, lt, PF_BM, 0, W.hist, W.perm, W.pos_of, W.tiles, W.n_tiles, W.n_slots, reinterpret_cast<unsigned int*>(ctx->dev_err) + kErrPlanMeet, ctx->dev_err};
    int plan_ctas = (P + 2047) / 2048;
    if (plan_ctas > PLAN_MAX_CTAS) plan_ctas = PLAN_MAX_CTAS;
    if (plan_ctas > ctx->sm_count) plan_ctas = ctx->sm_count;                   // the CTAs meet inside the kernel: all must be resident
    if ((r = hb_launch(ctx, "pf_plan", false, pf_plan_kernel, dim3(plan_ctas), dim3(PLAN_THREADS), 0, st, pl))) return r;
    // x quantised once per row and written straight into its pairs' slots
    if ((r = hbk_quant_rows_scatter(ctx, x + (size_t)s0 * H, H, n, H, W.pos_of, K, W.xq_s, W.xs_s, W.xg_s, st))) return r;
    PfGemmArgs a{};
    a.tiles = W.tiles; a.n_tiles = W.n_tiles; a.perm = W.perm; a.tab = lt; a.L = L; a.tmB = W.tmB; a.limit = limit; a.err = ctx->dev_err;
    a.as = W.xs_s; a.ag = W.xg_s; a.Kd = H; a.N = I; a.out = W.y; a.ldo = I;
    if ((r = pf_launch<PF_GU>(ctx, "pf_gemm_gu", a, tm_x, tm_x, st))) return r;
    if ((r = hbk_quant_rows_scatter(ctx, W.y, I, P, I, nullptr, 1, W.yq, W.ys, W.yg, st, W.n_slots))) return r;   // only the slots that hold a pair
    a.as = W.ys; a.ag = W.yg; a.Kd = I; a.N = H; a.out = W.part; a.ldo = H;
    if ((r = pf_launch<PF_DOWN>(ctx, "pf_gemm_down", a, tm_y, tm_y, st))) return r;
    const __nv_bfloat16* sh = cmb ? reinterpret_cast<const __nv_bfloat16*>(cmb->shared) + (size_t)s0 * H : nullptr;
    if ((r = hb_launch(ctx, "pf_sum_pairs", false, pf_sum_pairs_kernel, dim3((unsigned)((n + SUM_ROWS - 1) / SUM_ROWS < ctx->sm_count * 8 ? (n + SUM_ROWS - 1) / SUM_ROWS : ctx->sm_count * 8)), dim3(256), 0, st,
                       (const __nv_bfloat16*)W.part, (const int*)W.pos_of, w + (size_t)s0 * K, n, K, H, cmb ? (float*)nullptr : out + (size_t)s0 * H, sh,
                       cmb && cmb->lg ? cmb->lg + (size_t)s0 * cmb->ld : (const float*)nullptr, cmb ? cmb->ld : 0, cmb ? cmb->col : 0,
                       cmb ? reinterpret_cast<__nv_bfloat16*>(cmb->out) + (size_t)s0 * H : (__nv_bfloat16*)nullptr)))
      return r;
  }
  return HB_OK;
}

int hb_nvfp4_gemm_a4(hb_ctx* ctx, const hb_qmat* W, const uint8_t* xq, const uint8_t* xs, const float* xg, int M, float* y, int ldy, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  HB_REQUIRE(ctx, W && W->w && W->s && xq && xs && xg && y, HB_ERR_INVALID, "nvfp4_gemm_a4: NULL argument");
  HB_REQUIRE(ctx, W->fmt == HB_FMT_NVFP4 && W->N > 0 && W->N % 256 == 0 && W->K > 0 && W->K % 256 == 0 && M >= 1 && ldy >= W->N && ldy % 4 == 0,
             HB_ERR_UNSUPPORTED, "nvfp4_gemm_a4: NVFP4 matrix with N and K multiples of 256 wanted (fmt %d N=%d K=%d M=%d ldy=%d)", W->fmt, W->N, W->K, M, ldy);
  HB_REQUIRE(ctx, hb_aligned(W->w, 16) && hb_aligned(W->s, 16) && hb_aligned(xq, 16) && hb_aligned(xs, 16) && hb_aligned(y, 16), HB_ERR_INVALID,
             "nvfp4_gemm_a4: operands must be 16-byte aligned");
  PfGemmArgs a{};
  a.M = M; a.as = xs; a.ag = xg; a.Kd = W->K; a.bs = reinterpret_cast<const uint8_t*>(W->s); a.bg = W->g; a.N = W->N;
  a.out = y; a.ldo = ldy; a.err = ctx->dev_err;
  CUtensorMap tm_a, tm_b;
  int r;
  if ((r = pf_make_map(ctx, &tm_a, xq, (size_t)W->K / 2, (size_t)M))) return r;
  if ((r = pf_make_map(ctx, &tm_b, W->w, (size_t)W->K / 2, (size_t)W->N))) return r;
  return pf_launch<PF_PLAIN>(ctx, "pf_gemm_plain", a, tm_a, tm_b, reinterpret_cast<cudaStream_t>(stream));
}

int hb_fp4_peak_probe(hb_ctx* ctx, int rounds, float* tflops) {
  if (!ctx) return HB_ERR_INVALID;
  HB_REQUIRE(ctx, rounds >= 1 && rounds <= (1 << 20) && tflops, HB_ERR_INVALID, "fp4_peak_probe: rounds 1..2^20");
  cudaEvent_t e0, e1;
  HB_CUDA(ctx, cudaEventCreate(&e0)); HB_CUDA(ctx, cudaEventCreate(&e1));
  int r = hb_launch(ctx, "pf_peak", false, pf_peak_kernel, dim3(ctx->sm_count), dim3(128), (size_t)PF_STAGE + 2048, (cudaStream_t)0, 64, ctx->dev_err);   // warm-up
  cudaEventRecord(e0, 0);
  if (!r) r = hb_launch(ctx, "pf_peak", false, pf_peak_kernel, dim3(ctx->sm_count), dim3(128), (size_t)PF_STAGE + 2048, (cudaStream_t)0, rounds, ctx->dev_err);
  cudaEventRecord(e1, 0);
  const cudaError_t e = cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  if (r) return r;
  if (e != cudaSuccess) return hb_fail(ctx, HB_ERR_CUDA, "fp4_peak_probe: %s", cudaGetErrorString(e));
  *tflops = (float)(2.0 * PF_BM * PF_BN * 64.0 * 4.0 * rounds * ctx->sm_count / (ms * 1e-3) / 1e12);
  return HB_OK;
}

}  // extern "C"
