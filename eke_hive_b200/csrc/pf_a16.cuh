// Grouped GEMM of the prefill operator with bf16 activations (W4A16, the reference's default prefill arithmetic,
// engine/src/qwen/fn_moe_pf.cu:118-437) on the 5th-generation tensor cores: tcgen05.mma kind::f16, bf16 × bf16 → fp32 in tensor memory.
//
// The NVFP4 weights are the A operand (M = 128 rows of the record's matrix), the activation rows of one expert's pairs the B operand
// (N ≤ 256 pairs, N a multiple of 16 chosen per tile), so one dequantised weight value serves up to 256 multiply-adds and the
// accumulator's lanes are weight rows — the epilogue thread of a lane owns one output row of the expert, as in the decode kernels.
// Dequantisation: e2m1 → bf16 by byte permutes, × the e4m3 block scale as bf16 — the product has ≤ 6 significant bits, exact in bf16 —
// written into the K-major 128-byte-swizzle operand tile by sixteen warps; every product of the MMA is therefore the exact product of
// the decode operators, sums are fp32.  Rounding points after the sums are the reference's (g, u → bf16 after the
// global scale, y → bf16, down → bf16 before the routing weight).
//
// A work item is 256 weight rows (two A tiles of 128) × one tile of pairs; the two accumulators fill the CTA's tensor memory, so
// the MMAs of the next item wait for the epilogue.  Per 64 k values an item moves 32 KB of activations and 8 KB of codes from L2 into
// shared memory (with one A tile per item the activation stream alone ran into what the SMs can pull out of L2).
//
// Per CTA (persistent, one per SM, 26 warps): warp 9 (one thread) streams by TMA the raw code boxes of the weights (128 bytes × 64
// rows, 256 k values per row, through the anchored tensor map of the decode path) and the activation boxes (64 values × 64 rows of
// bf16) of the tile; warps 10-25 (eight per A tile) turn a raw box into four operand tiles, fetching their row's block scales from
// global memory a raw box ahead; warp 8 (one thread) issues the MMAs (128 × N × 16, four per A tile and step); warps 0-3 and 4-7 run
// the epilogues of the two accumulators.  Gate/up: an A tile holds 64 gate and 64 up rows arranged so that lanes l and l + 16 of a
// warp hold the gate and the up value of the same row of I — SwiGLU needs one exchange.  Every wait is bounded; a barrier gets one
// arrival per warp, not per thread (arrivals on one barrier are taken one after the other).
#pragma once
#include "tc_common.cuh"

namespace hb {

constexpr int A16_BN = 256;                     // pairs of a tile (MMA N), at most
constexpr int A16_STA = 2, A16_STB = 3;         // operand rings: dequantised weight tiles, activation tiles
constexpr int A16_A1 = 128 * 128;               // one A tile: 128 rows × 64 bf16
constexpr int A16_A = 2 * A16_A1;               // both A tiles of a step
constexpr int A16_B = A16_BN * 128;             // 256 rows × 64 bf16
constexpr int A16_RAW = 2 * 128 * 128;          // raw codes of both A tiles: 128 rows × 128 bytes each (256 k values per row)
constexpr int A16_SMEM = 1024 + A16_STA * A16_A + A16_STB * A16_B + 2 * A16_RAW + 1024;
constexpr int A16_THREADS = 26 * 32;            // warps 0-3 and 4-7 epilogues of the two A tiles, 8 MMA issue, 9 TMA, 10-17 and 18-25 dequantisation
constexpr int A16_W_MMA = 8, A16_W_TMA = 9, A16_W_DQ0 = 10, A16_DQ_THREADS = 512;
constexpr int A16_TMEM_COLS = 512;              // the accumulators of the two A tiles, 256 columns each
static_assert(A16_SMEM <= 227 * 1024, "shared memory");

struct A16Args {
  const TileRef* tiles; const int* n_tiles;     // tiles of ≤ A16_BN consecutive slots of one expert's run of the sorted pairs
  const int* perm;                              // pair of a slot (the down pass writes its rows by pair)
  const uint8_t* const* tab;                    // expert records of the layer
  int down;                                     // 0: gate/up (out = y bf16 [slot, I]); 1: down (out = bf16 [pair, H])
  int K, n_out;                                 // inner dimension (H | I), output rows per expert (I | H)
  uint32_t off_w, off_s0, off_s1, off_g;        // record offsets: first matrix, scales of the matrix of lanes 0-15 / 16-31 of a warp (gate / up; down:
                                                // the same matrix twice), global scales
  int row2;                                     // matrix rows between the two 64-row boxes of an A tile
  const CUtensorMap* maps; const unsigned long long* anchor; int vmax;   // anchored weight map (variants) of this pass
  int pitch, gstep, pshift;
  float limit;
  __nv_bfloat16* out;
  uint32_t* err;
};

__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// two f16 values (exactly representable in bf16) → bf16x2, element order kept
__device__ __forceinline__ uint32_t f16x2_to_bf16x2(uint32_t h2) {
  const __half2 h = *reinterpret_cast<const __half2*>(&h2);
  const float2 f = __half22float2(h);
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t*>(&b);
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t bmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Eight e2m1 codes (one word, element 0 in the low nibble) → eight bf16 values times the block scale `sv` (bf16x2, both halves the same), as
// four bf16x2 words in element order — on the integer pipe: the conversion unit is too slow for one conversion per element.  The bf16
// pattern of a magnitude code m is looked up bytewise with byte permutes (high bytes 00 3F 3F 3F 40 40 40 40, low bytes 00 00 80 C0 00 40
// 80 C0 for 0, .5, 1, 1.5, 2, 3, 4, 6), the sign bits come from a permute in sign-replication mode; the product of such a value and an
// e4m3 scale has at most 6 significant bits: exact in bf16.
__device__ __forceinline__ uint4 a16_dequant8(uint32_t w, uint32_t sv) {
  const uint32_t wa = w << 4;
  uint32_t o[4];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint32_t sel = (half ? (w >> 16) : w) & 0x7777u;
    const uint32_t hi = prmt(0x3F3F3F00u, 0x40404040u, sel), lo = prmt(0xC0800000u, 0xC0804000u, sel);
    const uint32_t sg = prmt(wa, w, half ? 0xFBEAu : 0xD9C8u);            // byte i = 0xFF where element i is negative
    const uint32_t hs = hi | (sg & 0x80808080u);
    o[2 * half] = bmul2_u32(prmt(lo, hs, 0x5140u), sv);
    o[2 * half + 1] = bmul2_u32(prmt(lo, hs, 0x7362u), sv);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// The slot-ordered copy of the activation rows: row `slot` = x[perm[slot] / K].  One CTA per slot at a time.
__global__ void __launch_bounds__(256) a16_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ perm, const int* __restrict__ n_slots, int K,
                                                         int H, __nv_bfloat16* __restrict__ out) {
  const int n = *n_slots;
  for (int s = blockIdx.x; s < n; s += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(perm[s] / K) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)s * H);
    for (int i = threadIdx.x; i < H / 8; i += 256) dst[i] = __ldg(src + i);
  }
}

// Optional in-kernel timing (compile with -DHB_A16_TRACE): the roles of every CTA sum the clocks they spend in each kind of wait.
#ifdef HB_A16_TRACE
__device__ long long g_a16_trace[2 * 256 * 16];   // gate/up launch, down launch
#define A16_TIMED(acc, stmt) do { const long long t_ = clock64(); stmt; acc += clock64() - t_; } while (0)
#define A16_PUT(slot, v) g_a16_trace[(a.down * 256 + blockIdx.x) * 16 + (slot)] = (v)
#else
#define A16_TIMED(acc, stmt) do { stmt; } while (0)
#define A16_PUT(slot, v) do { } while (0)
#endif

__global__ void __launch_bounds__(A16_THREADS, 1) a16_gemm_kernel(const A16Args a, const __grid_constant__ CUtensorMap tmB) {
  extern __shared__ uint8_t a16_raw[];
  const uint32_t raw0 = smem_u32(a16_raw), base = (raw0 + 1023u) & ~1023u;
  uint8_t* sm = a16_raw + (base - raw0);
  uint8_t* smA = sm;                                   // [STA][2 A tiles][16 KB]
  uint8_t* smB = smA + A16_STA * A16_A;                // [STB][32 KB]
  uint8_t* smR = smB + A16_STB * A16_B;                // [2][2 A tiles][16 KB] raw codes
  uint64_t* fullA = reinterpret_cast<uint64_t*>(smR + 2 * A16_RAW);
  uint64_t* emptyA = fullA + A16_STA;
  uint64_t* fullB = emptyA + A16_STA;
  uint64_t* emptyB = fullB + A16_STB;
  uint64_t* fullR = emptyB + A16_STB;
  uint64_t* emptyR = fullR + 2;
  uint64_t* acc_full = emptyR + 2;
  uint64_t* acc_empty = acc_full + 1;
  uint64_t* mma_done = acc_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < A16_STA; ++s) { mbar_init(&fullA[s], A16_DQ_THREADS / 32); mbar_init(&emptyA[s], 1); }   // one arrival per dequantisation warp
    for (int s = 0; s < A16_STB; ++s) { mbar_init(&fullB[s], 1); mbar_init(&emptyB[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&fullR[s], 1); mbar_init(&emptyR[s], A16_DQ_THREADS / 32); }
    mbar_init(acc_full, 1); mbar_init(acc_empty, 8);
    mbar_init(mma_done, 1);
    mbar_fence_init();
  }
  if (warp == A16_W_MMA) { tmem_alloc(tmem_slot, A16_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int arows = a.down ? 128 : 64;                        // matrix rows an A tile advances (gate/up: 64 of each matrix)
  const int nT = a.n_out / (2 * arows);                       // items per tile: two A tiles each
  const int n_items_all = *a.n_tiles * nT;
  const int nk = a.K >> 6;                                    // steps per item (a multiple of 4)

  if (warp == A16_W_TMA) {
    // ------------------------------------------------------------------------------------------------ loads: one thread
    if (lane == 0) {
      uint32_t rit = 0, kit = 0, seen = 0u;
      bool ok = true;
      [[maybe_unused]] long long tw = 0, t0 = clock64();
      const unsigned long long anchor = *a.anchor;
      for (int item = blockIdx.x; item < n_items_all && ok; item += gridDim.x) {
        const int ti = item / nT, t = item - ti * nT;
        const TileRef tl = a.tiles[ti];
        const uint8_t* rec = a.tab[tl.expert];
        const unsigned long long addr = reinterpret_cast<unsigned long long>(rec) + a.off_w, delta = addr - anchor;
        unsigned long long row;
        int v = 0;
        if (!rec || addr < anchor) { atomicOr(a.err, 0x400000u); break; }
        if (a.pshift >= 0) row = delta >> a.pshift;
        else {
          const unsigned long long rem = delta % (unsigned long long)a.pitch;
          row = (delta - rem) / (unsigned long long)a.pitch;
          v = (int)(rem / (unsigned long long)a.gstep);
          if (rem % (unsigned long long)a.gstep || v >= a.vmax) { atomicOr(a.err, 0x400000u); break; }
        }
        if (row + (1ull << 24) >= (1ull << 31)) { atomicOr(a.err, 0x400000u); break; }
        const CUtensorMap* map = a.maps + v;
        if (!((seen >> v) & 1u)) { tmap_acquire(map); seen |= 1u << v; }
        const int r0 = (int)row + 2 * t * arows;
        const int nbox = (tl.rows + 63) >> 6;
        for (int rs = 0; rs < nk / 4 && ok; ++rs, ++rit) {
          const uint32_t sl = rit & 1u;
          A16_TIMED(tw, ok = mbar_wait(&emptyR[sl], ((rit >> 1) & 1u) ^ 1u, a.err, 0x1u));
          if (!ok) break;
          const uint32_t rb = smem_u32(smR + sl * A16_RAW);
          mbar_expect_tx(&fullR[sl], A16_RAW);
#pragma unroll
          for (int uu = 0; uu < 2; ++uu) {
            tma_load_2d(rb + uu * A16_A1, map, rs * 128, r0 + uu * arows, &fullR[sl]);
            tma_load_2d(rb + uu * A16_A1 + A16_A1 / 2, map, rs * 128, r0 + uu * arows + a.row2, &fullR[sl]);
          }
          for (int kq = 0; kq < 4; ++kq, ++kit) {
            const uint32_t sb = kit % A16_STB;
            A16_TIMED(tw, ok = mbar_wait(&emptyB[sb], ((kit / A16_STB) & 1u) ^ 1u, a.err, 0x2u));
            if (!ok) break;
            const uint32_t bb = smem_u32(smB + sb * A16_B);
            mbar_expect_tx(&fullB[sb], (uint32_t)nbox * 8192u);
            for (int i = 0; i < nbox; ++i) tma_load_2d(bb + i * 8192, &tmB, (rs * 4 + kq) * 64, tl.slot0 + i * 64, &fullB[sb]);
          }
        }
      }
      A16_PUT(0, tw); A16_PUT(1, clock64() - t0);
    }
  } else if (warp >= A16_W_DQ0) {
    // ------------------------------------------------------------------------------------------------ dequantisation: thread (u, r, h) owns half a row
    // of A tile u in every step: A row r, k values [32 h, 32 h + 32) of the step's 64
    const int dt = threadIdx.x - A16_W_DQ0 * 32, u = dt >> 8, r = (dt & 255) >> 1, h = dt & 1;
    int rr, srow; uint32_t soff;                               // raw row, row of the scale matrix inside the A tile, which scale matrix
    if (a.down) { rr = r; srow = r; soff = a.off_s0; }
    else {
      const int q = r >> 5, j = r & 31;
      rr = j < 16 ? 16 * q + j : 64 + 16 * q + (j - 16);
      srow = 16 * q + (j & 15);
      soff = j < 16 ? a.off_s0 : a.off_s1;
    }
    const int sbytes = a.K >> 4;                               // scale bytes per matrix row
    uint32_t rit = 0, kit = 0;
    bool ok = true;
    [[maybe_unused]] long long tw = 0, tc = 0, t0 = clock64(), tl0 = 0;
    for (int item = blockIdx.x; item < n_items_all && ok; item += gridDim.x) {
      const int ti = item / nT, t = item - ti * nT;
      const uint8_t* rec = a.tab[a.tiles[ti].expert];
      if (!rec) break;
      const uint8_t* srowp = rec + soff + (size_t)((2 * t + u) * arows + srow) * sbytes;
      uint4 sc = __ldg(reinterpret_cast<const uint4*>(srowp));
      for (int rs = 0; rs < nk / 4 && ok; ++rs, ++rit) {
        uint4 sc_next = sc;
        if (rs + 1 < nk / 4) sc_next = __ldg(reinterpret_cast<const uint4*>(srowp + (size_t)(rs + 1) * 16));
        const uint32_t sl = rit & 1u;
        if (lane == 0) A16_TIMED(tw, ok = mbar_wait(&fullR[sl], (rit >> 1) & 1u, a.err, 0x4u));
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const uint8_t* rawrow = smR + sl * A16_RAW + u * A16_A1 + rr * 128;
        const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
        for (int kq = 0; kq < 4; ++kq, ++kit) {
#ifdef HB_A16_TRACE
          tl0 = clock64();
#endif
          const uint4 cw = *reinterpret_cast<const uint4*>(rawrow + (((kq * 2 + h) ^ (rr & 7)) << 4));     // 32 codes
          const uint32_t s2 = (scw[kq] >> (16 * h)) & 0xffffu;                                              // the two block scales
          const uint32_t sh = f16x2_to_bf16x2(cvt_e4m3x2_f16x2(s2));
          const uint32_t slo = __byte_perm(sh, sh, 0x1010), shi = __byte_perm(sh, sh, 0x3232);             // (s0, s0), (s1, s1) as bf16
          const uint4 o0 = a16_dequant8(cw.x, slo), o1 = a16_dequant8(cw.y, slo), o2 = a16_dequant8(cw.z, shi), o3 = a16_dequant8(cw.w, shi);
#ifdef HB_A16_TRACE
          if (o0.x == 0x12345u && o3.w == 0x54321u) tc += 1;            // keeps the values' computation in front of the clock read
          tc += clock64() - tl0;
#endif
          // one lane waits for the slot and one lane announces the warp's rows
          const uint32_t sa = kit % A16_STA;
          if (lane == 0) A16_TIMED(tw, ok = mbar_wait(&emptyA[sa], ((kit / A16_STA) & 1u) ^ 1u, a.err, 0x8u));
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          uint8_t* arow = smA + sa * A16_A + u * A16_A1 + r * 128;
          *reinterpret_cast<uint4*>(arow + (((h * 4 + 0) ^ (r & 7)) << 4)) = o0;
          *reinterpret_cast<uint4*>(arow + (((h * 4 + 1) ^ (r & 7)) << 4)) = o1;
          *reinterpret_cast<uint4*>(arow + (((h * 4 + 2) ^ (r & 7)) << 4)) = o2;
          *reinterpret_cast<uint4*>(arow + (((h * 4 + 3) ^ (r & 7)) << 4)) = o3;
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&fullA[sa]);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&emptyR[sl]);
        sc = sc_next;
      }
    }
    if (dt == 0) { A16_PUT(2, tw); A16_PUT(3, clock64() - t0); A16_PUT(4, tc); }
  } else if (warp == A16_W_MMA) {
    // ------------------------------------------------------------------------------------------------ MMA issue: one thread
    if (lane == 0) {
      uint32_t kit = 0, n_it = 0;
      bool ok = true;
      [[maybe_unused]] long long twa = 0, twb = 0, twe = 0, t0 = clock64();
      for (int item = blockIdx.x; item < n_items_all && ok; item += gridDim.x, ++n_it) {
        const int rows = a.tiles[item / nT].rows;
        const uint32_t N = (uint32_t)((rows + 15) & ~15);
        // kind::f16: D fp32 (bit 4), A and B bf16 (format 1 at bits 7 and 10), both K-major, N / 8 at bit 17, M / 16 at bit 24
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((128u >> 4) << 24);
        if (n_it >= 1) A16_TIMED(twe, ok = mbar_wait(acc_empty, (n_it - 1u) & 1u, a.err, 0x10u));   // the epilogue has read the previous item's sums
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < nk; ++kb, ++kit) {
          const uint32_t sa = kit % A16_STA, sb = kit % A16_STB;
          A16_TIMED(twb, ok = mbar_wait(&fullB[sb], (kit / A16_STB) & 1u, a.err, 0x40u));
          if (!ok) break;
          A16_TIMED(twa, ok = mbar_wait(&fullA[sa], (kit / A16_STA) & 1u, a.err, 0x20u));
          if (!ok) break;
          tc_fence_after();
          const uint64_t ad = tc_desc_sw128(base + sa * A16_A), bd = tc_desc_sw128(base + A16_STA * A16_A + sb * A16_B);
#pragma unroll
          for (uint32_t uu = 0; uu < 2; ++uu) {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j)
              tc_mma_f16(tmem + uu * 256, ad + uu * (A16_A1 >> 4) + 2 * j, bd + 2 * j, idesc, (kb | (int)j) != 0 ? 1u : 0u);
          }
          tc_commit(&emptyA[sa]);
          tc_commit(&emptyB[sb]);
        }
        if (ok) tc_commit(acc_full);
      }
      tc_commit(mma_done);
      mbar_wait(mma_done, 0, a.err, 0x80u);
      A16_PUT(5, twa); A16_PUT(6, twb); A16_PUT(7, twe); A16_PUT(8, clock64() - t0); A16_PUT(9, (long long)kit);
    }
  } else {
    // ------------------------------------------------------------------------------------------------ epilogues: warp 4 u + q reads lanes [32 q, 32 q + 32) of accumulator u
    const int u = warp >> 2, q = warp & 3, tl_ = threadIdx.x & 127;   // tl_ = row of the A tile
    bool ok = true;
    uint32_t n_it = 0;
    [[maybe_unused]] long long tw = 0, t0 = clock64(), tld = 0;
    for (int item = blockIdx.x; item < n_items_all && ok; item += gridDim.x, ++n_it) {
      const int ti = item / nT, t = item - ti * nT;
      const TileRef tl = a.tiles[ti];
      const uint8_t* rec = a.tab[tl.expert];
      if (!rec) break;
      const float gsc = __ldg(reinterpret_cast<const float*>(rec + a.off_g) + (a.down ? 2 : lane < 16 ? 0 : 1));
      // down: the pairs (output rows) of the tile's columns, lane l those of columns 32 i + l — fetched while the MMAs run and handed
      // round by shuffles below
      int my_pair[A16_BN / 32];
#pragma unroll
      for (int i = 0; i < A16_BN / 32; ++i) my_pair[i] = a.down && 32 * i + lane < tl.rows ? __ldg(a.perm + tl.slot0 + 32 * i + lane) : 0;
      A16_TIMED(tw, ok = mbar_wait(acc_full, n_it & 1u, a.err, 0x100u));
      if (!ok) break;
      tc_fence_after();
      const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16) + u * 256;
#pragma unroll
      for (int ci = 0; ci < A16_BN / 32; ++ci) {
        const int c0 = 32 * ci;
        if (c0 >= tl.rows) break;
        uint32_t rg[32];
        A16_TIMED(tld, tc_ld32(trow + c0, rg); tc_wait_ld());
        if (a.down) {
          unsigned short* orow = reinterpret_cast<unsigned short*>(a.out) + (size_t)(2 * t + u) * 128 + tl_;
#pragma unroll
          for (int c = 0; c < 32; c += 2) {                     // two columns per conversion
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(rg[c]) * gsc, __uint_as_float(rg[c + 1]) * gsc);
            const uint32_t bw = *reinterpret_cast<const uint32_t*>(&b2);
            const int p0 = __shfl_sync(0xffffffffu, my_pair[ci], c), p1 = __shfl_sync(0xffffffffu, my_pair[ci], c + 1);
            if (c0 + c < tl.rows) orow[(size_t)p0 * a.n_out] = (unsigned short)(bw & 0xffffu);
            if (c0 + c + 1 < tl.rows) orow[(size_t)p1 * a.n_out] = (unsigned short)(bw >> 16);
          }
        } else {
          // lanes 0-15 hold the gate values of 16 rows of I, lanes 16-31 the up values of the same rows.  Of a pair of columns the low
          // half-warp finishes the even one and the high half-warp the odd one: one exchange per pair, every lane computes
          const bool hi = lane >= 16;
          __nv_bfloat16* orow = a.out + (size_t)(tl.slot0 + c0 + (hi ? 1 : 0)) * a.n_out + (2 * t + u) * 64 + 16 * q + (lane & 15);
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float v0 = bf16r(__uint_as_float(rg[c]) * gsc), v1 = bf16r(__uint_as_float(rg[c + 1]) * gsc);
            const float got = __shfl_xor_sync(0xffffffffu, hi ? v0 : v1, 16);      // low lanes get u of the even column, high lanes g of the odd one
            float gv = hi ? got : v0, uv = hi ? v1 : got;
            if (a.limit > 0.f) { uv = fminf(fmaxf(uv, -a.limit), a.limit); gv = fminf(gv, a.limit); }
            // silu by the fast reciprocal (the decode kernels divide exactly; the difference is below the bf16 rounding that follows in
            // all but a few cases in a thousand — the accumulators are not double-buffered, and the exact division's instructions
            // were the longest part of the time the MMAs wait for this epilogue)
            if (c0 + c + (hi ? 1 : 0) < tl.rows) orow[(size_t)c * a.n_out] = __float2bfloat16(__fdividef(gv, 1.f + __expf(-gv)) * uv);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
    }
    if (threadIdx.x == 0) { A16_PUT(10, tw); A16_PUT(11, clock64() - t0); A16_PUT(12, tld); A16_PUT(13, (long long)n_it); }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == A16_W_MMA) { tc_fence_after(); tmem_dealloc(tmem, A16_TMEM_COLS); }
}

}  // namespace hb
