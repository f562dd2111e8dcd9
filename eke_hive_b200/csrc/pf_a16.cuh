// Grouped GEMM of the prefill operator with bf16 activations (W4A16, the reference's default prefill arithmetic,
// engine/src/qwen/fn_moe_pf.cu:118-437) on the 5th-generation tensor cores: tcgen05.mma kind::f16, bf16 × bf16 → fp32 in tensor memory.
//
// The NVFP4 weights are the A operand (M = 128 rows of the record's matrix), the activation rows of one expert's pairs the B operand
// (N ≤ 256 pairs, N a multiple of 16 chosen per tile), so one dequantised weight value serves up to 256 multiply-adds and the
// accumulator's lanes are weight rows — the epilogue thread of a lane owns one output row of the expert, as in the decode kernels.
// Dequantisation: e2m1 → f16 (hardware converter) × e4m3 block scale as f16 — the product has ≤ 6 significant bits, exact in f16 and
// in bf16 — written as bf16 into the K-major 128-byte-swizzle operand tile by eight warps; every product of the MMA is therefore the
// exact product of the decode operators, sums are fp32.  Rounding points after the sums are the reference's (g, u → bf16 after the
// global scale, y → bf16, down → bf16 before the routing weight).
//
// Per CTA (persistent, one per SM, 14 warps): warp 5 (one thread) streams raw code boxes (128 bytes × 64 rows, 256 k values per row)
// of the weights through the anchored tensor map of the decode path and the activation boxes (64 values × 64 rows of bf16) of the
// tile; warps 6-13 turn a raw box into four operand tiles (64 k values each), fetching their row's block scales from global memory
// a raw box ahead; warp 4 (one thread) issues the MMAs (128 × N × 16, four per operand tile) into two accumulator buffers of 256
// columns; warps 0-3 run the epilogue.  Gate/up: an A tile holds 64 gate and 64 up rows arranged so that lanes l and l + 16 of a
// warp hold the gate and the up value of the same row of I — SwiGLU is one shuffle.  Every wait is bounded.
#pragma once
#include "tc_common.cuh"

namespace hb {

constexpr int A16_BN = 256;                     // pairs of a tile (MMA N), at most
constexpr int A16_STA = 3, A16_STB = 4;         // operand rings: dequantised weight tiles, activation tiles
constexpr int A16_A = 128 * 128;                // 128 rows × 64 bf16
constexpr int A16_B = A16_BN * 128;             // 256 rows × 64 bf16
constexpr int A16_RAW = 128 * 128;              // raw codes: 128 rows × 128 bytes (256 k values per row)
constexpr int A16_SMEM = 1024 + A16_STA * A16_A + A16_STB * A16_B + 2 * A16_RAW + 1024;
constexpr int A16_THREADS = 14 * 32;            // warps 0-3 epilogue, 4 MMA issue, 5 TMA, 6-13 dequantisation
constexpr int A16_W_MMA = 4, A16_W_TMA = 5, A16_W_DQ0 = 6, A16_DQ_THREADS = 256;
constexpr int A16_TMEM_COLS = 512;              // two accumulators of 256 columns
static_assert(A16_SMEM <= 227 * 1024, "shared memory");

struct A16Args {
  const TileRef* tiles; const int* n_tiles;     // tiles of ≤ A16_BN consecutive slots of one expert's run of the sorted pairs
  const int* perm;                              // pair of a slot (the down pass writes its rows by pair)
  const uint8_t* const* tab;                    // expert records of the layer
  int down;                                     // 0: gate/up (out = y bf16 [slot, I]); 1: down (out = bf16 [pair, H])
  int K, n_out;                                 // inner dimension (H | I), output rows per expert (I | H)
  uint32_t off_w, off_s0, off_s1, off_g;        // record offsets: first matrix, scales of both halves of an A tile, global scales
  int row2, trows;                              // matrix rows between the two 64-row boxes of an item; matrix rows an item advances per half
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

__global__ void __launch_bounds__(A16_THREADS, 1) a16_gemm_kernel(const A16Args a, const __grid_constant__ CUtensorMap tmB) {
  extern __shared__ uint8_t a16_raw[];
  const uint32_t raw0 = smem_u32(a16_raw), base = (raw0 + 1023u) & ~1023u;
  uint8_t* sm = a16_raw + (base - raw0);
  uint8_t* smA = sm;                                   // [STA][16 KB]
  uint8_t* smB = smA + A16_STA * A16_A;                // [STB][32 KB]
  uint8_t* smR = smB + A16_STB * A16_B;                // [2][16 KB]
  uint64_t* fullA = reinterpret_cast<uint64_t*>(smR + 2 * A16_RAW);
  uint64_t* emptyA = fullA + A16_STA;
  uint64_t* fullB = emptyA + A16_STA;
  uint64_t* emptyB = fullB + A16_STB;
  uint64_t* fullR = emptyB + A16_STB;
  uint64_t* emptyR = fullR + 2;
  uint64_t* acc_full = emptyR + 2;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* mma_done = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < A16_STA; ++s) { mbar_init(&fullA[s], A16_DQ_THREADS); mbar_init(&emptyA[s], 1); }
    for (int s = 0; s < A16_STB; ++s) { mbar_init(&fullB[s], 1); mbar_init(&emptyB[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&fullR[s], 1); mbar_init(&emptyR[s], A16_DQ_THREADS); mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 128); }
    mbar_init(mma_done, 1);
    mbar_fence_init();
  }
  if (warp == A16_W_MMA) { tmem_alloc(tmem_slot, A16_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int nT = a.down ? a.n_out / 128 : a.n_out / 64;       // items per tile
  const int n_items_all = *a.n_tiles * nT;
  const int nraw = a.K >> 8;                                  // raw boxes per item; four operand tiles each

  if (warp == A16_W_TMA) {
    // ------------------------------------------------------------------------------------------------ loads: one thread
    if (lane == 0) {
      uint32_t rit = 0, kit = 0, seen = 0u;
      bool ok = true;
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
        const int r0 = (int)row + t * a.trows, r1 = r0 + a.row2;
        const int nbox = (tl.rows + 63) >> 6;
        for (int rs = 0; rs < nraw && ok; ++rs, ++rit) {
          const uint32_t sl = rit & 1u;
          if (!(ok = mbar_wait(&emptyR[sl], ((rit >> 1) & 1u) ^ 1u, a.err, 0x1u))) break;
          const uint32_t rb = smem_u32(smR + sl * A16_RAW);
          mbar_expect_tx(&fullR[sl], A16_RAW);
          tma_load_2d(rb, map, rs * 128, r0, &fullR[sl]);
          tma_load_2d(rb + A16_RAW / 2, map, rs * 128, r1, &fullR[sl]);
          for (int kq = 0; kq < 4; ++kq, ++kit) {
            const uint32_t sb = kit % A16_STB;
            if (!(ok = mbar_wait(&emptyB[sb], ((kit / A16_STB) & 1u) ^ 1u, a.err, 0x2u))) break;
            const uint32_t bb = smem_u32(smB + sb * A16_B);
            mbar_expect_tx(&fullB[sb], (uint32_t)nbox * 8192u);
            for (int i = 0; i < nbox; ++i) tma_load_2d(bb + i * 8192, &tmB, (rs * 4 + kq) * 64, tl.slot0 + i * 64, &fullB[sb]);
          }
        }
      }
    }
  } else if (warp >= A16_W_DQ0) {
    // ------------------------------------------------------------------------------------------------ dequantisation: thread (r, h) owns half a row
    // of every operand tile: A row r, k values [32 h, 32 h + 32) of the tile's 64
    const int dt = threadIdx.x - A16_W_DQ0 * 32, r = dt >> 1, h = dt & 1;
    int rr, srow; uint32_t soff;                               // raw row, row of the scale matrix inside the item, which scale matrix
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
    for (int item = blockIdx.x; item < n_items_all && ok; item += gridDim.x) {
      const int ti = item / nT, t = item - ti * nT;
      const uint8_t* rec = a.tab[a.tiles[ti].expert];
      if (!rec) break;
      const uint8_t* srowp = rec + soff + (size_t)(t * a.trows + srow) * sbytes;
      uint4 sc = __ldg(reinterpret_cast<const uint4*>(srowp));
      for (int rs = 0; rs < nraw && ok; ++rs, ++rit) {
        uint4 sc_next = sc;
        if (rs + 1 < nraw) sc_next = __ldg(reinterpret_cast<const uint4*>(srowp + (size_t)(rs + 1) * 16));
        const uint32_t sl = rit & 1u;
        if (!(ok = mbar_wait(&fullR[sl], (rit >> 1) & 1u, a.err, 0x4u))) break;
        const uint8_t* rawrow = smR + sl * A16_RAW + rr * 128;
        const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
        for (int kq = 0; kq < 4; ++kq, ++kit) {
          const uint4 cw = *reinterpret_cast<const uint4*>(rawrow + (((kq * 2 + h) ^ (rr & 7)) << 4));     // 32 codes
          const uint32_t s2 = (scw[kq] >> (16 * h)) & 0xffffu;                                              // the two block scales
          const uint32_t sh = cvt_e4m3x2_f16x2(s2);
          const uint32_t slo = __byte_perm(sh, sh, 0x1010), shi = __byte_perm(sh, sh, 0x3232);             // (s0, s0), (s1, s1)
          const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
          const uint32_t sa = kit % A16_STA;
          if (!(ok = mbar_wait(&emptyA[sa], ((kit / A16_STA) & 1u) ^ 1u, a.err, 0x8u))) break;
          uint8_t* arow = smA + sa * A16_A + r * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t hh[4];
            cvt_e2m1x8_f16x2(cws[c], hh);
            const uint32_t sv = c < 2 ? slo : shi;
            uint4 o;
            o.x = f16x2_to_bf16x2(hmul2_u32(hh[0], sv)); o.y = f16x2_to_bf16x2(hmul2_u32(hh[1], sv));
            o.z = f16x2_to_bf16x2(hmul2_u32(hh[2], sv)); o.w = f16x2_to_bf16x2(hmul2_u32(hh[3], sv));
            *reinterpret_cast<uint4*>(arow + (((h * 4 + c) ^ (r & 7)) << 4)) = o;
          }
          fence_proxy_async_smem();
          mbar_arrive(&fullA[sa]);
        }
        if (!ok) break;
        mbar_arrive(&emptyR[sl]);
        sc = sc_next;
      }
    }
  } else if (warp == A16_W_MMA) {
    // ------------------------------------------------------------------------------------------------ MMA issue: one thread
    if (lane == 0) {
      uint32_t kit = 0, n_it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items_all && ok; item += gridDim.x, ++n_it) {
        const int ti = item / nT;
        const int rows = a.tiles[ti].rows;
        const uint32_t N = (uint32_t)((rows + 15) & ~15);
        // kind::f16: D fp32 (bit 4), A and B bf16 (format 1 at bits 7 and 10), both K-major, N / 8 at bit 17, M / 16 at bit 24
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t buf = n_it & 1u;
        if (n_it >= 2 && !(ok = mbar_wait(&acc_empty[buf], ((n_it >> 1) - 1u) & 1u, a.err, 0x10u))) break;
        tc_fence_after();
        const int nk = a.K >> 6;
        for (int kb = 0; kb < nk; ++kb, ++kit) {
          const uint32_t sa = kit % A16_STA, sb = kit % A16_STB;
          if (!(ok = mbar_wait(&fullA[sa], (kit / A16_STA) & 1u, a.err, 0x20u))) break;
          if (!(ok = mbar_wait(&fullB[sb], (kit / A16_STB) & 1u, a.err, 0x40u))) break;
          tc_fence_after();
          const uint64_t ad = tc_desc_sw128(base + sa * A16_A), bd = tc_desc_sw128(base + A16_STA * A16_A + sb * A16_B);
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) tc_mma_f16(tmem + buf * 256, ad + 2 * j, bd + 2 * j, idesc, (kb | (int)j) != 0 ? 1u : 0u);
          tc_commit(&emptyA[sa]);
          tc_commit(&emptyB[sb]);
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
      tc_commit(mma_done);
      mbar_wait(mma_done, 0, a.err, 0x80u);
    }
  } else {
    // ------------------------------------------------------------------------------------------------ epilogue: warp q reads lanes [32 q, 32 q + 32)
    const int q = warp, tl_ = threadIdx.x;                     // tl_ = row of the A tile
    bool ok = true;
    uint32_t n_it = 0;
    for (int item = blockIdx.x; item < n_items_all && ok; item += gridDim.x, ++n_it) {
      const int ti = item / nT, t = item - ti * nT;
      const TileRef tl = a.tiles[ti];
      const uint8_t* rec = a.tab[tl.expert];
      if (!rec) break;
      const float gsc = __ldg(reinterpret_cast<const float*>(rec + a.off_g) + (a.down ? 2 : lane < 16 ? 0 : 1));
      const uint32_t buf = n_it & 1u;
      if (!(ok = mbar_wait(&acc_full[buf], (n_it >> 1) & 1u, a.err, 0x100u))) break;
      tc_fence_after();
      const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16) + buf * 256;
      for (int c0 = 0; c0 < tl.rows; c0 += 32) {
        uint32_t rg[32];
        tc_ld32(trow + c0, rg);
        tc_wait_ld();
        if (a.down) {
          __nv_bfloat16* orow = a.out + (size_t)t * 128 + tl_;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c0 + c < tl.rows) {
              const int pair = __ldg(a.perm + tl.slot0 + c0 + c);
              orow[(size_t)pair * a.n_out] = __float2bfloat16(__uint_as_float(rg[c]) * gsc);
            }
          }
        } else {
          __nv_bfloat16* orow = a.out + (size_t)(tl.slot0 + c0) * a.n_out + t * 64 + 16 * q + (lane & 15);
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float v = bf16r(__uint_as_float(rg[c]) * gsc);
            float uv = __shfl_down_sync(0xffffffffu, v, 16);
            if (lane < 16 && c0 + c < tl.rows) {
              float gv = v;
              if (a.limit > 0.f) { uv = fminf(fmaxf(uv, -a.limit), a.limit); gv = fminf(gv, a.limit); }
              orow[(size_t)c * a.n_out] = __float2bfloat16(gv / (1.f + __expf(-gv)) * uv);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == A16_W_MMA) { tc_fence_after(); tmem_dealloc(tmem, A16_TMEM_COLS); }
}

}  // namespace hb
