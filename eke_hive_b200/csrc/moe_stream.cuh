// Shared pieces of the routed-expert decode kernels: workspace carve-up, the item geometry of the weight stream, the
// B-fragment loader and the per-warp e2m1 → f16 → tensor-core slice product.  Included by the unfused kernels
// (k_moe_decode.cu) and the fused layer kernel (k_moe_fused.cu).
#pragma once
#include "hb_common.cuh"
#include "hb_kernels.h"

namespace hb {

constexpr int kGroupRows = 8;         // activation rows per group = columns of one m16n8k16 tile
constexpr int kSlice = 256;           // K elements per consumer warp
constexpr int kMaxStages = 8;
constexpr int kGroupThreads = 1024;

struct Group { const uint8_t* rec; int start; int n; };
static_assert(sizeof(Group) == 16, "Group layout");

struct DecodeWs {
  int* hdr;               // [0] number of groups, [1] number of valid pairs
  Group* groups;          // [n_pairs]
  int* s_row;             // [n_pairs] activation row of each sorted position
  int* pos_of;            // [n_pairs] sorted position of each original pair, -1 = skipped (invalid id / null record)
  int* prow;              // [n_pairs] activation row of each original pair
  float* pw;              // [n_pairs] routing weight of each original pair
  __nv_bfloat16* y;       // [n_pairs, I]
  __nv_bfloat16* part;    // [n_pairs, H]
  int* done;              // [n_pairs] fused kernel: gate/up items finished per group (zeroed by the grouping kernel); hdr[2] counts down items
};

__host__ __device__ inline size_t al256(size_t b) { return (b + 255) / 256 * 256; }

inline DecodeWs carve(void* ws, int n, int H, int I) {
  uint8_t* p = reinterpret_cast<uint8_t*>(ws);
  DecodeWs w;
  w.hdr = reinterpret_cast<int*>(p); p += 256;
  w.groups = reinterpret_cast<Group*>(p); p += al256((size_t)n * sizeof(Group));
  w.s_row = reinterpret_cast<int*>(p); p += al256((size_t)n * 4);
  w.pos_of = reinterpret_cast<int*>(p); p += al256((size_t)n * 4);
  w.prow = reinterpret_cast<int*>(p); p += al256((size_t)n * 4);
  w.pw = reinterpret_cast<float*>(p); p += al256((size_t)n * 4);
  w.y = reinterpret_cast<__nv_bfloat16*>(p); p += al256((size_t)n * I * 2);
  w.part = reinterpret_cast<__nv_bfloat16*>(p); p += al256((size_t)n * H * 2);
  w.done = reinterpret_cast<int*>(p);
  return w;
}

// Routed reduce of two adjacent columns of one row: Σ_k w·part in k order, then either the fp32 sum or the shared-expert combine.
struct ReduceArgs {
  const __nv_bfloat16* part; const int* pos_of; const float* pw; int M, K, H, shared_pairs;
  const __nv_bfloat16* shared; const float* lg; int ld, col;
  __nv_bfloat16* out_bf16; float* out_f32;
  __nv_bfloat16* shared_out = nullptr; int sh_row0 = 0, sh_rows = 0;   // fp32 form: the shared expert's output rows, written apart
  hbk_ep_push ep = {};                            // ep.world > 0: the routed sums go to the owning ranks' partial buffers
  uint32_t* err = nullptr; int n_pos = 0;         // debug build (-DHB_BOUNDS): the context's error word and the number of positions of `part`
};

struct StreamArgs {
  const int* hdr; const Group* groups; const int* s_row;
  const __nv_bfloat16* act; int act_ld;        // gate/up: x rows (indexed through s_row); down: y (indexed by sorted position)
  __nv_bfloat16* outp;                         // gate/up: y [pos, I]; down: part [pos, H]
  int H, I; float limit;
  uint32_t off_wa, off_sa, off_wb, off_sb, off_g;   // record offsets: gate/up = w1,s1,w3,s3 ; down = w2,s2 (wb/sb unused)
  int stages;
  uint32_t* err;
  // down kernel, routed form: when red_on, the CTAs meet at the end (fin: two counters in the workspace header, zeroed by the grouping
  // kernel) and add the rows' pairs up themselves — the k-order sum and the shared-expert combine without a launch of their own
  int red_on; unsigned int* fin; ReduceArgs red;
};

template <int WK, int WM, bool DOWN>
struct StreamCfg {
  static constexpr int NW = WK * WM;                       // consumer warps
  static constexpr int THREADS = (NW + 2) * 32;            // + one producer warp + one epilogue warp
  static constexpr int K = WK * kSlice;
  static constexpr int RB = K / 2, RS = K / 16;            // bytes of one row: weights, scales
  static constexpr int TR = (DOWN ? 16 : 8) * WM;          // matrix rows per item (gate/up: TR gate rows + TR up rows)
  static constexpr int MAT = TR * (RB + RS);               // bytes of one matrix part of a stage
  static constexpr int UP_OFF = MAT + 16;                  // the up part sits 16 B off a 128-B boundary: its rows use other banks than gate's
  static constexpr int STAGE = DOWN ? MAT : ((UP_OFF + MAT + 127) / 128 * 128);
  static constexpr int TX = DOWN ? MAT : 2 * MAT;          // bytes a full stage receives
  static constexpr int CTAS_PER_SM = THREADS <= 320 ? 2 : 1;   // resident CTAs the register and shared-memory budgets are planned for
  static constexpr int SLOT = NW * 32 * 16;                // one split-K exchange slot: a float4 per consumer thread
  static constexpr int BARS = 2 * kMaxStages * 8 + (kMaxStages + 1) * (WM + 1) * 8;
  __host__ __device__ static constexpr size_t head(int stages) { return (size_t)(((WK > 1 ? (stages + 1) * SLOT : 0) + BARS + 127) / 128 * 128); }
  __host__ __device__ static constexpr size_t smem(int stages) { return head(stages) + (size_t)stages * STAGE; }
};

// Loads this warp's 256-column slice of ≤ 8 activation rows as the B fragments of 16 m16n8k16 tiles (f16): lane (g, t) holds
// columns [64t, 64t+64) of activation row g of the group.  Each row slice is scaled by a power of two so its largest magnitude
// lands in [2^14, 2^15) before the bf16 → f16 conversion (no overflow, small values keep their bits); inv[0], inv[1] return
// the inverse factors of the two tile columns this lane accumulates.
// COHERENT: the rows were written earlier in the same kernel by other CTAs — read them through L2 (ld.global.cg), never the
// non-coherent path.
template <bool COHERENT = false>
__device__ __forceinline__ void load_b_frags(const __nv_bfloat16* src /* slice of the row of column g, or nullptr */, int t, uint32_t (&b)[32],
                                             float (&inv)[2]) {
  // two passes over the lane's 128 bytes (the second hits L1/L2): max magnitude first, then scale + convert, so that at most
  // the 32 result registers are live
  const uint4* p = src ? reinterpret_cast<const uint4*>(src + 64 * t) : nullptr;
  uint32_t am = 0;                                              // max |x| as bf16 bits (sign cleared): integer order = magnitude order
  if (p) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 r = COHERENT ? __ldcg(p + i) : __ldg(p + i);
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { am = max(am, w[j] & 0x7fffu); am = max(am, (w[j] >> 16) & 0x7fffu); }
    }
  }
  am = max(am, __shfl_xor_sync(0xffffffffu, am, 1));
  am = max(am, __shfl_xor_sync(0xffffffffu, am, 2));
  int e = (int)(am >> 7);                                       // biased exponent of the largest magnitude
  e = min(max(e, 27), 254);                                     // tiny rows: keep the factor finite
  const float fac = __int_as_float((uint32_t)(127 + 14 + 127 - e) << 23);       // 2^(14 - (e - 127))
  const float myinv = __int_as_float((uint32_t)(e - 14) << 23);                 // 2^((e - 127) - 14)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint4 r = p ? (COHERENT ? __ldcg(p + i) : __ldg(p + i)) : make_uint4(0, 0, 0, 0);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = __uint_as_float(w[j] << 16) * fac, hi = __uint_as_float(w[j] & 0xffff0000u) * fac;
      const __half2 hh = __floats2half2_rn(lo, hi);
      b[i * 4 + j] = *reinterpret_cast<const uint32_t*>(&hh);
    }
  }
  inv[0] = __shfl_sync(0xffffffffu, myinv, (2 * t) * 4);
  inv[1] = __shfl_sync(0xffffffffu, myinv, (2 * t + 1) * 4);
}

// One warp: 16 tile rows (this lane: rowA for the low half, rowB for the high half) × 256 columns against the B fragments.
// wa / wb point at this lane's 32 weight bytes of the two rows (columns [64t, 64t+64) of the slice), sa / sb at its 4 scale bytes.
// The two 16-byte halves are fetched one after the other to keep few registers live; the stage is handed back to the producer
// as soon as the second half is in registers.
__device__ __forceinline__ void warp_slice_mma(const uint8_t* wa, const uint8_t* wb, const uint8_t* sa, const uint8_t* sb,
                                               const uint32_t (&b)[32], float (&acc)[4], uint64_t* empty_bar) {
  const uint32_t s4a = *reinterpret_cast<const uint32_t*>(sa), s4b = *reinterpret_cast<const uint32_t*>(sb);
  // four e4m3 block scales per row → f16 (exact)
  const uint32_t fa[2] = {cvt_e4m3x2_f16x2(s4a & 0xffffu), cvt_e4m3x2_f16x2(s4a >> 16)};
  const uint32_t fb[2] = {cvt_e4m3x2_f16x2(s4b & 0xffffu), cvt_e4m3x2_f16x2(s4b >> 16)};
  float c[2][4];                                        // two independent accumulator chains, summed at the end
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 qa = *reinterpret_cast<const uint4*>(wa + 16 * h), qb = *reinterpret_cast<const uint4*>(wb + 16 * h);
    if (h == 1) {                                       // everything this warp needs from the stage is in registers
      __syncwarp();
      if (empty_bar && (threadIdx.x & 31) == 0) mbar_arrive(empty_bar);
    }
    const uint32_t wqa[4] = {qa.x, qa.y, qa.z, qa.w}, wqb[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {                    // word j = 8 columns = two tiles; its 16-column block is j >> 1
      const int j = 4 * h + jj;
      // the block's f16 scale broadcast to both halves of a register
      const uint32_t sca = __byte_perm(fa[h], 0, (jj >> 1) ? 0x3232 : 0x1010), scb = __byte_perm(fb[h], 0, (jj >> 1) ? 0x3232 : 0x1010);
      uint32_t ha[4], hb_[4];
      cvt_e2m1x8_f16x2(wqa[jj], ha);
      cvt_e2m1x8_f16x2(wqb[jj], hb_);
#pragma unroll
      for (int i = 0; i < 4; ++i) { ha[i] = hmul2_u32(ha[i], sca); hb_[i] = hmul2_u32(hb_[i], scb); }
      { const uint32_t afr[4] = {ha[0], hb_[0], ha[1], hb_[1]}; mma_f16_16816(c[0], afr, b[4 * j], b[4 * j + 1]); }
      { const uint32_t afr[4] = {ha[2], hb_[2], ha[3], hb_[3]}; mma_f16_16816(c[1], afr, b[4 * j + 2], b[4 * j + 3]); }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) acc[j] = c[0][j] + c[1][j];
}

// Epilogue of one 16-row tile held in m16n8k16 accumulator layout: acc[c] = (tile row g + 8·(c>>1), activation row 2t + (c&1)).
// Gate/up tiles alternate gate and up rows (even g = gate, odd g = up of the same output row): bf16 roundings, optional clamp,
// SiLU·up → y.  Down tiles: bf16(v · g2) → part.  gl = the record's three global scales.
template <bool DOWN>
__device__ __forceinline__ void tile_epilogue(const float (&acc)[4], const Group& grp, const float (&gl)[3], int row0 /* first matrix row of the tile */,
                                              int lane, int H, int I, float limit, __nv_bfloat16* outp) {
  const int g = lane >> 2, tok0 = 2 * (lane & 3);
  if (DOWN) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int tok = tok0 + (c & 1), n = row0 + g + (c >> 1) * 8;
      if (tok < grp.n) outp[(size_t)(grp.start + tok) * H + n] = __float2bfloat16(acc[c] * gl[2]);
    }
  } else {
    float oth[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) oth[c] = __shfl_xor_sync(0xffffffffu, acc[c], 4);
    const bool odd = g & 1;
    const int i = row0 + (g >> 1) + (odd ? 4 : 0);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float gv = odd ? oth[2 + c] : acc[c], uv = odd ? acc[2 + c] : oth[c];
      gv = bf16r(gv * gl[0]); uv = bf16r(uv * gl[1]);
      if (limit > 0.f) { uv = fminf(fmaxf(uv, -limit), limit); gv = fminf(gv, limit); }
      const float yv = gv / (1.f + __expf(-gv)) * uv;
      const int tok = tok0 + c;
      if (tok < grp.n) outp[(size_t)(grp.start + tok) * I + i] = __float2bfloat16(yv);
    }
  }
}

__device__ __forceinline__ void reduce_routed_unit(const ReduceArgs& r, size_t i) {
  const int m = (int)(i / (r.H / 2)), d = (int)(i % (r.H / 2)) * 2;
  float a0 = 0.f, a1 = 0.f;
  // four terms at a time: fetch them first (independent loads in flight together), then add in k order
#pragma unroll 1
  for (int k0 = 0; k0 < r.K; k0 += 4) {
    uint32_t raw[4]; float wv[4]; int ps[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      raw[k] = 0u; wv[k] = 0.f; ps[k] = -1;
      if (k0 + k < r.K) {
        ps[k] = r.pos_of[m * r.K + k0 + k];
        if (ps[k] >= 0 && !HB_BOUND(r.err, ps[k] < r.n_pos, 0x121u, ps[k])) ps[k] = -1;
        if (ps[k] >= 0) { wv[k] = r.pw[m * r.K + k0 + k]; raw[k] = __ldcg(reinterpret_cast<const unsigned int*>(r.part + (size_t)ps[k] * r.H + d)); }
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (ps[k] >= 0) {                                    // a skipped pair adds nothing (not even +0: keeps -0 sums as they are)
        a0 = __fadd_rn(a0, __fmul_rn(wv[k], __uint_as_float(raw[k] << 16)));
        a1 = __fadd_rn(a1, __fmul_rn(wv[k], __uint_as_float(raw[k] & 0xffff0000u)));
      }
    }
  }
  const int sh_pos = (r.shared_pairs || r.shared_out) ? r.pos_of[r.M * r.K + m] : -1;
  if (r.ep.world > 0) {                            // row m belongs to rank m / B: slot `rank` of that rank's partial buffer
    const int pr = m / r.ep.B;
    *reinterpret_cast<float2*>(r.ep.rs[pr] + ((size_t)r.ep.rank * r.ep.B + (m - pr * r.ep.B)) * r.H + d) = make_float2(a0, a1);
  } else if (r.out_f32) { r.out_f32[(size_t)m * r.H + d] = a0; r.out_f32[(size_t)m * r.H + d + 1] = a1; }
  if (r.shared_out && m >= r.sh_row0 && m < r.sh_row0 + r.sh_rows) {
    *reinterpret_cast<unsigned int*>(r.shared_out + (size_t)(m - r.sh_row0) * r.H + d) =
        sh_pos >= 0 ? __ldcg(reinterpret_cast<const unsigned int*>(r.part + (size_t)sh_pos * r.H + d)) : 0u;
  }
  if (!r.out_bf16) return;
  float s0 = 0.f, s1 = 0.f;
  bool have = false;
  if (r.shared_pairs) {
    const uint32_t raw = __ldcg(reinterpret_cast<const unsigned int*>(r.part + (size_t)sh_pos * r.H + d));
    s0 = __uint_as_float(raw << 16); s1 = __uint_as_float(raw & 0xffff0000u); have = true;
  } else if (r.shared) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(r.shared + (size_t)m * r.H + d);
    s0 = __bfloat162float(v.x); s1 = __bfloat162float(v.y); have = true;
  }
  if (have && r.lg) {
    const float gt = bf16r(sigmoid_portable(bf16r(r.lg[(size_t)m * r.ld + r.col])));
    s0 = bf16r(__fmul_rn(gt, s0)); s1 = bf16r(__fmul_rn(gt, s1));
  }
  __nv_bfloat162 o;
  o.x = __float2bfloat16(__fadd_rn(bf16r(a0), s0)); o.y = __float2bfloat16(__fadd_rn(bf16r(a1), s1));
  *reinterpret_cast<__nv_bfloat162*>(r.out_bf16 + (size_t)m * r.H + d) = o;
}

}  // namespace hb

// fused layer kernel (k_moe_fused.cu)
bool hbk_moe_fused_available(int H, int I);
int hbk_moe_fused_setup(hb_ctx* ctx);
int hbk_moe_fused_launch(hb_ctx* ctx, const hb::DecodeWs& w, const void* x, int H, int I, float limit, const hb_rec_layout& L, const hb::ReduceArgs* red,
                         cudaStream_t st);
