// Dense decode GEMV for one weight matrix, M ≤ 8 activation rows per pass: NVFP4 and the 3-/2-bit group-64 formats
// (hb_qmat).  HBM-bound: every weight byte is read once, decoded in registers and fed to m16n8k16 tensor-core tiles whose 8
// columns are the activation rows (fp32 accumulation).
//
//   stream   persistent CTAs, grid = (CTAs per K split, K splits).  A CTA first turns the activation columns of its K range into
//            f16 B fragments in shared memory, in the order the tiles consume them; every (row, 256-column slice) gets its own
//            power-of-two rescale so bf16 outliers cannot overflow f16, undone in fp32 when the slice is accumulated.  The CTA
//            then walks strips of 16 weight rows (b, b + CTAs, ...): warp w streams the strip's slice w through its own cp.async
//            ring, which keeps running across strips, and the 8 partial tiles are summed in warp order in shared memory
//   reduce   fixed-order sum over the K splits, output conversion, or the fused SiLU·up activation of the gate/up pair
//
// Low-bit decode without shifts or subtractions per element: a 2-bit field left at bit 2j of an f16 mantissa under exponent
// 0x64 reads as 1024 + q·4^j, a 1-bit field at bit j as 1024 + b·2^j.  The B fragments carry the matching 4^-j / 2^-j factors
// (exact), and the 1024·Σx' offset is removed per group together with the zero-point:  y += s·(tile − zp·S0 − S1),
// S0 = Σ x, S1 = 1024·Σ x'.  One logic instruction per element pair, scales and zero-points applied in fp32.
#include "moe_stream.cuh"

namespace hb {

constexpr int kDSlice = 256;            // columns per pipeline stage
constexpr int kDWarps = 8;              // streaming warps per CTA (one slice of K each); a ninth warp sums their partial tiles
constexpr int kDSlots = 4;              // ring of partial-tile slots between the streaming warps and the summing warp
__host__ __device__ constexpr int dense_stages(int fmt) { return fmt == HB_FMT_NVFP4 ? 3 : 4; }
// K range of one CTA (slices of 256 columns whose B fragments sit in shared memory): sized for two CTAs per SM
__host__ __device__ constexpr int dense_max_slices(int) { return kDWarps; }     // one slice per warp

struct DenseFmt {
  int planes;         // B-fragment planes (LB3 has two)
  int pitch_w;        // shared-memory row pitch of the first code plane (padded: rows of a quarter-warp hit different banks)
  int bytes_w;        // code bytes per row per slice, first plane
  int pitch_h, bytes_h;   // second plane (LB3 high bits)
  int bytes_s;        // scale (+ zero-point) bytes per row per slice
};
__host__ __device__ constexpr DenseFmt dense_fmt(int fmt) {
  return fmt == HB_FMT_NVFP4 ? DenseFmt{1, 144, 128, 0, 0, 16}
       : fmt == HB_FMT_LB2_G64 ? DenseFmt{1, 80, 64, 0, 0, 16}
                               : DenseFmt{2, 80, 64, 48, 32, 16};
}
__host__ __device__ constexpr int dense_stage_bytes(int fmt) {
  return 16 * (dense_fmt(fmt).pitch_w + dense_fmt(fmt).pitch_h + dense_fmt(fmt).bytes_s);
}

// Workspace = fp32 partial sums [mats][K splits][8][N].
//
// Fragment order.  Register r (0..31) of lane (tok = lane >> 2, t = lane & 3) of a slice sits at uint32 index
// ((r >> 2) * 32 + lane) * 4 + (r & 3) of the slice's plane; its halves hold, with gq = r >> 3 and pr = r & 7:
//   NVFP4          columns 64t + 2r, 64t + 2r + 1
//   2-bit plane    columns 64gq + 16t + pr and + 8, times 4^-j, j = pr < 5 ? pr : pr - 5   (the lane's 32-bit word of the group)
//   1-bit plane    columns 64gq + 32(t >> 1) + 8(t & 1) + pr and + 16, times 4 / 2^pr      (lanes 0,1 share word 0, lanes 2,3 word 1)

// B fragments, slice factor and group sums of row `tok`, slice `cs` (of the CTA's range) from the 8 columns [8·lane, 8·lane+8)
// this lane holds in v.  One warp per (slice, row).
template <int FMT>
__device__ __forceinline__ void dense_build_row_slice(uint4 v, int cs, int tok, int lane, uint4* xb_s, float2* sums_s, float* inv_s) {
  constexpr int PL = dense_fmt(FMT).planes;
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  unsigned int am = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) { am = max(am, w[j] & 0x7fffu); am = max(am, (w[j] >> 16) & 0x7fffu); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) am = max(am, __shfl_xor_sync(0xffffffffu, am, o));
  const int e = min(max((int)(am >> 7), 27), 254);                       // bf16 exponent field of the largest magnitude
  const float f = __int_as_float((uint32_t)(127 + 12 + 127 - e) << 23);  // the maximum lands in [2^12, 2^13): 4·x (high-bit plane) stays inside f16
  if (lane == 0) inv_s[cs * 8 + tok] = __int_as_float((uint32_t)(e - 12) << 23);
  float xv[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) { xv[2 * j] = __int_as_float(w[j] << 16) * f; xv[2 * j + 1] = __int_as_float(w[j] & 0xffff0000u) * f; }
  if (FMT == HB_FMT_NVFP4) {
    uint4 o;
    __half2 h;
    h = __floats2half2_rn(xv[0], xv[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(xv[2], xv[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(xv[4], xv[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(xv[6], xv[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
    xb_s[(size_t)cs * 256 + (lane & 7) * 32 + tok * 4 + (lane >> 3)] = o;
    return;
  }
  const int gq = lane >> 3, l7 = lane & 7;
  float s0 = 0.f, s1 = 0.f;
  {                                                                      // 2-bit plane: partner lane ^1 holds the other half of each register
    float sv[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int j = p < 5 ? p : p - 5;
      sv[p] = __half2float(__float2half_rn(xv[p] * (1.f / (float)(1 << (2 * j)))));
      s0 += __half2float(__float2half_rn(xv[p]));
      s1 += sv[p];
    }
    const int hi = lane & 1, t = l7 >> 1;
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float got = __shfl_xor_sync(0xffffffffu, hi ? sv[q] : sv[4 + q], 1);
      const __half2 h = hi ? __floats2half2_rn(got, sv[4 + q]) : __floats2half2_rn(sv[q], got);
      o[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    xb_s[(size_t)cs * PL * 256 + (2 * gq + hi) * 32 + tok * 4 + t] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (FMT == HB_FMT_LB3_G64) {                                           // 1-bit plane: partner lane ^2
    float hv[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) { hv[p] = __half2float(__float2half_rn(xv[p] * (4.f / (float)(1 << p)))); s1 += hv[p]; }
    const int hi = (l7 >> 1) & 1, t = 2 * (l7 >> 2) + (l7 & 1);
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float got = __shfl_xor_sync(0xffffffffu, hi ? hv[q] : hv[4 + q], 2);
      const __half2 h = hi ? __floats2half2_rn(got, hv[4 + q]) : __floats2half2_rn(hv[q], got);
      o[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    xb_s[(size_t)cs * PL * 256 + 256 + (2 * gq + hi) * 32 + tok * 4 + t] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  // the tile of a 64-column group sums (1024 + q·4^j)·x' (+ (1024 + b·2^j)·x''): S0 = Σ x removes the zero-point, S1 = 1024·Σ x' the offset
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) { s0 += __shfl_xor_sync(0xffffffffu, s0, o); s1 += __shfl_xor_sync(0xffffffffu, s1, o); }
  if (l7 == 0) sums_s[(size_t)cs * 32 + gq * 8 + tok] = make_float2(s0, 1024.f * s1);
}

// ------------------------------------------------------------------------------------------------ stream
struct DenseMat { const uint8_t* w; const uint8_t* wh; const uint8_t* s; const uint8_t* zp; float g; };
struct DenseArgs {
  DenseMat mat[2]; int n_mats;
  uint32_t* err;                          // the context's error word (bounded waits)
  int N, K, M, ksplit, slices, ldx;       // slices = K / 256
  const __nv_bfloat16* x;
  float* part;                            // [n_mats][ksplit][8][N]
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }

// Persistent CTAs: blockIdx.y = K split (the CTA keeps that range's B fragments in shared memory for its whole life), blockIdx.x = one
// of the CTAs sharing the split.  Work unit of a CTA = a strip of 16 weight rows of one matrix over the split's columns; CTA b takes
// strips b, b + gridDim.x, ...  Warp w streams slice w of every strip through its own cp.async ring (so the CTA's requests cover
// 8 consecutive slices of the same 16 rows: long contiguous runs per row), and the warps' partial tiles meet in shared memory
// in warp order once per strip.
template <int FMT>
__global__ void __launch_bounds__((kDWarps + 1) * 32, 2) dense_stream_kernel(DenseArgs a) {
  constexpr DenseFmt F = dense_fmt(FMT);
  constexpr int STG = dense_stage_bytes(FMT), NST = dense_stages(FMT), MAXSL = dense_max_slices(FMT);
  extern __shared__ __align__(128) uint8_t dsm[];
  uint4* xb_s = reinterpret_cast<uint4*>(dsm);                                            // [MAXSL][planes][256] uint4
  float2* sums_s = reinterpret_cast<float2*>(dsm + (size_t)MAXSL * F.planes * 4096);      // [MAXSL][4 groups][8 rows] (S0, S1)
  float* inv_s = reinterpret_cast<float*>(dsm + (size_t)MAXSL * F.planes * 4096 + (size_t)MAXSL * 256);   // [MAXSL][8 rows] 1 / slice factor
  float4* red_s = reinterpret_cast<float4*>(inv_s + MAXSL * 8);                           // [kDSlots][warps][32 lanes] partial tiles
  uint64_t* redbar = reinterpret_cast<uint64_t*>(red_s + kDSlots * kDWarps * 32);         // [kDSlots] the slot's partial tiles are written
  uint64_t* redfree = redbar + kDSlots;                                                   // [kDSlots] the slot has been summed and may be reused
  uint8_t* rings = reinterpret_cast<uint8_t*>(redfree + kDSlots);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int ks = blockIdx.y;
  const int sl0 = (int)((long long)a.slices * ks / a.ksplit), sl1 = (int)((long long)a.slices * (ks + 1) / a.ksplit), nsl = sl1 - sl0;
  const int strips_per_mat = (a.N + 15) / 16, n_strips = strips_per_mat * a.n_mats;
  uint8_t* ring = rings + (size_t)warp * NST * STG;
  const int K = a.K;
  const bool active = warp < nsl;                                   // this warp's slice of the split: sl0 + warp
  auto issue = [&](int strip, int sl, int stage) {                  // slice sl (absolute) of a strip → ring stage
    const bool m1 = strip >= strips_per_mat;                        // (selects, not an index: a dynamic index would copy the parameter to local memory)
    DenseMat W;
    W.w = m1 ? a.mat[1].w : a.mat[0].w; W.wh = m1 ? a.mat[1].wh : a.mat[0].wh; W.s = m1 ? a.mat[1].s : a.mat[0].s; W.zp = m1 ? a.mat[1].zp : a.mat[0].zp;
    const int n0 = (m1 ? strip - strips_per_mat : strip) * 16;
    uint8_t* st = ring + (size_t)stage * STG;
    if (FMT == HB_FMT_NVFP4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = lane + 32 * i, row = c >> 3, col = c & 7, n = min(n0 + row, a.N - 1);
        cp_async16(st + row * F.pitch_w + col * 16, W.w + (size_t)n * (K / 2) + (size_t)sl * 128 + col * 16);
      }
      if (lane < 16) { const int n = min(n0 + lane, a.N - 1); cp_async16(st + 16 * F.pitch_w + lane * 16, W.s + (size_t)n * (K / 16) + (size_t)sl * 16); }
    } else {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int c = lane + 32 * i, row = c >> 2, col = c & 3, n = min(n0 + row, a.N - 1);
        cp_async16(st + row * F.pitch_w + col * 16, W.w + (size_t)n * (K / 4) + (size_t)sl * 64 + col * 16);
      }
      if (FMT == HB_FMT_LB3_G64) {
        const int row = lane >> 1, col = lane & 1, n = min(n0 + row, a.N - 1);
        cp_async16(st + 16 * F.pitch_w + row * F.pitch_h + col * 16, W.wh + (size_t)n * (K / 8) + (size_t)sl * 32 + col * 16);
      }
      const int row = lane & 15, which = lane >> 4, n = min(n0 + row, a.N - 1);
      cp_async8(st + 16 * (F.pitch_w + F.pitch_h) + row * 16 + which * 8, (which ? W.zp : W.s) + ((size_t)n * (K / 64) + (size_t)sl * 4) * 2);
    }
  };
  int istrip = blockIdx.x, istage = 0;                             // issue cursor, NST-1 strips ahead of the compute cursor
  auto issue_next = [&]() {
    if (active && istrip < n_strips) issue(istrip, sl0 + warp, istage);
    istrip += gridDim.x;
    if (++istage == NST) istage = 0;
    cp_async_commit();                                              // always commit: the group count stays in step with the strip count
  };
  if (threadIdx.x == 0) {
    for (int q = 0; q < kDSlots; ++q) { mbar_init(&redbar[q], (uint32_t)nsl); mbar_init(&redfree[q], 1); }
    mbar_fence_init();
  }
  if (warp < kDWarps) for (int i = 0; i < NST - 1; ++i) issue_next();   // weights do not depend on the previous kernel: fetch before waiting for it
  griddep_wait();
  for (int it = warp; it < nsl * 8; it += kDWarps + 1) {                // B fragments of this K range, one warp per (slice, row)
    const int bs = it >> 3, tok = it & 7;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (tok < a.M) v = __ldcg(reinterpret_cast<const uint4*>(a.x + (size_t)tok * a.ldx + (size_t)(sl0 + bs) * kDSlice) + lane);
    dense_build_row_slice<FMT>(v, bs, tok, lane, xb_s, sums_s, inv_s);
  }
  __syncthreads();
  griddep_launch();
  const int cs = active ? warp : 0;                                 // slice index inside the CTA's range
  const uint4* xb_i = xb_s + (size_t)cs * F.planes * 256;
  const float2 iv = *reinterpret_cast<const float2*>(inv_s + cs * 8 + 2 * t);             // undo the slice factor of rows 2t, 2t+1
  uint32_t bq[32];
  if constexpr (FMT == HB_FMT_NVFP4) {                                        // the warp's slice never changes: its B fragments stay in registers
#pragma unroll
    for (int q = 0; q < 8; ++q) { const uint4 v = xb_i[q * 32 + lane]; bq[4 * q] = v.x; bq[4 * q + 1] = v.y; bq[4 * q + 2] = v.z; bq[4 * q + 3] = v.w; }
  }
  if (warp == kDWarps) {
    // ------------------------------------------------------------------------------------------------ summing warp
    // waits for a slot's partial tiles, adds them in warp order (fixed: deterministic), writes [mat][ks][row 0..7][N], frees the slot
    int slot = 0; uint32_t rph = 0;
    for (int strip = blockIdx.x; strip < n_strips; strip += gridDim.x) {
      if (!mbar_wait(&redbar[slot], rph, a.err, 0x10000u)) break;
      const int mat_i = strip >= strips_per_mat ? 1 : 0, n0 = (mat_i ? strip - strips_per_mat : strip) * 16;
      const float gsc = FMT == HB_FMT_NVFP4 ? (mat_i ? a.mat[1].g : a.mat[0].g) : 1.f;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      for (int w2 = 0; w2 < nsl; ++w2) { const float4 p = red_s[(slot * kDWarps + w2) * 32 + lane]; v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w; }
      __syncwarp();
      if (lane == 0) mbar_arrive(&redfree[slot]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int tok = 2 * t + (c & 1), n = n0 + g + (c >> 1) * 8;
        if (tok < a.M && n < a.N) a.part[(((size_t)mat_i * a.ksplit + ks) * 8 + tok) * a.N + n] = v[c] * gsc;
      }
      if (++slot == kDSlots) { slot = 0; rph ^= 1u; }
    }
    return;
  }
  if (!active) { cp_async_wait<0>(); return; }
  int cstage = 0, slot = 0;
  uint32_t rph = 0;
  for (int strip = blockIdx.x; strip < n_strips; strip += gridDim.x) {
    issue_next();
    cp_async_wait<NST - 1>();
    __syncwarp();
    float total[4] = {0.f, 0.f, 0.f, 0.f};
    {
    const uint8_t* st = ring + (size_t)cstage * STG;
    if constexpr (FMT == HB_FMT_NVFP4) {
      float acc[4];
      warp_slice_mma(st + g * F.pitch_w + 32 * t, st + (g + 8) * F.pitch_w + 32 * t, st + 16 * F.pitch_w + g * 16 + 4 * t,
                     st + 16 * F.pitch_w + (g + 8) * 16 + 4 * t, bq, acc, nullptr);
#pragma unroll
      for (int c = 0; c < 4; ++c) total[c] = fmaf(acc[c], (c & 1) ? iv.y : iv.x, total[c]);
    } else {
      const uint8_t* sz = st + 16 * (F.pitch_w + F.pitch_h);
      const uint4 szA = *reinterpret_cast<const uint4*>(sz + g * 16), szB = *reinterpret_cast<const uint4*>(sz + (g + 8) * 16);
      const uint32_t szAw[4] = {szA.x, szA.y, szA.z, szA.w}, szBw[4] = {szB.x, szB.y, szB.z, szB.w};   // {s01, s23, zp01, zp23} as f16 pairs
      float sub[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int gq = 0; gq < 4; ++gq) {
        float tmp[4] = {0.f, 0.f, 0.f, 0.f};
        {                                                           // low two bits: one 32-bit word = 16 columns per lane and row
          const uint32_t wA = *reinterpret_cast<const uint32_t*>(st + g * F.pitch_w + gq * 16 + 4 * t);
          const uint32_t wB = *reinterpret_cast<const uint32_t*>(st + (g + 8) * F.pitch_w + gq * 16 + 4 * t);
          const uint32_t wA2 = wA >> 10, wB2 = wB >> 10;
          uint32_t pA[8], pB[8];
#pragma unroll
          for (int p2 = 0; p2 < 8; ++p2) {
            const uint32_t m = 0x00030003u << (2 * (p2 < 5 ? p2 : p2 - 5));
            pA[p2] = ((p2 < 5 ? wA : wA2) & m) | 0x64006400u;
            pB[p2] = ((p2 < 5 ? wB : wB2) & m) | 0x64006400u;
          }
          const uint4 b0 = xb_i[(gq * 2) * 32 + lane], b1 = xb_i[(gq * 2 + 1) * 32 + lane];
          const uint32_t b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
          for (int m4 = 0; m4 < 4; ++m4) { const uint32_t afr[4] = {pA[2 * m4], pB[2 * m4], pA[2 * m4 + 1], pB[2 * m4 + 1]}; mma_f16_16816(tmp, afr, b[2 * m4], b[2 * m4 + 1]); }
        }
        if (FMT == HB_FMT_LB3_G64) {                                // high bit: lanes 0,1 share word 0 of the group, lanes 2,3 word 1
          const uint8_t* hb = st + 16 * F.pitch_w;
          uint32_t wA = *reinterpret_cast<const uint32_t*>(hb + g * F.pitch_h + gq * 8 + 4 * (t >> 1));
          uint32_t wB = *reinterpret_cast<const uint32_t*>(hb + (g + 8) * F.pitch_h + gq * 8 + 4 * (t >> 1));
          if (t & 1) { wA >>= 8; wB >>= 8; }
          uint32_t pA[8], pB[8];
#pragma unroll
          for (int p2 = 0; p2 < 8; ++p2) { pA[p2] = (wA & (0x00010001u << p2)) | 0x64006400u; pB[p2] = (wB & (0x00010001u << p2)) | 0x64006400u; }
          const uint4 b0 = xb_i[256 + (gq * 2) * 32 + lane], b1 = xb_i[256 + (gq * 2 + 1) * 32 + lane];
          const uint32_t b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
          for (int m4 = 0; m4 < 4; ++m4) { const uint32_t afr[4] = {pA[2 * m4], pB[2 * m4], pA[2 * m4 + 1], pB[2 * m4 + 1]}; mma_f16_16816(tmp, afr, b[2 * m4], b[2 * m4 + 1]); }
        }
        // scale and zero-point in fp32: y += s·(tile − zp·S0 − S1)
        const float4 su = *reinterpret_cast<const float4*>(sums_s + (size_t)cs * 32 + gq * 8 + 2 * t);   // (S0, S1) of rows 2t, 2t+1
        const __half2 sA2 = *reinterpret_cast<const __half2*>(&szAw[gq >> 1]), zA2 = *reinterpret_cast<const __half2*>(&szAw[2 + (gq >> 1)]);
        const __half2 sB2 = *reinterpret_cast<const __half2*>(&szBw[gq >> 1]), zB2 = *reinterpret_cast<const __half2*>(&szBw[2 + (gq >> 1)]);
        const float sA = (gq & 1) ? __high2float(sA2) : __low2float(sA2), zA = (gq & 1) ? __high2float(zA2) : __low2float(zA2);
        const float sB = (gq & 1) ? __high2float(sB2) : __low2float(sB2), zB = (gq & 1) ? __high2float(zB2) : __low2float(zB2);
        sub[0] = fmaf(sA, tmp[0] - fmaf(zA, su.x, su.y), sub[0]);
        sub[1] = fmaf(sA, tmp[1] - fmaf(zA, su.z, su.w), sub[1]);
        sub[2] = fmaf(sB, tmp[2] - fmaf(zB, su.x, su.y), sub[2]);
        sub[3] = fmaf(sB, tmp[3] - fmaf(zB, su.z, su.w), sub[3]);
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) total[c] = fmaf(sub[c], (c & 1) ? iv.y : iv.x, total[c]);
    }
    }
    __syncwarp();
    if (++cstage == NST) cstage = 0;
    // hand the partial tile to the summing warp through the slot ring; no streaming warp waits for another one
    if (!mbar_wait(&redfree[slot], rph ^ 1u, a.err, 0x20000u)) break;   // the slot's previous contents have been summed
    red_s[(slot * kDWarps + warp) * 32 + lane] = make_float4(total[0], total[1], total[2], total[3]);
    __syncwarp();
    if (lane == 0) mbar_arrive(&redbar[slot]);
    if (++slot == kDSlots) { slot = 0; rph ^= 1u; }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------------------ reduce
// mode 0: y fp32; 1: y bf16; 2: act = bf16( bf16(silu(bf16 g)) · bf16 u ) from the two matrices' sums
__global__ void dense_reduce_kernel(const float* __restrict__ part, int n_mats, int ksplit, int M, int N, int mode, void* __restrict__ y, int ldy) {
  griddep_wait();
  griddep_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  float v[2] = {0.f, 0.f};
  for (int mt = 0; mt < n_mats; ++mt)
    for (int k = 0; k < ksplit; ++k) v[mt] += part[(((size_t)mt * ksplit + k) * 8 + m) * N + n];      // fixed order
  if (mode == 0) reinterpret_cast<float*>(y)[(size_t)m * ldy + n] = v[0];
  else if (mode == 1) reinterpret_cast<__nv_bfloat16*>(y)[(size_t)m * ldy + n] = __float2bfloat16(v[0]);
  else {
    const float gv = bf16r(v[0]), uv = bf16r(v[1]);
    reinterpret_cast<__nv_bfloat16*>(y)[(size_t)m * ldy + n] = __float2bfloat16(bf16r(gv / (1.f + __expf(-gv))) * uv);
  }
}

// ------------------------------------------------------------------------------------------------ low-bit dequant (bit-exact definition)
__global__ void lb_dequant_kernel(int bits, const uint8_t* __restrict__ w, const uint8_t* __restrict__ wh, const __half* __restrict__ s,
                                  const __half* __restrict__ zp, int N, int K, __nv_bfloat16* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)N * K; i += (size_t)gridDim.x * blockDim.x) {
    const size_t n = i / K; const int k = (int)(i % K);
    int q = (w[n * (K / 4) + k / 4] >> (2 * (k & 3))) & 3;
    if (bits == 3) q |= ((wh[n * (K / 8) + k / 8] >> (k & 7)) & 1) << 2;
    const float sf = __half2float(s[n * (K / 64) + k / 64]), zf = __half2float(zp[n * (K / 64) + k / 64]);
    out[i] = __float2bfloat16(__fmul_rn(__fsub_rn((float)q, zf), sf));
  }
}

}  // namespace hb

using namespace hb;

namespace {
int dense_ksplit(int fmt, int K) { const int sl = K / kDSlice, mx = dense_max_slices(fmt); return (sl + mx - 1) / mx; }
size_t dense_smem(int fmt) {
  const DenseFmt F = dense_fmt(fmt);
  return (size_t)dense_max_slices(fmt) * F.planes * 4096 + (size_t)dense_max_slices(fmt) * 256 + (size_t)dense_max_slices(fmt) * 32 + kDSlots * kDWarps * 32 * 16 + 2 * kDSlots * 8 + (size_t)kDWarps * dense_stages(fmt) * dense_stage_bytes(fmt);
}
int check_mat(hb_ctx* ctx, const hb_qmat* W, const char* fn) {
  HB_REQUIRE(ctx, W && W->w && W->s, HB_ERR_INVALID, "%s: NULL matrix", fn);
  HB_REQUIRE(ctx, W->fmt == HB_FMT_NVFP4 || W->fmt == HB_FMT_LB3_G64 || W->fmt == HB_FMT_LB2_G64, HB_ERR_INVALID, "%s: unknown format %d", fn, W->fmt);
  HB_REQUIRE(ctx, W->N > 0 && W->K > 0 && W->K % kDSlice == 0, HB_ERR_UNSUPPORTED, "%s: N=%d K=%d (K must be a multiple of %d)", fn, W->N, W->K, kDSlice);
  HB_REQUIRE(ctx, W->fmt == HB_FMT_NVFP4 || W->zp, HB_ERR_INVALID, "%s: low-bit matrix without zero-points", fn);
  HB_REQUIRE(ctx, hb_aligned(W->w, 16) && hb_aligned(W->s, 16) && (W->fmt == HB_FMT_NVFP4 || hb_aligned(W->zp, 8)), HB_ERR_INVALID,
             "%s: weight / scale pointers must be 16-byte aligned", fn);
  return HB_OK;
}
DenseMat to_mat(const hb_qmat* W) {
  DenseMat m;
  m.w = W->w; m.s = reinterpret_cast<const uint8_t*>(W->s); m.zp = reinterpret_cast<const uint8_t*>(W->zp); m.g = W->g;
  m.wh = W->fmt == HB_FMT_LB3_G64 ? W->w + (size_t)W->N * (W->K / 4) : nullptr;
  return m;
}
// one pass of ≤ 8 rows: stream → reduce
int dense_pass(hb_ctx* ctx, const hb_qmat* A, const hb_qmat* B2, const void* x, int ldx, int M, int mode, void* y, int ldy, void* ws, cudaStream_t st) {
  const int fmt = A->fmt, N = A->N, K = A->K, slices = K / kDSlice, ksplit = dense_ksplit(fmt, K), mats = B2 ? 2 : 1;
  float* part = reinterpret_cast<float*>(ws);
  DenseArgs a{};
  a.mat[0] = to_mat(A); if (B2) a.mat[1] = to_mat(B2);
  a.n_mats = mats; a.N = N; a.K = K; a.M = M; a.ksplit = ksplit; a.slices = slices; a.ldx = ldx;
  a.x = reinterpret_cast<const __nv_bfloat16*>(x); a.part = part; a.err = ctx->dev_err;
  int r;
  int per_split = (2 * ctx->sm_count) / ksplit;                    // two CTAs per SM in all, shared out over the K splits
  const int strips = ((N + 15) / 16) * mats, max_useful = strips;
  if (per_split < 1) per_split = 1;
  if (per_split > max_useful) per_split = max_useful;
  const dim3 grid(per_split, ksplit, 1);
  auto fn = fmt == HB_FMT_NVFP4 ? dense_stream_kernel<HB_FMT_NVFP4> : fmt == HB_FMT_LB2_G64 ? dense_stream_kernel<HB_FMT_LB2_G64> : dense_stream_kernel<HB_FMT_LB3_G64>;
  if ((r = hb_launch(ctx, fmt == HB_FMT_NVFP4 ? "dense_stream_nvfp4" : fmt == HB_FMT_LB2_G64 ? "dense_stream_lb2" : "dense_stream_lb3", true, fn, grid,
                     dim3((kDWarps + 1) * 32), dense_smem(fmt), st, a))) return r;
  return hb_launch(ctx, "dense_reduce", true, dense_reduce_kernel, dim3((unsigned)(((size_t)M * N + 255) / 256)), dim3(256), 0, st, (const float*)part, mats,
                   ksplit, M, N, mode, y, ldy);
}
}  // namespace

int hbk_dense_setup(hb_ctx* ctx) {
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(dense_stream_kernel<HB_FMT_NVFP4>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dense_smem(HB_FMT_NVFP4)));
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(dense_stream_kernel<HB_FMT_LB2_G64>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dense_smem(HB_FMT_LB2_G64)));
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(dense_stream_kernel<HB_FMT_LB3_G64>), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dense_smem(HB_FMT_LB3_G64)));
  return HB_OK;
}

extern "C" {

size_t hb_dense_gemv_ws_bytes(int fmt, int N, int K, int n_mats) {
  if (K <= 0 || N <= 0 || K % kDSlice || n_mats < 1 || n_mats > 2) return 0;
  return al256((size_t)n_mats * dense_ksplit(fmt, K) * 8 * N * 4);
}

int hb_dense_gemv(hb_ctx* ctx, const hb_qmat* W, const void* x, int ldx, int M, void* yb, float* yf, int ldy, void* ws, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  int r = check_mat(ctx, W, "dense_gemv");
  if (r) return r;
  HB_REQUIRE(ctx, x && ((yb != nullptr) != (yf != nullptr)), HB_ERR_INVALID, "dense_gemv: x NULL, or not exactly one of yb / yf given");
  HB_REQUIRE(ctx, hb_aligned(x, 16) && ldx % 8 == 0, HB_ERR_INVALID, "dense_gemv: x must be 16-byte aligned with ldx a multiple of 8");
  HB_REQUIRE(ctx, M >= 1 && M <= 16 && ldx >= W->K && ldy >= W->N, HB_ERR_UNSUPPORTED, "dense_gemv: M=%d (1..16) ldx=%d ldy=%d", M, ldx, ldy);
  HB_REQUIRE(ctx, ws && hb_aligned(ws, 256), HB_ERR_WORKSPACE, "dense_gemv: ws NULL or not 256-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  for (int m0 = 0; m0 < M; m0 += 8) {                         // passes of ≤ 8 rows: per-row arithmetic does not depend on the batch
    const int mm = M - m0 < 8 ? M - m0 : 8;
    const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)m0 * ldx;
    void* yp = yf ? static_cast<void*>(yf + (size_t)m0 * ldy) : static_cast<void*>(reinterpret_cast<__nv_bfloat16*>(yb) + (size_t)m0 * ldy);
    if ((r = dense_pass(ctx, W, nullptr, xp, ldx, mm, yf ? 0 : 1, yp, ldy, ws, st))) return r;
  }
  return HB_OK;
}

int hb_dense_gemv_gu(hb_ctx* ctx, const hb_qmat* G, const hb_qmat* U, const void* x, int ldx, int M, void* act, int lda, void* ws, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  int r = check_mat(ctx, G, "dense_gemv_gu");
  if (!r) r = check_mat(ctx, U, "dense_gemv_gu");
  if (r) return r;
  HB_REQUIRE(ctx, G->fmt == U->fmt && G->N == U->N && G->K == U->K, HB_ERR_INVALID, "dense_gemv_gu: gate and up must share format and shape");
  HB_REQUIRE(ctx, x && hb_aligned(x, 16) && ldx % 8 == 0, HB_ERR_INVALID, "dense_gemv_gu: x must be 16-byte aligned with ldx a multiple of 8");
  HB_REQUIRE(ctx, x && act && M >= 1 && M <= 16 && ldx >= G->K && lda >= G->N, HB_ERR_UNSUPPORTED, "dense_gemv_gu: M=%d (1..16) ldx=%d lda=%d", M, ldx, lda);
  HB_REQUIRE(ctx, ws && hb_aligned(ws, 256), HB_ERR_WORKSPACE, "dense_gemv_gu: ws NULL or not 256-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  for (int m0 = 0; m0 < M; m0 += 8) {
    const int mm = M - m0 < 8 ? M - m0 : 8;
    if ((r = dense_pass(ctx, G, U, reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)m0 * ldx, ldx, mm, 2,
                        reinterpret_cast<__nv_bfloat16*>(act) + (size_t)m0 * lda, lda, ws, st))) return r;
  }
  return HB_OK;
}

int hb_lb_dequant(hb_ctx* ctx, const hb_qmat* W, void* out_bf16, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  HB_REQUIRE(ctx, W && W->w && W->s && W->zp && out_bf16, HB_ERR_INVALID, "lb_dequant: NULL argument");
  HB_REQUIRE(ctx, (W->fmt == HB_FMT_LB3_G64 || W->fmt == HB_FMT_LB2_G64) && W->N > 0 && W->K > 0 && W->K % 64 == 0, HB_ERR_UNSUPPORTED,
             "lb_dequant: format %d N=%d K=%d", W->fmt, W->N, W->K);
  const size_t n = (size_t)W->N * W->K;
  size_t blocks = (n + 255) / 256, cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  return hb_launch(ctx, "lb_dequant", false, lb_dequant_kernel, dim3((unsigned)blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                   W->fmt == HB_FMT_LB3_G64 ? 3 : 2, W->w, W->fmt == HB_FMT_LB3_G64 ? W->w + (size_t)W->N * (W->K / 4) : (const uint8_t*)nullptr,
                   reinterpret_cast<const __half*>(W->s), reinterpret_cast<const __half*>(W->zp), W->N, W->K, reinterpret_cast<__nv_bfloat16*>(out_bf16));
}

}  // extern "C"
