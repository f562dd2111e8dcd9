// Dense decode GEMV for one weight matrix, M ≤ 8 activation rows per pass: NVFP4 and the 3-/2-bit group-64 formats
// (hb_qmat).  HBM-bound: every weight byte is read once, decoded in registers and fed to m16n8k16 tensor-core tiles whose 8
// columns are the activation rows (fp32 accumulation).
//
//   prep     the activation rows become f16 B fragments in the order the tiles consume them (per-row power-of-two rescale so
//            bf16 outliers cannot overflow f16), plus, for the low-bit formats, two sums per 64-column group (see below)
//   stream   grid = (128-row tiles, K splits).  A CTA keeps the B fragments of its K range in shared memory; each of its 8
//            warps owns 16 weight rows and streams them through a private 4-stage cp.async ring, 256 columns per stage
//   reduce   fixed-order sum over the K splits, output conversion, or the fused SiLU·up activation of the gate/up pair
//
// Low-bit decode without shifts or subtractions per element: a 2-bit field left at bit 2j of an f16 mantissa under exponent
// 0x64 reads as 1024 + q·4^j, a 1-bit field at bit j as 1024 + b·2^j.  The B fragments carry the matching 4^-j / 2^-j factors
// (exact), and the 1024·Σx' offset is removed per group together with the zero-point:  y += s·(tile − zp·S0 − S1),
// S0 = Σ x, S1 = 1024·Σ x'.  One logic instruction per element pair, scales and zero-points applied in fp32.
#include "moe_stream.cuh"

namespace hb {

constexpr int kDSlice = 256;            // columns per pipeline stage
constexpr int kDWarps = 8;              // consumer warps per CTA, 16 weight rows each
constexpr int kDRows = kDWarps * 16;    // rows per CTA tile
__host__ __device__ constexpr int dense_stages(int fmt) { return fmt == HB_FMT_NVFP4 ? 3 : 4; }
// K range of one CTA (slices of 256 columns whose B fragments sit in shared memory): sized for two CTAs per SM
__host__ __device__ constexpr int dense_max_slices(int fmt) { return fmt == HB_FMT_LB3_G64 ? 4 : 8; }

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

struct DenseWs {
  uint32_t* xb;      // [slices][planes][1024] B fragments: index ((r >> 2) * 32 + lane) * 4 + (r & 3), r = register 0..31 of the slice
  float2* sums;      // [slices][4 groups][8 rows] (S0, S1), low-bit formats
  unsigned int* amax; // [8] max |x| of each row as bf16 bits, then [8..] the strip counters of the K splits
  float* part;       // [mats][K splits][8][N] fp32 partial sums
};
inline DenseWs dense_carve(void* ws, int slices, int planes, int mats, int ksplit, int N) {
  uint8_t* p = reinterpret_cast<uint8_t*>(ws);
  DenseWs w;
  w.xb = reinterpret_cast<uint32_t*>(p); p += al256((size_t)slices * planes * 4096);
  w.sums = reinterpret_cast<float2*>(p); p += al256((size_t)slices * 256);
  w.amax = reinterpret_cast<unsigned int*>(p); p += 256;
  w.part = reinterpret_cast<float*>(p);
  (void)mats; (void)ksplit; (void)N;
  return w;
}

// ------------------------------------------------------------------------------------------------ prep
// max |x| of each row as bf16 bits (integer order = magnitude order), over a grid of (row, column chunk) blocks; also zeroes
// the strip counters of the stream kernel.  amax must be zero on entry (the reduce kernel of the previous pass leaves it so;
// the first pass clears it with a memset).
__global__ void dense_amax_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int M, int K, unsigned int* __restrict__ amax, int* __restrict__ counters,
                                  int n_counters) {
  griddep_wait();
  const int m = blockIdx.x;
  if (blockIdx.x == 0 && blockIdx.y == 0) for (int i = threadIdx.x; i < n_counters; i += blockDim.x) counters[i] = 0;
  if (m >= M) return;
  unsigned int am = 0;
  const uint4* row = reinterpret_cast<const uint4*>(x + (size_t)m * ldx);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < K / 8; i += gridDim.y * blockDim.x) {
    const uint4 v = __ldg(row + i);
    const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { am = max(am, w[j] & 0x7fffu); am = max(am, (w[j] >> 16) & 0x7fffu); }
  }
  for (int o = 16; o > 0; o >>= 1) am = max(am, __shfl_xor_sync(0xffffffffu, am, o));
  if ((threadIdx.x & 31) == 0 && am) atomicMax(&amax[m], am);
}
// rescale factor of a row from its max magnitude: the max lands in [2^12, 2^13), so 4·x (high-bit plane) stays inside f16
__device__ __forceinline__ float dense_fac(unsigned int am) {
  int e = (int)(am >> 7);
  e = min(max(e, 27), 254);
  return __int_as_float((uint32_t)(127 + 12 + 127 - e) << 23);
}
__device__ __forceinline__ float dense_inv(unsigned int am) {
  int e = (int)(am >> 7);
  e = min(max(e, 27), 254);
  return __int_as_float((uint32_t)(e - 12) << 23);
}

// element (within the slice) and position factor of half `hi` (0 / 1) of B register r of lane (tok, t), plane p
__device__ __forceinline__ void dense_b_elem(int fmt, int p, int r, int t, int hi, int* elem, float* scale) {
  if (fmt == HB_FMT_NVFP4) { *elem = 64 * t + 2 * r + hi; *scale = 1.f; return; }
  const int gq = r >> 3, i = (r >> 1) & 3, h = r & 1, pr = 2 * i + h;      // group of the slice, tile of the group, pair of the lane's word
  if (p == 0) {                                              // 2-bit plane: the lane's word = columns [16t, 16t+16) of the group
    *elem = 64 * gq + 16 * t + pr + 8 * hi;
    const int j = pr < 5 ? pr : pr - 5;
    *scale = 1.f / (float)(1 << (2 * j));
  } else {                                                   // 1-bit plane: lanes 0,1 share word 0, lanes 2,3 word 1; odd lanes take its upper bytes
    *elem = 64 * gq + 32 * (t >> 1) + 8 * (t & 1) + pr + 16 * hi;
    *scale = 4.f / (float)(1 << pr);
  }
}

// one block per slice: B fragments (both planes) and the group sums
__global__ void __launch_bounds__(256) dense_prep_kernel(int fmt, const __nv_bfloat16* __restrict__ x, int ldx, int M, const unsigned int* __restrict__ amax,
                                                         uint32_t* __restrict__ xb, float2* __restrict__ sums) {
  griddep_wait();
  const int sl = blockIdx.x, planes = dense_fmt(fmt).planes;
  for (int p = 0; p < planes; ++p)
    for (int idx = threadIdx.x; idx < 1024; idx += blockDim.x) {
      const int r = idx >> 5, lane = idx & 31, tok = lane >> 2, t = lane & 3;
      float v[2] = {0.f, 0.f};
      int e0, e1; float sc0, sc1;
      dense_b_elem(fmt, p, r, t, 0, &e0, &sc0);
      dense_b_elem(fmt, p, r, t, 1, &e1, &sc1);
      if (tok < M) {
        const float f = dense_fac(amax[tok]);
        v[0] = __bfloat162float(x[(size_t)tok * ldx + (size_t)sl * kDSlice + e0]) * f * sc0;
        v[1] = __bfloat162float(x[(size_t)tok * ldx + (size_t)sl * kDSlice + e1]) * f * sc1;
      }
      const __half2 hh = __floats2half2_rn(v[0], v[1]);
      xb[((size_t)sl * planes + p) * 1024 + ((r >> 2) * 32 + lane) * 4 + (r & 3)] = *reinterpret_cast<const uint32_t*>(&hh);
    }
  if (fmt == HB_FMT_NVFP4) return;
  if (threadIdx.x < 32) {                                    // (group, row): S0 = Σ x (rescaled, as f16), S1 = 1024·Σ x' — serial, fixed order
    const int gq = threadIdx.x >> 3, tok = threadIdx.x & 7;
    float s0 = 0.f, s1 = 0.f;
    if (tok < M) {
      const float f = dense_fac(amax[tok]);
      for (int k = 0; k < 64; ++k) {
        const float xn = __bfloat162float(x[(size_t)tok * ldx + (size_t)sl * kDSlice + 64 * gq + k]) * f;
        s0 += __half2float(__float2half_rn(xn));
        const int pr = k & 7, j = pr < 5 ? pr : pr - 5;      // the factors dense_b_elem gives column k of a group
        s1 += __half2float(__float2half_rn(xn / (float)(1 << (2 * j))));
        if (planes > 1) s1 += __half2float(__float2half_rn(xn * 4.f / (float)(1 << pr)));
      }
    }
    sums[(size_t)sl * 32 + gq * 8 + tok] = make_float2(s0, 1024.f * s1);
  }
}

// ------------------------------------------------------------------------------------------------ stream
struct DenseMat { const uint8_t* w; const uint8_t* wh; const uint8_t* s; const uint8_t* zp; float g; };
struct DenseArgs {
  DenseMat mat[2]; int n_mats;
  int N, K, M, ksplit, slices;            // slices = K / 256
  const uint32_t* xb; const float2* sums; const unsigned int* amax;
  int* counters;                          // [ksplit] next unclaimed strip of each K split (zeroed by the amax kernel)
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

// Persistent CTAs: blockIdx.y = K split (the CTA keeps that range's B fragments in shared memory for its whole life),
// blockIdx.x = one of the CTAs sharing the split.  Work unit of a warp = a strip of 16 weight rows of one matrix over the
// split's columns, claimed from the split's counter; the warp's cp.async ring runs on across strip boundaries.
template <int FMT>
__global__ void __launch_bounds__((kDWarps) * 32, 2) dense_stream_kernel(DenseArgs a) {
  constexpr DenseFmt F = dense_fmt(FMT);
  constexpr int STG = dense_stage_bytes(FMT), NST = dense_stages(FMT), MAXSL = dense_max_slices(FMT);
  extern __shared__ __align__(128) uint8_t dsm[];
  uint4* xb_s = reinterpret_cast<uint4*>(dsm);                                            // [MAXSL][planes][256] uint4
  float4* sums_s = reinterpret_cast<float4*>(dsm + (size_t)MAXSL * F.planes * 4096);      // [MAXSL][4 groups][4] float4 = rows (2i, 2i+1)
  int* claimed_s = reinterpret_cast<int*>(dsm + (size_t)MAXSL * F.planes * 4096 + (size_t)MAXSL * 256);   // [warps][8]
  uint8_t* rings = reinterpret_cast<uint8_t*>(claimed_s) + 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int ks = blockIdx.y;
  const int sl0 = (int)((long long)a.slices * ks / a.ksplit), sl1 = (int)((long long)a.slices * (ks + 1) / a.ksplit), nsl = sl1 - sl0;
  griddep_wait();
  {                                                                 // B fragments (and group sums) of this K range → shared memory
    const uint4* src = reinterpret_cast<const uint4*>(a.xb) + (size_t)sl0 * F.planes * 256;
    for (int i = threadIdx.x; i < nsl * F.planes * 256; i += blockDim.x) xb_s[i] = __ldg(src + i);
    if (FMT != HB_FMT_NVFP4) {
      const float4* ss = reinterpret_cast<const float4*>(a.sums) + (size_t)sl0 * 16;
      for (int i = threadIdx.x; i < nsl * 16; i += blockDim.x) sums_s[i] = __ldg(ss + i);
    }
  }
  __syncthreads();
  griddep_launch();
  const int strips_per_mat = (a.N + 15) / 16, n_strips = strips_per_mat * a.n_mats;
  uint8_t* ring = rings + (size_t)warp * NST * STG;
  int* claimed = claimed_s + warp * 8;
  const int K = a.K;
  auto claim = [&]() -> int {
    int v = 0;
    if (lane == 0) v = atomicAdd(&a.counters[ks], 1);
    return __shfl_sync(0xffffffffu, v, 0);
  };
  auto issue = [&](int strip, int sl, int stage) {                  // slice sl (absolute) of a strip → ring stage
    const DenseMat& W = a.mat[strip >= strips_per_mat ? 1 : 0];
    const int n0 = (strip >= strips_per_mat ? strip - strips_per_mat : strip) * 16;
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
  // issue cursor: ordinal of the strip being fetched (io), its slice (is); compute cursor (co, cs) follows NST-1 slices behind
  int io = 0, is = 0, istage = 0, istrip = claim();
  if (lane == 0) claimed[0] = istrip;
  auto issue_next = [&]() {
    if (istrip < n_strips) {
      issue(istrip, sl0 + is, istage);
      if (++is == nsl) { is = 0; ++io; istrip = claim(); if (lane == 0) claimed[io & 7] = istrip; }
      if (++istage == NST) istage = 0;
    }
    cp_async_commit();                                              // always commit: the group count stays in step with the slice count
  };
  for (int i = 0; i < NST - 1; ++i) issue_next();
  __syncwarp();
  int co = 0, cs = 0, cstage = 0;
  float total[4] = {0.f, 0.f, 0.f, 0.f};
  for (;;) {
    const int strip = claimed[co & 7];
    if (strip >= n_strips) break;
    issue_next();
    cp_async_wait<NST - 1>();
    __syncwarp();
    const uint8_t* st = ring + (size_t)cstage * STG;
    const uint4* xb_i = xb_s + (size_t)cs * F.planes * 256;
    if (FMT == HB_FMT_NVFP4) {
      uint32_t b[32];
#pragma unroll
      for (int q = 0; q < 8; ++q) { const uint4 v = xb_i[q * 32 + lane]; b[4 * q] = v.x; b[4 * q + 1] = v.y; b[4 * q + 2] = v.z; b[4 * q + 3] = v.w; }
      float acc[4];
      warp_slice_mma(st + g * F.pitch_w + 32 * t, st + (g + 8) * F.pitch_w + 32 * t, st + 16 * F.pitch_w + g * 16 + 4 * t,
                     st + 16 * F.pitch_w + (g + 8) * 16 + 4 * t, b, acc, nullptr);
#pragma unroll
      for (int c = 0; c < 4; ++c) total[c] += acc[c];
    } else {
      const uint8_t* sz = st + 16 * (F.pitch_w + F.pitch_h);
      const uint4 szA = *reinterpret_cast<const uint4*>(sz + g * 16), szB = *reinterpret_cast<const uint4*>(sz + (g + 8) * 16);
      const uint32_t szAw[4] = {szA.x, szA.y, szA.z, szA.w}, szBw[4] = {szB.x, szB.y, szB.z, szB.w};   // {s01, s23, zp01, zp23} as f16 pairs
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
        const float4 su = sums_s[(size_t)cs * 16 + gq * 4 + t];     // (S0, S1) of rows 2t, 2t+1
        const __half2 sA2 = *reinterpret_cast<const __half2*>(&szAw[gq >> 1]), zA2 = *reinterpret_cast<const __half2*>(&szAw[2 + (gq >> 1)]);
        const __half2 sB2 = *reinterpret_cast<const __half2*>(&szBw[gq >> 1]), zB2 = *reinterpret_cast<const __half2*>(&szBw[2 + (gq >> 1)]);
        const float sA = (gq & 1) ? __high2float(sA2) : __low2float(sA2), zA = (gq & 1) ? __high2float(zA2) : __low2float(zA2);
        const float sB = (gq & 1) ? __high2float(sB2) : __low2float(sB2), zB = (gq & 1) ? __high2float(zB2) : __low2float(zB2);
        total[0] = fmaf(sA, tmp[0] - fmaf(zA, su.x, su.y), total[0]);
        total[1] = fmaf(sA, tmp[1] - fmaf(zA, su.z, su.w), total[1]);
        total[2] = fmaf(sB, tmp[2] - fmaf(zB, su.x, su.y), total[2]);
        total[3] = fmaf(sB, tmp[3] - fmaf(zB, su.z, su.w), total[3]);
      }
    }
    __syncwarp();
    if (++cstage == NST) cstage = 0;
    if (++cs == nsl) {                                              // strip finished: its partial sums of this K split → [mat][ks][row 0..7][N]
      const int mat_i = strip >= strips_per_mat ? 1 : 0, n0 = (mat_i ? strip - strips_per_mat : strip) * 16;
      float* part = a.part + ((size_t)mat_i * a.ksplit + ks) * 8 * a.N;
      const float gsc = FMT == HB_FMT_NVFP4 ? a.mat[mat_i].g : 1.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int tok = 2 * t + (c & 1), n = n0 + g + (c >> 1) * 8;
        if (tok < a.M && n < a.N) part[(size_t)tok * a.N + n] = total[c] * dense_inv(a.amax[tok]) * gsc;
        total[c] = 0.f;
      }
      cs = 0; ++co;
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------------------ reduce
// mode 0: y fp32; 1: y bf16; 2: act = bf16( bf16(silu(bf16 g)) · bf16 u ) from the two matrices' sums
__global__ void dense_reduce_kernel(const float* __restrict__ part, int n_mats, int ksplit, int M, int N, int mode, void* __restrict__ y, int ldy) {
  griddep_wait();
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
  return (size_t)dense_max_slices(fmt) * F.planes * 4096 + (size_t)dense_max_slices(fmt) * 256 + 256 + (size_t)kDWarps * dense_stages(fmt) * dense_stage_bytes(fmt);
}
int check_mat(hb_ctx* ctx, const hb_qmat* W, const char* fn) {
  HB_REQUIRE(ctx, W && W->w && W->s, HB_ERR_INVALID, "%s: NULL matrix", fn);
  HB_REQUIRE(ctx, W->fmt == HB_FMT_NVFP4 || W->fmt == HB_FMT_LB3_G64 || W->fmt == HB_FMT_LB2_G64, HB_ERR_INVALID, "%s: unknown format %d", fn, W->fmt);
  HB_REQUIRE(ctx, W->N > 0 && W->K > 0 && W->K % kDSlice == 0, HB_ERR_UNSUPPORTED, "%s: N=%d K=%d (K must be a multiple of %d)", fn, W->N, W->K, kDSlice);
  HB_REQUIRE(ctx, W->K / kDSlice <= 56 * dense_max_slices(W->fmt), HB_ERR_UNSUPPORTED, "%s: K=%d beyond the %d K splits the workspace header holds", fn, W->K, 56);
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
// one pass of ≤ 8 rows: prep → stream → reduce
int dense_pass(hb_ctx* ctx, const hb_qmat* A, const hb_qmat* B2, const void* x, int ldx, int M, int mode, void* y, int ldy, void* ws, cudaStream_t st) {
  const int fmt = A->fmt, N = A->N, K = A->K, slices = K / kDSlice, planes = dense_fmt(fmt).planes, ksplit = dense_ksplit(fmt, K), mats = B2 ? 2 : 1;
  DenseWs w = dense_carve(ws, slices, planes, mats, ksplit, N);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  int* counters = reinterpret_cast<int*>(w.amax + 8);
  cudaError_t e = cudaMemsetAsync(w.amax, 0, 32, st);
  if (e != cudaSuccess) return hb_fail(ctx, HB_ERR_CUDA, "memset amax: %s", cudaGetErrorString(e));
  int r = hb_launch(ctx, "dense_amax", false, dense_amax_kernel, dim3(8, 16), dim3(256), 0, st, xb, ldx, M, K, w.amax, counters, ksplit);
  if (r) return r;
  if ((r = hb_launch(ctx, "dense_prep", true, dense_prep_kernel, dim3(slices), dim3(256), 0, st, fmt, xb, ldx, M, (const unsigned int*)w.amax, w.xb, w.sums))) return r;
  DenseArgs a{};
  a.mat[0] = to_mat(A); if (B2) a.mat[1] = to_mat(B2);
  a.n_mats = mats; a.N = N; a.K = K; a.M = M; a.ksplit = ksplit; a.slices = slices;
  a.xb = w.xb; a.sums = w.sums; a.amax = w.amax; a.counters = counters; a.part = w.part;
  int per_split = (2 * ctx->sm_count) / ksplit;                    // two CTAs per SM in all, shared out over the K splits
  const int strips = ((N + 15) / 16) * mats, max_useful = (strips + kDWarps - 1) / kDWarps;
  if (per_split < 1) per_split = 1;
  if (per_split > max_useful) per_split = max_useful;
  const dim3 grid(per_split, ksplit, 1);
  auto fn = fmt == HB_FMT_NVFP4 ? dense_stream_kernel<HB_FMT_NVFP4> : fmt == HB_FMT_LB2_G64 ? dense_stream_kernel<HB_FMT_LB2_G64> : dense_stream_kernel<HB_FMT_LB3_G64>;
  if ((r = hb_launch(ctx, fmt == HB_FMT_NVFP4 ? "dense_stream_nvfp4" : fmt == HB_FMT_LB2_G64 ? "dense_stream_lb2" : "dense_stream_lb3", true, fn, grid,
                     dim3(kDWarps * 32), dense_smem(fmt), st, a))) return r;
  return hb_launch(ctx, "dense_reduce", true, dense_reduce_kernel, dim3((unsigned)(((size_t)M * N + 255) / 256)), dim3(256), 0, st, (const float*)w.part, mats,
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
  const int slices = K / kDSlice;
  return al256((size_t)slices * dense_fmt(fmt).planes * 4096) + al256((size_t)slices * 256) + 256 + al256((size_t)n_mats * dense_ksplit(fmt, K) * 8 * N * 4);
}

int hb_dense_gemv(hb_ctx* ctx, const hb_qmat* W, const void* x, int ldx, int M, void* yb, float* yf, int ldy, void* ws, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  int r = check_mat(ctx, W, "dense_gemv");
  if (r) return r;
  HB_REQUIRE(ctx, x && ((yb != nullptr) != (yf != nullptr)), HB_ERR_INVALID, "dense_gemv: x NULL, or not exactly one of yb / yf given");
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
