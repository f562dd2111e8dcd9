// NVFP4 matrix kernels: dequantise to bf16, small-batch GEMV for one matrix, fp32 → NVFP4 weight quantisation and the
// per-row activation quantisation of the W4A4 prefill path.  Formats: e2m1 nibbles [N, K/2] (low nibble = even column),
// one e4m3 scale per 16 columns [N, K/16], one fp32 scale per tensor (multiplies).
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "hb_common.cuh"
#include "hb_kernels.h"

namespace hb {

// ---- dequant: out[n, k] = bf16( E2M1[nib] * (e4m3(s[n, k/16]) * g) ) — the reference's expression order, so bit-exact
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ W, const uint8_t* __restrict__ S, float g, const float* __restrict__ g_dev,
                                     size_t n_blocks16, __nv_bfloat16* __restrict__ out) {
  if (g_dev) g = __ldg(g_dev);                          // the global sits on the device (inside an expert record)
  // one thread per 16-column block: 8 weight bytes in, 32 bytes out
  for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks16; b += (size_t)gridDim.x * blockDim.x) {
    const float s = __fmul_rn(e4m3_to_f32(S[b]), g);
    const uint2 q = *reinterpret_cast<const uint2*>(W + b * 8);
    const uint32_t w[2] = {q.x, q.y};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t byte = (w[j >> 2] >> (8 * (j & 3))) & 0xFF;
      const __nv_bfloat16 lo = __float2bfloat16(__fmul_rn(e2m1_to_f32(byte & 15), s));
      const __nv_bfloat16 hi = __float2bfloat16(__fmul_rn(e2m1_to_f32(byte >> 4), s));
      o[j] = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + b * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// ---- GEMV for one matrix, M ≤ 16 activation rows: one warp per weight row, lanes stride over K in 32-column pieces.
// Per 16-column block the partial dot is formed in fp32 and then multiplied by the block scale (scale never rounded into the
// weight); the warp sum is a 16,8,4,2,1 butterfly; the tensor scale multiplies last.
template <int MT>
__global__ void __launch_bounds__(256) nvfp4_gemv_kernel(const uint8_t* __restrict__ W, const uint8_t* __restrict__ S, float g, int N, int K,
                                                         const __nv_bfloat16* __restrict__ x, int ldx, int M, float* __restrict__ y, int ldy) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const uint8_t* wr = W + (size_t)n * (K / 2);
  const uint8_t* sr = S + (size_t)n * (K / 16);
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  for (int k0 = lane * 32; k0 < K; k0 += 32 * 32) {
    const uint4 q = *reinterpret_cast<const uint4*>(wr + k0 / 2);
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    const uint16_t s2 = *reinterpret_cast<const uint16_t*>(sr + k0 / 16);
    const float sc[2] = {e4m3_to_f32(s2 & 0xFF), e4m3_to_f32(s2 >> 8)};
    float wv[32];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t byte = (qw[j >> 2] >> (8 * (j & 3))) & 0xFF;
      wv[2 * j] = e2m1_to_f32(byte & 15); wv[2 * j + 1] = e2m1_to_f32(byte >> 4);
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < M) {
        const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k0);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float d = 0.f;
#pragma unroll
          for (int v = 0; v < 2; ++v) {
            const uint4 xv = __ldg(xp + h * 2 + v);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              d = fmaf(__uint_as_float(xw[j] << 16), wv[h * 16 + v * 8 + 2 * j], d);
              d = fmaf(__uint_as_float(xw[j] & 0xffff0000u), wv[h * 16 + v * 8 + 2 * j + 1], d);
            }
          }
          acc[m] = fmaf(d, sc[h], acc[m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float v = acc[m];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && m < M) y[(size_t)m * ldy + n] = v * g;
  }
}

// ---- fp32 → NVFP4 (the device rule of the reference's requant kernels: one global scale from the tensor's largest magnitude, block
// scale = e4m3(block amax · gs / 6), code = e2m1(v · gs / scale); no per-block scale search).  Four lanes share a block of 16: a lane
// loads ONE float4 (a warp reads 512 contiguous bytes), the block's amax is two shuffles away, the four lanes work out the same scale
// and each turns its own four values into 16 bits of codes (a warp writes 64 contiguous bytes).
// The source of four consecutive values: an fp32 matrix, or an FP8 (e4m3) matrix with one fp32 scale per row (value = fp8 · row scale,
// the reference's FP8ROW weights).
struct SrcF32 {
  const float4* w4;
  __device__ __forceinline__ float4 load(size_t i) const { return __ldg(w4 + i); }
};
struct SrcFp8Row {
  const uint32_t* w8; const float* row_scale; int K4;                       // K4 = K / 4 groups per row
  __device__ __forceinline__ float4 load(size_t i) const {
    const uint32_t u = __ldg(w8 + i);
    const float sr = __ldg(row_scale + i / (size_t)K4);
    return make_float4(__fmul_rn(e4m3_to_f32(u & 0xffu), sr), __fmul_rn(e4m3_to_f32((u >> 8) & 0xffu), sr), __fmul_rn(e4m3_to_f32((u >> 16) & 0xffu), sr),
                       __fmul_rn(e4m3_to_f32(u >> 24), sr));
  }
};
template <class SRC>
__global__ void __launch_bounds__(256) tensor_absmax_kernel(const SRC src, size_t n4, float* __restrict__ amax) {
  __shared__ float part[8];
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (size_t)gridDim.x * 256) {
    const float4 v = src.load(i);
    m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
  }
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 8) {
    m = part[threadIdx.x];
    for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffu, m, o));
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(m));   // one atomic per block; magnitudes order like their bits
  }
}
template <class SRC>
__global__ void __launch_bounds__(256) nvfp4_encode_kernel(const SRC src, size_t n4, const float* __restrict__ amax, uint16_t* __restrict__ q16,
                                                           uint8_t* __restrict__ s, float* __restrict__ g_mul) {
  const float am = *amax;
  const bool live = am > 0.f;
  const float gs = live ? __fdiv_rn(448.f * 6.f, am) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *g_mul = live ? __fdiv_rn(am, 448.f * 6.f) : 1.f;
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;                   // four values per thread; n4 is a multiple of 4, whole quads stay in range together
  if (i >= n4) return;
  const float4 v = src.load(i);
  float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  const unsigned quad = 0xfu << (threadIdx.x & 28);
  m = fmaxf(m, __shfl_xor_sync(quad, m, 1));
  m = fmaxf(m, __shfl_xor_sync(quad, m, 2));
  const __nv_fp8_storage_t sc = __nv_cvt_float_to_fp8(__fdiv_rn(__fmul_rn(m, gs), 6.f), __NV_SATFINITE, __NV_E4M3);
  const float sd = e4m3_to_f32(sc);
  if ((threadIdx.x & 3) == 0) s[i >> 2] = (uint8_t)sc;
  const float f[4] = {v.x, v.y, v.z, v.w};
  uint32_t c = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (sd > 0.f) c |= ((uint32_t)__nv_cvt_float_to_fp4(__fdiv_rn(__fmul_rn(f[j], gs), sd), __NV_E2M1, cudaRoundNearest) & 0xFu) << (4 * j);
  q16[i] = (uint16_t)c;
}

// ---- per-row dynamic NVFP4 quantisation of bf16 rows (the rule of the reference's activation quantiser: gx = amax / (6·448), block
// scale = e4m3((block amax / 6) / gx), code = e2m1(v · (1/gx) / scale)), written to any number of destination rows at once.
// A CTA takes one row at a time: the row is staged in shared memory once, the quantised row (codes, scales) is built there, and then
// copied to each place it is wanted — with a destination list this is quantise + gather-into-expert-order in one pass (a row is
// quantised once however many experts it goes to, and the quantised row never makes a round trip through global memory).
//   dest == nullptr: row r goes to slot r.  Else: row r goes to slots dest[r·nd + j], j < nd, negative entries skipped.
constexpr int QS_THREADS = 256;
// TG threads work on a row together (256 for long rows, 64 for short ones: 256 / TG rows are then in progress in a CTA, each group
// with its own staging buffers and its own named barrier).
template <int TG>
__global__ void __launch_bounds__(QS_THREADS) quant_rows_scatter_kernel(const __nv_bfloat16* __restrict__ x, int ld, int n_cap, const int* __restrict__ n_dev, int Kd,
                                                                        const int* __restrict__ dest, int nd, uint8_t* __restrict__ q, uint8_t* __restrict__ s,
                                                                        float* __restrict__ g) {
  constexpr int NG = QS_THREADS / TG;
  extern __shared__ __align__(16) uint8_t qs_sm[];
  __shared__ float red[NG][TG / 32];
  __shared__ int dst_s[NG][32];
  const int grp = threadIdx.x / TG, t = threadIdx.x % TG, lane = t & 31, wp = t >> 5, bar = 1 + grp;
  const size_t stage = (size_t)Kd * 2 + Kd / 2 + (Kd / 16 + 15) / 16 * 16;
  uint32_t* row32 = reinterpret_cast<uint32_t*>(qs_sm + grp * stage);         // Kd bf16 values
  uint8_t* codes = reinterpret_cast<uint8_t*>(row32) + (size_t)Kd * 2;       // Kd / 2 bytes
  uint8_t* scl = codes + Kd / 2;                                             // Kd / 16 bytes
  const int nb = Kd / 16;
  const int n = n_dev ? min(n_cap, *n_dev) : n_cap;                           // a row count known only on the device (rows beyond it are not touched)
  for (int r = blockIdx.x * NG + grp; r < n; r += gridDim.x * NG) {
    const __nv_bfloat16* xr = x + (size_t)r * ld;
    if (dest) {                                                               // a row nobody wants (all its experts live elsewhere) is not even read
      if (t < nd) dst_s[grp][t] = dest[(size_t)r * nd + t];
      named_bar_sync(bar, TG);
      bool wanted = false;
      for (int j = 0; j < nd; ++j) wanted |= dst_s[grp][j] >= 0;
      if (!wanted) { named_bar_sync(bar, TG); continue; }
    }
    float a = 0.f;
    if ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
      for (int i = t; i < Kd / 8; i += TG) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(xr) + i);
        reinterpret_cast<uint4*>(row32)[i] = u;
        const uint32_t wv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) a = fmaxf(a, fmaxf(fabsf(__uint_as_float(wv[j] << 16)), fabsf(__uint_as_float(wv[j] & 0xffff0000u))));
      }
    } else {
      for (int i = t; i < Kd; i += TG) {
        const __nv_bfloat16 v = xr[i];
        reinterpret_cast<__nv_bfloat16*>(row32)[i] = v;
        a = fmaxf(a, fabsf(__bfloat162float(v)));
      }
    }
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    if (lane == 0) red[grp][wp] = a;
    named_bar_sync(bar, TG);
#pragma unroll
    for (int i = 0; i < TG / 32; ++i) a = fmaxf(a, red[grp][i]);
    const float gx = a > 0.f ? __fdiv_rn(a, 6.f * 448.f) : 1.f, inv = __fdiv_rn(1.f, gx);
    for (int b = t; b < nb; b += TG) {
      float v[16], ab = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t u = row32[b * 8 + j];
        v[2 * j] = __uint_as_float(u << 16); v[2 * j + 1] = __uint_as_float(u & 0xffff0000u);
        ab = fmaxf(ab, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
      }
      const __nv_fp8_storage_t se = __nv_cvt_float_to_fp8(__fmul_rn(__fdiv_rn(ab, 6.f), inv), __NV_SATFINITE, __NV_E4M3);
      const float sv = e4m3_to_f32(se), f = sv > 0.f ? __fdiv_rn(inv, sv) : 0.f;
      uint32_t lo = 0u, hi = 0u;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        lo |= ((uint32_t)__nv_cvt_float_to_fp4(__fmul_rn(v[j], f), __NV_E2M1, cudaRoundNearest) & 0xFu) << (4 * j);
        hi |= ((uint32_t)__nv_cvt_float_to_fp4(__fmul_rn(v[8 + j], f), __NV_E2M1, cudaRoundNearest) & 0xFu) << (4 * j);
      }
      reinterpret_cast<uint2*>(codes)[b] = make_uint2(lo, hi);
      scl[b] = (uint8_t)se;
    }
    named_bar_sync(bar, TG);
    // the quantised row leaves for its destinations: 16-byte pieces when the row length allows (Kd a multiple of 256), else bytes
    const int ndest = dest ? nd : 1;
    for (int j = 0; j < ndest; ++j) {
      const int slot = dest ? dst_s[grp][j] : r;
      if (slot < 0) continue;
      uint8_t* qd = q + (size_t)slot * (Kd / 2);
      uint8_t* sd = s + (size_t)slot * nb;
      if (Kd % 256 == 0 && ((reinterpret_cast<uintptr_t>(qd) | reinterpret_cast<uintptr_t>(sd)) & 15) == 0) {
        for (int i = t; i < Kd / 32 + Kd / 256; i += TG) {
          if (i < Kd / 32) reinterpret_cast<uint4*>(qd)[i] = reinterpret_cast<const uint4*>(codes)[i];
          else reinterpret_cast<uint4*>(sd)[i - Kd / 32] = reinterpret_cast<const uint4*>(scl)[i - Kd / 32];
        }
      } else {
        for (int i = t; i < nb; i += TG) { reinterpret_cast<uint2*>(qd)[i] = reinterpret_cast<const uint2*>(codes)[i]; sd[i] = scl[i]; }
      }
      if (t == 0) g[slot] = gx;
    }
    named_bar_sync(bar, TG);                                                  // the staging buffers are reused by the group's next row
  }
}

}  // namespace hb

using namespace hb;

int hbk_nvfp4_dequant(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, void* out, cudaStream_t st, const float* g_dev) {
  const size_t nb = (size_t)N * K / 16;
  size_t blocks = (nb + 255) / 256, cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  return hb_launch(ctx, "nvfp4_dequant", false, nvfp4_dequant_kernel, dim3((unsigned)blocks), dim3(256), 0, st, w, s, g, g_dev, nb,
                   reinterpret_cast<__nv_bfloat16*>(out));
}

int hbk_nvfp4_gemv(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, const void* x, int ldx, int M, float* y, int ldy,
                   cudaStream_t st) {
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const dim3 grid((N + 7) / 8), block(256);
  auto fn = M <= 1 ? nvfp4_gemv_kernel<1> : M <= 2 ? nvfp4_gemv_kernel<2> : M <= 4 ? nvfp4_gemv_kernel<4> : M <= 8 ? nvfp4_gemv_kernel<8>
                                                                                                                  : nvfp4_gemv_kernel<16>;
  return hb_launch(ctx, "nvfp4_gemv", false, fn, grid, block, 0, st, w, s, g, N, K, xb, ldx, M, y, ldy);
}

template <class SRC>
static int quantize_from(hb_ctx* ctx, const SRC& src, size_t n4, uint8_t* q, uint8_t* s, float* g_mul, float* amax, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(amax, 0, 4, st);
  if (e != cudaSuccess) return hb_fail(ctx, HB_ERR_CUDA, "memset amax: %s", cudaGetErrorString(e));
  size_t blocks = (n4 + 255) / 256, cap = (size_t)ctx->sm_count * 8;
  int r = hb_launch(ctx, "tensor_absmax", false, tensor_absmax_kernel<SRC>, dim3((unsigned)(blocks < cap ? blocks : cap)), dim3(256), 0, st, src, n4, amax);
  if (r) return r;
  return hb_launch(ctx, "nvfp4_encode", false, nvfp4_encode_kernel<SRC>, dim3((unsigned)blocks), dim3(256), 0, st, src, n4, (const float*)amax,
                   reinterpret_cast<uint16_t*>(q), s, g_mul);
}
int hbk_nvfp4_quantize(hb_ctx* ctx, const float* w, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax, cudaStream_t st) {
  return quantize_from(ctx, SrcF32{reinterpret_cast<const float4*>(w)}, (size_t)N * K / 4, q, s, g_mul, amax, st);   // K is a multiple of 16
}
int hbk_requant_nvfp4(hb_ctx* ctx, const uint8_t* w_fp8, const float* row_scale, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax, cudaStream_t st) {
  return quantize_from(ctx, SrcFp8Row{reinterpret_cast<const uint32_t*>(w_fp8), row_scale, K / 4}, (size_t)N * K / 4, q, s, g_mul, amax, st);
}

int hbk_quant_rows_scatter(hb_ctx* ctx, const void* x, int ld, int n, int K, const int* dest, int nd, uint8_t* q, uint8_t* s, float* g, cudaStream_t st,
                           const int* n_dev) {
  HB_REQUIRE(ctx, nd >= 1 && nd <= 32, HB_ERR_UNSUPPORTED, "quant_rows: %d destinations per row (at most 32)", nd);
  const bool small = K <= 4096;                                              // short rows: four at a time per CTA
  const size_t stage = (size_t)K * 2 + K / 2 + (K / 16 + 15) / 16 * 16, smem = stage * (small ? 4 : 1);
  HB_REQUIRE(ctx, smem <= 96 * 1024, HB_ERR_UNSUPPORTED, "quant_rows: rows of %d values do not fit the staging buffer", K);
  const int per = small ? 4 : 1;
  int grid = ctx->sm_count * 4;
  if (grid > (n + per - 1) / per) grid = (n + per - 1) / per;
  const char* name = dest ? "quant_rows_scatter" : "a4_quant";
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  if (small) return hb_launch(ctx, name, false, quant_rows_scatter_kernel<64>, dim3(grid), dim3(QS_THREADS), smem, st, xb, ld, n, n_dev, K, dest, nd, q, s, g);
  return hb_launch(ctx, name, false, quant_rows_scatter_kernel<256>, dim3(grid), dim3(QS_THREADS), smem, st, xb, ld, n, n_dev, K, dest, nd, q, s, g);
}

int hbk_a4_quant(hb_ctx* ctx, const void* x, int ld, int n, int K, uint8_t* q, uint8_t* s, float* g, cudaStream_t st) {
  return hbk_quant_rows_scatter(ctx, x, ld, n, K, nullptr, 1, q, s, g, st, nullptr);
}

int hbk_nvfp4_setup(hb_ctx* ctx) {
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(quant_rows_scatter_kernel<64>), cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(quant_rows_scatter_kernel<256>), cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  return HB_OK;
}
