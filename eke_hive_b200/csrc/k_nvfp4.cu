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

// ---- fp32 → NVFP4, the device rule of the reference's requant kernels (no per-block scale search)
__global__ void amax_f32_kernel(const float* __restrict__ w, size_t n, float* __restrict__ amax) {
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) m = fmaxf(m, fabsf(w[i]));
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));   // non-negative floats order like ints
}
__global__ void nvfp4_quant_kernel(const float* __restrict__ w, size_t n_blocks16, const float* __restrict__ amax, uint8_t* __restrict__ q,
                                   uint8_t* __restrict__ s, float* __restrict__ g_mul) {
  const float am = *amax;
  const float gs = am > 0.f ? __fdiv_rn(448.f * 6.f, am) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *g_mul = am > 0.f ? __fdiv_rn(am, 448.f * 6.f) : 1.f;
  const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks16) return;
  float f[16], m = 0.f;
  const float4* src = reinterpret_cast<const float4*>(w + b * 16);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 v = src[j];
    f[4 * j] = v.x; f[4 * j + 1] = v.y; f[4 * j + 2] = v.z; f[4 * j + 3] = v.w;
    m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
  const __nv_fp8_storage_t sc = __nv_cvt_float_to_fp8(__fdiv_rn(__fmul_rn(m, gs), 6.f), __NV_SATFINITE, __NV_E4M3);
  const float sd = e4m3_to_f32(sc);
  s[b] = (uint8_t)sc;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t v = sd > 0.f ? ((uint32_t)__nv_cvt_float_to_fp4(__fdiv_rn(__fmul_rn(f[j], gs), sd), __NV_E2M1, cudaRoundNearest) & 0xFu) : 0u;
    if (j < 8) lo |= v << (4 * j); else hi |= v << (4 * (j - 8));
  }
  reinterpret_cast<uint2*>(q)[b] = make_uint2(lo, hi);
}

// ---- per-row dynamic NVFP4 activation quantisation: one warp per row
__global__ void a4_quant_kernel(const __nv_bfloat16* __restrict__ x, int ld, int n, int K, uint8_t* __restrict__ q, uint8_t* __restrict__ s,
                                float* __restrict__ g) {
  const int row = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const __nv_bfloat16* xr = x + (size_t)row * ld;
  const int nb = K / 16;
  const bool vec = (reinterpret_cast<uintptr_t>(xr) & 15) == 0;              // 16-byte loads when the row allows them
  auto load16 = [&](int b, float* v) {
    if (vec) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(xr + b * 16)), u1 = __ldg(reinterpret_cast<const uint4*>(xr + b * 16) + 1);
      const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[2 * j] = __uint_as_float(w[j] << 16); v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __bfloat162float(xr[b * 16 + j]);
    }
  };
  float a = 0.f;
  for (int b = lane; b < nb; b += 32) {
    float v[16];
    load16(b, v);
#pragma unroll
    for (int j = 0; j < 16; ++j) a = fmaxf(a, fabsf(v[j]));
  }
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  const float gx = a > 0.f ? __fdiv_rn(a, 6.f * 448.f) : 1.f, inv = __fdiv_rn(1.f, gx);
  if (lane == 0) g[row] = gx;
  for (int b = lane; b < nb; b += 32) {
    float v[16], ab = 0.f;
    load16(b, v);
#pragma unroll
    for (int j = 0; j < 16; ++j) ab = fmaxf(ab, fabsf(v[j]));
    const __nv_fp8_storage_t se = __nv_cvt_float_to_fp8(__fmul_rn(__fdiv_rn(ab, 6.f), inv), __NV_SATFINITE, __NV_E4M3);
    const float sv = e4m3_to_f32(se);
    const float f = sv > 0.f ? __fdiv_rn(inv, sv) : 0.f;
    uint32_t o[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; ++j)
      o[j / 8] |= ((uint32_t)__nv_cvt_float_to_fp4(__fmul_rn(v[j], f), __NV_E2M1, cudaRoundNearest) & 0xFu) << (4 * (j % 8));
    *reinterpret_cast<uint2*>(q + (size_t)row * (K / 2) + (size_t)b * 8) = make_uint2(o[0], o[1]);
    s[(size_t)row * nb + b] = (uint8_t)se;
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

int hbk_nvfp4_quantize(hb_ctx* ctx, const float* w, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax, cudaStream_t st) {
  const size_t n = (size_t)N * K, nb = n / 16;
  cudaError_t e = cudaMemsetAsync(amax, 0, 4, st);
  if (e != cudaSuccess) return hb_fail(ctx, HB_ERR_CUDA, "memset amax: %s", cudaGetErrorString(e));
  size_t blocks = (n / 4 + 255) / 256, cap = (size_t)ctx->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  int r = hb_launch(ctx, "amax_f32", false, amax_f32_kernel, dim3((unsigned)blocks), dim3(256), 0, st, w, n, amax);
  if (r) return r;
  return hb_launch(ctx, "nvfp4_quant", false, nvfp4_quant_kernel, dim3((unsigned)((nb + 255) / 256)), dim3(256), 0, st, w, nb, (const float*)amax, q, s,
                   g_mul);
}

int hbk_a4_quant(hb_ctx* ctx, const void* x, int ld, int n, int K, uint8_t* q, uint8_t* s, float* g, cudaStream_t st) {
  return hb_launch(ctx, "a4_quant", false, a4_quant_kernel, dim3((n + 7) / 8), dim3(256), 0, st, reinterpret_cast<const __nv_bfloat16*>(x), ld, n, K,
                   q, s, g);
}
