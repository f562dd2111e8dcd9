// Routing and the small row kernels around the expert compute: softmax / sigmoid top-k routers, pair building, the
// shared-expert combine, and the gather / SwiGLU / scatter-add helpers of the composed prefill path.
#include "hb_common.cuh"
#include "hb_kernels.h"
#include "router.cuh"

namespace hb {

// One warp per row (see router.cuh)
__global__ void router_softmax_kernel(const float* __restrict__ logits, int ld, int M, int E, int k, int renorm, int logits_bf16,
                                      int32_t* __restrict__ ids, float* __restrict__ w) {
  extern __shared__ float sm_p[];
  griddep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * (blockDim.x >> 5) + warp;
  if (m >= M) return;
  route_softmax_row(logits + (size_t)m * ld, E, k, renorm, logits_bf16, sm_p + (size_t)warp * E, lane, ids + (size_t)m * k, w + (size_t)m * k);
}

__global__ void router_sigmoid_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int M, int E, int k, float scale,
                                      int32_t* __restrict__ ids, float* __restrict__ w) {
  extern __shared__ float sm_p[];
  griddep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x * (blockDim.x >> 5) + warp;
  if (m >= M) return;
  route_sigmoid_row(logits + (size_t)m * E, bias, E, k, scale, sm_p + (size_t)warp * 2 * E, lane, ids + (size_t)m * k, w + (size_t)m * k);
}

__global__ void build_pairs_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w, int M, int K, const uint8_t* const* __restrict__ tab,
                                   int li, int E, hb_moe_pair* __restrict__ pairs) {
  griddep_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * K) return;
  const int e = ids[i];
  hb_moe_pair p;
  p.row = i / K;
  p.rec = (e >= 0 && e < E) ? tab[(size_t)li * E + e] : nullptr;   // a null record is skipped by the decode kernels
  p.w = p.rec ? w[i] : 0.f;
  pairs[i] = p;
}

__global__ void moe_combine_kernel(const float* __restrict__ routed, const __nv_bfloat16* __restrict__ shared, const float* __restrict__ lg, int ld,
                                   int col, int M, int H, __nv_bfloat16* __restrict__ out) {
  griddep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)M * H) return;
  const int m = (int)(i / H);
  float sh = __bfloat162float(shared[i]);
  if (lg) sh = bf16r(__fmul_rn(bf16r(sigmoid_portable(bf16r(lg[(size_t)m * ld + col]))), sh));
  out[i] = __float2bfloat16(__fadd_rn(bf16r(routed[i]), sh));
}

__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ rows, int R, int H8, uint4* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)R * H8; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / H8), c = (int)(i % H8);
    out[i] = x[(size_t)rows[r] * H8 + c];
  }
}
__global__ void swiglu_rows_kernel(const __nv_bfloat16* __restrict__ gu, int R, int I, float limit, __nv_bfloat16* __restrict__ y) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)R * I; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / I, c = i % I;
    float g = __bfloat162float(gu[r * 2 * I + c]), u = __bfloat162float(gu[r * 2 * I + I + c]);
    if (limit > 0.f) { u = fminf(fmaxf(u, -limit), limit); g = fminf(g, limit); }
    y[i] = __float2bfloat16(__fmul_rn(silu_portable(g), u));
  }
}
__global__ void scatter_add_rows_kernel(const __nv_bfloat16* __restrict__ e, const int32_t* __restrict__ rows, const float* __restrict__ w, int R, int H,
                                        float* __restrict__ out) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)R * H; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / H, c = i % H;
    float* o = out + (size_t)rows[r] * H + c;
    *o = __fadd_rn(*o, __fmul_rn(w[r], __bfloat162float(e[i])));
  }
}
__global__ void add_f32_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) a[i] = __fadd_rn(a[i], b[i]);
}

}  // namespace hb

using namespace hb;

static inline int grid_for(hb_ctx* ctx, size_t n, int per_block) {
  size_t b = (n + per_block - 1) / per_block;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  return b ? (int)b : 1;
}

int hbk_route_softmax_topk(hb_ctx* ctx, const float* logits, int ld, int M, int E, int k, int renorm, int logits_bf16, int32_t* ids, float* w,
                           cudaStream_t st, bool pdl) {
  const int warps = 4;
  return hb_launch(ctx, "router_softmax", pdl, router_softmax_kernel, dim3((M + warps - 1) / warps), dim3(warps * 32), (size_t)warps * E * 4, st,
                   logits, ld, M, E, k, renorm, logits_bf16, ids, w);
}
int hbk_route_sigmoid_topk(hb_ctx* ctx, const float* logits, const float* bias, int M, int E, int k, float scale, int32_t* ids, float* w,
                           cudaStream_t st, bool pdl) {
  const int warps = 4;
  return hb_launch(ctx, "router_sigmoid", pdl, router_sigmoid_kernel, dim3((M + warps - 1) / warps), dim3(warps * 32), (size_t)warps * 2 * E * 4, st,
                   logits, bias, M, E, k, scale, ids, w);
}
int hbk_build_pairs(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* tab, int li, int E, hb_moe_pair* pairs,
                    cudaStream_t st, bool pdl) {
  return hb_launch(ctx, "build_pairs", pdl, build_pairs_kernel, dim3((M * K + 255) / 256), dim3(256), 0, st, ids, w, M, K, tab, li, E, pairs);
}
int hbk_moe_combine(hb_ctx* ctx, const float* routed, const void* shared, const float* lg, int ld, int col, int M, int H, void* out, cudaStream_t st,
                    bool pdl) {
  return hb_launch(ctx, "moe_combine", pdl, moe_combine_kernel, dim3((unsigned)(((size_t)M * H + 255) / 256)), dim3(256), 0, st, routed,
                   reinterpret_cast<const __nv_bfloat16*>(shared), lg, ld, col, M, H, reinterpret_cast<__nv_bfloat16*>(out));
}
__global__ void layer_prep_kernel(const uint8_t** tab1, int32_t* ids1, float* w1, int M, const uint8_t* shared_rec) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) tab1[0] = shared_rec;
  if (i < M) { ids1[i] = 0; w1[i] = 1.f; }
}
__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = __float2bfloat16(in[i]);
}
// the always-on shared expert as a one-expert routing: table {shared_rec}, ids 0, weights 1
int hbk_layer_prep(hb_ctx* ctx, const uint8_t** tab1, int32_t* ids1, float* w1, int M, const uint8_t* shared_rec, cudaStream_t st) {
  return hb_launch(ctx, "layer_prep", false, layer_prep_kernel, dim3((M + 255) / 256), dim3(256), 0, st, tab1, ids1, w1, M, shared_rec);
}
int hbk_f32_to_bf16(hb_ctx* ctx, const float* in, void* out, size_t n, cudaStream_t st) {
  return hb_launch(ctx, "f32_to_bf16", false, f32_to_bf16_kernel, dim3(grid_for(ctx, n, 256)), dim3(256), 0, st, in, reinterpret_cast<__nv_bfloat16*>(out), n);
}
int hbk_gather_rows(hb_ctx* ctx, const void* x, const int32_t* rows, int R, int H, void* out, cudaStream_t st) {
  return hb_launch(ctx, "gather_rows", false, gather_rows_kernel, dim3(grid_for(ctx, (size_t)R * (H / 8), 256)), dim3(256), 0, st,
                   reinterpret_cast<const uint4*>(x), rows, R, H / 8, reinterpret_cast<uint4*>(out));
}
int hbk_swiglu_rows(hb_ctx* ctx, const void* gu, int R, int I, float limit, void* y, cudaStream_t st) {
  return hb_launch(ctx, "swiglu_rows", false, swiglu_rows_kernel, dim3(grid_for(ctx, (size_t)R * I, 256)), dim3(256), 0, st,
                   reinterpret_cast<const __nv_bfloat16*>(gu), R, I, limit, reinterpret_cast<__nv_bfloat16*>(y));
}
int hbk_scatter_add_rows(hb_ctx* ctx, const void* e, const int32_t* rows, const float* w, int R, int H, float* out, cudaStream_t st) {
  return hb_launch(ctx, "scatter_add_rows", false, scatter_add_rows_kernel, dim3(grid_for(ctx, (size_t)R * H, 256)), dim3(256), 0, st,
                   reinterpret_cast<const __nv_bfloat16*>(e), rows, w, R, H, out);
}
int hbk_add_f32(hb_ctx* ctx, float* a, const float* b, size_t n, cudaStream_t st) {
  return hb_launch(ctx, "add_f32", false, add_f32_kernel, dim3(grid_for(ctx, n, 256)), dim3(256), 0, st, a, (const float*)b, n);
}
