// Per-row routing by one warp, shared by the stand-alone router kernels (k_router.cu) and the fused route + group kernel
// (k_moe_decode.cu).  The exp is the portable polynomial form, sums are taken per lane (e = lane, lane+32, …) and then by a
// 16,8,4,2,1 butterfly, the k picks are summed in pick order — the CPU oracle does the same operations in the same order, so
// ids and weights agree with it to the bit.
#pragma once
#include "hb_common.cuh"

namespace hb {

// (value, id) maximum with ties to the smaller id, over the warp
__device__ __forceinline__ void warp_argmax(float& best, int& bid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bid, o);
    if (ob > best || (ob == best && oi < bid)) { best = ob; bid = oi; }
  }
}

// Softmax top-k of one row.  p: E floats of shared memory owned by this warp.  Lanes 0..k-1 write ids[lane], w[lane].
__device__ __forceinline__ void route_softmax_row(const float* __restrict__ lr, int E, int k, int renorm, int logits_bf16, float* p, int lane,
                                                  int32_t* __restrict__ ids, float* __restrict__ w) {
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    const float v = logits_bf16 ? bf16r(lr[e]) : lr[e];
    p[e] = v;
    mx = fmaxf(mx, v);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float v = exp_portable(__fsub_rn(p[e], mx));
    p[e] = v;
    sum = __fadd_rn(sum, v);
  }
  for (int o = 16; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
  const float inv = __fdiv_rn(1.f, sum);
  __syncwarp();
  float my_w = 0.f, tot = 0.f;
  int my_id = 0;
  for (int r = 0; r < k; ++r) {
    float best = -1.f;
    int bid = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = p[e];
      if (v >= 0.f && v > best) { best = v; bid = e; }      // ascending e per lane: the first (smaller) id keeps a tie
    }
    warp_argmax(best, bid);
    const float sw = __fmul_rn(best, inv);
    tot = __fadd_rn(tot, sw);
    if (lane == r) { my_id = bid; my_w = sw; }
    if (bid != 0x7fffffff && (bid & 31) == lane) p[bid] = -1.f;
    __syncwarp();
  }
  if (lane < k) {
    const float sc = renorm ? __fdiv_rn(1.f, tot) : 1.f;
    ids[lane] = my_id;
    w[lane] = __fmul_rn(my_w, sc);
  }
}

// Sigmoid top-k of one row: s = sigmoid(logit), pick k maxima of s + bias (first maximum = smaller id), w = s/(Σs + 1e-20)·scale
// with Σ in pick order.  sc: 2·E floats of shared memory owned by this warp.
__device__ __forceinline__ void route_sigmoid_row(const float* __restrict__ lr, const float* __restrict__ bias, int E, int k, float scale, float* sc,
                                                  int lane, int32_t* __restrict__ ids, float* __restrict__ w) {
  float* s = sc;
  float* c = sc + E;
  for (int e = lane; e < E; e += 32) {
    const float v = sigmoid_portable(lr[e]);
    s[e] = v;
    c[e] = bias ? __fadd_rn(v, bias[e]) : v;
  }
  __syncwarp();
  float my_s = 0.f, sum = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bid = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = c[e];
      if (v > best) { best = v; bid = e; }
    }
    warp_argmax(best, bid);
    if (bid == 0x7fffffff) bid = 0;                           // every candidate already taken or NaN: keep a valid id
    const float sv = s[bid];
    sum = __fadd_rn(sum, sv);
    if (lane == j) { my_id = bid; my_s = sv; }
    __syncwarp();
    if ((bid & 31) == lane) c[bid] = -INFINITY;
    __syncwarp();
  }
  if (lane < k) {
    const float inv = __fdiv_rn(1.f, __fadd_rn(sum, 1e-20f));
    ids[lane] = my_id;
    w[lane] = __fmul_rn(__fmul_rn(my_s, inv), scale);
  }
}

}  // namespace hb
