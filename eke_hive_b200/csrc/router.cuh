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

// ---- one row routed by G warps (G a power of two ≤ 32): a two-level tournament.  Warp w takes the experts [w·C, (w+1)·C), finds its own
// k best in k rounds of two warp reductions (largest key, then the smallest id that has it) and leaves them as a sorted list; warp 0
// then merges the G lists in k more rounds.  The order (value descending, id ascending) is the order the one-warp forms above pick
// in, the softmax sum is taken by warp 0 in their order too (per lane e = lane, lane + 32, …, then the butterfly), and the picks are
// summed in pick order: ids and weights are the same bits as theirs.  A one-warp row spends its time waiting on its own
// instructions; G warps share the exponentials and the scans.
__device__ __forceinline__ uint32_t f32_sort_key(float v) {          // monotone map float → uint32, > 0x007fffff for every v > -inf
  const uint32_t b = __float_as_uint(v);
  return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
}

struct RouteScratch {                                                 // shared memory of one group: floats
  // [0, E) p (softmax) / s (sigmoid); [E, 2E) candidates; then G lists of k (key, id) pairs; then G + 2 words
  __host__ __device__ static size_t floats(int E, int k, int G) { return 2 * (size_t)E + 2 * (size_t)G * k + G + 2; }
};

// mode 1 = softmax, 2 = sigmoid + bias.  wg = this warp's index inside the group, bar = a named barrier id owned by the group.
// Lanes 0..k-1 of warp 0 return their pick in (out_id, out_w); the other warps return nothing.
__device__ __forceinline__ void route_row_group(int mode, const float* __restrict__ lr, const float* __restrict__ bias, int E, int k, int renorm, int logits_bf16,
                                                float sig_scale, float* sm, int G, int wg, int lane, int bar, int32_t& out_id, float& out_w) {
  float* p = sm;
  float* cand = sm + E;
  uint32_t* lkey = reinterpret_cast<uint32_t*>(sm + 2 * (size_t)E);    // [G][k]
  int* lid = reinterpret_cast<int*>(lkey + (size_t)G * k);             // [G][k]
  float* misc = reinterpret_cast<float*>(lid + (size_t)G * k);         // [G] warp maxima, then inv
  const int C = ((E + 32 * G - 1) / (32 * G)) * 32, e0 = wg * C, e1 = min(E, e0 + C);
  // ---- values
  if (mode == 1) {
    float mx = -INFINITY;
#pragma unroll 1
    for (int e = e0 + lane; e < e1; e += 32) { const float v = logits_bf16 ? bf16r(lr[e]) : lr[e]; cand[e] = v; mx = fmaxf(mx, v); }
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) misc[wg] = mx;
    named_bar_sync(bar, 32 * G);
    for (int g = 0; g < G; ++g) mx = fmaxf(mx, misc[g]);
#pragma unroll 1
    for (int e = e0 + lane; e < e1; e += 32) { const float v = exp_portable(__fsub_rn(cand[e], mx)); p[e] = v; cand[e] = v; }
  } else {
#pragma unroll 1
    for (int e = e0 + lane; e < e1; e += 32) {
      const float v = sigmoid_portable(lr[e]);
      p[e] = v;
      cand[e] = bias ? __fadd_rn(v, bias[e]) : v;
    }
  }
  // ---- this warp's k best.  A candidate is valid when the one-warp forms would pick it: softmax v ≥ 0 (not NaN), sigmoid c > -inf.
  auto key_of = [&](float v) -> uint32_t {
    if (mode == 1) return v >= 0.f ? __float_as_uint(v) + 1u : 0u;     // non-negative floats order like their bits
    return v > -INFINITY ? f32_sort_key(v) : 0u;
  };
  uint32_t lb = 0u;
  int le = 0x7fffffff;
  auto rescan = [&]() {
    lb = 0u; le = 0x7fffffff;
#pragma unroll 1
    for (int e = e0 + lane; e < e1; e += 32) { const uint32_t kk = key_of(cand[e]); if (kk > lb) { lb = kk; le = e; } }   // ascending e: the first of equal keys stays
  };
  __syncwarp();
  rescan();
#pragma unroll 1
  for (int r = 0; r < k; ++r) {
    const uint32_t m = __reduce_max_sync(0xffffffffu, lb);
    const int bid = (int)__reduce_min_sync(0xffffffffu, (lb == m && m != 0u) ? (uint32_t)le : 0x7fffffffu);
    if (lane == 0) { lkey[wg * k + r] = m; lid[wg * k + r] = bid; }
    if (m != 0u && le == bid) { cand[bid] = mode == 1 ? -1.f : -INFINITY; rescan(); }
  }
  named_bar_sync(bar, 32 * G);
  if (wg != 0) return;
  // ---- warp 0: the sum of the softmax in the one-warp order, then the merge
  float inv = 1.f;
  if (mode == 1) {
    float sum = 0.f;
#pragma unroll 4
    for (int e = lane; e < E; e += 32) sum = __fadd_rn(sum, p[e]);
    for (int o = 16; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    inv = __fdiv_rn(1.f, sum);
  }
  int head = 0;
  uint32_t hk = lane < G ? lkey[lane * k] : 0u;
  int hid = lane < G ? lid[lane * k] : 0x7fffffff;
  float my_v = 0.f, tot = 0.f;
  int my_id = 0;
#pragma unroll 1
  for (int r = 0; r < k; ++r) {
    const uint32_t m = __reduce_max_sync(0xffffffffu, hk);
    int bid = (int)__reduce_min_sync(0xffffffffu, (hk == m && m != 0u) ? (uint32_t)hid : 0x7fffffffu);
    if (m != 0u && hid == bid && hk == m) {                             // this lane's list gave the pick: next entry
      ++head;
      hk = head < k ? lkey[lane * k + head] : 0u;
      hid = head < k ? lid[lane * k + head] : 0x7fffffff;
    }
    float v;
    if (mode == 1) {
      v = __fmul_rn(m ? __uint_as_float(m - 1u) : -1.f, inv);           // softmaxed weight of the pick
    } else {
      if (bid == 0x7fffffff) bid = 0;                                   // every candidate already taken or NaN: keep a valid id
      v = p[bid];
    }
    tot = __fadd_rn(tot, v);
    if (lane == r) { my_id = bid; my_v = v; }
  }
  out_id = my_id;
  if (mode == 1) out_w = __fmul_rn(my_v, renorm ? __fdiv_rn(1.f, tot) : 1.f);
  else out_w = __fmul_rn(__fmul_rn(my_v, __fdiv_rn(1.f, __fadd_rn(tot, 1e-20f))), sig_scale);
}

}  // namespace hb
