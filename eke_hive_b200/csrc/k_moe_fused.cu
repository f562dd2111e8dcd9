// The decode MoE layer's expert compute as ONE persistent kernel: gate/up stream → down stream → routed reduce + combine.
//
// The three stages of the unfused path cost a launch, a pipeline fill and a drain each (≈ 5 µs per kernel at these sizes, more
// than the 3–40 µs the weights themselves take).  Here every CTA first takes its share of the gate/up items, then its share
// of the down items, then its share of the output rows; the producer warp keeps the weight ring full across the stage
// boundaries, so HBM never idles between them.  Cross-CTA dependencies are counters in global memory:
//   done[g]  gate/up items of group g finished (the down consumers of group g wait for it to reach I / 8·WM before reading y)
//   hdr[2]   down items finished (the reduce waits for all of them)
// Every CTA of the grid is resident at once (the grid is sized from the occupancy query), all waits are bounded and set the
// context's error word instead of hanging.  Layout of work and arithmetic are those of moe_stream_kernel (moe_stream.cuh).
#include "moe_stream.cuh"

namespace hb {

struct FusedArgs {
  int* hdr; const Group* groups; const int* s_row; int* done;
  const __nv_bfloat16* x; __nv_bfloat16* y; __nv_bfloat16* part;
  int H, I; float limit;
  uint32_t off_w1, off_s1, off_w3, off_s3, off_w2, off_s2, off_g;
  int stages;
  uint32_t* err;
  int do_reduce;            // 1: routed reduce / combine as the last stage; 0: a separate kernel finishes (pair-list form)
  ReduceArgs red;
};

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded spin on a global counter (one lane); false after ~seconds, with the site recorded.
__device__ __forceinline__ bool wait_counter(const int* p, int target, uint32_t* err, uint32_t site) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (ld_acquire(p) >= target) return true;
    if (it > 4096) __nanosleep(64);
  }
  if (err) atomicOr(err, site);
  return false;
}

template <int WKA, int WKB, int NW>
struct FusedCfg {
  using A = StreamCfg<WKA, NW / WKA, false>;
  using B = StreamCfg<WKB, NW / WKB, true>;
  static_assert(NW % WKA == 0 && NW % WKB == 0, "consumer warps must tile both stages");
  static constexpr int THREADS = (NW + 2) * 32;
  static constexpr int CTAS_PER_SM = THREADS <= 320 ? 2 : 1;
  static constexpr int STAGE = A::STAGE > B::STAGE ? A::STAGE : B::STAGE;
  static constexpr int SLOT = NW * 32 * 16;
  static constexpr int BARS = (2 * kMaxStages + 2 * (kMaxStages + 1)) * 8;
  __host__ __device__ static constexpr size_t head(int stages) { return (size_t)(((stages + 1) * SLOT + BARS + 127) / 128 * 128); }
  __host__ __device__ static constexpr size_t smem(int stages) { return head(stages) + (size_t)stages * STAGE; }
};

// Ring / slot cursors carried across the two streaming stages.
struct Cursor { int s = 0; uint32_t ph = 0; int slot = 0; uint32_t rph = 0; };

struct SmemView { float4* red; uint64_t* full; uint64_t* empty; uint64_t* redbar; uint64_t* redfree; uint8_t* ring; int S, NSLOT, stage_bytes; };

template <class C, bool DOWN>
__device__ __forceinline__ bool producer_stage(const FusedArgs& a, const SmemView& v, Cursor& c, int i_begin, int n_items, int tiles, int* issued_total) {
  int gi = i_begin / tiles, tile = i_begin - gi * tiles, cur = -1;
  Group g = {nullptr, 0, 0};
  const uint32_t off_wa = DOWN ? a.off_w2 : a.off_w1, off_sa = DOWN ? a.off_s2 : a.off_s1;
  for (int it = 0; it < n_items; ++it) {
    if (!mbar_wait(&v.empty[c.s], c.ph ^ 1u, a.err, 1u)) return false;
    if (gi != cur) { g = a.groups[gi]; cur = gi; }
    uint8_t* st = v.ring + (size_t)c.s * v.stage_bytes;
    mbar_expect_tx(&v.full[c.s], C::TX);
    const size_t r0 = (size_t)tile * C::TR;
    bulk_g2s(st, g.rec + off_wa + r0 * C::RB, C::TR * C::RB, &v.full[c.s]);
    bulk_g2s(st + C::TR * C::RB, g.rec + off_sa + r0 * C::RS, C::TR * C::RS, &v.full[c.s]);
    if (!DOWN) {
      bulk_g2s(st + C::UP_OFF, g.rec + a.off_w3 + r0 * C::RB, C::TR * C::RB, &v.full[c.s]);
      bulk_g2s(st + C::UP_OFF + C::TR * C::RB, g.rec + a.off_s3 + r0 * C::RS, C::TR * C::RS, &v.full[c.s]);
    }
    ++*issued_total;
    if (++tile == tiles) { tile = 0; ++gi; }
    if (++c.s == v.S) { c.s = 0; c.ph ^= 1u; }
  }
  return true;
}

template <class C, bool DOWN>
__device__ __forceinline__ bool epilogue_stage(const FusedArgs& a, const SmemView& v, Cursor& c, int i_begin, int n_items, int tiles, int lane) {
  constexpr int WK = C::NW / (C::TR / (DOWN ? 16 : 8)), WM = C::TR / (DOWN ? 16 : 8);
  int gi = i_begin / tiles, tile = i_begin - gi * tiles, cur = -1, pending = 0;
  Group grp = {nullptr, 0, 0};
  float gl[3] = {1.f, 1.f, 1.f};
  // Finished items are counted once per run of items of one group (a device-wide fence per item would serialise this warp):
  // fence, then add the run length to the group's counter (gate/up) or to the down total.
  auto publish = [&]() {
    if (pending == 0) return;
    __syncwarp();                                          // every lane's stores of the run are ordered before lane 0's fence …
    if (lane == 0) {
      __threadfence();                                     // … which makes them visible device-wide before they are counted
      atomicAdd(DOWN ? &a.hdr[2] : &a.done[cur], pending);
    }
    pending = 0;
  };
  for (int it = 0; it < n_items; ++it) {
    if (gi != cur) {
      if (!DOWN) publish();
      cur = gi;
      grp = a.groups[gi];
      const float* gp = reinterpret_cast<const float*>(grp.rec + a.off_g);
      gl[0] = __ldg(gp); gl[1] = __ldg(gp + 1); gl[2] = __ldg(gp + 2);
    }
    if (!mbar_wait(&v.redbar[c.slot], c.rph, a.err, 8u)) return false;
    const float4* rb = v.red + (size_t)c.slot * C::NW * 32;
#pragma unroll
    for (int mt = 0; mt < WM; ++mt) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k2 = 0; k2 < WK; ++k2) {                    // fixed order over the K slices: deterministic
        const float4 q = rb[(mt * WK + k2) * 32 + lane];
        acc[0] += q.x; acc[1] += q.y; acc[2] += q.z; acc[3] += q.w;
      }
      tile_epilogue<DOWN>(acc, grp, gl, tile * C::TR + (DOWN ? 16 : 8) * mt, lane, a.H, a.I, a.limit, DOWN ? a.part : a.y);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&v.redfree[c.slot]);
    ++pending;
    if (++tile == tiles) { tile = 0; ++gi; }
    if (++c.slot == v.NSLOT) { c.slot = 0; c.rph ^= 1u; }
  }
  publish();
  return true;
}

template <class C, bool DOWN>
__device__ __forceinline__ bool consumer_stage(const FusedArgs& a, const SmemView& v, Cursor& c, int i_begin, int n_items, int tiles, int warp, int lane,
                                               int tiles_gate_up) {
  constexpr int WM = C::TR / (DOWN ? 16 : 8), WK = C::NW / WM;
  const int mt = warp / WK, ks = warp % WK;
  const int g = lane >> 2, t = lane & 3;
  int rowA, rowB, matoff = 0;
  if (DOWN) { rowA = 16 * mt + g; rowB = rowA + 8; }
  else { rowA = 8 * mt + (g >> 1); rowB = rowA + 4; matoff = (g & 1) ? C::UP_OFF : 0; }
  const int wA = matoff + rowA * C::RB + ks * (kSlice / 2) + 32 * t, wB = matoff + rowB * C::RB + ks * (kSlice / 2) + 32 * t;
  const int sA = matoff + C::TR * C::RB + rowA * C::RS + ks * (kSlice / 16) + 4 * t, sB = matoff + C::TR * C::RB + rowB * C::RS + ks * (kSlice / 16) + 4 * t;
  uint32_t bfr[32];
  float inv[2] = {1.f, 1.f};
  int gi = i_begin / tiles, tile = i_begin - gi * tiles, cur = -1;
  for (int it = 0; it < n_items; ++it) {
    if (gi != cur) {
      cur = gi;
      const Group grp = a.groups[gi];
      if (DOWN) {                                          // y of this group is complete once all its gate/up items are counted
        bool ok = true;
        if (lane == 0) ok = wait_counter(&a.done[gi], tiles_gate_up, a.err, 32u);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
      }
      const __nv_bfloat16* src = nullptr;
      if (g < grp.n) src = DOWN ? a.y + (size_t)(grp.start + g) * a.I + ks * kSlice : a.x + (size_t)a.s_row[grp.start + g] * a.H + ks * kSlice;
      load_b_frags<DOWN>(src, t, bfr, inv);
    }
    if (!mbar_wait(&v.full[c.s], c.ph, a.err, 2u)) return false;
    const uint8_t* st = v.ring + (size_t)c.s * v.stage_bytes;
    float acc[4];
    warp_slice_mma(st + wA, st + wB, st + sA, st + sB, bfr, acc, &v.empty[c.s]);
    acc[0] *= inv[0]; acc[1] *= inv[1]; acc[2] *= inv[0]; acc[3] *= inv[1];
    if (!mbar_wait(&v.redfree[c.slot], c.rph ^ 1u, a.err, 16u)) return false;      // the slot's previous contents have been read
    v.red[(size_t)c.slot * C::NW * 32 + warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncwarp();
    if (lane == 0) mbar_arrive(&v.redbar[c.slot]);
    if (++tile == tiles) { tile = 0; ++gi; }
    if (++c.s == v.S) { c.s = 0; c.ph ^= 1u; }
    if (++c.slot == v.NSLOT) { c.slot = 0; c.rph ^= 1u; }
  }
  return true;
}

template <int WKA, int WKB, int NW>
__global__ void __launch_bounds__(FusedCfg<WKA, WKB, NW>::THREADS, FusedCfg<WKA, WKB, NW>::CTAS_PER_SM) moe_fused_kernel(FusedArgs a) {
  using F = FusedCfg<WKA, WKB, NW>;
  using CA = typename F::A;
  using CB = typename F::B;
  extern __shared__ __align__(128) uint8_t smem[];
  SmemView v;
  v.S = a.stages; v.NSLOT = a.stages + 1; v.stage_bytes = F::STAGE;
  v.red = reinterpret_cast<float4*>(smem);                                        // [NSLOT][NW][32]
  v.full = reinterpret_cast<uint64_t*>(smem + (size_t)v.NSLOT * F::SLOT);         // [kMaxStages]
  v.empty = v.full + kMaxStages;                                                  // [kMaxStages]
  v.redbar = v.empty + kMaxStages;                                                // [kMaxStages + 1]
  v.redfree = v.redbar + kMaxStages + 1;                                          // [kMaxStages + 1]
  v.ring = smem + F::head(a.stages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < v.S; ++s) { mbar_init(&v.full[s], 1); mbar_init(&v.empty[s], NW); }
    for (int s = 0; s < v.NSLOT; ++s) { mbar_init(&v.redbar[s], NW); mbar_init(&v.redfree[s], 1); }
    mbar_fence_init();
  }
  __syncthreads();
  griddep_wait();                                          // the grouping kernel's list and zeroed counters
  const int n_groups = a.hdr[0];
  const int tilesA = a.I / CA::TR, tilesB = a.H / CB::TR;
  griddep_launch();
  // Work split, aligned to groups: with no more groups than CTAs, a team of T = ⌊CTAs / groups⌋ CTAs shares one group (each
  // member a contiguous share of its gate/up tiles, then of its down tiles), so a CTA loads its activation fragments once per
  // stage and only waits for its own team before the down stage; with more groups than CTAs every CTA takes whole groups.
  const int G = (int)gridDim.x, cta = (int)blockIdx.x;
  const int T = n_groups > 0 && n_groups <= G ? G / n_groups : 1;
  const int g_first = cta / T, member = cta % T, g_stride = n_groups <= G ? n_groups : G;   // one pass when teams are used
  const int ta0 = tilesA * member / T, ta1 = tilesA * (member + 1) / T;
  const int tb0 = tilesB * member / T, tb1 = tilesB * (member + 1) / T;
  Cursor c;

  if (warp == NW) {                                        // ---- producer: one lane keeps the ring full across stages and groups
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int gi = g_first; gi < n_groups && ok; gi += g_stride) {
        ok = producer_stage<CA, false>(a, v, c, gi * tilesA + ta0, ta1 - ta0, tilesA, &issued);
        if (ok) ok = producer_stage<CB, true>(a, v, c, gi * tilesB + tb0, tb1 - tb0, tilesB, &issued);
      }
      // copies still in flight land before the CTA leaves (immediate when the consumers took every stage)
      for (int j = issued > v.S ? issued - v.S : 0; j < issued; ++j) mbar_wait(&v.full[j % v.S], (uint32_t)((j / v.S) & 1), a.err, 4u);
    }
    return;
  }
  if (warp == NW + 1) {                                    // ---- epilogue warp
    bool ok = true;
    for (int gi = g_first; gi < n_groups && ok; gi += g_stride) {
      ok = epilogue_stage<CA, false>(a, v, c, gi * tilesA + ta0, ta1 - ta0, tilesA, lane);
      if (ok) ok = epilogue_stage<CB, true>(a, v, c, gi * tilesB + tb0, tb1 - tb0, tilesB, lane);
    }
    return;
  }
  // ---- consumers
  for (int gi = g_first; gi < n_groups; gi += g_stride) {
    if (!consumer_stage<CA, false>(a, v, c, gi * tilesA + ta0, ta1 - ta0, tilesA, warp, lane, tilesA)) return;
    if (!consumer_stage<CB, true>(a, v, c, gi * tilesB + tb0, tb1 - tb0, tilesB, warp, lane, tilesA)) return;
  }
  if (!a.do_reduce) return;
  // ---- routed reduce + combine over this CTA's share of (row, column pair) units, once every down item is counted
  const long long totB = (long long)n_groups * tilesB;
  const size_t units = (size_t)a.red.M * a.H / 2;
  const size_t per = (units + gridDim.x - 1) / gridDim.x;
  const size_t u0 = per * blockIdx.x, u1 = u0 + per < units ? u0 + per : units;
  if (u0 >= units) return;
  bool ok = true;
  if (lane == 0) ok = wait_counter(&a.hdr[2], (int)totB, a.err, 64u);
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (!ok) return;
  for (size_t u = u0 + threadIdx.x; u < u1; u += NW * 32) reduce_routed_unit(a.red, u);
}

}  // namespace hb

using namespace hb;

namespace {
using FusedFn = void (*)(FusedArgs);
struct FusedKernel { FusedFn fn; int threads; int ctas; size_t (*smem)(int); int wka, wkb; };

template <int WKA, int WKB, int NW>
FusedKernel mk() {
  using F = FusedCfg<WKA, WKB, NW>;
  return FusedKernel{moe_fused_kernel<WKA, WKB, NW>, F::THREADS, F::CTAS_PER_SM, &F::smem, WKA, WKB};
}
// (H/256, I/256) pairs with a fused kernel; other shapes of the streaming path run the three separate kernels
const FusedKernel* fused_table(int* n) {
  static const FusedKernel t[] = {
      mk<8, 2, 8>(),    // H 2048, I 512  (Qwen3-Next-shaped decode)
      mk<16, 2, 16>(),  // H 4096, I 512
      mk<8, 8, 8>(),    // H 2048, I 2048
      mk<8, 4, 8>(),    // H 2048, I 1024
      mk<4, 2, 8>(),    // H 1024, I 512
      mk<4, 4, 8>(),    // H 1024, I 1024
      mk<2, 2, 8>(),    // H 512,  I 512
      mk<1, 1, 8>(),    // H 256,  I 256
      mk<16, 8, 16>(),  // H 4096, I 2048
      mk<16, 4, 16>(),  // H 4096, I 1024
      mk<16, 16, 16>(), // H 4096, I 4096
      mk<2, 1, 8>(),    // H 512,  I 256
      mk<16, 1, 16>(),  // H 4096, I 256
      mk<4, 1, 8>(),    // H 1024, I 256
  };
  *n = (int)(sizeof t / sizeof t[0]);
  return t;
}
const FusedKernel* find_fused(int H, int I) {
  if (H % kSlice || I % kSlice) return nullptr;
  int n;
  const FusedKernel* t = fused_table(&n);
  for (int i = 0; i < n; ++i)
    if (t[i].wka == H / kSlice && t[i].wkb == I / kSlice) {
      // both stages must tile the matrices: I rows in gate/up tiles of 8·WM, H rows in down tiles of 16·WM
      const int nw = (t[i].threads / 32) - 2;
      if (I % (8 * (nw / t[i].wka)) == 0 && H % (16 * (nw / t[i].wkb)) == 0) return &t[i];
    }
  return nullptr;
}
void plan_fused(const hb_ctx* ctx, const FusedKernel& k, int* stages) {
  const long long avail = k.ctas == 1 ? ctx->smem_optin : (228 * 1024) / k.ctas - 2048;
  int s = kMaxStages;
  while (s > 2 && (long long)k.smem(s) > avail) --s;
  *stages = s;
}
}  // namespace

bool hbk_moe_fused_available(int H, int I) { return find_fused(H, I) != nullptr; }

int hbk_moe_fused_setup(hb_ctx* ctx) {
  int n;
  const FusedKernel* t = fused_table(&n);
  for (int i = 0; i < n; ++i) {
    int s;
    plan_fused(ctx, t[i], &s);
    HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(t[i].fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t[i].smem(s)));
  }
  return HB_OK;
}

// Launches the fused kernel on the grouped workspace `w`.  red == nullptr: no reduce stage (the caller launches its own).
int hbk_moe_fused_launch(hb_ctx* ctx, const DecodeWs& w, const void* x, int H, int I, float limit, const hb_rec_layout& L, const ReduceArgs* red,
                         cudaStream_t st) {
  const FusedKernel* k = find_fused(H, I);
  if (!k) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "no fused kernel for H=%d I=%d", H, I);
  FusedArgs a{};
  a.hdr = w.hdr; a.groups = w.groups; a.s_row = w.s_row; a.done = w.done;
  a.x = reinterpret_cast<const __nv_bfloat16*>(x); a.y = w.y; a.part = w.part;
  a.H = H; a.I = I; a.limit = limit;
  a.off_w1 = (uint32_t)L.w1; a.off_s1 = (uint32_t)L.s1; a.off_w3 = (uint32_t)L.w3; a.off_s3 = (uint32_t)L.s3;
  a.off_w2 = (uint32_t)L.w2; a.off_s2 = (uint32_t)L.s2; a.off_g = (uint32_t)L.g;
  a.err = ctx->dev_err;
  a.do_reduce = red ? 1 : 0;
  if (red) a.red = *red;
  plan_fused(ctx, *k, &a.stages);
  // every CTA must be resident at once (they wait on each other's counters): size the grid from the occupancy query
  int per_sm = 0;
  HB_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, reinterpret_cast<const void*>(k->fn), k->threads, k->smem(a.stages)));
  if (per_sm < 1) return hb_fail(ctx, HB_ERR_CUDA, "fused kernel does not fit an SM (H=%d I=%d)", H, I);
  if (per_sm > k->ctas) per_sm = k->ctas;
  int grid = ctx->sm_count * per_sm;
  if (ctx->max_ctas > 0 && grid > ctx->max_ctas) grid = ctx->max_ctas;
  return hb_launch(ctx, "moe_fused", true, k->fn, dim3(grid), dim3(k->threads), k->smem(a.stages), st, a);
}
