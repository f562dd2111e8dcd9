// Routed-expert decode for NVFP4 expert records (1–16 tokens per expert): a memory-bound streaming path.
//
//   group   one CTA: sorts the (row, expert) pairs by expert into groups of ≤ 8 rows, so a record streams once per group
//   gate/up persistent CTAs: item = (group, 8 gate + 8 up rows of I).  A producer warp streams the packed rows into a
//           shared-memory ring with 1-D bulk asynchronous copies (mbarrier transaction counts); consumer warps split K,
//           decode e2m1 → f16 in registers with the hardware converter, multiply by the exact f16 e4m3 block scale and
//           feed m16n8k16 tensor-core tiles whose 8 columns are the group's activation rows (fp32 accumulation); split-K
//           partials meet in shared memory in a fixed order; SwiGLU epilogue → y[pair, I] (bf16)
//   down    same machinery over [H, I]: part[pair, H] = bf16(down · g2)
//   reduce  out[row] = Σ_k w·part in k (or pair) order, fused with the shared-expert combine where asked
//
// HBM traffic per layer is the records touched plus O(pairs·(H+I)) bytes of activations; weights are read once per group.
// Shapes the streaming path takes: H, I multiples of 256, at most 4096; anything else (H, I multiples of 32) runs on the
// generic CUDA-core kernels at the end of this file.
#include "ep.cuh"
#include "moe_stream.cuh"
#include "router.cuh"

namespace hb {

// ================================================================================================ grouping
struct GroupArgs {
  const hb_moe_pair* pairs; int n_pairs;                 // list form (ids == nullptr)
  const int32_t* ids; const float* w; int M, K;          // routed form
  const uint8_t* const* tab; int li, E;
  const uint8_t* shared_rec;
  int ld_ids, sh_row0, sh_rows;                          // pitch of ids / w rows; rows [sh_row0, sh_row0 + sh_rows) get the shared pair
  const uint32_t* wait_flags; int wait_n; const uint32_t* wait_step; uint32_t* wait_err;   // expert parallel: the gathered rows' flags
  DecodeWs ws;
  // optional routing stage (routed form): logits → ids / w by one warp per row before the grouping
  int route; const float* logits; int ld, renorm, logits_bf16; const float* bias; float sig_scale;
  int32_t* ids_out; float* w_out;
  int group_rows;       // rows per group (≤ kGroupRows)
};

// Exclusive scan of two int arrays of length n in shared memory, by the whole block (blockDim.x == kGroupThreads).
__device__ void block_scan2(int* a, int* b, int n, int* tot_a, int* tot_b, int* warp_tmp /* [2][32] */) {
  const int per = (n + kGroupThreads - 1) / kGroupThreads;
  const int i0 = threadIdx.x * per, i1 = min(n, i0 + per);
  int sa = 0, sb = 0;
  for (int i = i0; i < i1; ++i) { sa += a[i]; sb += b[i]; }
  int xa = sa, xb = sb;                                  // inclusive warp scan of the per-thread sums
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 1; o < 32; o <<= 1) {
    const int ta = __shfl_up_sync(0xffffffffu, xa, o), tb = __shfl_up_sync(0xffffffffu, xb, o);
    if (lane >= o) { xa += ta; xb += tb; }
  }
  if (lane == 31) { warp_tmp[warp] = xa; warp_tmp[32 + warp] = xb; }
  __syncthreads();
  if (warp == 0) {
    int va = warp_tmp[lane], vb = warp_tmp[32 + lane];
    const int ia = va, ib = vb;
    for (int o = 1; o < 32; o <<= 1) {
      const int ta = __shfl_up_sync(0xffffffffu, va, o), tb = __shfl_up_sync(0xffffffffu, vb, o);
      if (lane >= o) { va += ta; vb += tb; }
    }
    warp_tmp[lane] = va - ia; warp_tmp[32 + lane] = vb - ib;          // exclusive warp offsets
    if (lane == 31) { *tot_a = va; *tot_b = vb; }
  }
  __syncthreads();
  int ba = warp_tmp[warp] + xa - sa, bb = warp_tmp[32 + warp] + xb - sb;
  for (int i = i0; i < i1; ++i) { const int ca = a[i], cb = b[i]; a[i] = ba; b[i] = bb; ba += ca; bb += cb; }
  __syncthreads();
}

constexpr int kTcGuMinPairs = 40;                   // unpinned contexts: pairs per call from which gate/up runs on the tensor-memory kernel

__global__ void __launch_bounds__(kGroupThreads) moe_group_kernel(GroupArgs a) {
  extern __shared__ __align__(16) uint8_t gsm[];
  griddep_wait();
  griddep_launch();                                     // what follows in the stream may start its prologue (each kernel waits for its own inputs)
  if (a.wait_flags) {                                   // the rows, ids and weights this pass reads are pushed by the other ranks
    if ((int)threadIdx.x < a.wait_n && !*reinterpret_cast<volatile uint32_t*>(a.wait_err))
      ep_wait_flag(a.wait_flags + threadIdx.x, *a.wait_step + 1u, a.wait_err, 0x40000u);
    __syncthreads();
  }
  const bool routed = a.ids != nullptr;
  const int P = routed ? a.M * a.K + (a.shared_rec ? a.M : 0) : a.n_pairs;
  const int NK = routed ? a.E + 1 : P;                  // key space: expert id (E = the shared expert) or leader pair index
  int* key = reinterpret_cast<int*>(gsm);               // [P]
  int* cnt = key + P;                                   // [NK] → exclusive offsets
  int* ngr = cnt + NK;                                  // [NK] → exclusive group bases
  int* fill = ngr + NK;                                 // [NK]
  int* misc = fill + NK;                                // [64 + 2]
  const uint8_t** recs = reinterpret_cast<const uint8_t**>(gsm + ((size_t)(P + 3 * NK + 68) * 4 + 7) / 8 * 8);   // [P], list form only
  if (a.route) {                                        // routed form with routing: recs is unused, the router scratch sits there
    float* rsm = reinterpret_cast<float*>(recs);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int m = warp; m < a.M; m += nwarps) {
      if (a.route == 1) route_softmax_row(a.logits + (size_t)m * a.ld, a.E, a.K, a.renorm, a.logits_bf16, rsm + (size_t)warp * a.E, lane,
                                          a.ids_out + (size_t)m * a.K, a.w_out + (size_t)m * a.K);
      else route_sigmoid_row(a.logits + (size_t)m * a.ld, a.bias, a.E, a.K, a.sig_scale, rsm + (size_t)warp * 2 * a.E, lane,
                             a.ids_out + (size_t)m * a.K, a.w_out + (size_t)m * a.K);
    }
    __syncthreads();                                    // ids / w of every row are written (same CTA): the grouping below reads them
  }
  for (int k = threadIdx.x; k < NK; k += blockDim.x) { cnt[k] = 0; fill[k] = 0; }
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    int row, kk = -1; float wv;
    if (routed) {
      if (i < a.M * a.K) {
        row = i / a.K;
        const size_t src = (size_t)row * a.ld_ids + (i - row * a.K);
        const int e = a.ids[src];
        wv = a.w[src];
        if (e >= 0 && e < a.E && a.tab[(size_t)a.li * a.E + e] != nullptr) kk = e;
      } else { row = i - a.M * a.K; wv = 1.f; kk = row >= a.sh_row0 && row < a.sh_row0 + a.sh_rows ? a.E : -1; }
    } else {
      const hb_moe_pair p = a.pairs[i];
      row = p.row; wv = p.w; recs[i] = p.rec;
      kk = p.rec ? i : -1;                              // replaced by the leader index below
    }
    key[i] = kk; a.ws.prow[i] = row; a.ws.pw[i] = wv;
  }
  __syncthreads();
  if (!routed) {
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
      const uint8_t* r = recs[i];
      if (!r) continue;
      int l = i;
      for (int j = 0; j < i; ++j) if (recs[j] == r) { l = j; break; }
      key[i] = l;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < P; i += blockDim.x) if (key[i] >= 0) atomicAdd(&cnt[key[i]], 1);
  __syncthreads();
  const int GR = a.group_rows;                          // rows per group: 8 for the streaming gate/up kernel, 2 for the tensor-memory one
  for (int k = threadIdx.x; k < NK; k += blockDim.x) ngr[k] = (cnt[k] + GR - 1) / GR;
  __syncthreads();
  // keep the counts: the scan overwrites cnt with offsets, so copy them into fill's slot first (fill is re-zeroed after)
  for (int k = threadIdx.x; k < NK; k += blockDim.x) fill[k] = cnt[k];
  __syncthreads();
  block_scan2(cnt, ngr, NK, &misc[64], &misc[65], misc);
  // groups of every key that has pairs
  for (int k = threadIdx.x; k < NK; k += blockDim.x) {
    const int c = fill[k];
    if (c == 0) continue;
    const uint8_t* rec = routed ? (k == a.E ? a.shared_rec : a.tab[(size_t)a.li * a.E + k]) : recs[k];
    for (int j = 0; j * GR < c; ++j)
      if (HB_BOUND(a.wait_err, ngr[k] + j >= 0 && ngr[k] + j < P, 0x101u, ngr[k] + j))
        a.ws.groups[ngr[k] + j] = Group{rec, cnt[k] + j * GR, min(GR, c - j * GR)};
  }
  __syncthreads();
  for (int k = threadIdx.x; k < NK; k += blockDim.x) fill[k] = 0;
  __syncthreads();
  // slot inside the expert's run: any order gives the same results (columns of a tile are independent)
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    const int kk = key[i];
    int pos = -1;
    if (kk >= 0) { pos = cnt[kk] + atomicAdd(&fill[kk], 1); if (HB_BOUND(a.wait_err, pos >= 0 && pos < P, 0x102u, pos)) a.ws.s_row[pos] = a.ws.prow[i]; }
    a.ws.pos_of[i] = pos;
  }
  for (int i = threadIdx.x; i < P; i += blockDim.x) a.ws.done[i] = 0;
  if (threadIdx.x == 0) { a.ws.hdr[0] = misc[65]; a.ws.hdr[1] = misc[64]; a.ws.hdr[2] = 0; a.ws.hdr[3] = 0; }
}

static size_t group_smem(bool routed, int P, int E, int route = 0) {
  const int NK = routed ? E + 1 : P;
  size_t b = (size_t)P * 4 + (size_t)NK * 12 + 68 * 4;
  b = (b + 7) / 8 * 8;
  if (route) return b + (size_t)(kGroupThreads / 32) * E * 4 * (route == 2 ? 2 : 1);
  return b + (routed ? 0 : (size_t)P * 8);
}

// ================================================================================================ streaming kernels
template <int WK, int WM, bool DOWN>
__device__ __forceinline__ void moe_stream_roles(const StreamArgs& a) {
  using C = StreamCfg<WK, WM, DOWN>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int S = a.stages, NSLOT = S + 1;
  // split-K exchange: NSLOT slots of one float4 per consumer thread.  Consumer warps drop their partial sums into the item's slot
  // and go on to the next item; a dedicated epilogue warp waits for the slot (redbar), adds the K slices in fixed order, applies
  // the epilogue and hands the slot back (redfree).  No consumer ever waits for another consumer.
  float4* red = reinterpret_cast<float4*>(smem);                                                // [NSLOT][NW][32]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (WK > 1 ? NSLOT * C::SLOT : 0));          // [kMaxStages]
  uint64_t* empty = full + kMaxStages;                                                          // [kMaxStages]
  uint64_t* redbar = empty + kMaxStages;                                                        // [NSLOT][WM]
  uint64_t* redfree = redbar + (kMaxStages + 1) * WM;                                           // [NSLOT]
  uint8_t* ring = smem + C::head(S);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], C::NW); }
    for (int s = 0; s < NSLOT * WM; ++s) mbar_init(&redbar[s], WK);
    for (int s = 0; s < NSLOT; ++s) mbar_init(&redfree[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  // the group list was written by the grouping kernel two launches back (see hbk_moe_decode_run for why that is complete here);
  // the activations of the down pass are not: consumers wait for the previous kernel before touching them
  if (!DOWN) griddep_wait();
  const int n_groups = a.hdr[0];
  const int N = DOWN ? a.H : a.I;
  const int tiles = N / C::TR;
  const long long total = (long long)n_groups * tiles;
  const int i_begin = (int)(total * blockIdx.x / gridDim.x), i_end = (int)(total * (blockIdx.x + 1) / gridDim.x);
  const int n_items = i_end - i_begin;
  int gi = i_begin / tiles, tile = i_begin - gi * tiles;
  griddep_launch();

  if (warp == C::NW) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      int s = 0, issued = 0;
      uint32_t ph = 0;
      Group g = {nullptr, 0, 0};
      int cur = -1;
      for (; issued < n_items; ++issued) {
        if (!mbar_wait(&empty[s], ph ^ 1u, a.err, 1u)) break;
        if (!HB_BOUND(a.err, gi >= 0 && gi < n_groups && tile < tiles, 0x113u, gi)) break;
        if (gi != cur) { g = a.groups[gi]; cur = gi; }
        uint8_t* st = ring + (size_t)s * C::STAGE;
        mbar_expect_tx(&full[s], C::TX);
        const size_t r0 = (size_t)tile * C::TR;
        bulk_g2s(st, g.rec + a.off_wa + r0 * C::RB, C::TR * C::RB, &full[s]);
        bulk_g2s(st + C::TR * C::RB, g.rec + a.off_sa + r0 * C::RS, C::TR * C::RS, &full[s]);
        if (!DOWN) {
          bulk_g2s(st + C::UP_OFF, g.rec + a.off_wb + r0 * C::RB, C::TR * C::RB, &full[s]);
          bulk_g2s(st + C::UP_OFF + C::TR * C::RB, g.rec + a.off_sb + r0 * C::RS, C::TR * C::RS, &full[s]);
        }
        if (++tile == tiles) { tile = 0; ++gi; }
        if (++s == S) { s = 0; ph ^= 1u; }
      }
      // copies still in flight land before the CTA leaves (immediate when the consumers took every stage)
      for (int j = issued > S ? issued - S : 0; j < issued; ++j) mbar_wait(&full[j % S], (uint32_t)((j / S) & 1), a.err, 4u);
    }
    return;
  }

  const int g = lane >> 2, t = lane & 3;
  const int tok0 = 2 * t;
  // epilogue of one 16-row tile held in fragment layout: acc[c] = (row g + 8·(c>>1), activation row tok0 + (c&1))
  auto epilogue = [&](const float (&acc)[4], const Group& grp, const float (&gl)[3], int mt, int tile_) {
    if (DOWN) {
      const int n0 = tile_ * C::TR + 16 * mt + g;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int tok = tok0 + (c & 1), n = n0 + (c >> 1) * 8;
        if (tok < grp.n && HB_BOUND(a.err, grp.start + tok >= 0 && grp.start + tok < a.hdr[1] && n < a.H, 0x111u, grp.start + tok))
          a.outp[(size_t)(grp.start + tok) * a.H + n] = __float2bfloat16(acc[c] * gl[2]);
      }
    } else {
      float oth[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) oth[c] = __shfl_xor_sync(0xffffffffu, acc[c], 4);
      const bool odd = g & 1;
      const int i = tile_ * C::TR + 8 * mt + (g >> 1) + (odd ? 4 : 0);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float gv = odd ? oth[2 + c] : acc[c], uv = odd ? acc[2 + c] : oth[c];
        gv = bf16r(gv * gl[0]); uv = bf16r(uv * gl[1]);
        if (a.limit > 0.f) { uv = fminf(fmaxf(uv, -a.limit), a.limit); gv = fminf(gv, a.limit); }
        const float yv = gv / (1.f + __expf(-gv)) * uv;
        const int tok = tok0 + c;
        if (tok < grp.n && HB_BOUND(a.err, grp.start + tok >= 0 && grp.start + tok < a.hdr[1] && i < a.I, 0x112u, grp.start + tok))
          a.outp[(size_t)(grp.start + tok) * a.I + i] = __float2bfloat16(yv);
      }
    }
  };

  if (warp == C::NW + 1) {
    // ---------------------------------------------------------------- epilogue warp (split-K kernels only)
    if (WK == 1) return;
    int cur_group = -1, slot = 0;
    uint32_t rph = 0;
    Group grp = {nullptr, 0, 0};
    float gl[3] = {1.f, 1.f, 1.f};
    for (int it = 0; it < n_items; ++it) {
      if (gi != cur_group) {
        cur_group = gi;
        grp = a.groups[gi];
        const float* gp = reinterpret_cast<const float*>(grp.rec + a.off_g);
        gl[0] = __ldg(gp); gl[1] = __ldg(gp + 1); gl[2] = __ldg(gp + 2);
      }
      const float4* rb = red + (size_t)slot * C::NW * 32;
      bool ok = true;
#pragma unroll
      for (int mt = 0; mt < WM; ++mt) {
        ok = mbar_wait(&redbar[slot * WM + mt], rph, a.err, 8u);
        if (!ok) break;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k2 = 0; k2 < WK; ++k2) {                  // fixed order over the K slices: deterministic
          const float4 v = rb[(mt * WK + k2) * 32 + lane];
          acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        }
        epilogue(acc, grp, gl, mt, tile);
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&redfree[slot]);
      if (++tile == tiles) { tile = 0; ++gi; }
      if (++slot == NSLOT) { slot = 0; rph ^= 1u; }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  if (DOWN) griddep_wait();
  const int mt = warp / WK, ks = warp % WK;
  int rowA, rowB, matoff = 0;
  if (DOWN) { rowA = 16 * mt + g; rowB = rowA + 8; }
  else { rowA = 8 * mt + (g >> 1); rowB = rowA + 4; matoff = (g & 1) ? C::UP_OFF : 0; }
  const int wA = matoff + rowA * C::RB + ks * (kSlice / 2) + 32 * t, wB = matoff + rowB * C::RB + ks * (kSlice / 2) + 32 * t;
  const int sA = matoff + C::TR * C::RB + rowA * C::RS + ks * (kSlice / 16) + 4 * t, sB = matoff + C::TR * C::RB + rowB * C::RS + ks * (kSlice / 16) + 4 * t;

  uint32_t bfr[32];
  float inv[2] = {1.f, 1.f};
  float gl[3] = {1.f, 1.f, 1.f};
  int cur_group = -1;
  Group grp = {nullptr, 0, 0};
  int s = 0, slot = 0;
  uint32_t ph = 0, rph = 0;
  for (int it = 0; it < n_items; ++it) {
    if (gi != cur_group) {
      cur_group = gi;
      grp = a.groups[gi];
      const __nv_bfloat16* src = nullptr;
      if (g < grp.n) src = DOWN ? a.act + (size_t)(grp.start + g) * a.act_ld + ks * kSlice
                                : a.act + (size_t)a.s_row[grp.start + g] * a.act_ld + ks * kSlice;
      load_b_frags(src, t, bfr, inv);
      if (WK == 1) {
        const float* gp = reinterpret_cast<const float*>(grp.rec + a.off_g);
        gl[0] = __ldg(gp); gl[1] = __ldg(gp + 1); gl[2] = __ldg(gp + 2);
      }
    }
    if (!mbar_wait(&full[s], ph, a.err, 2u)) break;
    const uint8_t* st = ring + (size_t)s * C::STAGE;
    float acc[4];
    warp_slice_mma(st + wA, st + wB, st + sA, st + sB, bfr, acc, &empty[s]);
    acc[0] *= inv[0]; acc[1] *= inv[1]; acc[2] *= inv[0]; acc[3] *= inv[1];
    if (WK > 1) {
      if (!mbar_wait(&redfree[slot], rph ^ 1u, a.err, 16u)) break;      // the slot's previous contents have been read
      red[(size_t)slot * C::NW * 32 + warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(&redbar[slot * WM + mt]);
    } else {
      epilogue(acc, grp, gl, mt, tile);
    }
    if (++tile == tiles) { tile = 0; ++gi; }
    if (++s == S) { s = 0; ph ^= 1u; }
    if (++slot == NSLOT) { slot = 0; rph ^= 1u; }
  }
}

// The streaming kernel: the roles above, and for the down pass of the routed form the sums over each row's pairs at the end.  All CTAs
// of the grid are resident (the grid is sized by the occupancy the launcher planned), so they can meet: a CTA announces that its
// partial rows are written, waits (bounded) until every CTA has, and takes its share of the (row, column pair) units.
template <int WK, int WM, bool DOWN>
__global__ void __launch_bounds__(StreamCfg<WK, WM, DOWN>::THREADS, StreamCfg<WK, WM, DOWN>::CTAS_PER_SM) moe_stream_kernel(const StreamArgs a) {
  moe_stream_roles<WK, WM, DOWN>(a);
  if (!DOWN || !a.red_on) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(a.fin, 1u);
    uint32_t spins = 0;
    while (*reinterpret_cast<volatile unsigned int*>(a.fin) < gridDim.x) {
      if (++spins > (1u << 22)) { atomicOr(a.err, 0x8000u); break; }
      __nanosleep(32);
    }
    __threadfence();
  }
  __syncthreads();
  const size_t units = (size_t)a.red.M * a.red.H / 2, step = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < units; i += step) reduce_routed_unit(a.red, i);
  if (a.red.ep.world > 0) {
    // expert parallel: the sums were stored into the owning ranks' memory; when the last CTA is through, tell every rank
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(a.red.ep.done, 1u) == gridDim.x - 1) {
      *a.red.ep.done = 0;
      __threadfence_system();
      const uint32_t stepno = *a.red.ep.step + 1u;
      for (int p = 0; p < a.red.ep.world; ++p) st_release_sys(a.red.ep.flag[p] + a.red.ep.rank, stepno);
    }
  }
}

// ================================================================================================ reduce / combine
// Routed form: out[m] = Σ_k w[m,k]·part[pos] in k order; then either fp32 (overwritten) or the shared-expert combine → bf16.
__global__ void moe_reduce_routed_kernel(ReduceArgs r) {
  griddep_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // one thread per (row, 2 columns)
  if (i < (size_t)r.M * r.H / 2) reduce_routed_unit(r, i);
  if (r.ep.world > 0) {
    // expert parallel: the sums were stored into the owning ranks' memory; when the last block is through, tell every rank
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(r.ep.done, 1u) == gridDim.x - 1) {
      *r.ep.done = 0;
      __threadfence_system();
      const uint32_t step = *r.ep.step + 1u;
      for (int p = 0; p < r.ep.world; ++p) st_release_sys(r.ep.flag[p] + r.ep.rank, step);
    }
  }
}

// List form: out[row] += w·part, pairs visited in list order.  One block column per pair that is the first of its row.
__global__ void moe_reduce_list_kernel(const __nv_bfloat16* __restrict__ part, const int* __restrict__ pos_of, const int* __restrict__ prow,
                                       const float* __restrict__ pw, int n_pairs, int H, float* __restrict__ out) {
  griddep_wait();
  const int p = blockIdx.y;
  const int row = prow[p];
  for (int j = 0; j < p; ++j) if (prow[j] == row) return;             // not the first pair of its row
  const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (d >= H) return;
  float2 v = *reinterpret_cast<float2*>(out + (size_t)row * H + d);
  for (int q = p; q < n_pairs; ++q) {
    if (prow[q] != row) continue;
    const int pos = pos_of[q];
    if (pos < 0) continue;
    const __nv_bfloat162 e = *reinterpret_cast<const __nv_bfloat162*>(part + (size_t)pos * H + d);
    const float wv = pw[q];
    v.x = __fadd_rn(v.x, __fmul_rn(__bfloat162float(e.x), wv));
    v.y = __fadd_rn(v.y, __fmul_rn(__bfloat162float(e.y), wv));
  }
  *reinterpret_cast<float2*>(out + (size_t)row * H + d) = v;
}

// ================================================================================================ generic shapes (CUDA cores)
// One block per (sorted pair position, 8 output rows): a warp per output row, the activation row in shared memory as fp32.
template <bool DOWN>
__global__ void __launch_bounds__(256) moe_generic_kernel(StreamArgs a) {
  extern __shared__ float xs[];
  griddep_wait();
  const int n_valid = a.hdr[1];
  const int pos = blockIdx.y;
  if (pos >= n_valid) return;
  const int K = DOWN ? a.I : a.H, N = DOWN ? a.H : a.I;
  // the group that holds this position
  const int n_groups = a.hdr[0];
  int gi = 0;
  for (int lo = 0, hi = n_groups - 1; lo <= hi;) {
    const int mid = (lo + hi) >> 1;
    if (a.groups[mid].start <= pos) { gi = mid; lo = mid + 1; } else hi = mid - 1;
  }
  const uint8_t* rec = a.groups[gi].rec;
  const __nv_bfloat16* src = DOWN ? a.act + (size_t)pos * a.act_ld : a.act + (size_t)a.s_row[pos] * a.act_ld;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = __bfloat162float(src[k]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const float* gp = reinterpret_cast<const float*>(rec + a.off_g);
  float res[2] = {0.f, 0.f};
  for (int mat = 0; mat < (DOWN ? 1 : 2); ++mat) {
    const uint8_t* wr = rec + (mat ? a.off_wb : a.off_wa) + (size_t)n * (K / 2);
    const uint8_t* sr = rec + (mat ? a.off_sb : a.off_sa) + (size_t)n * (K / 16);
    float acc = 0.f;
    for (int b = lane; b < K / 16; b += 32) {
      const uint2 q = *reinterpret_cast<const uint2*>(wr + b * 8);
      const uint32_t w[2] = {q.x, q.y};
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) d = fmaf(xs[b * 16 + j], e2m1_to_f32((w[j >> 3] >> (4 * (j & 7))) & 15), d);
      acc = fmaf(d, e4m3_to_f32(sr[b]), acc);
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    res[mat] = acc;
  }
  if (lane != 0) return;
  if (DOWN) {
    a.outp[(size_t)pos * a.H + n] = __float2bfloat16(res[0] * gp[2]);
  } else {
    float gv = bf16r(res[0] * gp[0]), uv = bf16r(res[1] * gp[1]);
    if (a.limit > 0.f) { uv = fminf(fmaxf(uv, -a.limit), a.limit); gv = fminf(gv, a.limit); }
    a.outp[(size_t)pos * a.I + n] = __float2bfloat16(gv / (1.f + __expf(-gv)) * uv);
  }
}

}  // namespace hb

using namespace hb;

// ================================================================================================ host side
namespace {

constexpr int kWkList[] = {1, 2, 3, 4, 6, 8, 12, 16};
constexpr size_t kRouteSmemMax = 160 * 1024;       // shared memory the route + group kernel may ask for
constexpr int wm_for(int wk) { return wk >= 8 ? 1 : (wk >= 4 ? 2 : (wk == 3 ? 2 : (wk == 2 ? 4 : 8))); }

using StreamFn = void (*)(StreamArgs);
struct StreamKernel { StreamFn fn; int threads; int stage; size_t (*smem)(int); int tr; };

template <int WK, bool DOWN>
StreamKernel make_kernel() {
  constexpr int WM = wm_for(WK);
  using C = StreamCfg<WK, WM, DOWN>;
  return StreamKernel{moe_stream_kernel<WK, WM, DOWN>, C::THREADS, C::STAGE, &C::smem, C::TR};
}
template <bool DOWN>
bool pick_kernel(int K, StreamKernel* out) {
  if (K % kSlice) return false;
  switch (K / kSlice) {
    case 1: *out = make_kernel<1, DOWN>(); return true;
    case 2: *out = make_kernel<2, DOWN>(); return true;
    case 3: *out = make_kernel<3, DOWN>(); return true;
    case 4: *out = make_kernel<4, DOWN>(); return true;
    case 6: *out = make_kernel<6, DOWN>(); return true;
    case 8: *out = make_kernel<8, DOWN>(); return true;
    case 12: *out = make_kernel<12, DOWN>(); return true;
    case 16: *out = make_kernel<16, DOWN>(); return true;
    default: return false;
  }
}

// stages and CTAs per SM for a streaming kernel: as deep a ring as the shared memory allows, two CTAs per SM when the
// block is small enough
void plan_stream(const hb_ctx* ctx, const StreamKernel& k, int* stages, int* ctas_per_sm) {
  const int budget = ctx->smem_optin;                       // per block opt-in limit (227 KB on sm_100)
  const int per_sm = 228 * 1024;
  int cps = (k.threads <= 320) ? 2 : 1;
  for (;; --cps) {
    const int avail = (cps == 1 ? budget : per_sm / cps - 1024 - 1024);
    int s = kMaxStages;
    while (s > 2 && (long long)k.smem(s) > avail) --s;
    if ((long long)k.smem(s) <= avail && (s >= 3 || cps == 1)) { *stages = s; *ctas_per_sm = cps; return; }
  }
}

}  // namespace

bool hbk_moe_decode_fast(int H, int I) {
  StreamKernel a, b;
  return H > 0 && I > 0 && pick_kernel<false>(H, &a) && pick_kernel<true>(I, &b) && I % a.tr == 0 && H % b.tr == 0;
}

size_t hbk_moe_decode_ws_stream_bytes(int n, int H, int I) {
  if (n < 1) n = 1;
  return 256 + al256((size_t)n * sizeof(Group)) + 5 * al256((size_t)n * 4) + al256((size_t)n * I * 2) + al256((size_t)n * H * 2);
}
size_t hbk_moe_decode_ws_bytes(int n, int H, int I) { return hbk_moe_decode_ws_stream_bytes(n, H, I) + hbk_moe_dtc_ws_extra(n < 1 ? 1 : n, H, I); }

int hbk_moe_decode_setup(hb_ctx* ctx) {
  int n_down = 0;
  static_assert(sizeof(kWkList) / sizeof(kWkList[0]) <= 8, "hb_ctx::down_fn");
  for (int wk : kWkList) {
    StreamKernel k[2];
    pick_kernel<false>(wk * kSlice, &k[0]);
    pick_kernel<true>(wk * kSlice, &k[1]);
    for (auto& kk : k) {
      int s, c;
      plan_stream(ctx, kk, &s, &c);
      HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(kk.fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kk.smem(s)));
    }
    {
      // may the down kernel's CTAs wait for one another?  Only if the runtime agrees that the planned CTAs per SM fit
      int s, c, occ = 0;
      plan_stream(ctx, k[1], &s, &c);
      HB_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, reinterpret_cast<const void*>(k[1].fn), k[1].threads, k[1].smem(s)));
      ctx->down_fn[n_down] = reinterpret_cast<const void*>(k[1].fn);
      ctx->down_meet[n_down] = occ >= c;
      ++n_down;
    }
  }
  {
    int rf = hbk_moe_fused_setup(ctx);
    if (!rf) rf = hbk_moe_dtc_setup(ctx);
    if (rf) return rf;
  }
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(moe_group_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)kRouteSmemMax));
  return HB_OK;
}

int hbk_moe_decode_run(hb_ctx* ctx, const hbk_pair_src& src, const void* x, int H, int I, float limit, const hbk_reduce& red, void* ws,
                       cudaStream_t st) {
  const bool routed = src.ids != nullptr;
  const int P = routed ? src.M * src.K + (src.shared_rec ? src.M : 0) : src.n_pairs;
  if (P <= 0) return HB_OK;
  DecodeWs w = carve(ws, P, H, I);
  hb_rec_layout L;
  hb_rec_layout_make(H, I, &L);

  GroupArgs ga{};
  ga.pairs = src.pairs; ga.n_pairs = src.n_pairs; ga.ids = src.ids; ga.w = src.w; ga.M = src.M; ga.K = src.K;
  ga.tab = src.tab; ga.li = src.li; ga.E = src.E; ga.shared_rec = src.shared_rec; ga.ws = w;
  ga.ld_ids = src.ld_ids ? src.ld_ids : src.K; ga.sh_row0 = src.sh_row0; ga.sh_rows = src.sh_rows < 0 ? src.M : src.sh_rows;
  ga.wait_flags = src.wait_flags; ga.wait_n = src.wait_n; ga.wait_step = src.wait_step; ga.wait_err = ctx->dev_err;
  // Which gate/up engine: a context may pin either (HB_FLAG_DECODE_MMA_SYNC / HB_FLAG_DECODE_TC_GU).  Unpinned, the tensor-memory
  // kernel takes calls of kTcGuMinPairs pairs or more — below that its start-up (tensor-memory allocation, work table, first TMA
  // boxes) costs more than its faster stream saves (measured: 30.6 vs 27.6 µs per layer at 11 pairs, 73 vs 81 µs at 176).
  // Expert parallel (rows of all ranks, most pairs dead on this rank): what counts is this rank's share of the pairs, and with many
  // gathered rows the digit planes of rows this rank has nothing for cost more than the faster stream saves (measured at 8 ranks ×
  // 16 rows: 109 vs 99 µs per layer; at 4 ranks × 16 rows: 99 vs 103 µs; at 2 ranks: 101 vs 108 µs) — unpinned contexts take the
  // tensor-memory kernel up to 64 gathered rows.
  bool tc_gu = false;
  if (routed && !src.ws_stream_only && src.tab && hbk_moe_decode_fast(H, I) && hbk_moe_dtc_supported(H, I) && hbk_moe_dtc_gu_fits(ctx, P, src.E, H, I) &&
      !(ctx->flags & (HB_FLAG_DECODE_MMA_SYNC | HB_FLAG_FUSED))) {
    const int ranks = red.ep ? red.ep->world : 1;
    const int pairs_eff = (P > src.pairs_hint ? P : src.pairs_hint) / ranks;
    const bool auto_tc = pairs_eff >= kTcGuMinPairs && (ranks == 1 || src.M <= 64);
    tc_gu = (ctx->flags & (HB_FLAG_DECODE_TC_GU | HB_FLAG_DECODE_TC)) || auto_tc;
  }
  ga.group_rows = tc_gu ? 2 : kGroupRows;
  const int x_ld = src.x_ld ? src.x_ld : H;
  if (src.route && ga.ld_ids != src.K) return hb_fail(ctx, HB_ERR_INVALID, "moe_decode: in-kernel routing writes dense ids / w rows");
  int route = src.route;
  if (route && group_smem(true, P, src.E, route) > kRouteSmemMax) {
    // the per-warp router scratch does not fit beside the grouping arrays (large E): route with the stand-alone kernel first
    int rr = route == 1 ? hbk_route_softmax_topk(ctx, src.logits, src.ld, src.M, src.E, src.K, src.renorm, src.logits_bf16, const_cast<int32_t*>(src.ids),
                                                 const_cast<float*>(src.w), st, true)
                        : hbk_route_sigmoid_topk(ctx, src.logits, src.bias, src.M, src.E, src.K, src.sig_scale, const_cast<int32_t*>(src.ids),
                                                 const_cast<float*>(src.w), st, true);
    if (rr) return rr;
    route = 0;
  }
  ga.route = route; ga.logits = src.logits; ga.ld = src.ld; ga.renorm = src.renorm; ga.logits_bf16 = src.logits_bf16; ga.bias = src.bias;
  ga.sig_scale = src.sig_scale; ga.ids_out = const_cast<int32_t*>(src.ids); ga.w_out = const_cast<float*>(src.w);
  int r = hb_launch(ctx, route ? "moe_route_group" : "moe_group", true, moe_group_kernel, dim3(1), dim3(kGroupThreads), group_smem(routed, P, src.E, route),
                    st, ga);
  if (r) return r;

  StreamArgs sa{};
  sa.hdr = w.hdr; sa.groups = w.groups; sa.s_row = w.s_row; sa.H = H; sa.I = I; sa.limit = limit; sa.err = ctx->dev_err;
  sa.off_g = (uint32_t)L.g;
  StreamArgs sd = sa;
  sa.act = reinterpret_cast<const __nv_bfloat16*>(x); sa.act_ld = x_ld; sa.outp = w.y;
  sa.off_wa = (uint32_t)L.w1; sa.off_sa = (uint32_t)L.s1; sa.off_wb = (uint32_t)L.w3; sa.off_sb = (uint32_t)L.s3;
  sd.act = w.y; sd.act_ld = I; sd.outp = w.part;
  sd.off_wa = (uint32_t)L.w2; sd.off_sa = (uint32_t)L.s2;

  if (x_ld != H && !hbk_moe_decode_fast(H, I)) return hb_fail(ctx, HB_ERR_UNSUPPORTED, "moe_decode: strided activation rows need a shape of the streaming path");
  if (hbk_moe_fused_available(H, I) && (ctx->flags & HB_FLAG_FUSED) && x_ld == H && !red.ep) {
    // one persistent kernel: gate/up → down → (routed form) reduce + combine
    if (routed) {
      ReduceArgs ra{w.part, w.pos_of, w.pw, src.M, src.K, H, src.shared_rec ? 1 : 0, reinterpret_cast<const __nv_bfloat16*>(red.shared), red.lg, red.ld, red.col,
                    reinterpret_cast<__nv_bfloat16*>(red.out_bf16), red.out_f32, reinterpret_cast<__nv_bfloat16*>(red.shared_out), ga.sh_row0, ga.sh_rows,
                  red.ep ? *red.ep : hbk_ep_push{}, ctx->dev_err, P};
      return hbk_moe_fused_launch(ctx, w, x, H, I, limit, L, &ra, st);
    }
    if ((r = hbk_moe_fused_launch(ctx, w, x, H, I, limit, L, nullptr, st))) return r;
  } else if (hbk_moe_decode_fast(H, I)) {
    // PDL chain: group → gate/up → down → reduce.  Each streaming kernel calls griddepcontrol.launch_dependents only after its own
    // griddepcontrol.wait returned (gate/up) or after reading the group list (down), so when the down kernel's producer starts,
    // the grouping kernel has completed and its list is visible; the down consumers wait for gate/up before reading y.
    StreamKernel kg, kd;
    pick_kernel<false>(H, &kg);
    pick_kernel<true>(I, &kd);
    int s, c;
    plan_stream(ctx, kg, &s, &c);
    sa.stages = s;
    int grid = ctx->sm_count * c;
    if (ctx->max_ctas > 0 && grid > ctx->max_ctas) grid = ctx->max_ctas;
    if (tc_gu) {
      // gate/up on the block-scaled tensor cores: digit planes of the rows (beside the grouping kernel), then the tensor-memory kernel
      if ((r = hbk_moe_dtc_gu_run(ctx, x, x_ld, src.M, src.tab + (size_t)src.li * src.E, src.E, src.shared_rec, P, H, I, limit, ws, src.wait_flags, src.wait_n, src.wait_step, st)))
        return r;
    } else if ((r = hb_launch(ctx, "moe_gate_up", true, kg.fn, dim3(grid), dim3(kg.threads), kg.smem(s), st, sa))) return r;
    if (tc_gu && routed && !red.ep && (ctx->flags & HB_FLAG_DECODE_TC_DOWN) && hbk_moe_dtc_down_fits(ctx, P, src.E, H, I)) {
      const ReduceArgs ra{w.part, w.pos_of, w.pw, src.M, src.K, H, src.shared_rec ? 1 : 0, reinterpret_cast<const __nv_bfloat16*>(red.shared), red.lg, red.ld, red.col,
                          reinterpret_cast<__nv_bfloat16*>(red.out_bf16), red.out_f32, reinterpret_cast<__nv_bfloat16*>(red.shared_out), ga.sh_row0, ga.sh_rows,
                          hbk_ep_push{}, ctx->dev_err, P};
      return hbk_moe_dtc_down_run(ctx, P, H, I, ws, &ra, reinterpret_cast<unsigned int*>(w.hdr + 3), st);
    }
    plan_stream(ctx, kd, &s, &c);
    sd.stages = s;
    grid = ctx->sm_count * c;
    if (ctx->max_ctas > 0 && grid > ctx->max_ctas) grid = ctx->max_ctas;
    bool meet = false;
    for (int j = 0; j < 8; ++j) if (ctx->down_fn[j] == reinterpret_cast<const void*>(kd.fn)) meet = ctx->down_meet[j];
    if (routed && meet && !red.ep) {
      // the down pass sums the rows' pairs itself (its CTAs meet at the end): no reduce launch.  (Expert parallel keeps the separate
      // reduce kernel: pushing the sums to the other ranks from the down kernel's tail measured 2 µs slower per layer at 2 ranks and more
      // at 8 — the stores start only after every CTA of the long kernel has arrived.)
      sd.red_on = 1; sd.fin = reinterpret_cast<unsigned int*>(w.hdr + 3);
      sd.red = ReduceArgs{w.part, w.pos_of, w.pw, src.M, src.K, H, src.shared_rec ? 1 : 0, reinterpret_cast<const __nv_bfloat16*>(red.shared), red.lg, red.ld, red.col,
                          reinterpret_cast<__nv_bfloat16*>(red.out_bf16), red.out_f32, reinterpret_cast<__nv_bfloat16*>(red.shared_out), ga.sh_row0, ga.sh_rows,
                          red.ep ? *red.ep : hbk_ep_push{}, ctx->dev_err, P};
      return hb_launch(ctx, red.ep ? "moe_down_reduce_push" : "moe_down_reduce", true, kd.fn, dim3(grid), dim3(kd.threads), kd.smem(s), st, sd);
    }
    if ((r = hb_launch(ctx, "moe_down", true, kd.fn, dim3(grid), dim3(kd.threads), kd.smem(s), st, sd))) return r;
  } else {
    if ((r = hb_launch(ctx, "moe_gate_up_generic", true, moe_generic_kernel<false>, dim3((I + 7) / 8, P), dim3(256), (size_t)H * 4, st, sa))) return r;
    if ((r = hb_launch(ctx, "moe_down_generic", true, moe_generic_kernel<true>, dim3((H + 7) / 8, P), dim3(256), (size_t)I * 4, st, sd))) return r;
  }

  if (routed) {
    ReduceArgs ra{w.part, w.pos_of, w.pw, src.M, src.K, H, src.shared_rec ? 1 : 0, reinterpret_cast<const __nv_bfloat16*>(red.shared), red.lg, red.ld, red.col,
                  reinterpret_cast<__nv_bfloat16*>(red.out_bf16), red.out_f32, reinterpret_cast<__nv_bfloat16*>(red.shared_out), ga.sh_row0, ga.sh_rows,
                  red.ep ? *red.ep : hbk_ep_push{}, ctx->dev_err, P};
    return hb_launch(ctx, "moe_reduce_routed", true, moe_reduce_routed_kernel, dim3((unsigned)(((size_t)src.M * H / 2 + 255) / 256)), dim3(256), 0, st, ra);
  }
  return hb_launch(ctx, "moe_reduce_list", true, moe_reduce_list_kernel, dim3((H / 2 + 255) / 256, P), dim3(256), 0, st, (const __nv_bfloat16*)w.part,
                   (const int*)w.pos_of, (const int*)w.prow, (const float*)w.pw, P, H, red.out_accum);
}
