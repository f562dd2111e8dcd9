// Routed-expert decode on the block-scaled tensor cores: the NVFP4 records go from HBM through shared memory into
// `tcgen05.mma kind::mxf4nvf4` untouched — no instruction ever handles a weight.
//
// The tensor core multiplies FP4 by FP4, the operators take bf16 activations (the reference's W4A16 arithmetic).  A bf16 row is
// therefore written, exactly, as eight FP4 "digit planes": with the row's largest exponent E, every element is the integer
// X = x / 2^(E-21) (|X| < 2^22; exact for elements down to 2^-15 of the row maximum, rounded to nearest below that — finer than
// an fp32 accumulation resolves), and X = Σ_p d_p·8^(7-p) in balanced base 8, digits d_p ∈ {-4 … 4}, all of which e2m1 holds.
// The eight planes are eight B-operand rows (block scales 1.0); the weights are the A operand with their own e4m3 block scales
// applied by the tensor core; the accumulator columns of one activation row are recombined in fp32 by Horner's rule:
//     Σ_k w_k·x_k = 2^(E-21) · Σ_p 8^(7-p) · D[·, p].
// Every product is exact; sums are fp32.  Rounding points after the products are the reference's (g, u → bf16 after the global
// scale, y → bf16, down → bf16, fp32 sum in k order).
//
// Two launches per layer:
//   prep   one CTA per activation row: (optional) routing of the row, the row's digit planes; the last CTA to finish sorts the
//          (row, expert) pairs into groups of ≤ 8 rows per expert and clears the hand-over flags
//   layer  persistent CTAs, one per SM.  Work items: gate/up = (group, 64 rows of I: 64 gate rows + 64 up rows form one 128-row
//          A tile), down = (group, 128 rows of H).  Items are dealt round-robin; a CTA's list interleaves the gate/up items of
//          round r with the down items of the groups whose gate/up finished in round r-1, so no down item ever waits for a
//          gate/up item that is not already done or in its last microseconds.  Per CTA: a TMA thread streams weight boxes
//          (128 bytes × 64/128 rows, 128-byte swizzle) through tensor maps anchored below the records, a second thread brings the
//          digit planes (pre-swizzled 1 KB atoms, plain bulk copies), four warps fetch the e4m3 scales two windows ahead and
//          lay them out as the 32 × 16-byte chunks `tcgen05.cp` moves to tensor memory, one thread issues the MMAs
//          (128 × N × 64, N = 16 … 64) into double-buffered accumulators, four warps run the epilogues: SwiGLU → y → (last
//          finisher of a group) y's digit planes; down → bf16 partial rows → (last arriver of a row's 128-column block) the
//          k-order sum and the shared-expert combine.
// Every wait is bounded and reports through the context's error word.
#include "moe_stream.cuh"
#include "router.cuh"
#include "ep.cuh"
#include "tc_common.cuh"

namespace hb {

constexpr int DT_ST = 10;                       // pipeline stages
constexpr int DT_A = 16384;                    // weight tile of a stage: 128 rows × 128 bytes (256 k values)
constexpr int DT_B = 2048;                     // digit planes of a stage: 2 activation rows × 8 planes × 128 bytes (the grouping kernel makes groups of ≤ 2 rows
                                               // for this kernel: most experts of a decode batch get one or two rows, and a small slot leaves room for more stages)
constexpr int DT_STAGE = DT_A + DT_B;
constexpr int DT_RAWD = 3;                     // windows the scale fetch runs ahead of its use
constexpr int DT_RAW = (DT_RAWD + 1) * 2048;   // ring of fetched scale rows: 128 rows × 16 bytes per window
constexpr int DT_EX = 8 * 64 * 4;              // SwiGLU exchange: up values of 64 rows × 8 activation rows
constexpr int DT_TBL = 256;                    // work-list entries a CTA can hold (16 bytes + 8 row indices + 8 row units each)
constexpr int DT_SFBC = 16 * 8 * 32;              // block-scale codes of the down items in flight: [16 items][8 rows][≤ 32 slices]
constexpr int DT_SMEM = 1024 + DT_ST * DT_STAGE + DT_RAW + 2 * DT_EX + DT_SFBC + 1024 + DT_TBL * 64;
constexpr int DT_THREADS = 16 * 32;            // warps 0-7 epilogues (two sets of four), then one warp each: MMA issue, weight TMA, digit copies,
                                               // (one idle); warps 12-15 fetch the scales and store them into tensor memory
constexpr int DT_W_MMA = 8, DT_W_TMA = 9, DT_W_DIG = 10, DT_W_SC0 = 12;   // warp 11 idles: the scale warps must be warps 0-3 modulo 4
constexpr int DT_TMEM_COLS = 512;              // accumulators 2 × 64, then 32 columns per stage (16 of weight scales), then 16 columns of 1.0
constexpr int DT_SFA_COL0 = 128;               // per stage 32 columns: 16 of weight scales, 16 of digit-plane scales (down items)
constexpr int DT_SFB1_COL = DT_SFA_COL0 + DT_ST * 32;   // 16 columns of 1.0: the digit-plane scales of gate/up items
constexpr int DT_VMAX = 32;                    // tensor-map variants per matrix kind (see DtcMeta)
constexpr int DT_GU_ROWS = 64;                 // rows of I per gate/up item
constexpr int DT_DN_ROWS = 128;                // rows of H per down item
static_assert(DT_STAGE % 1024 == 0, "stage buffers keep the swizzle atom's alignment");
static_assert(DT_SFB1_COL + 16 <= DT_TMEM_COLS, "tensor memory");
static_assert(DT_SMEM <= 227 * 1024, "shared memory");

// Tensor maps for the weight boxes cannot be made per record ahead of time (the table may change between calls) and records sit
// at arbitrary 4096-aligned addresses.  One map per matrix kind covers them all: a 2-D byte matrix [2^31 rows][pitch] whose base
// lies 2^30 rows below the lowest record seen when the maps were made.  A matrix whose distance from that base is not a multiple
// of the pitch uses variant v of the map, shifted by v·gcd(pitch, 4096) bytes (pitch / gcd variants cover every residue).
struct DtcMeta { unsigned long long anchor[2]; };

struct DtcWs {
  uint8_t* xdig;        // [rows][H/256][8 planes][128 bytes], swizzled
  uint8_t* ydig;        // [pairs][I/256][8][128]; the 64 values of a gate/up item are digitised against their own exponent
  uint8_t* yexp;        // [pairs][I/64, padded to 8] that exponent (biased), per pair and 64-value slice; 0 = slice not written yet
  float* xs;            // [rows] unit of a row's digits (a power of two)
  unsigned int* fin;    // CTAs of the layer kernel whose partial rows are all written
  uint16_t* g_row;      // [groups][8] activation rows of a group
  float* g_unit;        // [groups][8] digit units of those rows
};

// Division of a 32-bit unsigned number by a divisor fixed for the whole launch: multiply-high and shift (exact for n < 2^31).
struct DtDiv {
  uint32_t d, m, l;
  __host__ __device__ void set(uint32_t d_) {
    d = d_; l = 0;
    while ((1u << l) < d) ++l;
    m = (uint32_t)(((1ull << 32) * ((1ull << l) - d)) / d + 1);
  }
  __device__ uint32_t div(uint32_t n) const { return (uint32_t)(((unsigned long long)__umulhi(n, m) + n) >> l); }
};

struct DtcArgs {
  int gu_only;          // 1: only the gate/up items run, y leaves as bf16 rows [pos, I] (`y`) for the streaming down kernel; rows and units of a
                       //    group come from s_row / xs (the streaming path's grouping kernel made the list)
  const int* hdr; const Group* groups; const int* s_row;
  int H, I; float limit;
  DtDiv dIT, dHT, dG;                                    // dividers by the items per group (gate/up, down) and by the grid size
  hb_rec_layout L;
  const CUtensorMap* maps; const DtcMeta* meta;          // maps[kind · DT_VMAX + variant], kind 0 = gate/up, 1 = down
  int pitch[2], gstep[2], pshift[2];                     // pshift: log2(pitch) when the pitch divides 4096, else -1
  DtcWs dw;
  __nv_bfloat16* y; __nv_bfloat16* part;
  unsigned int* done;
  ReduceArgs red;
  uint32_t* err;
};

// ---- digit planes ------------------------------------------------------------------------------------------------------------------
// One bf16 value → its eight digits, nibble p = the e2m1 code of plane p.
__device__ __forceinline__ uint32_t dt_digits1(uint32_t b, int eb) {
  const uint32_t ex = (b >> 7) & 0xffu;
  const uint32_t mant = ex ? ((b & 0x7fu) | 0x80u) : (b & 0x7fu);
  const int sh = (int)(ex ? ex : 1u) - eb + 14;
  uint32_t X;
  if (sh >= 0) X = mant << sh;
  else if (sh < -9) X = 0u;
  else {
    const int s2 = -sh;
    const uint32_t q = mant >> s2, rem = mant & ((1u << s2) - 1u), half = 1u << (s2 - 1);
    X = q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u);
  }
  const uint32_t Y = X + 0x924924u;
  const uint32_t tbl = (b & 0x8000u) ? 0xDCA02456u : 0x5420ACDEu;
  uint32_t w = 0u;
#pragma unroll
  for (int p = 0; p < 8; ++p) w |= ((tbl >> (((Y >> (3 * (7 - p))) & 7u) << 2)) & 0xfu) << (4 * p);
  return w;
}
// Eight consecutive bf16 values (v: four packed pairs) of a row whose largest biased exponent is eb → one 32-bit word per plane
// (plane 0 = most significant digit), nibble j = element j as an e2m1 code.
__device__ __forceinline__ void dt_digits8(const uint32_t (&v)[4], int eb, uint32_t (&plane)[8]) {
#pragma unroll
  for (int p = 0; p < 8; ++p) plane[p] = 0u;
  unsigned long long lo = ((unsigned long long)v[1] << 32) | v[0], hi = ((unsigned long long)v[3] << 32) | v[2];
#pragma unroll 1
  for (int j = 0; j < 8; ++j) {                                       // rolled: this runs once per thread and launch, its size is its cost
    const uint32_t w = dt_digits1((uint32_t)lo & 0xffffu, eb);
    lo = (lo >> 16) | (hi << 48); hi >>= 16;
#pragma unroll
    for (int p = 0; p < 8; ++p) plane[p] |= ((w >> (4 * p)) & 0xfu) << (4 * j);
  }
}
// Eight consecutive lanes hold one such word each (lane l: the digits of element l); afterwards lane l holds plane l's word of the
// eight elements (nibble e = element e): an 8 × 8 transpose of nibbles in three exchange steps.
__device__ __forceinline__ uint32_t dt_transpose8(uint32_t x, int lane) {
#pragma unroll
  for (int s = 4; s >= 1; s >>= 1) {
    const uint32_t m = s == 4 ? 0x0000ffffu : s == 2 ? 0x00ff00ffu : 0x0f0f0f0fu;     // nibbles whose index has bit s clear
    const uint32_t y = __shfl_xor_sync(0xffffffffu, x, s);
    x = (lane & s) ? ((x & ~m) | ((y & ~m) >> (4 * s))) : ((x & m) | ((y & m) << (4 * s)));
  }
  return x;
}
__device__ __forceinline__ int dt_row_exponent(uint32_t amax_bits) {   // biased exponent the digits are taken against
  int eb = (int)(amax_bits >> 7) & 0xff;
  return min(max(eb, 30), 254);                                       // tiny rows: keep the unit a normal float
}
__device__ __forceinline__ float dt_unit(int eb) { return __int_as_float((uint32_t)(eb - 21) << 23); }   // 2^(eb - 148)
// where the word of plane p for elements [k0, k0 + 8) of row `r` goes (rows of K values)
__device__ __forceinline__ size_t dt_dig_off(size_t r, int K, int k0, int p) {
  const int kb = k0 >> 8, bo = ((k0 & 255) >> 3) << 2;
  return ((r * (size_t)(K >> 8) + kb) * 8 + p) * 128 + (size_t)((((bo >> 4) ^ p) << 4) + (bo & 15));
}

// ---- the work list of a CTA -----------------------------------------------------------------------------------------------------------
// Items: gate/up = (group g, rows [64 t, 64 t + 64) of I), down = (group g, rows [128 t, 128 t + 128) of H).  Gate/up item j of the
// launch goes to CTA j mod grid in round j / grid; the down items of a group follow `lag` rounds after the round in which the
// group's last gate/up item runs, dealt round-robin in their own numbering.  A CTA's list is: round 0's gate/up item, round 0's
// down items, round 1's ….  Every CTA builds its list once, into shared memory, before its pipeline starts.
struct DtEnt { const uint8_t* rec; int start; uint32_t info; };      // info: bit 0 kind, bits 1-4 rows of the group, bits 5-15 t, bits 16-31 g
static_assert(sizeof(DtEnt) == 16, "DtEnt layout");
__device__ __forceinline__ int ent_kind(const DtEnt& e) { return (int)(e.info & 1u); }
__device__ __forceinline__ int ent_n(const DtEnt& e) { return (int)((e.info >> 1) & 15u); }
__device__ __forceinline__ int ent_t(const DtEnt& e) { return (int)((e.info >> 5) & 0x7ffu); }
__device__ __forceinline__ int ent_g(const DtEnt& e) { return (int)(e.info >> 16); }

// A CTA's list: first its gate/up items, then its down items.  Gate/up item j of the launch goes to CTA j mod grid, so the items of
// one group run on different CTAs at the same time and the groups finish in the order of their numbers; down item d (numbered
// group by group) is dealt so that every CTA streams about the same number of bytes — the gate/up items do not divide evenly over
// the CTAs (rem "heavy" CTAs have one more than the others):
//   d < D1           all CTAs in turn               (q_h passes: what a heavy CTA can take before it exceeds the mean)
//   D1 ≤ d < D2      the light CTAs in turn         (the extra passes that bring them up to the mean)
//   D2 ≤ d           all CTAs in turn               (what is left)
// Both parts of a CTA's list ascend in group number, so its down items meet y rows that were finished long before, except at the
// very end of the list.  The list is four arithmetic progressions: entry x is computed directly.
struct DtList {
  int grid, nIT, nHT, L, cntGU, cnt1, cnt2, first2, first3, total, c;
  DtDiv dIT, dHT;
  __device__ void init(int G, const DtDiv& dIT_, const DtDiv& dHT_, const DtDiv& dG, int sGU, int sDN, int c_) {
    dIT = dIT_; dHT = dHT_; nIT = (int)dIT.d; nHT = (int)dHT.d; grid = (int)dG.d; c = c_;
    const int nGU = G * nIT, nD = G * nHT;
    const int gu_l = (int)dG.div(nGU), rem = nGU - gu_l * grid, gu_h = gu_l + (rem ? 1 : 0);
    L = grid - rem;
    const int target = (int)dG.div((uint32_t)(nGU * sGU + nD * sDN));
    const int q_h = max(0, (target - gu_h * sGU) / sDN), q_l = max(q_h, (target - gu_l * sGU) / sDN);
    const int D1 = min(nD, q_h * grid), D2 = rem ? min(nD, D1 + (q_l - q_h) * L) : D1;
    cntGU = c < nGU ? (int)dG.div((uint32_t)(nGU - 1 - c)) + 1 : 0;
    cnt1 = c < D1 ? (int)dG.div((uint32_t)(D1 - 1 - c)) + 1 : 0;
    first2 = D1 + (c - rem);
    cnt2 = (c >= rem && first2 < D2) ? (D2 - 1 - first2) / L + 1 : 0;
    first3 = D2 + c;
    cnt3_ = first3 < nD ? (int)dG.div((uint32_t)(nD - 1 - first3)) + 1 : 0;
    total = cntGU + cnt1 + cnt2 + cnt3_;
  }
  int cnt3_;
  __device__ uint32_t info(int x) const {                 // kind | t << 5 | g << 16 of entry x
    if (x < cntGU) { const int j = c + x * grid, g = (int)dIT.div((uint32_t)j); return 0u | ((uint32_t)(j - g * nIT) << 5) | ((uint32_t)g << 16); }
    x -= cntGU;
    int d;
    if (x < cnt1) d = c + x * grid;
    else if (x < cnt1 + cnt2) d = first2 + (x - cnt1) * L;
    else d = first3 + (x - cnt1 - cnt2) * grid;
    const int g = (int)dHT.div((uint32_t)d);
    return 1u | ((uint32_t)(d - g * nHT) << 5) | ((uint32_t)g << 16);
  }
};

// Optional in-kernel timing (compile with -DHB_DTC_TRACE): every role of every CTA sums the clocks it spends in each kind of wait.
#ifdef HB_DTC_TRACE
__device__ long long g_dt_trace[256 * 32];
#define DT_TIMED(acc, stmt) do { const long long t_ = clock64(); stmt; acc += clock64() - t_; } while (0)
#define DT_TRACE_PUT(slot, v) g_dt_trace[blockIdx.x * 32 + (slot)] = (v)
__device__ __forceinline__ void g_dt_trace_prep_put(long long v) { g_dt_trace[200 * 32] = v; }
__device__ long long g_dt_stage[2 * 128 * 8];
#define DT_STAMP(it, col) do { if ((blockIdx.x == 0 || blockIdx.x == 77) && (it) < 128) g_dt_stage[((blockIdx.x ? 1 : 0) * 128 + (it)) * 8 + (col)] = clock64(); } while (0)
#else
#define DT_TIMED(acc, stmt) do { stmt; } while (0)
#define DT_TRACE_PUT(slot, v) do { } while (0)
__device__ __forceinline__ void g_dt_trace_prep_put(long long) {}
#define DT_STAMP(it, col) do { } while (0)
#endif

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_u32(const unsigned int* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(unsigned int* p, uint32_t v) { asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

// ---- the layer kernel -------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(DT_THREADS, 1) moe_dtc_layer_kernel(const DtcArgs a) {
  extern __shared__ uint8_t dt_raw[];
  const uint32_t raw = smem_u32(dt_raw), base = (raw + 1023u) & ~1023u;
  uint8_t* sm = dt_raw + (base - raw);
  uint8_t* rawsc = sm + DT_ST * DT_STAGE;                                       // fetched scale rows
  float* ex_all = reinterpret_cast<float*>(rawsc + DT_RAW);                     // [2 sets][8][64]
  uint8_t* sfbc = reinterpret_cast<uint8_t*>(ex_all) + 2 * DT_EX;               // [16][8][32] e4m3 codes 2^(slice exponent - row reference) of down items
  uint64_t* full = reinterpret_cast<uint64_t*>(sfbc + DT_SFBC);                     // [ST] weights and digits of the stage are in shared memory, its scales in tensor memory
  uint64_t* empty = full + DT_ST;                                               // [ST] the MMAs that read the stage are done
  uint64_t* bmeta = empty + DT_ST;                                              // [ST] the stage's digit-plane scale codes are in shared memory
  uint64_t* acc_full = bmeta + DT_ST;                                           // [2]
  uint64_t* acc_empty = acc_full + 2;                                           // [2]
  uint64_t* mma_done = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + 1);
  volatile int* flag_all = reinterpret_cast<volatile int*>(tmem_slot + 1);      // [2 sets][24] epilogue hand-over words: [8..23] the two gate warps' row maxima
  float* rowsc = reinterpret_cast<float*>(const_cast<int*>(flag_all) + 48);     // [16 items in flight][8] units of the item's activation rows
  DtEnt* tbl = reinterpret_cast<DtEnt*>(sfbc + DT_SFBC + 1024);                     // [DT_TBL] this CTA's work list
  uint16_t* tbl_row = reinterpret_cast<uint16_t*>(tbl + DT_TBL);                // [DT_TBL][8] activation rows of the item's group
  float* tbl_unit = reinterpret_cast<float*>(tbl_row + DT_TBL * 8);             // [DT_TBL][8] digit units of those rows (gate/up items)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  [[maybe_unused]] const long long t_k0 = clock64();
  if (threadIdx.x == 0) {
    for (int s = 0; s < DT_ST; ++s) { mbar_init(&full[s], 128 + 2); mbar_init(&empty[s], 1); mbar_init(&bmeta[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
    mbar_init(mma_done, 1);
    mbar_fence_init();
  }
  if (warp == DT_W_MMA) { tmem_alloc(tmem_slot, DT_TMEM_COLS); tmem_relinquish(); }
  // the first variant of each kind's tensor map (the only one when the pitch divides 4096) is made visible to the TMA thread before
  // the wait: the maps were stamped by an earlier launch that has completed
  if (threadIdx.x == DT_W_TMA * 32) { tmap_acquire(a.maps); tmap_acquire(a.maps + DT_VMAX); }
  griddep_wait();                                                               // the prep kernel's lists, digit planes and cleared flags
  griddep_launch();
  [[maybe_unused]] const long long t_k1 = clock64();
  const int nIT = a.I / DT_GU_ROWS, nHT = a.H / DT_DN_ROWS;
  DtList lst;
  lst.init(a.hdr[0], a.dIT, a.dHT, a.dG, a.H >> 8, a.I >> 8, (int)blockIdx.x);
  int n_items = a.gu_only ? lst.cntGU : 0;                                      // only the gate/up form is dispatched (the digit-plane slot holds two rows)
  if (!a.gu_only && threadIdx.x == 0) atomicOr(a.err, 0x1000u);
  if (n_items > DT_TBL) { if (threadIdx.x == 0) atomicOr(a.err, 0x1000u); n_items = 0; }   // the launcher sizes the grid so that this does not happen
  for (int j = threadIdx.x; j < n_items * kGroupRows; j += DT_THREADS) {       // records, row ranges, activation rows and their digit units
    const int i = j >> 3, c = j & 7;
    const uint32_t info = lst.info(i);
    const Group g = a.groups[info >> 16];
    if (a.gu_only) {
      const int row = c < g.n ? a.s_row[g.start + c] : 0;
      tbl_row[j] = (uint16_t)row; tbl_unit[j] = 0.f;                            // the epilogue fetches the rows' units itself, off the start-up path
    } else {
      const size_t gj = (size_t)(info >> 16) * kGroupRows + c;
      tbl_row[j] = a.dw.g_row[gj]; tbl_unit[j] = a.dw.g_unit[gj];
    }
    if (c == 0) {
      if (g.n > DT_B / 1024) atomicOr(a.err, 0x1000u);                            // the grouping kernel was asked for groups of ≤ 2 rows
      tbl[i].rec = g.rec; tbl[i].start = g.start; tbl[i].info = info | ((uint32_t)min(g.n, DT_B / 1024) << 1);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  [[maybe_unused]] const long long t_k2 = clock64();

  if (warp == DT_W_TMA) {
    // ------------------------------------------------------------------------------------------------ weight boxes: one thread
    if (lane == 0) {
      uint32_t it = 0, seen[2] = {1u, 1u};                                      // variant 0 of both kinds: acquired in the prologue
      bool ok = true;
      [[maybe_unused]] long long tw = 0, t_begin = clock64();
      const unsigned long long anchor[2] = {a.meta->anchor[0], a.meta->anchor[1]};
      const int up_rows = (int)((a.L.w3 - a.L.w1) / (unsigned long long)a.pitch[0]);
      for (int ii = 0; ii < n_items && ok; ++ii) {
        const DtEnt e = tbl[ii];
        const int k = ent_kind(e);
        const unsigned long long addr = reinterpret_cast<unsigned long long>(e.rec) + (k ? a.L.w2 : a.L.w1), delta = addr - anchor[k];
        unsigned long long row;
        int v = 0;
        if (a.pshift[k] >= 0) row = delta >> a.pshift[k];                          // the pitch divides 4096: every matrix is a whole number of rows above the anchor
        else {
          const unsigned long long rem = delta % (unsigned long long)a.pitch[k];
          row = (delta - rem) / (unsigned long long)a.pitch[k];
          v = (int)(rem / (unsigned long long)a.gstep[k]);
          if (rem % (unsigned long long)a.gstep[k] || v >= DT_VMAX) { atomicOr(a.err, 0x400000u); break; }
        }
        if (addr < anchor[k] || row + (1ull << 24) >= (1ull << 31)) { atomicOr(a.err, 0x400000u); break; }
        const CUtensorMap* map = a.maps + k * DT_VMAX + v;
        if (!((seen[k] >> v) & 1u)) { tmap_acquire(map); seen[k] |= 1u << v; }
        const int r0 = (int)row + ent_t(e) * (k ? DT_DN_ROWS : DT_GU_ROWS), r1 = r0 + up_rows;
        const int nkb = (k ? a.I : a.H) >> 8;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t stage = it % DT_ST;
          DT_TIMED(tw, ok = mbar_wait(&empty[stage], ((it / DT_ST) & 1) ^ 1, a.err, 0x1u));
          if (!ok) break;
          DT_STAMP(it, 0);
          const uint32_t sb = base + stage * DT_STAGE;
          mbar_expect_tx(&full[stage], DT_A);
          if (k) tma_load_2d(sb, map, kb * 128, r0, &full[stage]);
          else { tma_load_2d(sb, map, kb * 128, r0, &full[stage]); tma_load_2d(sb + DT_A / 2, map, kb * 128, r1, &full[stage]); }
          DT_STAMP(it, 1);
        }
      }
      DT_TRACE_PUT(0, tw); DT_TRACE_PUT(1, clock64() - t_begin); DT_TRACE_PUT(2, (long long)it);
    }
  } else if (warp == DT_W_DIG) {
    // ------------------------------------------------------------------------------------------------ digit planes: one thread walks the items' stages in ring
    // order — wait for the slot, announce the bytes, copy the 1 KB plane atoms of the group's one or two rows (a row's planes of
    // consecutive k windows are contiguous in global memory).  (In order, by one thread: a wait by parity tells apart only
    // neighbouring phases of a slot, so nobody may wait for a slot more than one ring cycle ahead.)
    if (lane == 0) {
      const int nkb = a.H >> 8;
      uint32_t it = 0;
      bool ok = true;
      for (int ii = 0; ii < n_items && ok; ++ii) {
        const int n = ent_n(tbl[ii]);
        const uint8_t* s0 = a.dw.xdig + (size_t)tbl_row[ii * kGroupRows] * nkb * 1024;
        const uint8_t* s1 = n > 1 ? a.dw.xdig + (size_t)tbl_row[ii * kGroupRows + 1] * nkb * 1024 : nullptr;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t stage = it % DT_ST;
          if (!(ok = mbar_wait(&empty[stage], ((it / DT_ST) & 1) ^ 1, a.err, 0x2u))) break;
          uint8_t* dst = sm + stage * DT_STAGE + DT_A;
          mbar_expect_tx(&full[stage], (uint32_t)n * 1024u);
          bulk_g2s(dst, s0 + (size_t)kb * 1024, 1024, &full[stage]);
          if (s1) bulk_g2s(dst + 1024, s1 + (size_t)kb * 1024, 1024, &full[stage]);
        }
      }
    }
  } else if (warp >= DT_W_SC0) {
    // ------------------------------------------------------------------------------------------------ weight scales: thread r owns row r of each A tile
    // A row's 16 scale bytes of a window = 4 k-steps × 4 scales.  In tensor memory the scales of a k-step take four columns; the
    // tensor core reads, for the accumulator rows of lane quarter q, column q of those four: lane l there holds the 4 scales of row
    // 32 q + l — which is this thread's own row.  Each thread copies its row's 16 bytes asynchronously DT_RAWD windows ahead (a
    // cursor of its own over the same work list) and stores the four words with one tcgen05.st into its own lane.
    const int r = threadIdx.x - DT_W_SC0 * 32, q = r >> 5;
    const uint32_t sf_lane = tmem + ((uint32_t)(q * 32) << 16);
    const uint8_t* prow = nullptr;
    int pii = 0, pkb = 0, pnkb = 0;
    uint32_t pw = 0;
    auto prefetch = [&]() {
      if (pkb == pnkb) {
        prow = nullptr;
        if (pii < n_items) {
          const DtEnt e = tbl[pii++];
          if (ent_kind(e)) { prow = e.rec + a.L.s2 + (size_t)(ent_t(e) * DT_DN_ROWS + r) * (a.I / 16); pnkb = a.I >> 8; }
          else { prow = e.rec + (r < 64 ? a.L.s1 : a.L.s3) + (size_t)(ent_t(e) * DT_GU_ROWS + (r & 63)) * (a.H / 16); pnkb = a.H >> 8; }
          pkb = 0;
        }
      }
      if (prow) { pf_cp16(smem_u32(rawsc + (pw % (DT_RAWD + 1)) * 2048 + r * 16), prow + (size_t)pkb * 16); ++pkb; }
      pf_cp_commit();
      ++pw;
    };
#pragma unroll
    for (int i = 0; i < DT_RAWD; ++i) prefetch();
    uint32_t it = 0;
    bool ok = true;
    [[maybe_unused]] long long tw = 0, tg = 0;
    // the digit planes of gate/up items have block scales 1.0: four columns written once, read by all their MMAs
    {
      uint32_t one16[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) one16[i] = 0x38383838u;
      tc_st16(sf_lane + DT_SFB1_COL, one16);
    }
    int pend = -1;                                                               // stage whose scales are stored but not yet announced
    for (int ii = 0; ii < n_items && ok; ++ii) {
      const int kind = ent_kind(tbl[ii]), nkb = (kind ? a.I : a.H) >> 8;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        prefetch();
        DT_TIMED(tg, pf_cp_wait<DT_RAWD>());                                       // this window's own 16 bytes have landed
        const uint4 v = *reinterpret_cast<const uint4*>(rawsc + (it % (DT_RAWD + 1)) * 2048 + r * 16);
        const uint32_t stage = it % DT_ST;
        // columns [0, 16) of the stage's 32: the weight scales — the word of k-step j goes to column 4 j + q of this thread's own lane
        // (the other columns of the quarter are never read).  Columns [16, 32), down items only: the block scales of the digit
        // planes — plane row 8 c + p sits in lane (8 c + p) mod 32, column (8 c + p) / 32 of the k-step's four columns, in every
        // quarter; k-step j of window kb is the 64-value slice 4 kb + j of the y rows.
        uint32_t w32[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) w32[i] = i < 16 ? 0u : 0x38383838u;
        const uint32_t vj[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) if (qq == q) w32[4 * j + qq] = vj[j];
        }
        // the previous stage's stores have had this long to land: announce it before anything below can wait
        if (pend >= 0) { tc_wait_st(); tc_fence_before(); mbar_arrive(&full[pend]); pend = -1; }
        if (kind) {
          if (!(ok = mbar_wait(&bmeta[stage], (it / DT_ST) & 1, a.err, 0x400u))) break;
          const uint8_t* codes = sfbc + (ii & 15) * 256 + kb * 4;
          const int l = r & 31;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            w32[16 + 4 * j] = 0x01010101u * codes[(l >> 3) * 32 + j];
            w32[16 + 4 * j + 1] = 0x01010101u * codes[(4 + (l >> 3)) * 32 + j];
          }
        }
        DT_TIMED(tw, ok = mbar_wait(&empty[stage], ((it / DT_ST) & 1) ^ 1, a.err, 0x4u));   // the MMAs that read this stage's scale columns are done
        if (!ok) break;
        tc_fence_after();
        if (kind) tc_st32(sf_lane + DT_SFA_COL0 + stage * 32, w32);
        else tc_st16(sf_lane + DT_SFA_COL0 + stage * 32, reinterpret_cast<const uint32_t(&)[16]>(w32));
        pend = (int)stage;
        if (r == 0) DT_STAMP(it, 2);
      }
    }
    if (pend >= 0 && ok) { tc_wait_st(); tc_fence_before(); mbar_arrive(&full[pend]); }
    pf_cp_wait<0>();
    if (r == 0) { DT_TRACE_PUT(5, tw); DT_TRACE_PUT(6, tg); }
  } else if (warp == DT_W_MMA) {
    // ------------------------------------------------------------------------------------------------ MMA issue: one thread
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      [[maybe_unused]] long long tf = 0, te = 0, t_begin = clock64();
      for (int ii = 0; ii < n_items && ok; ++ii) {
        const DtEnt e = tbl[ii];
        const uint32_t n_eff = (uint32_t)((ent_n(e) + 1) >> 1) * 16u, buf = (uint32_t)ii & 1u;
        const uint32_t idesc = (1u << 7) | (1u << 10) | ((n_eff >> 3) << 17) | ((128u >> 4) << 24);
        if (ii >= 2) DT_TIMED(te, ok = mbar_wait(&acc_empty[buf], ((ii >> 1) - 1) & 1, a.err, 0x8u));
        if (!ok) break;
        tc_fence_after();
        const int nkb = (ent_kind(e) ? a.I : a.H) >> 8;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t stage = it % DT_ST;
          DT_TIMED(tf, ok = mbar_wait(&full[stage], (it / DT_ST) & 1, a.err, 0x10u));
          if (!ok) break;
          DT_STAMP(it, 5);
          tc_fence_after();
          const uint32_t sb = base + stage * DT_STAGE, sfc = tmem + DT_SFA_COL0 + stage * 32, sfb = ent_kind(e) ? sfc + 16 : tmem + DT_SFB1_COL;
          const uint64_t ad = tc_desc_sw128(sb), bd = tc_desc_sw128(sb + DT_A);
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j)
            tc_mma_nvf4(tmem + buf * 64, ad + 2 * j, bd + 2 * j, idesc, sfc + 4 * j, sfb + 4 * j, (kb | (int)j) != 0 ? 1u : 0u);
          tc_commit(&empty[stage]);
          DT_STAMP(it, 6);
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
      tc_commit(mma_done);                                                       // nothing of this thread's is in flight when tensor memory is freed
      mbar_wait(mma_done, 0, a.err, 0x40u);
      DT_TRACE_PUT(7, tf); DT_TRACE_PUT(8, te); DT_TRACE_PUT(9, clock64() - t_begin); DT_TRACE_PUT(10, (long long)n_items);
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------------------------------------ epilogues: two sets of four warps, set s takes the items whose
    // accumulator buffer is s; warp q of a set reads tensor-memory lanes [32 q, 32 q + 32)
    const int set = warp >> 2, tl = threadIdx.x & 127;                           // tl = row of the A tile
    const int bar_id = 1 + set;
    float* ex = ex_all + set * (DT_EX / 4);
    volatile int* flag = flag_all + set * 24;
    const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16) + set * 64;
    bool ok = true;
    [[maybe_unused]] long long ta = 0, tgu = 0, tdn = 0, tdig = 0;
    for (int ii = set; ii < n_items && ok; ii += 2) {
      const DtEnt e = tbl[ii];
      const int n = ent_n(e), kind = ent_kind(e), t = ent_t(e), g = ent_g(e);
      const float* gp = reinterpret_cast<const float*>(e.rec + a.L.g);
      const float gsc = __ldg(gp + (kind ? 2 : (tl < 64 ? 0 : 1)));               // the record's global scale this thread applies
      float un[kGroupRows];
      if (a.gu_only) {
#pragma unroll
        for (int c = 0; c < kGroupRows; ++c) un[c] = c < n ? __ldg(a.dw.xs + tbl_row[ii * kGroupRows + c]) : 0.f;
      }
      DT_TIMED(ta, ok = mbar_wait(&acc_full[set], (ii >> 1) & 1, a.err, 0x80u));
      if (!ok) break;
      const float* units = rowsc + (ii & 15) * 8;
      [[maybe_unused]] const long long t_item = clock64();
      tc_fence_after();
      float val[kGroupRows];
#pragma unroll
      for (int c2 = 0; c2 < kGroupRows / 2; ++c2) {
        val[2 * c2] = val[2 * c2 + 1] = 0.f;
        if (2 * c2 < n) {
          uint32_t rr[16];
          tc_ld16(trow + 16 * c2, rr);
          tc_wait_ld();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float acc = __uint_as_float(rr[8 * h]);
#pragma unroll
            for (int p = 1; p < 8; ++p) acc = __fmaf_rn(acc, 8.f, __uint_as_float(rr[8 * h + p]));
            val[2 * c2 + h] = acc;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[set]);
      if (kind == 0) {
        // gate rows in lanes 0-63 (warps 0, 1 of the set), up rows in lanes 64-127 (warps 2, 3): up values cross through shared memory
        float gu[kGroupRows];
#pragma unroll
        for (int c = 0; c < kGroupRows; ++c) {
          gu[c] = 0.f;
          if (c < n) gu[c] = bf16r(val[c] * (a.gu_only ? un[c] : units[c]) * gsc);
        }
        if (tl >= 64) {
#pragma unroll
          for (int c = 0; c < kGroupRows; ++c) if (c < n) ex[c * 64 + (tl - 64)] = gu[c];
        }
        named_bar_sync(bar_id, 128);
        float upv[kGroupRows];
#pragma unroll
        for (int c = 0; c < kGroupRows; ++c) upv[c] = (tl < 64 && c < n) ? ex[c * 64 + tl] : 0.f;
        named_bar_sync(bar_id, 128);                                              // the up values are read: the item after next may overwrite them
        if (tl < 64) {
          // y = bf16(silu(g)·u) of the item's 64 values per row; its digit planes are taken against the largest exponent among the 64
          uint32_t yb[kGroupRows];
#pragma unroll
          for (int c = 0; c < kGroupRows; ++c) {
            yb[c] = 0u;
            if (c < n) {
              float gv = gu[c], uv = upv[c];
              if (a.limit > 0.f) { uv = fminf(fmaxf(uv, -a.limit), a.limit); gv = fminf(gv, a.limit); }
              const __nv_bfloat16 yv = __float2bfloat16(gv / (1.f + __expf(-gv)) * uv);
              yb[c] = (uint32_t)__bfloat16_as_ushort(yv);
              if (a.gu_only) { a.y[(size_t)(e.start + c) * a.I + t * DT_GU_ROWS + tl] = yv; continue; }   // 64 threads, 128 contiguous bytes per row
              const uint32_t am = __reduce_max_sync(0xffffffffu, yb[c] & 0x7fffu);
              if (lane == 0) flag[8 + (warp & 1) * 8 + c] = (int)am;
            }
          }
          if (a.gu_only) continue;                                               // (uniform over the kernel) nothing is digitised: the down pass reads bf16
          named_bar_sync(3 + set, 64);
          int ebs[kGroupRows];
#pragma unroll
          for (int c = 0; c < kGroupRows; ++c) {
            ebs[c] = 0;
            if (c < n) {
              const int eb = dt_row_exponent((uint32_t)max(flag[8 + c], flag[16 + c]));
              ebs[c] = eb;
              const uint32_t pw = dt_transpose8(dt_digits1(yb[c], eb), lane);
              *reinterpret_cast<uint32_t*>(a.dw.ydig + dt_dig_off((size_t)(e.start + c), a.I, t * DT_GU_ROWS + (tl & ~7), lane & 7)) = pw;
            }
          }
          named_bar_sync(3 + set, 64);
          // the slice's exponents are also what tells the down items that its planes are written: they go out last, behind a fence
          // (a slice whose exponent byte reads non-zero has all its planes in memory)
          if (tl == 0) {
            fence_proxy_async_all();
            __threadfence();
#pragma unroll
            for (int c = 0; c < kGroupRows; ++c) if (c < n) a.dw.yexp[(size_t)(e.start + c) * (((nIT + 7) >> 3) << 3) + t] = (uint8_t)ebs[c];
          }
        }
#ifdef HB_DTC_TRACE
        tgu += clock64() - t_item;
#endif
      } else {
        const int h = t * DT_DN_ROWS + tl;
#pragma unroll
        for (int c = 0; c < kGroupRows; ++c)
          if (c < n) a.part[(size_t)(e.start + c) * a.H + h] = __float2bfloat16(val[c] * units[c] * gsc);
#ifdef HB_DTC_TRACE
        tdn += clock64() - t_item;
#endif
      }
    }
    if (tl == 0 && set == 0) { DT_TRACE_PUT(11, ta); DT_TRACE_PUT(12, tgu); DT_TRACE_PUT(13, tdn); DT_TRACE_PUT(14, tdig); }
  }
  tc_fence_before();
  __syncthreads();
  [[maybe_unused]] const long long t_k3 = clock64();
  if (warp == DT_W_MMA) { tc_fence_after(); tmem_dealloc(tmem, DT_TMEM_COLS); }
  if (a.gu_only) return;                                                        // y is written; the streaming down kernel takes over
  // ---- every CTA's partial rows are written once all CTAs have come this far: then the k-order sums, one (row, 128 columns) block per
  // group of 64 threads
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(a.dw.fin, 1u);
    uint32_t spins = 0;
    while (ld_acquire_u32(a.dw.fin) < gridDim.x) {
      if (++spins > (1u << 22)) { atomicOr(a.err, 0x800u); break; }
      __nanosleep(40);
    }
  }
  __syncthreads();
  [[maybe_unused]] const long long t_k4 = clock64();
  {
    const int blocks = a.red.M * nHT, sub = threadIdx.x >> 6, l64 = threadIdx.x & 63, nsub = DT_THREADS / 64;
    for (int b = (int)blockIdx.x + sub * (int)gridDim.x; b < blocks; b += nsub * (int)gridDim.x) {
      const int m = b / nHT, ht = b - m * nHT;
      reduce_routed_unit(a.red, (size_t)m * (a.H / 2) + (size_t)ht * (DT_DN_ROWS / 2) + l64);
    }
  }
  if (threadIdx.x == 0) { DT_TRACE_PUT(20, t_k1 - t_k0); DT_TRACE_PUT(21, t_k2 - t_k1); DT_TRACE_PUT(22, t_k3 - t_k2); DT_TRACE_PUT(23, t_k4 - t_k3); DT_TRACE_PUT(24, clock64() - t_k4); }
}

// The digit planes of the activation rows alone (the gate/up pass on the tensor cores behind the streaming path's grouping kernel):
// one CTA per row.  It is launched right behind the grouping kernel, which triggers its dependents as soon as its own wait for the
// stream's earlier work has returned — so the rows are final when this kernel starts, it runs beside the grouping, and it does its
// own wait (for the grouping kernel to finish) LAST: the kernel behind it then finds both the planes and the group list complete.
// wait_flags: the rows are pushed by other ranks (expert parallel) — every CTA waits, bounded, for the same flags the grouping kernel
// waits for before it reads its row.
struct XdigArgs { const __nv_bfloat16* x; int x_ld, H; DtcWs dw; const uint32_t* wait_flags; int wait_n; const uint32_t* wait_step; uint32_t* err; };
__global__ void __launch_bounds__(256) moe_xdig_kernel(const XdigArgs a) {
  __shared__ int s_red[8];
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  griddep_launch();
  if (a.wait_flags) {
    if ((int)threadIdx.x < a.wait_n && !*reinterpret_cast<volatile uint32_t*>(a.err)) ep_wait_flag(a.wait_flags + threadIdx.x, *a.wait_step + 1u, a.err, 0x40000u);
    __syncthreads();
  }
  const uint32_t* xr = reinterpret_cast<const uint32_t*>(a.x + (size_t)m * a.x_ld);
  uint32_t am = 0;
  for (int e2 = threadIdx.x; e2 < a.H / 2; e2 += 256) { const uint32_t w2 = __ldg(xr + e2); am = max(am, max(w2 & 0x7fffu, (w2 >> 16) & 0x7fffu)); }
  for (int o = 16; o > 0; o >>= 1) am = max(am, __shfl_xor_sync(0xffffffffu, am, o));
  if (lane == 0) s_red[warp] = (int)am;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) am = max(am, (uint32_t)s_red[i]);
  const int eb = dt_row_exponent(am);
  if (threadIdx.x == 0) a.dw.xs[m] = dt_unit(eb);
  for (int u = threadIdx.x; u < a.H / 8; u += 256) {
    const uint4 q4 = __ldg(reinterpret_cast<const uint4*>(xr) + u);
    const uint32_t v4[4] = {q4.x, q4.y, q4.z, q4.w};
    uint32_t pl[8];
    dt_digits8(v4, eb, pl);
#pragma unroll
    for (int p = 0; p < 8; ++p) *reinterpret_cast<uint32_t*>(a.dw.xdig + dt_dig_off((size_t)m, a.H, u * 8, p)) = pl[p];
  }
  fence_proxy_async_global();                                                  // the planes are read through the async proxy (bulk copies) by the next kernel
  griddep_wait();
}

// Stamps the anchored bases into the tensor-map variants of both matrix kinds (one block; runs when the maps are first needed).
struct DtcMapTpl { CUtensorMap t[2]; };
__global__ void moe_dtc_anchor_kernel(const __grid_constant__ DtcMapTpl tpl, const uint8_t* const* __restrict__ tab, int n_tab, const uint8_t* shared_rec,
                                      int pitch0, int pitch1, int gstep0, int gstep1, CUtensorMap* __restrict__ maps, DtcMeta* __restrict__ meta) {
  __shared__ unsigned long long s_min;
  if (threadIdx.x == 0) s_min = shared_rec ? reinterpret_cast<unsigned long long>(shared_rec) : ~0ull;
  __syncthreads();
  unsigned long long mn = ~0ull;
  for (int i = threadIdx.x; i < n_tab; i += blockDim.x) { const unsigned long long p = reinterpret_cast<unsigned long long>(tab[i]); if (p) mn = min(mn, p); }
  atomicMin(&s_min, mn);
  __syncthreads();
  const unsigned long long lo = s_min == ~0ull ? (1ull << 40) : (s_min & ~4095ull);
  const int pitch[2] = {pitch0, pitch1}, gstep[2] = {gstep0, gstep1};
  for (int i = threadIdx.x; i < 2 * DT_VMAX; i += blockDim.x) {
    const int k = i / DT_VMAX, v = i - k * DT_VMAX;
    if (v >= pitch[k] / gstep[k]) continue;
    unsigned long long anchor = lo - ((unsigned long long)pitch[k] << 30);
    anchor &= ~4095ull;
    if (v == 0) meta->anchor[k] = anchor;
    const uint4* src = reinterpret_cast<const uint4*>(&tpl.t[k]);
    uint4* dst = reinterpret_cast<uint4*>(maps + i);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = src[j];
    const unsigned long long addr = anchor + (unsigned long long)v * gstep[k];
    asm volatile("tensormap.replace.tile.global_address.global.b1024.b64 [%0], %1;" ::"l"(dst), "l"(addr) : "memory");
    asm volatile("fence.proxy.tensormap::generic.release.gpu;" ::: "memory");
  }
}

}  // namespace hb

using namespace hb;

namespace {
int gcd_int(int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; }

size_t dtc_carve(void* ws, size_t off, int n, int H, int I, DtcWs* w) {
  auto take = [&](size_t b) { void* r = ws ? static_cast<char*>(ws) + off : nullptr; off += al256(b); return r; };
  DtcWs t;
  t.xdig = (uint8_t*)take((size_t)n * 4 * H); t.ydig = (uint8_t*)take((size_t)n * 4 * I);
  t.xs = (float*)take((size_t)n * 4); t.yexp = (uint8_t*)take((size_t)n * ((I / DT_GU_ROWS + 7) / 8 * 8)); t.fin = (unsigned int*)take(4);
  t.g_row = (uint16_t*)take((size_t)n * 8 * 2); t.g_unit = (float*)take((size_t)n * 8 * 4);
  if (w) *w = t;
  return off;
}
}  // namespace

bool hbk_moe_dtc_supported(int H, int I) {
  if (H <= 0 || I <= 0 || H % 256 || I % 256 || I / DT_GU_ROWS > 32) return false;
  const int p0 = H / 2, p1 = I / 2;
  return p0 / gcd_int(p0, 4096) <= DT_VMAX && p1 / gcd_int(p1, 4096) <= DT_VMAX;
}

// the gate/up-only form: a CTA's list holds its share of the gate/up items
bool hbk_moe_dtc_gu_fits(const hb_ctx* ctx, int P, int E, int H, int I) {
  int grid = ctx->sm_count;
  if (ctx->max_ctas > 0 && grid > ctx->max_ctas) grid = ctx->max_ctas;
  const long long G = P < E + 1 + P / 2 ? P : E + 1 + P / 2;              // groups of ≤ 2 rows: at most one odd group per expert
  return (G * (I / DT_GU_ROWS) + grid - 1) / grid <= DT_TBL;
}

size_t hbk_moe_dtc_ws_extra(int n, int H, int I) { return hbk_moe_dtc_supported(H, I) ? dtc_carve(nullptr, 0, n, H, I, nullptr) : 0; }

int hbk_moe_dtc_setup(hb_ctx* ctx) {
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(moe_dtc_layer_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, DT_SMEM));
  HB_CUDA(ctx, cudaMalloc(&ctx->dtc_maps, (size_t)2 * DT_VMAX * sizeof(CUtensorMap) + 256));
  HB_CUDA(ctx, cudaMemset(ctx->dtc_maps, 0, (size_t)2 * DT_VMAX * sizeof(CUtensorMap) + 256));
  return HB_OK;
}

// the tensor maps for (H, I), anchored below the records of `tab`: made on first use and whenever the shape changes
static int dtc_maps_for(hb_ctx* ctx, const uint8_t* const* tab, int n_tab, const uint8_t* shared_rec, int H, int I, cudaStream_t st) {
  if (ctx->dtc_H == H && ctx->dtc_I == I) return HB_OK;
  TcEncodeFn fn = tc_encode_fn();
  HB_REQUIRE(ctx, fn, HB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  DtcMapTpl tpl;
  const int pitch[2] = {H / 2, I / 2};
  const cuuint32_t rows[2] = {DT_GU_ROWS, DT_DN_ROWS};
  for (int k = 0; k < 2; ++k) {
    const cuuint64_t dims[2] = {(cuuint64_t)pitch[k], (cuuint64_t)1 << 31}, strides[1] = {(cuuint64_t)pitch[k]};
    const cuuint32_t box[2] = {128u, rows[k]}, estr[2] = {1, 1};
    const CUresult r = fn(&tpl.t[k], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, ctx->dtc_maps, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    HB_REQUIRE(ctx, r == CUDA_SUCCESS, HB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for pitch %d", (int)r, pitch[k]);
  }
  CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(ctx->dtc_maps);
  DtcMeta* meta = reinterpret_cast<DtcMeta*>(maps + 2 * DT_VMAX);
  const int r = hb_launch(ctx, "moe_dtc_anchor", false, moe_dtc_anchor_kernel, dim3(1), dim3(256), 0, st, tpl, tab, n_tab, shared_rec, pitch[0], pitch[1],
                          gcd_int(pitch[0], 4096), gcd_int(pitch[1], 4096), maps, meta);
  if (r) return r;
  ctx->dtc_H = H; ctx->dtc_I = I;
  return HB_OK;
}

#ifdef HB_DTC_TRACE
extern "C" __attribute__((visibility("default"))) int hb_dtc_trace_read(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_dt_trace, (size_t)n * 8);
}
extern "C" __attribute__((visibility("default"))) int hb_dtc_stage_read(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_dt_stage, (size_t)n * 8);
}
#endif

// The gate/up pass alone, behind the streaming path's grouping kernel (which wrote hdr / groups / s_row into the workspace `w`):
// digit planes of the M rows of x (row pitch x_ld), then the layer kernel in its gate/up-only form writing y bf16 into w.y.
int hbk_moe_dtc_gu_run(hb_ctx* ctx, const void* x, int x_ld, int M, const uint8_t* const* tab, int n_tab, const uint8_t* shared_rec, int P, int H, int I,
                       float limit, void* ws, const uint32_t* wait_flags, int wait_n, const uint32_t* wait_step, cudaStream_t st) {
  DecodeWs w = carve(ws, P, H, I);
  DtcWs dw;
  dtc_carve(ws, hbk_moe_decode_ws_bytes(P, H, I) - hbk_moe_dtc_ws_extra(P, H, I), P, H, I, &dw);
  hb_rec_layout L;
  hb_rec_layout_make(H, I, &L);
  int r = dtc_maps_for(ctx, tab, n_tab, shared_rec, H, I, st);
  if (r) return r;
  XdigArgs xa{reinterpret_cast<const __nv_bfloat16*>(x), x_ld, H, dw, wait_flags, wait_n, wait_step, ctx->dev_err};
  if ((r = hb_launch(ctx, "moe_xdig", true, moe_xdig_kernel, dim3(M), dim3(256), 0, st, xa))) return r;
  DtcArgs a{};
  a.gu_only = 1;
  a.hdr = w.hdr; a.groups = w.groups; a.s_row = w.s_row; a.H = H; a.I = I; a.limit = limit; a.L = L;
  a.maps = reinterpret_cast<const CUtensorMap*>(ctx->dtc_maps); a.meta = reinterpret_cast<const DtcMeta*>(a.maps + 2 * DT_VMAX);
  a.pitch[0] = H / 2; a.pitch[1] = I / 2; a.gstep[0] = gcd_int(H / 2, 4096); a.gstep[1] = gcd_int(I / 2, 4096);
  for (int k = 0; k < 2; ++k) { a.pshift[k] = -1; for (int b = 7; b <= 12; ++b) if (a.pitch[k] == (1 << b)) a.pshift[k] = b; }
  a.dw = dw; a.y = w.y; a.part = w.part; a.done = reinterpret_cast<unsigned int*>(w.done); a.err = ctx->dev_err;
  int grid = ctx->sm_count;
  if (ctx->max_ctas > 0 && grid > ctx->max_ctas) grid = ctx->max_ctas;
  a.dIT.set((uint32_t)(I / DT_GU_ROWS)); a.dHT.set((uint32_t)(H / DT_DN_ROWS)); a.dG.set((uint32_t)grid);
  return hb_launch(ctx, "moe_gate_up_tc", true, moe_dtc_layer_kernel, dim3(grid), dim3(DT_THREADS), (size_t)DT_SMEM, st, a);
}
