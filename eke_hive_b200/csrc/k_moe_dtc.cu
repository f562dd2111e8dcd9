// The gate/up pass of the routed decode operators on the block-scaled tensor cores: the NVFP4 weights go from HBM through shared
// memory into `tcgen05.mma kind::mxf4nvf4` untouched — no instruction ever handles a weight.
//
// The tensor core multiplies FP4 by FP4, the operators take bf16 activations (the reference's W4A16 arithmetic).  A bf16 row is
// therefore written, exactly, as eight FP4 "digit planes": with the row's largest biased exponent e, every element is the integer
// X = x / 2^(e-148) (|X| < 2^22; exact for elements down to 2^-15 of the row maximum, rounded to nearest below that — finer than
// an fp32 accumulation resolves), and X = Σ_p d_p·8^(7-p) in balanced base 8, digits d_p ∈ {-4 … 4}, all of which e2m1 holds.
// The eight planes are eight B-operand rows (block scales 1.0); the weights are the A operand with their own e4m3 block scales
// applied by the tensor core; the accumulator columns of one activation row are recombined in fp32 by Horner's rule:
//     Σ_k w_k·x_k = 2^(e-148) · Σ_p 8^(7-p) · D[·, p].
// Every product is exact; sums are fp32.  Rounding points after the products are the reference's (g, u → bf16 after the global
// scale, y → bf16).
//
// Where it sits: the streaming path's grouping kernel (k_moe_decode.cu; asked for groups of ≤ 2 rows) → beside it `moe_xdig_kernel`
// (one CTA per activation row: the row's digit planes) → `moe_dtc_layer_kernel` (this file) → the streaming down kernel, which
// reads y as bf16 rows.  A whole-layer form of this kernel (down items fed by digit planes of y published slice by slice, sums after
// the CTAs meet) was built first; it was slower than this chain and not run-to-run stable in its down phase, and is gone.
//
// The kernel: persistent CTAs, one per SM.  Work item = (group, 64 rows of I: 64 gate rows + 64 up rows form one 128-row A tile),
// dealt round-robin; a CTA's list is closed-form and built once into shared memory.  Per CTA: one thread streams weight boxes
// (128 bytes × 64 rows, 128-byte swizzle) by TMA through a tensor map anchored below the records; one thread copies the digit
// planes (pre-swizzled 1 KB atoms, plain bulk copies); four warps fetch the e4m3 scale rows ahead with cp.async and store them into
// tensor memory with tcgen05.st; one thread issues the MMAs (128 × 16 × 64) into two accumulator buffers; two sets of four warps
// run the epilogue (Horner, global scales, SwiGLU, y).  Every wait is bounded and reports through the context's error word.
#include "moe_stream.cuh"
#include "ep.cuh"
#include "tc_common.cuh"

namespace hb {

constexpr int DT_ST = 10;                      // pipeline stages
constexpr int DT_A = 16384;                    // weight tile of a stage: 128 rows × 128 bytes (256 k values)
constexpr int DT_B = 2048;                     // digit planes of a stage: 2 activation rows × 8 planes × 128 bytes (most experts of a decode batch get one
                                               // or two rows, and a small slot leaves room for more stages)
constexpr int DT_ROWS = DT_B / 1024;           // activation rows of a group
constexpr int DT_STAGE = DT_A + DT_B;
constexpr int DT_RAWD = 3;                     // windows the scale fetch runs ahead of its use
constexpr int DT_RAW = (DT_RAWD + 1) * 2048;   // ring of fetched scale rows: 128 rows × 16 bytes per window
constexpr int DT_EX = DT_ROWS * 64 * 4;        // SwiGLU exchange: up values of 64 rows × the group's activation rows
constexpr int DT_TBL = 256;                    // work-list entries a CTA can hold (16 bytes + DT_ROWS row indices each)
constexpr int DT_SMEM = 1024 + DT_ST * DT_STAGE + DT_RAW + 2 * DT_EX + 1024 + DT_TBL * (16 + 2 * DT_ROWS);
constexpr int DT_THREADS = 16 * 32;            // warps 0-7 epilogues (two sets of four), 8 MMA issue, 9 weight TMA, 10 digit copies, (11 idle),
                                               // 12-15 scales (they must be warps 0-3 modulo 4: a warp reaches the tensor-memory lanes of that quarter)
constexpr int DT_W_MMA = 8, DT_W_TMA = 9, DT_W_DIG = 10, DT_W_SC0 = 12;
constexpr int DT_TMEM_COLS = 512;              // accumulators 2 × 64 columns, then 16 columns of weight scales per stage, then 16 columns of 1.0
constexpr int DT_SFA_COL0 = 128;
constexpr int DT_SFB1_COL = DT_SFA_COL0 + DT_ST * 16;   // the digit planes' block scales: 1.0 for every plane, written once
constexpr int DT_VMAX = 32;                    // tensor-map variants (see DtcMeta)
constexpr int DT_GU_ROWS = 64;                 // rows of I per item
static_assert(DT_STAGE % 1024 == 0, "stage buffers keep the swizzle atom's alignment");
static_assert(DT_SFB1_COL + 16 <= DT_TMEM_COLS, "tensor memory");
static_assert(DT_SMEM <= 227 * 1024, "shared memory");
static_assert(DT_ROWS <= kGroupRows, "groups of the grouping kernel");

// A tensor map for the weight boxes cannot be made per record ahead of time (the table may change between calls) and records sit
// at arbitrary 4096-aligned addresses.  One map covers them all: a 2-D byte matrix [2^31 rows][pitch] whose base lies 2^30 rows
// below the lowest record seen when the map was made.  A matrix whose distance from that base is not a multiple of the pitch uses
// variant v of the map, shifted by v·gcd(pitch, 4096) bytes (pitch / gcd variants cover every residue).
struct DtcMeta { unsigned long long anchor; };

struct DtcWs {
  uint8_t* xdig;        // [rows][K/256][8 planes][128 bytes], swizzled
  float* xs;            // [rows] unit of a row's digits (a power of two)
};
struct DtcWs2 { DtcWs x, y; };   // planes of the activation rows (K = H) and of the y rows (K = I)

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
  const int* hdr; const Group* groups;                    // the grouping kernel's list: hdr[0] groups
  const int* s_row;                                       // gate/up: rows of a group = s_row[start .. start + n); down (nullptr): positions start .. start + n
  int down;                                               // 0: gate/up (A tile = 64 gate + 64 up rows, out = y); 1: down (A tile = 128 rows of w2, out = per-pair rows)
  int K, out_ld; float limit;                             // K: inner dimension (H | I); out_ld: row length of the output (I | H)
  DtDiv dIT, dG;                                          // dividers by the items per group and by the grid size
  uint32_t off_w, off_s0, off_s1, off_g;                  // record offsets: the matrix of the tile's first half, the scales of both halves, the global scales
  int row2, trows;                                        // matrix rows from the first 64-row box of an item to the second; matrix rows an item advances per half
  const CUtensorMap* maps; const DtcMeta* meta;           // maps[variant]
  int pitch, gstep, pshift;                               // pshift: log2(pitch) when the pitch divides 4096, else -1
  DtcWs dw;                                               // the digit planes of the B operand's rows
  __nv_bfloat16* out;                                     // bf16 [position, out_ld]
  unsigned int* fin; ReduceArgs red; int red_on;          // down: the sums over each row's pairs after the CTAs have met
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
// Item j of the launch = (group j / T, tile t = j mod T); gate/up: T = I/64, the tile = rows [64 t, 64 t + 64) of gate and of up; down:
// T = H/128, the tile = rows [128 t, 128 t + 128) of w2.  It goes to CTA j mod grid, so the items of one group run on different CTAs
// at the same time.  Entry x of CTA c is item c + x·grid: computed directly.
struct DtEnt { const uint8_t* rec; int start; uint32_t info; };      // info: bits 1-4 rows of the group, bits 5-15 t, bits 16-31 g
static_assert(sizeof(DtEnt) == 16, "DtEnt layout");
__device__ __forceinline__ int ent_n(const DtEnt& e) { return (int)((e.info >> 1) & 15u); }
__device__ __forceinline__ int ent_t(const DtEnt& e) { return (int)((e.info >> 5) & 0x7ffu); }

// Optional in-kernel timing (compile with -DHB_DTC_TRACE): every role of every CTA sums the clocks it spends in each kind of wait.
#ifdef HB_DTC_TRACE
__device__ long long g_dt_trace[256 * 32];
#define DT_TIMED(acc, stmt) do { const long long t_ = clock64(); stmt; acc += clock64() - t_; } while (0)
#define DT_TRACE_PUT(slot, v) g_dt_trace[blockIdx.x * 32 + (slot)] = (v)
__device__ long long g_dt_stage[2 * 128 * 8];
#define DT_STAMP(it, col) do { if ((blockIdx.x == 0 || blockIdx.x == 77) && (it) < 128) g_dt_stage[((blockIdx.x ? 1 : 0) * 128 + (it)) * 8 + (col)] = clock64(); } while (0)
#else
#define DT_TIMED(acc, stmt) do { stmt; } while (0)
#define DT_TRACE_PUT(slot, v) do { } while (0)
#define DT_STAMP(it, col) do { } while (0)
#endif

__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// ---- the kernel ---------------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(DT_THREADS, 1) moe_dtc_layer_kernel(const DtcArgs a) {
  extern __shared__ uint8_t dt_raw[];
  const uint32_t raw = smem_u32(dt_raw), base = (raw + 1023u) & ~1023u;
  uint8_t* sm = dt_raw + (base - raw);
  uint8_t* rawsc = sm + DT_ST * DT_STAGE;                                       // fetched scale rows
  float* ex_all = reinterpret_cast<float*>(rawsc + DT_RAW);                     // [2 sets][DT_ROWS][64]
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(ex_all) + 2 * DT_EX);   // [ST] weights and digits of the stage are in shared memory, its scales in tensor memory
  uint64_t* empty = full + DT_ST;                                               // [ST] the MMAs that read the stage are done
  uint64_t* acc_full = empty + DT_ST;                                           // [2]
  uint64_t* acc_empty = acc_full + 2;                                           // [2]
  uint64_t* mma_done = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_done + 1);
  DtEnt* tbl = reinterpret_cast<DtEnt*>(reinterpret_cast<uint8_t*>(full) + 1024);   // [DT_TBL] this CTA's work list
  uint16_t* tbl_row = reinterpret_cast<uint16_t*>(tbl + DT_TBL);                // [DT_TBL][DT_ROWS] activation rows of the item's group
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DT_ST; ++s) { mbar_init(&full[s], 128 + 2); mbar_init(&empty[s], 1); }   // full: 128 scale threads + the two copy threads
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
    mbar_init(mma_done, 1);
    mbar_fence_init();
  }
  if (warp == DT_W_MMA) { tmem_alloc(tmem_slot, DT_TMEM_COLS); tmem_relinquish(); }
  // the first variant of the tensor map (the only one when the pitch divides 4096) is made visible to the TMA thread before the
  // wait: the maps were stamped by an earlier launch that has completed
  if (threadIdx.x == DT_W_TMA * 32) tmap_acquire(a.maps);
  griddep_wait();                                                               // the group list and the digit planes of the rows
  griddep_launch();
  const int nIT = (int)a.dIT.d, grid = (int)a.dG.d, c0 = (int)blockIdx.x;
  const int n_gu = a.hdr[0] * nIT;
  int n_items = c0 < n_gu ? (int)a.dG.div((uint32_t)(n_gu - 1 - c0)) + 1 : 0;
  if (n_items > DT_TBL) { if (threadIdx.x == 0) atomicOr(a.err, 0x1000u); n_items = 0; }   // the launcher checks that this does not happen
  for (int j = threadIdx.x; j < n_items * DT_ROWS; j += DT_THREADS) {           // records, positions and activation rows of the items
    const int i = j / DT_ROWS, c = j - i * DT_ROWS;
    const int item = c0 + i * grid, gi = (int)a.dIT.div((uint32_t)item);
    const Group g = a.groups[gi];
    tbl_row[j] = (uint16_t)(c < g.n ? (a.s_row ? a.s_row[g.start + c] : g.start + c) : 0);
    if (c == 0) {
      if (g.n > DT_ROWS) atomicOr(a.err, 0x1000u);                               // the grouping kernel was asked for groups of ≤ DT_ROWS rows
      tbl[i].rec = g.rec; tbl[i].start = g.start;
      tbl[i].info = ((uint32_t)min(g.n, DT_ROWS) << 1) | ((uint32_t)(item - gi * nIT) << 5) | ((uint32_t)gi << 16);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int nkb = a.K >> 8;                                                     // stages per item

  if (warp == DT_W_TMA) {
    // ------------------------------------------------------------------------------------------------ weight boxes: one thread
    if (lane == 0) {
      uint32_t it = 0, seen = 1u;                                                // variant 0: acquired in the prologue
      bool ok = true;
      [[maybe_unused]] long long tw = 0, t_begin = clock64();
      const unsigned long long anchor = a.meta->anchor;
      for (int ii = 0; ii < n_items && ok; ++ii) {
        const DtEnt e = tbl[ii];
        const unsigned long long addr = reinterpret_cast<unsigned long long>(e.rec) + a.off_w, delta = addr - anchor;
        unsigned long long row;
        int v = 0;
        if (a.pshift >= 0) row = delta >> a.pshift;                               // the pitch divides 4096: every matrix is a whole number of rows above the anchor
        else {
          const unsigned long long rem = delta % (unsigned long long)a.pitch;
          row = (delta - rem) / (unsigned long long)a.pitch;
          v = (int)(rem / (unsigned long long)a.gstep);
          if (rem % (unsigned long long)a.gstep || v >= DT_VMAX) { atomicOr(a.err, 0x400000u); break; }
        }
        if (addr < anchor || row + (1ull << 24) >= (1ull << 31)) { atomicOr(a.err, 0x400000u); break; }
        const CUtensorMap* map = a.maps + v;
        if (!((seen >> v) & 1u)) { tmap_acquire(map); seen |= 1u << v; }
        const int r0 = (int)row + ent_t(e) * a.trows, r1 = r0 + a.row2;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t stage = it % DT_ST;
          DT_TIMED(tw, ok = mbar_wait(&empty[stage], ((it / DT_ST) & 1) ^ 1, a.err, 0x1u));
          if (!ok) break;
          DT_STAMP(it, 0);
          const uint32_t sb = base + stage * DT_STAGE;
          mbar_expect_tx(&full[stage], DT_A);
          tma_load_2d(sb, map, kb * 128, r0, &full[stage]);                       // 64 gate rows | rows 0-63 of the w2 tile
          tma_load_2d(sb + DT_A / 2, map, kb * 128, r1, &full[stage]);            // 64 up rows | rows 64-127
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
      uint32_t it = 0;
      bool ok = true;
      for (int ii = 0; ii < n_items && ok; ++ii) {
        const int n = ent_n(tbl[ii]);
        const uint8_t* s0 = a.dw.xdig + (size_t)tbl_row[ii * DT_ROWS] * nkb * 1024;
        const uint8_t* s1 = n > 1 ? a.dw.xdig + (size_t)tbl_row[ii * DT_ROWS + 1] * nkb * 1024 : nullptr;
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
    int pii = 0, pkb = nkb;
    uint32_t pw = 0;
    auto prefetch = [&]() {
      if (pkb == nkb) {
        prow = nullptr;
        if (pii < n_items) {
          const DtEnt e = tbl[pii++];
          prow = e.rec + (r < 64 ? a.off_s0 : a.off_s1) + (size_t)(ent_t(e) * a.trows + (r & 63)) * (a.K / 16);
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
    // the digit planes have block scales 1.0: sixteen columns written once, read by every MMA
    {
      uint32_t one16[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) one16[i] = 0x38383838u;
      tc_st16(sf_lane + DT_SFB1_COL, one16);
    }
    int pend = -1;                                                               // stage whose scales are stored but not yet announced
    const uint32_t n_stages = (uint32_t)n_items * (uint32_t)nkb;
    for (; it < n_stages && ok; ++it) {
      prefetch();
      DT_TIMED(tg, pf_cp_wait<DT_RAWD>());                                         // this window's own 16 bytes have landed
      const uint4 v = *reinterpret_cast<const uint4*>(rawsc + (it % (DT_RAWD + 1)) * 2048 + r * 16);
      const uint32_t stage = it % DT_ST;
      // the word of k-step j goes to column 4 j + q of this thread's own lane (the other columns of the quarter are never read)
      uint32_t w16[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) w16[i] = 0u;
      const uint32_t vj[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int qq = 0; qq < 4; ++qq) if (qq == q) w16[4 * j + qq] = vj[j];
      }
      // the previous stage's stores have had this long to land: announce it before anything below can wait
      if (pend >= 0) { tc_wait_st(); tc_fence_before(); mbar_arrive(&full[pend]); pend = -1; }
      DT_TIMED(tw, ok = mbar_wait(&empty[stage], ((it / DT_ST) & 1) ^ 1, a.err, 0x4u));   // the MMAs that read this stage's scale columns are done
      if (!ok) break;
      tc_fence_after();
      tc_st16(sf_lane + DT_SFA_COL0 + stage * 16, w16);
      pend = (int)stage;
      if (r == 0) DT_STAMP(it, 2);
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
      // 128 × 16 × 64 per instruction: A and B e2m1 (format 1), both K-major, N / 8 at bit 17, ue4m3 scales, M / 16 at bit 24
      constexpr uint32_t idesc = (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
      for (int ii = 0; ii < n_items && ok; ++ii) {
        const uint32_t buf = (uint32_t)ii & 1u;
        if (ii >= 2) DT_TIMED(te, ok = mbar_wait(&acc_empty[buf], ((ii >> 1) - 1) & 1, a.err, 0x8u));
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const uint32_t stage = it % DT_ST;
          DT_TIMED(tf, ok = mbar_wait(&full[stage], (it / DT_ST) & 1, a.err, 0x10u));
          if (!ok) break;
          DT_STAMP(it, 5);
          tc_fence_after();
          const uint32_t sb = base + stage * DT_STAGE, sfc = tmem + DT_SFA_COL0 + stage * 16, sfb = tmem + DT_SFB1_COL;
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
    // accumulator buffer is s; warp q of a set reads tensor-memory lanes [32 q, 32 q + 32): gate rows in lanes 0-63 (warps 0, 1 of the
    // set), up rows in lanes 64-127 (warps 2, 3) — the up values cross to the gate threads through shared memory
    const int set = warp >> 2, tl = threadIdx.x & 127;                           // tl = row of the A tile
    const int bar_id = 1 + set;
    float* ex = ex_all + set * (DT_EX / 4);
    const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16) + set * 64;
    bool ok = true;
    [[maybe_unused]] long long ta = 0;
    for (int ii = set; ii < n_items && ok; ii += 2) {
      const DtEnt e = tbl[ii];
      const int n = ent_n(e), t = ent_t(e);
      const float gsc = __ldg(reinterpret_cast<const float*>(e.rec + a.off_g) + (a.down ? 2 : tl < 64 ? 0 : 1));   // the record's global scale this thread applies
      float un[DT_ROWS];                                                         // units of the rows' digits: fetched while the MMAs run
#pragma unroll
      for (int c = 0; c < DT_ROWS; ++c) un[c] = c < n ? __ldg(a.dw.xs + tbl_row[ii * DT_ROWS + c]) : 0.f;
      DT_TIMED(ta, ok = mbar_wait(&acc_full[set], (ii >> 1) & 1, a.err, 0x80u));
      if (!ok) break;
      tc_fence_after();
      float val[DT_ROWS];
      {
        uint32_t rr[16];                                                         // two activation rows × eight planes
        tc_ld16(trow, rr);
        tc_wait_ld();
#pragma unroll
        for (int h = 0; h < DT_ROWS; ++h) {
          float acc = __uint_as_float(rr[8 * h]);
#pragma unroll
          for (int p = 1; p < 8; ++p) acc = __fmaf_rn(acc, 8.f, __uint_as_float(rr[8 * h + p]));
          val[h] = acc;
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[set]);
      float gu[DT_ROWS];
#pragma unroll
      for (int c = 0; c < DT_ROWS; ++c) gu[c] = c < n ? bf16r(val[c] * un[c] * gsc) : 0.f;
      if (a.down) {
        // a pair's row of the down projection, bf16 (the routing weight is applied where the pairs are summed): 128 threads, 256 contiguous bytes
#pragma unroll
        for (int c = 0; c < DT_ROWS; ++c)
          if (c < n) a.out[(size_t)(e.start + c) * a.out_ld + t * 128 + tl] = __float2bfloat16(gu[c]);
        continue;
      }
      if (tl >= 64) {
#pragma unroll
        for (int c = 0; c < DT_ROWS; ++c) if (c < n) ex[c * 64 + (tl - 64)] = gu[c];
      }
      named_bar_sync(bar_id, 128);
      float upv[DT_ROWS];
#pragma unroll
      for (int c = 0; c < DT_ROWS; ++c) upv[c] = (tl < 64 && c < n) ? ex[c * 64 + tl] : 0.f;
      named_bar_sync(bar_id, 128);                                               // the up values are read: the item after next may overwrite them
      if (tl < 64) {
        // y = bf16(silu(g)·u): 64 threads, 128 contiguous bytes per activation row
#pragma unroll
        for (int c = 0; c < DT_ROWS; ++c) {
          if (c < n) {
            float gv = gu[c], uv = upv[c];
            if (a.limit > 0.f) { uv = fminf(fmaxf(uv, -a.limit), a.limit); gv = fminf(gv, a.limit); }
            a.out[(size_t)(e.start + c) * a.out_ld + t * DT_GU_ROWS + tl] = __float2bfloat16(gv / (1.f + __expf(-gv)) * uv);
          }
        }
      }
    }
    if (tl == 0 && set == 0) DT_TRACE_PUT(11, ta);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == DT_W_MMA) { tc_fence_after(); tmem_dealloc(tmem, DT_TMEM_COLS); }
  if (!a.red_on) return;
  // Down pass of the routed form: the sums over each row's pairs.  One CTA per SM and no more CTAs than SMs — all are resident, so
  // they can meet: a CTA announces that its rows are written, waits (bounded) until every CTA has, and takes its share of the
  // (row, column pair) units.
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
}

// The digit planes of the activation rows alone (the gate/up pass on the tensor cores behind the streaming path's grouping kernel):
// one CTA per row.  It is launched right behind the grouping kernel, which triggers its dependents as soon as its own wait for the
// stream's earlier work has returned — so the rows are final when this kernel starts, it runs beside the grouping, and it does its
// own wait (for the grouping kernel to finish) LAST: the kernel behind it then finds both the planes and the group list complete.
// wait_flags: the rows are pushed by other ranks (expert parallel) — every CTA waits, bounded, for the same flags the grouping kernel
// waits for before it reads its row.
// wait_first: the rows are the previous kernel's output (the y rows between the two passes): wait for it before reading.
struct XdigArgs { const __nv_bfloat16* x; int x_ld, H; DtcWs dw; const uint32_t* wait_flags; int wait_n; const uint32_t* wait_step; uint32_t* err; int wait_first; };
__global__ void __launch_bounds__(256) moe_xdig_kernel(const XdigArgs a) {
  __shared__ int s_red[8];
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  griddep_launch();
  if (a.wait_first) griddep_wait();
  if (a.wait_flags) {
    if ((int)threadIdx.x < a.wait_n && !*reinterpret_cast<volatile uint32_t*>(a.err)) ep_wait_flag(a.wait_flags + threadIdx.x, *a.wait_step + 1u, a.err, 0x40000u);
    __syncthreads();
  }
  const uint32_t* xr = reinterpret_cast<const uint32_t*>(a.x + (size_t)m * a.x_ld);
  uint32_t am = 0;
  for (int e2 = threadIdx.x; e2 < a.H / 2; e2 += 256) { const uint32_t w2 = __ldcg(xr + e2); am = max(am, max(w2 & 0x7fffu, (w2 >> 16) & 0x7fffu)); }
  for (int o = 16; o > 0; o >>= 1) am = max(am, __shfl_xor_sync(0xffffffffu, am, o));
  if (lane == 0) s_red[warp] = (int)am;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) am = max(am, (uint32_t)s_red[i]);
  const int eb = dt_row_exponent(am);
  if (threadIdx.x == 0) a.dw.xs[m] = dt_unit(eb);
  for (int u = threadIdx.x; u < a.H / 8; u += 256) {
    const uint4 q4 = __ldcg(reinterpret_cast<const uint4*>(xr) + u);
    const uint32_t v4[4] = {q4.x, q4.y, q4.z, q4.w};
    uint32_t pl[8];
    dt_digits8(v4, eb, pl);
#pragma unroll
    for (int p = 0; p < 8; ++p) *reinterpret_cast<uint32_t*>(a.dw.xdig + dt_dig_off((size_t)m, a.H, u * 8, p)) = pl[p];
  }
  fence_proxy_async_global();                                                  // the planes are read through the async proxy (bulk copies) by the next kernel
  if (!a.wait_first) griddep_wait();
}

// Stamps the anchored base into the variants of the tensor map (one block; runs when the maps are first needed).
struct DtcMapTpl { CUtensorMap t; };
__global__ void moe_dtc_anchor_kernel(const __grid_constant__ DtcMapTpl tpl, const uint8_t* const* __restrict__ tab, int n_tab, const uint8_t* shared_rec,
                                      int pitch, int gstep, CUtensorMap* __restrict__ maps, DtcMeta* __restrict__ meta) {
  __shared__ unsigned long long s_min;
  if (threadIdx.x == 0) s_min = shared_rec ? reinterpret_cast<unsigned long long>(shared_rec) : ~0ull;
  __syncthreads();
  unsigned long long mn = ~0ull;
  for (int i = threadIdx.x; i < n_tab; i += blockDim.x) { const unsigned long long p = reinterpret_cast<unsigned long long>(tab[i]); if (p) mn = min(mn, p); }
  atomicMin(&s_min, mn);
  __syncthreads();
  const unsigned long long lo = s_min == ~0ull ? (1ull << 40) : (s_min & ~4095ull);
  for (int v = threadIdx.x; v < DT_VMAX; v += blockDim.x) {
    if (v >= pitch / gstep) continue;
    unsigned long long anchor = lo - ((unsigned long long)pitch << 30);
    anchor &= ~4095ull;
    if (v == 0) meta->anchor = anchor;
    const uint4* src = reinterpret_cast<const uint4*>(&tpl.t);
    uint4* dst = reinterpret_cast<uint4*>(maps + v);
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = src[j];
    const unsigned long long addr = anchor + (unsigned long long)v * gstep;
    asm volatile("tensormap.replace.tile.global_address.global.b1024.b64 [%0], %1;" ::"l"(dst), "l"(addr) : "memory");
    asm volatile("fence.proxy.tensormap::generic.release.gpu;" ::: "memory");
  }
}

}  // namespace hb

using namespace hb;

namespace {
int gcd_int(int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; }

size_t dtc_carve(void* ws, size_t off, int n, int H, int I, DtcWs2* w) {
  auto take = [&](size_t b) { void* r = ws ? static_cast<char*>(ws) + off : nullptr; off += al256(b); return r; };
  DtcWs2 t;
  t.x.xdig = (uint8_t*)take((size_t)n * 4 * H); t.x.xs = (float*)take((size_t)n * 4);
  t.y.xdig = (uint8_t*)take((size_t)n * 4 * I); t.y.xs = (float*)take((size_t)n * 4);
  if (w) *w = t;
  return off;
}
constexpr size_t kMapSetBytes = (size_t)DT_VMAX * sizeof(CUtensorMap) + 256;   // the variants of one map and its DtcMeta
int dtc_grid(const hb_ctx* ctx) {
  int grid = ctx->sm_count;
  if (ctx->max_ctas > 0 && grid > ctx->max_ctas) grid = ctx->max_ctas;
  return grid;
}
long long dtc_groups(int P, int E) { return P < E + 1 + P / DT_ROWS ? P : E + 1 + P / DT_ROWS; }   // groups of ≤ DT_ROWS rows: at most one partly filled group per expert
}  // namespace

bool hbk_moe_dtc_supported(int H, int I) {
  if (H <= 0 || I <= 0 || H % 256 || I % 256 || I / DT_GU_ROWS > 2047) return false;
  const int p0 = H / 2, p1 = I / 2;
  return p0 / gcd_int(p0, 4096) <= DT_VMAX && p1 / gcd_int(p1, 4096) <= DT_VMAX && H / 128 <= 2047;
}

// a CTA's list holds its share of the items
bool hbk_moe_dtc_gu_fits(const hb_ctx* ctx, int P, int E, int H, int I) {
  const int grid = dtc_grid(ctx);
  const long long G = dtc_groups(P, E);
  return G < 65536 && (G * (I / DT_GU_ROWS) + grid - 1) / grid <= DT_TBL;
}
bool hbk_moe_dtc_down_fits(const hb_ctx* ctx, int P, int E, int H, int I) {
  const int grid = dtc_grid(ctx);
  const long long G = dtc_groups(P, E);
  return G < 65536 && P < 65536 && (G * (H / 128) + grid - 1) / grid <= DT_TBL && grid <= ctx->sm_count;
}

size_t hbk_moe_dtc_ws_extra(int n, int H, int I) { return hbk_moe_dtc_supported(H, I) ? dtc_carve(nullptr, 0, n, H, I, nullptr) : 0; }

int hbk_moe_dtc_setup(hb_ctx* ctx) {
  HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(moe_dtc_layer_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, DT_SMEM));
  HB_CUDA(ctx, cudaMalloc(&ctx->dtc_maps, 2 * kMapSetBytes));
  HB_CUDA(ctx, cudaMemset(ctx->dtc_maps, 0, 2 * kMapSetBytes));
  return HB_OK;
}

// the tensor maps of both passes (row pitch H/2 for gate and up, I/2 for down), anchored below the records of `tab`: made on first
// use and whenever the shape changes
static int dtc_maps_for(hb_ctx* ctx, const uint8_t* const* tab, int n_tab, const uint8_t* shared_rec, int H, int I, cudaStream_t st) {
  if (ctx->dtc_H == H && ctx->dtc_I == I) return HB_OK;
  TcEncodeFn fn = tc_encode_fn();
  HB_REQUIRE(ctx, fn, HB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  for (int kind = 0; kind < 2; ++kind) {
    DtcMapTpl tpl;
    const int pitch = (kind ? I : H) / 2;
    const cuuint64_t dims[2] = {(cuuint64_t)pitch, (cuuint64_t)1 << 31}, strides[1] = {(cuuint64_t)pitch};
    const cuuint32_t box[2] = {128u, 64u}, estr[2] = {1, 1};
    CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(static_cast<char*>(ctx->dtc_maps) + kind * kMapSetBytes);
    const CUresult cr = fn(&tpl.t, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, maps, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    HB_REQUIRE(ctx, cr == CUDA_SUCCESS, HB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for pitch %d", (int)cr, pitch);
    DtcMeta* meta = reinterpret_cast<DtcMeta*>(maps + DT_VMAX);
    const int r = hb_launch(ctx, "moe_dtc_anchor", false, moe_dtc_anchor_kernel, dim3(1), dim3(256), 0, st, tpl, tab, n_tab, shared_rec, pitch,
                            gcd_int(pitch, 4096), maps, meta);
    if (r) return r;
  }
  ctx->dtc_H = H; ctx->dtc_I = I;
  return HB_OK;
}

// what both passes share: the list, the map set of the pass, the dividers
static void dtc_args_common(hb_ctx* ctx, const DecodeWs& w, int kind, int K, int items_per_group, DtcArgs* a) {
  a->hdr = w.hdr; a->groups = w.groups; a->down = kind; a->K = K; a->err = ctx->dev_err;
  a->maps = reinterpret_cast<const CUtensorMap*>(static_cast<const char*>(ctx->dtc_maps) + kind * kMapSetBytes);
  a->meta = reinterpret_cast<const DtcMeta*>(a->maps + DT_VMAX);
  a->pitch = K / 2; a->gstep = gcd_int(K / 2, 4096);
  a->pshift = -1;
  for (int b = 7; b <= 12; ++b) if (a->pitch == (1 << b)) a->pshift = b;
  a->dIT.set((uint32_t)items_per_group); a->dG.set((uint32_t)dtc_grid(ctx));
}

// the same maps for the prefill GEMM with bf16 activations, which streams raw code boxes through them
int hbk_moe_dtc_maps(hb_ctx* ctx, const uint8_t* const* tab, int n_tab, const uint8_t* shared_rec, int H, int I, cudaStream_t st) {
  return dtc_maps_for(ctx, tab, n_tab, shared_rec, H, I, st);
}
void hbk_moe_dtc_map_set(const hb_ctx* ctx, int kind, const void** maps, const unsigned long long** anchor) {
  const CUtensorMap* m = reinterpret_cast<const CUtensorMap*>(static_cast<const char*>(ctx->dtc_maps) + kind * kMapSetBytes);
  *maps = m;
  *anchor = &reinterpret_cast<const DtcMeta*>(m + DT_VMAX)->anchor;
}
int hbk_moe_dtc_vmax() { return DT_VMAX; }

#ifdef HB_DTC_TRACE
extern "C" __attribute__((visibility("default"))) int hb_dtc_trace_read(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_dt_trace, (size_t)n * 8);
}
extern "C" __attribute__((visibility("default"))) int hb_dtc_stage_read(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_dt_stage, (size_t)n * 8);
}
#endif

// The gate/up pass behind the streaming path's grouping kernel (which wrote hdr / groups / s_row into the workspace): digit planes
// of the M rows of x (row pitch x_ld), then the tensor-memory kernel writing y bf16 into the workspace's y rows.
int hbk_moe_dtc_gu_run(hb_ctx* ctx, const void* x, int x_ld, int M, const uint8_t* const* tab, int n_tab, const uint8_t* shared_rec, int P, int H, int I,
                       float limit, void* ws, const uint32_t* wait_flags, int wait_n, const uint32_t* wait_step, cudaStream_t st) {
  DecodeWs w = carve(ws, P, H, I);
  DtcWs2 dw;
  dtc_carve(ws, hbk_moe_decode_ws_bytes(P, H, I) - hbk_moe_dtc_ws_extra(P, H, I), P, H, I, &dw);
  hb_rec_layout L;
  hb_rec_layout_make(H, I, &L);
  int r = dtc_maps_for(ctx, tab, n_tab, shared_rec, H, I, st);
  if (r) return r;
  XdigArgs xa{reinterpret_cast<const __nv_bfloat16*>(x), x_ld, H, dw.x, wait_flags, wait_n, wait_step, ctx->dev_err, 0};
  if ((r = hb_launch(ctx, "moe_xdig", true, moe_xdig_kernel, dim3(M), dim3(256), 0, st, xa))) return r;
  DtcArgs a{};
  dtc_args_common(ctx, w, 0, H, I / DT_GU_ROWS, &a);
  a.s_row = w.s_row; a.out_ld = I; a.limit = limit;
  a.off_w = (uint32_t)L.w1; a.off_s0 = (uint32_t)L.s1; a.off_s1 = (uint32_t)L.s3; a.off_g = (uint32_t)L.g;
  a.row2 = (int)((L.w3 - L.w1) / (size_t)(H / 2)); a.trows = DT_GU_ROWS;
  a.dw = dw.x; a.out = w.y;
  return hb_launch(ctx, "moe_gate_up_tc", true, moe_dtc_layer_kernel, dim3(dtc_grid(ctx)), dim3(DT_THREADS), (size_t)DT_SMEM, st, a);
}

// The down pass the same way: digit planes of the P rows of y (launched behind the gate/up kernel; rows past the list's end hold
// nothing anyone reads), then the tensor-memory kernel over 128-row tiles of w2 writing the per-pair rows; with `red` it also sums
// the rows' pairs after its CTAs have met (fin: a counter the grouping kernel zeroed).
int hbk_moe_dtc_down_run(hb_ctx* ctx, int P, int H, int I, void* ws, const ReduceArgs* red, unsigned int* fin, cudaStream_t st) {
  DecodeWs w = carve(ws, P, H, I);
  DtcWs2 dw;
  dtc_carve(ws, hbk_moe_decode_ws_bytes(P, H, I) - hbk_moe_dtc_ws_extra(P, H, I), P, H, I, &dw);
  hb_rec_layout L;
  hb_rec_layout_make(H, I, &L);
  HB_REQUIRE(ctx, ctx->dtc_H == H && ctx->dtc_I == I, HB_ERR_INVALID, "moe_decode: the down pass on the tensor cores follows the gate/up pass of the same shape");
  XdigArgs xa{w.y, I, I, dw.y, nullptr, 0, nullptr, ctx->dev_err, 1};
  int r = hb_launch(ctx, "moe_ydig", true, moe_xdig_kernel, dim3(P), dim3(256), 0, st, xa);
  if (r) return r;
  DtcArgs a{};
  dtc_args_common(ctx, w, 1, I, H / 128, &a);
  a.s_row = nullptr; a.out_ld = H; a.limit = 0.f;
  a.off_w = (uint32_t)L.w2; a.off_s0 = (uint32_t)L.s2; a.off_s1 = (uint32_t)(L.s2 + (size_t)64 * (I / 16)); a.off_g = (uint32_t)L.g;
  a.row2 = 64; a.trows = 128;
  a.dw = dw.y; a.out = w.part;
  if (red) { a.red = *red; a.fin = fin; a.red_on = 1; }
  return hb_launch(ctx, red ? "moe_down_reduce_tc" : "moe_down_tc", true, moe_dtc_layer_kernel, dim3(dtc_grid(ctx)), dim3(DT_THREADS), (size_t)DT_SMEM, st, a);
}
