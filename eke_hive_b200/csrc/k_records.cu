// Expert-record assembly on the device: the step in front of the routed-expert path.  A checkpoint stores an expert as three NVFP4
// projections (packed e2m1 bytes, e4m3 block scales, one fp32 global each); the kernels read one contiguous record per expert.
// hb_record_pack builds that record in HBM from device-resident tensors, and decodes block scales that the checkpoint stores
// compressed ("CSF": per 16 rows, 16 base code bytes + 4-bit deltas, plus a list of exception words) straight into the record —
// the work of hive::glm::GlmExperts::load_all (engine/src/glm/glm_experts.cpp:216-287) and hive::ckq::csf_decode
// (engine/src/ckpt_quant.cpp:34-73), which the reference runs on host threads.
//
// All of it is byte work bound by HBM: the expansion reads 8·C + 16 bytes and writes 16·C bytes per group of 16 rows, one thread
// per 8 consecutive scales (one 4-byte load of deltas, one 8-byte store).  The data-dependent invariants the reference checks
// sequentially are evaluated in parallel and reduced so that the reported violation is the one the sequential decoder meets first:
// the lowest exception ordinal with its first failing check, else the lowest invalid scale index.  Exceptions are applied in
// parallel; a repeated exception index with different values (no sound encoder writes one) is noticed afterwards — some word
// does not find its value in place — and that tensor's words are then re-applied in order by one thread, so the last word wins
// as in the sequential loop.
//
// A record is 1-2 MB, microseconds of HBM time, so the unit of work is a BATCH of records: the caller hands over a device array of
// jobs (three projections and a destination each) and every kernel runs once per batch with the job index in blockIdx.y — a handful
// of launches however many records, instead of host threads walking the tensors one by one.
#include <algorithm>

#include "hb_common.cuh"

namespace hb {

struct CsfArgs {
  const uint8_t* fixed; long long fixed_cols;
  const uint32_t* exc; uint32_t n_exc;
  uint32_t C, total;             // columns of the scale matrix, R·C; total == 0: nothing to decode (plain scales, or refused by shape)
  uint8_t* out;
  uint32_t* keys;                // [0] lowest (exception ordinal · 4 + failing check), [1] lowest invalid scale index; ~0 = none
  int32_t* status;               // [2]: HB_CSF_* code, position
  // plain copies of the same job (record assembly): weight bytes, and the scale bytes when they are stored uncompressed
  const uint8_t* copy_src[2]; uint8_t* copy_dst[2]; unsigned long long copy_n[2];
};

__device__ __forceinline__ uint32_t csf_delta(const CsfArgs& a, uint32_t i) {
  const uint32_t per_group = 16u * a.C, g = i / per_group, n = i - g * per_group;
  return (a.fixed[(size_t)g * a.fixed_cols + 16 + (n >> 1)] >> ((n & 1) * 4)) & 15u;
}

// code = base[row] + delta; codes above 0x7E are written as 0xFF (not a scale unless an exception replaces them).  16 scales per
// thread and step: one 8-byte load of deltas, one 16-byte store (a unit never straddles a group: 16·C is a multiple of 16).
__device__ __forceinline__ void csf_expand(const CsfArgs& a, uint32_t bid, uint32_t nblk) {
  const uint32_t per_group = 16u * a.C, units = a.total / 16;
  for (uint32_t t = bid * blockDim.x + threadIdx.x; t < units; t += nblk * blockDim.x) {
    const uint32_t i = t * 16, g = i / per_group, n = i - g * per_group;
    const uint8_t* grp = a.fixed + (size_t)g * a.fixed_cols;
    const uint2 d = *reinterpret_cast<const uint2*>(grp + 16 + (n >> 1));             // 8-byte aligned: the group pitch and n/2 are multiples of 8
    uint32_t r = n / a.C, c = n - r * a.C, base = grp[r];
    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t code = base + (((j < 8 ? d.x : d.y) >> (4 * (j & 7))) & 15u);
      w[j >> 2] |= (code > 0x7Eu ? 0xFFu : code) << (8 * (j & 3));
      if (++c == a.C && j < 15) { c = 0; ++r; base = grp[r]; }                        // n + 16 ≤ 16·C: r stays below 16 while j < 15
    }
    *reinterpret_cast<uint4*>(a.out + i) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// per exception: the checks of the sequential decoder in its order (index range, stored delta is 0, value is a finite non-negative
// e4m3 code)
__device__ __forceinline__ void csf_exc_check(const CsfArgs& a, uint32_t bid, uint32_t nblk) {
  if (a.total == 0) return;
  for (uint32_t k = bid * blockDim.x + threadIdx.x; k < a.n_exc; k += nblk * blockDim.x) {
    const uint32_t w = a.exc[k], i = w & 0xFFFFFFu, v = w >> 24;
    int bad = -1;
    if (i >= a.total) bad = 0;
    else if (csf_delta(a, i) != 0u) bad = 1;
    else if (v > 0x7Eu) bad = 2;
    if (bad >= 0) atomicMin(&a.keys[0], k * 4u + (uint32_t)bad);
  }
}

// weights (and uncompressed scales) into the record: 16 bytes per thread where both sides allow it
__device__ __forceinline__ void record_copy(const CsfArgs& a, uint32_t bid, uint32_t nblk) {
  const size_t tid = (size_t)bid * blockDim.x + threadIdx.x, nth = (size_t)nblk * blockDim.x;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const uint8_t* s = a.copy_src[p];
    uint8_t* d = a.copy_dst[p];
    const size_t n = a.copy_n[p];
    if (n == 0) continue;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d) | n) & 15) == 0) {
      const uint4* s4 = reinterpret_cast<const uint4*>(s);
      uint4* d4 = reinterpret_cast<uint4*>(d);
      size_t i = tid;
      for (; i + 3 * nth < n / 16; i += 4 * nth) {                                    // four loads in flight per thread
        const uint4 v0 = __ldg(s4 + i), v1 = __ldg(s4 + i + nth), v2 = __ldg(s4 + i + 2 * nth), v3 = __ldg(s4 + i + 3 * nth);
        d4[i] = v0; d4[i + nth] = v1; d4[i + 2 * nth] = v2; d4[i + 3 * nth] = v3;
      }
      for (; i < n / 16; i += nth) d4[i] = __ldg(s4 + i);
    } else {
      for (size_t i = tid; i < n; i += nth) d[i] = s[i];
    }
  }
}

// The three independent parts of a job in ONE launch, so that the latency-bound expansion and the scattered exception checks run
// under the bandwidth-bound copies: blockIdx.x selects the part (copy | expand | exception checks), blockIdx.y the job.
__global__ void __launch_bounds__(256) record_main_kernel(const CsfArgs* __restrict__ jobs, uint32_t cb, uint32_t eb, uint32_t kb) {
  const CsfArgs a = jobs[blockIdx.y];
  const uint32_t b = blockIdx.x;
  if (b < cb) record_copy(a, b, cb);
  else if (b < cb + eb) csf_expand(a, b - cb, eb);
  else csf_exc_check(a, b - cb - eb, kb);
}

__global__ void __launch_bounds__(256) csf_apply_kernel(const CsfArgs* __restrict__ jobs) {
  const CsfArgs a = jobs[blockIdx.y];
  if (a.total == 0) return;
  for (uint32_t k = blockIdx.x * blockDim.x + threadIdx.x; k < a.n_exc; k += gridDim.x * blockDim.x) {
    const uint32_t w = a.exc[k], i = w & 0xFFFFFFu;
    if (i < a.total) a.out[i] = (uint8_t)(w >> 24);
  }
}

// One block per job.  Every exception word must find its value in place; if one does not, two words named the same entry with
// different values and the parallel writes raced: thread 0 re-applies the job's words in order (the last word wins).
__global__ void __launch_bounds__(256) csf_settle_kernel(const CsfArgs* __restrict__ jobs) {
  const CsfArgs a = jobs[blockIdx.x];
  if (a.total == 0 || a.n_exc == 0) return;
  int conflict = 0;
  for (uint32_t k = threadIdx.x; k < a.n_exc; k += blockDim.x) {
    const uint32_t w = a.exc[k], i = w & 0xFFFFFFu;
    if (i < a.total && a.out[i] != (uint8_t)(w >> 24)) conflict = 1;
  }
  if (__syncthreads_or(conflict) && threadIdx.x == 0) {
    for (uint32_t k = 0; k < a.n_exc; ++k) {
      const uint32_t w = a.exc[k], i = w & 0xFFFFFFu;
      if (i < a.total) a.out[i] = (uint8_t)(w >> 24);
    }
  }
}

// every decoded byte must be ≤ 0x7E: 16 bytes per thread, a byte fails when its top bit is set or its low seven bits are all ones
__global__ void __launch_bounds__(256) csf_check_kernel(const CsfArgs* __restrict__ jobs) {
  const CsfArgs a = jobs[blockIdx.y];
  const uint32_t units = a.total / 16;
  uint32_t first = 0xFFFFFFFFu;
  for (uint32_t t = blockIdx.x * blockDim.x + threadIdx.x; t < units; t += gridDim.x * blockDim.x) {
    const uint4 x = *reinterpret_cast<const uint4*>(a.out + (size_t)t * 16);
    const uint32_t v[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int q = 3; q >= 0; --q) {
      const uint32_t bad = (v[q] | ((v[q] & 0x7F7F7F7Fu) + 0x01010101u)) & 0x80808080u;
      if (bad) first = min(first, t * 16 + 4 * q + (uint32_t)(__ffs((int)bad) - 1) / 8);
    }
  }
  if (first != 0xFFFFFFFFu) atomicMin(&a.keys[1], first);
}

// Large batches: apply, settle, validation and verdict of one job by ONE block (the four steps are ordered only within a tensor),
// one launch instead of four.
__global__ void __launch_bounds__(512) csf_tail_kernel(const CsfArgs* __restrict__ jobs) {
  const CsfArgs a = jobs[blockIdx.x];
  if (a.total == 0) return;
  __shared__ uint32_t first_s;
  if (threadIdx.x == 0) first_s = 0xFFFFFFFFu;
  int conflict = 0;
  for (uint32_t k = threadIdx.x; k < a.n_exc; k += blockDim.x) {
    const uint32_t w = a.exc[k], i = w & 0xFFFFFFu;
    if (i < a.total) a.out[i] = (uint8_t)(w >> 24);
  }
  __syncthreads();
  for (uint32_t k = threadIdx.x; k < a.n_exc; k += blockDim.x) {
    const uint32_t w = a.exc[k], i = w & 0xFFFFFFu;
    if (i < a.total && a.out[i] != (uint8_t)(w >> 24)) conflict = 1;
  }
  if (__syncthreads_or(conflict)) {
    if (threadIdx.x == 0)
      for (uint32_t k = 0; k < a.n_exc; ++k) {
        const uint32_t w = a.exc[k], i = w & 0xFFFFFFu;
        if (i < a.total) a.out[i] = (uint8_t)(w >> 24);
      }
    __syncthreads();
  }
  uint32_t first = 0xFFFFFFFFu;
  for (uint32_t t = threadIdx.x; t < a.total / 16; t += blockDim.x) {
    const uint4 x = *reinterpret_cast<const uint4*>(a.out + (size_t)t * 16);
    const uint32_t v[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int q = 3; q >= 0; --q) {
      const uint32_t bad = (v[q] | ((v[q] & 0x7F7F7F7Fu) + 0x01010101u)) & 0x80808080u;
      if (bad) first = min(first, t * 16 + 4 * q + (uint32_t)(__ffs((int)bad) - 1) / 8);
    }
  }
  if (first != 0xFFFFFFFFu) atomicMin(&first_s, first);
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t ke = a.keys[0], kc = first_s;
    int32_t code = HB_CSF_OK, where = 0;
    if (ke != 0xFFFFFFFFu) { code = HB_CSF_EXC_INDEX + (int32_t)(ke & 3u); where = (int32_t)(ke >> 2); }
    else if (kc != 0xFFFFFFFFu) { code = HB_CSF_CODE; where = (int32_t)kc; }
    a.status[0] = code; a.status[1] = where;
  }
}

// one thread per job: the verdict.  A job refused by shape keeps the status the preparation wrote.
__global__ void csf_finish_kernel(const CsfArgs* __restrict__ jobs, int n_jobs) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n_jobs) return;
  const CsfArgs a = jobs[j];
  if (a.total == 0) return;
  const uint32_t ke = a.keys[0], kc = a.keys[1];
  int32_t code = HB_CSF_OK, where = 0;
  if (ke != 0xFFFFFFFFu) { code = HB_CSF_EXC_INDEX + (int32_t)(ke & 3u); where = (int32_t)(ke >> 2); }
  else if (kc != 0xFFFFFFFFu) { code = HB_CSF_CODE; where = (int32_t)kc; }
  a.status[0] = code; a.status[1] = where;
}

struct RecordPrep {
  const hb_record_job* jobs; int n;
  int H, I;
  hb_rec_layout L;
  CsfArgs* out;                  // [3n]
  uint32_t* keys;                // [3n][2]
  int32_t* status;               // [n][3][2]
};

// one thread per (record, projection): the job descriptor the other kernels read, the shape rules of the format, the record's global
__global__ void record_prep_kernel(RecordPrep p) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= 3 * p.n) return;
  const int r = t / 3, j = t - 3 * r;
  const hb_record_job job = p.jobs[r];
  const hb_proj_src s = job.src[j];
  const uint64_t w_off = j == 0 ? p.L.w1 : j == 1 ? p.L.w3 : p.L.w2, s_off = j == 0 ? p.L.s1 : j == 1 ? p.L.s3 : p.L.s2;
  const int rows = j == 2 ? p.H : p.I, cols = j == 2 ? p.I : p.H, C = cols / 16;
  const unsigned long long nw = (unsigned long long)rows * cols / 2, ns = nw / 8;
  CsfArgs a;
  a.fixed = s.csf_fixed; a.fixed_cols = s.csf_fixed_cols; a.exc = s.csf_exc; a.n_exc = (uint32_t)s.n_exc; a.C = (uint32_t)C; a.total = 0;
  a.out = job.rec + s_off;
  a.keys = p.keys + 2 * t;
  a.status = p.status + 2 * t;
  const bool dst_ok = job.rec && !(reinterpret_cast<uintptr_t>(job.rec) & 15);
  a.copy_src[0] = s.weight; a.copy_dst[0] = job.rec + w_off; a.copy_n[0] = s.weight && dst_ok ? nw : 0;
  a.copy_src[1] = s.scale; a.copy_dst[1] = job.rec + s_off; a.copy_n[1] = s.scale && dst_ok ? ns : 0;
  int32_t code = HB_CSF_OK;
  if (!s.weight || (!s.scale && !s.csf_fixed) || !job.rec || (reinterpret_cast<uintptr_t>(job.rec) & 15)) code = HB_CSF_MISSING;
  else if (!s.scale) {
    if (s.csf_fixed_rows != rows / 16 || s.csf_fixed_cols != 16 + 8 * (long long)C) code = HB_CSF_SHAPE;
    else if (s.n_exc >= (1ull << 30) || (s.n_exc && !s.csf_exc) || (reinterpret_cast<uintptr_t>(s.csf_fixed) & 7) || (reinterpret_cast<uintptr_t>(s.csf_exc) & 3))
      code = HB_CSF_MISSING;
    else a.total = (uint32_t)(rows * C);
  }
  a.keys[0] = 0xFFFFFFFFu; a.keys[1] = 0xFFFFFFFFu;
  a.status[0] = code; a.status[1] = 0;
  p.out[t] = a;
  if (dst_ok) reinterpret_cast<float*>(job.rec + p.L.g)[j] = s.global;
}

static size_t csf_ws_bytes(long long jobs) { return hb_align256((size_t)jobs * sizeof(CsfArgs)) + hb_align256((size_t)jobs * 8); }

struct CsfWs { CsfArgs* jobs; uint32_t* keys; };
static CsfWs csf_carve(void* ws, long long jobs) {
  uint8_t* p = static_cast<uint8_t*>(ws);
  CsfWs w;
  w.jobs = reinterpret_cast<CsfArgs*>(p); p += hb_align256((size_t)jobs * sizeof(CsfArgs));
  w.keys = reinterpret_cast<uint32_t*>(p);
  return w;
}

// expansion, exceptions, validation and verdict of n_jobs prepared jobs
static int csf_launch(hb_ctx* ctx, const CsfWs& w, int n_jobs, long long total, bool copies, cudaStream_t st) {
  // blocks per job: enough that the whole grid fills the device a few times over, no more than the job has work for
  const unsigned per = (unsigned)std::max(1, ctx->sm_count * 8 / n_jobs);
  const unsigned eb = (unsigned)std::max<long long>(1, std::min<long long>((total / 16 + 255) / 256, per));
  const unsigned cb = copies ? std::max(2 * eb, 8u) : 0u, kb = eb;
  const dim3 blk(256);
  const CsfArgs* jobs = w.jobs;
  int r;
  if ((r = hb_launch(ctx, copies ? "record_main" : "csf_main", false, record_main_kernel, dim3(cb + eb + kb, (unsigned)n_jobs), blk, 0, st, jobs, cb, eb, kb)))
    return r;
  if (n_jobs >= ctx->sm_count)                          // enough tensors to fill the device with one block each
    return hb_launch(ctx, "csf_tail", false, csf_tail_kernel, dim3((unsigned)n_jobs), dim3(512), 0, st, jobs);
  if ((r = hb_launch(ctx, "csf_apply", false, csf_apply_kernel, dim3(eb, (unsigned)n_jobs), blk, 0, st, jobs))) return r;
  if ((r = hb_launch(ctx, "csf_settle", false, csf_settle_kernel, dim3((unsigned)n_jobs), blk, 0, st, jobs))) return r;
  if ((r = hb_launch(ctx, "csf_check", false, csf_check_kernel, dim3(eb, (unsigned)n_jobs), blk, 0, st, jobs))) return r;
  return hb_launch(ctx, "csf_finish", false, csf_finish_kernel, dim3((unsigned)(n_jobs + 127) / 128), dim3(128), 0, st,
                   static_cast<const CsfArgs*>(w.jobs), n_jobs);
}

}  // namespace hb

using namespace hb;

extern "C" {

size_t hb_csf_ws_bytes(int R, int C) { return R > 0 && C > 0 ? csf_ws_bytes(1) : 0; }

int hb_csf_decode(hb_ctx* ctx, const uint8_t* fixed, int64_t fixed_rows, int64_t fixed_cols, const uint32_t* exc, uint64_t n_exc, int R, int C,
                  uint8_t* out, int32_t* status, void* ws, size_t ws_bytes, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // shape rules of the format: refused before any launch
  HB_REQUIRE(ctx, R > 0 && C > 0 && R % 16 == 0, HB_ERR_INVALID, "CSF: rows not a multiple of 16 (R=%d C=%d)", R, C);
  HB_REQUIRE(ctx, fixed_rows == R / 16 && fixed_cols == 16 + 8 * (long long)C, HB_ERR_INVALID, "CSF: fixed shape [%lld, %lld] for scales [%d, %d]",
             (long long)fixed_rows, (long long)fixed_cols, R, C);
  const long long total = (long long)R * C;
  HB_REQUIRE(ctx, total <= (1ll << 24), HB_ERR_INVALID, "CSF: more scales than a 24-bit index addresses");
  HB_REQUIRE(ctx, n_exc < (1ull << 30), HB_ERR_UNSUPPORTED, "CSF: %llu exception words (limit 2^30)", (unsigned long long)n_exc);
  HB_REQUIRE(ctx, fixed && out && status && (n_exc == 0 || exc), HB_ERR_INVALID, "CSF: NULL tensor");
  HB_REQUIRE(ctx, hb_aligned(fixed, 8) && hb_aligned(exc, 4) && hb_aligned(out, 16) && hb_aligned(status, 4), HB_ERR_INVALID,
             "CSF: fixed 8-byte, exceptions / status 4-byte, out 16-byte aligned");
  HB_REQUIRE(ctx, ws && hb_aligned(ws, 256) && ws_bytes >= csf_ws_bytes(1), HB_ERR_WORKSPACE, "CSF: workspace of %zu bytes, 256-byte aligned",
             csf_ws_bytes(1));
  const CsfWs w = csf_carve(ws, 1);
  CsfArgs a = {};
  a.fixed = fixed; a.fixed_cols = fixed_cols; a.exc = exc; a.n_exc = (uint32_t)n_exc; a.C = (uint32_t)C; a.total = (uint32_t)total; a.out = out;
  a.keys = w.keys; a.status = status;
  HB_CUDA(ctx, cudaMemcpyAsync(w.jobs, &a, sizeof a, cudaMemcpyHostToDevice, st));      // pageable source: staged before the call returns
  HB_CUDA(ctx, cudaMemsetAsync(w.keys, 0xFF, 8, st));
  return csf_launch(ctx, w, 1, total, false, st);
}

size_t hb_record_pack_ws_bytes(int H, int I, int n) {
  return H > 0 && I > 0 && n > 0 ? hb_align256((size_t)n * sizeof(hb_record_job)) + csf_ws_bytes(3ll * n) : 0;
}

int hb_record_pack_batch(hb_ctx* ctx, const hb_record_job* jobs, int n, int H, int I, int32_t* status, void* ws, size_t ws_bytes, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  if (n == 0) return HB_OK;
  HB_REQUIRE(ctx, jobs && status && n > 0, HB_ERR_INVALID, "record_pack: NULL argument or negative count");
  hb_rec_layout L;
  HB_REQUIRE(ctx, hb_rec_layout_make(H, I, &L) == HB_OK && H % 16 == 0 && I % 16 == 0, HB_ERR_UNSUPPORTED, "record_pack: H=%d I=%d", H, I);
  const long long total = (long long)H * I / 16;
  HB_REQUIRE(ctx, total <= (1ll << 24), HB_ERR_UNSUPPORTED, "record_pack: more scales per projection than a 24-bit index addresses");
  HB_REQUIRE(ctx, hb_aligned(jobs, 8) && hb_aligned(status, 4), HB_ERR_INVALID, "record_pack: jobs 8-byte, status 4-byte aligned");
  HB_REQUIRE(ctx, ws && hb_aligned(ws, 256) && ws_bytes >= hb_record_pack_ws_bytes(H, I, n), HB_ERR_WORKSPACE,
             "record_pack: workspace of %zu bytes, 256-byte aligned", hb_record_pack_ws_bytes(H, I, n));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const CsfWs w = csf_carve(static_cast<uint8_t*>(ws) + hb_align256((size_t)n * sizeof(hb_record_job)), 3ll * n);
  RecordPrep p;
  p.jobs = jobs; p.n = n; p.H = H; p.I = I; p.L = L; p.out = w.jobs; p.keys = w.keys; p.status = status;
  int r = hb_launch(ctx, "record_prep", false, record_prep_kernel, dim3((unsigned)(3 * n + 127) / 128), dim3(128), 0, st, p);
  if (r) return r;
  return csf_launch(ctx, w, 3 * n, total, true, st);
}

int hb_record_pack(hb_ctx* ctx, const hb_proj_src* src, int H, int I, uint8_t* rec, int32_t* status, void* ws, size_t ws_bytes, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  HB_REQUIRE(ctx, src && rec && status, HB_ERR_INVALID, "record_pack: NULL argument");
  HB_REQUIRE(ctx, ws && hb_aligned(ws, 256) && ws_bytes >= hb_record_pack_ws_bytes(H, I, 1), HB_ERR_WORKSPACE,
             "record_pack: workspace of %zu bytes, 256-byte aligned", hb_record_pack_ws_bytes(H, I, 1));
  hb_record_job job;
  for (int j = 0; j < 3; ++j) job.src[j] = src[j];
  job.rec = rec;
  HB_CUDA(ctx, cudaMemcpyAsync(ws, &job, sizeof job, cudaMemcpyHostToDevice, reinterpret_cast<cudaStream_t>(stream)));   // pageable: staged before return
  return hb_record_pack_batch(ctx, static_cast<const hb_record_job*>(ws), 1, H, I, status, ws, ws_bytes, stream);
}

}  // extern "C"
