// Expert-parallel exchange over NVLink peer memory, without a collective library: the two exchanges of a decode layer are
// written by this GPU's kernels straight into the other GPUs' buffers (plain peer stores) and announced with a step number.
//
//   push rows       every rank packs its B rows [bf16 row | int32 ids | fp32 weights] into slot `rank` of every peer's gather
//                   buffer, then stores the step number into that peer's flag `rank`                      (an all-gather)
//   wait            a peer's data is complete once its flag holds the step number                          (bounded polls)
//   push partials   after the local experts ran over all G·B rows, the fp32 sums of the rows that belong to rank p go into slot
//                   `rank` of p's partial buffer, then the flag                                            (a reduce-scatter,
//   combine         waits for the G partial slots, adds them in rank order (fixed: deterministic and identical on every
//                   run), applies the shared-expert combine, and advances the step counter                  minus the reduction)
//
// Buffers are reused every layer without double buffering: a rank can only run ahead of a peer by less than one exchange,
// because its next push of rows needs its own combine to have finished, which needs every peer's partials of this layer, which a
// peer sends only after it has finished reading its gather buffer — and symmetrically for the partial buffers.
// Every wait is bounded; a wait that gives up sets the context's error word, and once that word is set all later waits return at
// once, so a lost peer ends the step in seconds instead of hanging the GPU.  No kernel here is ever launched twice on one GPU
// to wait for itself: the kernel a wait depends on runs on another GPU.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>

#include "ep.cuh"
#include "hb_common.cuh"
#include "hb_kernels.h"
#include "router.cuh"

namespace hb {

constexpr int kEpMaxRanks = 8;
struct EpPeers {
  uint8_t* recv[kEpMaxRanks];        // peer p's gather buffer [G·B, rec_bytes]
  uint32_t* ag_flag[kEpMaxRanks];    // peer p's gather flags [G]
  float* rs[kEpMaxRanks];            // peer p's partial buffer [G, B, H]
  uint32_t* rs_flag[kEpMaxRanks];    // peer p's partial flags [G]
};

// grid = G (one CTA per destination rank)
__global__ void __launch_bounds__(512) ep_push_rows_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int32_t* __restrict__ ids,
                                                           const float* __restrict__ w, int B, int H, int K, int rec_bytes, EpPeers peers, int rank,
                                                           const uint32_t* __restrict__ step_ctr) {
  const int pi = blockIdx.x;
  const uint32_t step = *step_ctr + 1u;
  uint8_t* dst = peers.recv[pi] + (size_t)rank * B * rec_bytes;
  const int xc = H / 8;                                                     // 16-byte pieces of a row's activations
  for (int i = threadIdx.x; i < B * xc; i += blockDim.x) {
    const int r = i / xc, c = i - r * xc;
    reinterpret_cast<uint4*>(dst + (size_t)r * rec_bytes)[c] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * ldx) + c);
  }
  for (int i = threadIdx.x; i < B * 2 * K; i += blockDim.x) {               // ids then weights, 4 bytes each
    const int r = i / (2 * K), c = i - r * 2 * K;
    const uint32_t v = c < K ? (uint32_t)ids[(size_t)r * K + c] : __float_as_uint(w[(size_t)r * K + c - K]);
    reinterpret_cast<uint32_t*>(dst + (size_t)r * rec_bytes + (size_t)H * 2)[c] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) st_release_sys(peers.ag_flag[pi] + rank, step);
}

// Router and push in one launch: every CTA (one per destination rank) routes all B rows itself — the routing is a deterministic
// function of the logits, so the G copies agree — and sends rows, ids and weights to its rank.  CTA 0 also stores ids / w for
// the caller.  Dynamic shared memory: (warps·E + 2·B·K) words.
__global__ void __launch_bounds__(512) ep_route_push_kernel(const float* __restrict__ logits, int ld, int E, int K, int renorm, int logits_bf16,
                                                            const __nv_bfloat16* __restrict__ x, int ldx, int32_t* __restrict__ ids_out,
                                                            float* __restrict__ w_out, int B, int H, int rec_bytes, EpPeers peers, int rank,
                                                            const uint32_t* __restrict__ step_ctr) {
  extern __shared__ float ep_sm[];
  griddep_wait();                                                          // the previous step's combine has advanced the step counter
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  int32_t* ids_s = reinterpret_cast<int32_t*>(ep_sm + (size_t)nw * E);
  float* w_s = reinterpret_cast<float*>(ids_s + B * K);
  for (int m = warp; m < B; m += nw)
    route_softmax_row(logits + (size_t)m * ld, E, K, renorm, logits_bf16, ep_sm + (size_t)warp * E, lane, ids_s + m * K, w_s + m * K);
  __syncthreads();
  const int pi = blockIdx.x;
  if (pi == 0)
    for (int i = threadIdx.x; i < B * K; i += blockDim.x) { ids_out[i] = ids_s[i]; w_out[i] = w_s[i]; }
  const uint32_t step = *step_ctr + 1u;
  uint8_t* dst = peers.recv[pi] + (size_t)rank * B * rec_bytes;
  const int xc = H / 8;
  for (int i = threadIdx.x; i < B * xc; i += blockDim.x) {
    const int r = i / xc, c = i - r * xc;
    reinterpret_cast<uint4*>(dst + (size_t)r * rec_bytes)[c] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * ldx) + c);
  }
  for (int i = threadIdx.x; i < B * 2 * K; i += blockDim.x) {
    const int r = i / (2 * K), c = i - r * 2 * K;
    const uint32_t v = c < K ? (uint32_t)ids_s[r * K + c] : __float_as_uint(w_s[r * K + c - K]);
    reinterpret_cast<uint32_t*>(dst + (size_t)r * rec_bytes + (size_t)H * 2)[c] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) st_release_sys(peers.ag_flag[pi] + rank, step);
}

// one CTA: thread r waits for rank r's flag
__global__ void ep_wait_kernel(const uint32_t* __restrict__ flags, int G, const uint32_t* __restrict__ step_ctr, uint32_t* err, uint32_t site) {
  if (*reinterpret_cast<volatile uint32_t*>(err)) return;
  if ((int)threadIdx.x < G) ep_wait_flag(flags + threadIdx.x, *step_ctr + 1u, err, site);
}

// grid = (G destination ranks, chunks): the rows of `part` that belong to rank p → slot `rank` of p's partial buffer
__global__ void __launch_bounds__(256) ep_push_partials_kernel(const float* __restrict__ part, int B, int H, EpPeers peers, int rank,
                                                               const uint32_t* __restrict__ step_ctr, unsigned int* __restrict__ done) {
  const int pi = blockIdx.x;
  const uint32_t step = *step_ctr + 1u;
  const float4* src = reinterpret_cast<const float4*>(part + (size_t)pi * B * H);
  float4* dst = reinterpret_cast<float4*>(peers.rs[pi] + (size_t)rank * B * H);
  const int n4 = B * H / 4;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n4; i += gridDim.y * blockDim.x) dst[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&done[pi], 1u) == gridDim.y - 1) {                        // last chunk of this destination: everything is on its way
      done[pi] = 0;
      __threadfence_system();
      st_release_sys(peers.rs_flag[pi] + rank, step);
    }
  }
}

// out = bf16(bf16(Σ_ranks partial) + bf16(bf16(sigmoid(bf16 gate logit))·shared)), one thread per element
__global__ void __launch_bounds__(256) ep_combine_kernel(const float* __restrict__ rs, const uint32_t* __restrict__ rs_flag, int G, int B, int H,
                                                         const __nv_bfloat16* __restrict__ shared, const float* __restrict__ lg, int ld, int col,
                                                         __nv_bfloat16* __restrict__ out, uint32_t* __restrict__ step_ctr, unsigned int* __restrict__ done,
                                                         uint32_t* err) {
  __shared__ int ok_s;
  griddep_wait();
  const uint32_t step = *step_ctr + 1u;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < G && !*reinterpret_cast<volatile uint32_t*>(err)) {
    if (!ep_wait_flag(rs_flag + threadIdx.x, step, err, 0x80000u)) ok_s = 0;
  }
  __syncthreads();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (ok_s && i < (size_t)B * H) {
    float a = 0.f;
    for (int r = 0; r < G; ++r) a = __fadd_rn(a, __ldcg(rs + (size_t)r * B * H + i));      // rank order
    float sh = 0.f;
    if (shared) {
      sh = __bfloat162float(shared[i]);
      if (lg) sh = bf16r(__fmul_rn(bf16r(sigmoid_portable(bf16r(lg[(size_t)(i / H) * ld + col]))), sh));
    }
    out[i] = __float2bfloat16(__fadd_rn(bf16r(a), sh));
  }
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(done, 1u) == gridDim.x - 1) { *done = 0; *step_ctr = step; }   // last block: the layer's exchanges are over
}

}  // namespace hb

using namespace hb;

struct hb_ep {
  hb_ctx* ctx;
  int rank, world, B, H, K, rec_bytes;
  EpPeers peers;
  uint8_t* recv; uint32_t* ag_flag; float* rs; uint32_t* rs_flag;      // this rank's own buffers (= peers.*[rank])
  uint32_t* step_ctr; unsigned int* done;                              // device words owned by this object: step counter, completion counters [G + 1]
};

extern "C" {

size_t hb_ep_rec_bytes(int H, int K) { return H > 0 && K > 0 ? ((size_t)H * 2 + (size_t)K * 8 + 15) / 16 * 16 : 0; }

// Sharing exchange memory between the ranks' processes.  The importing side opens the handle with ITS OWN device current and lazy
// peer access, which is the documented way to make another device's allocation addressable from this device's kernels
// (opening it under the exporting device's context and enabling peer access afterwards left the range unmapped for this device).
int hb_ep_export(hb_ctx* ctx, const void* ptr, void* handle64, size_t* offset) {
  if (!ctx) return HB_ERR_INVALID;
  HB_REQUIRE(ctx, ptr && handle64 && offset, HB_ERR_INVALID, "ep_export: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  HB_CUDA(ctx, cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range = nullptr;
  if (!range) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) range = reinterpret_cast<RangeFn>(f);
  }
  HB_REQUIRE(ctx, range, HB_ERR_CUDA, "ep_export: cuMemGetAddressRange is not available from this driver");
  CUdeviceptr base = 0; size_t size = 0;
  HB_REQUIRE(ctx, range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS, HB_ERR_CUDA, "ep_export: cuMemGetAddressRange failed");
  memcpy(handle64, &h, 64);
  *offset = reinterpret_cast<uintptr_t>(ptr) - static_cast<uintptr_t>(base);      // the handle names the whole allocation
  return HB_OK;
}

int hb_ep_import(hb_ctx* ctx, const void* handle64, size_t offset, void** ptr, void** base_out) {
  if (!ctx) return HB_ERR_INVALID;
  HB_REQUIRE(ctx, handle64 && ptr && base_out, HB_ERR_INVALID, "ep_import: NULL argument");
  int cur = -1;
  HB_CUDA(ctx, cudaGetDevice(&cur));
  HB_REQUIRE(ctx, cur == ctx->device, HB_ERR_INVALID, "ep_import: the context's device %d must be current (current: %d)", ctx->device, cur);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* base = nullptr;
  HB_CUDA(ctx, cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *base_out = base;
  *ptr = static_cast<uint8_t*>(base) + offset;
  return HB_OK;
}

int hb_ep_close(hb_ctx* ctx, void* base) {
  if (!ctx) return HB_ERR_INVALID;
  if (base) HB_CUDA(ctx, cudaIpcCloseMemHandle(base));
  return HB_OK;
}

int hb_ep_create(hb_ctx* ctx, int rank, int world, int B, int H, int K, void* const* recv, void* const* ag_flag, void* const* rs, void* const* rs_flag,
                 hb_ep** out) {
  if (!ctx || !out) return HB_ERR_INVALID;
  HB_REQUIRE(ctx, world >= 1 && world <= kEpMaxRanks && rank >= 0 && rank < world && B >= 1 && H >= 8 && H % 8 == 0 && K >= 1 && recv && ag_flag && rs &&
                      rs_flag, HB_ERR_INVALID, "ep_create: rank %d of %d, B=%d H=%d K=%d", rank, world, B, H, K);
  hb_ep* e = new hb_ep();
  e->ctx = ctx; e->rank = rank; e->world = world; e->B = B; e->H = H; e->K = K; e->rec_bytes = (int)hb_ep_rec_bytes(H, K);
  for (int p = 0; p < world; ++p) {
    if (!recv[p] || !ag_flag[p] || !rs[p] || !rs_flag[p]) { delete e; return hb_fail(ctx, HB_ERR_INVALID, "ep_create: NULL buffer of rank %d", p); }
    e->peers.recv[p] = static_cast<uint8_t*>(recv[p]); e->peers.ag_flag[p] = static_cast<uint32_t*>(ag_flag[p]);
    e->peers.rs[p] = static_cast<float*>(rs[p]); e->peers.rs_flag[p] = static_cast<uint32_t*>(rs_flag[p]);
  }
  e->recv = e->peers.recv[rank]; e->ag_flag = e->peers.ag_flag[rank]; e->rs = e->peers.rs[rank]; e->rs_flag = e->peers.rs_flag[rank];
  void* words = nullptr;
  if (cudaMalloc(&words, 256) != cudaSuccess || cudaMemset(words, 0, 256) != cudaSuccess) { delete e; cudaGetLastError(); return hb_fail(ctx, HB_ERR_CUDA, "ep_create: cudaMalloc"); }
  e->step_ctr = static_cast<uint32_t*>(words); e->done = reinterpret_cast<unsigned int*>(words) + 8;
  *out = e;
  return HB_OK;
}

void hb_ep_destroy(hb_ep* e) {
  if (!e) return;
  cudaFree(e->step_ctr);
  delete e;
}

int hb_ep_push_rows(hb_ep* e, const void* x_bf16, int ldx, const int32_t* ids, const float* w, void* stream) {
  if (!e) return HB_ERR_INVALID;
  hb_ctx* ctx = e->ctx;
  HB_REQUIRE(ctx, x_bf16 && ids && w && ldx >= e->H && ldx % 8 == 0 && hb_aligned(x_bf16, 16), HB_ERR_INVALID, "ep_push_rows: bad arguments");
  return hb_launch(ctx, "ep_push_rows", false, ep_push_rows_kernel, dim3(e->world), dim3(512), 0, reinterpret_cast<cudaStream_t>(stream),
                   reinterpret_cast<const __nv_bfloat16*>(x_bf16), ldx, ids, w, e->B, e->H, e->K, e->rec_bytes, e->peers, e->rank,
                   (const uint32_t*)e->step_ctr);
}

int hb_ep_route_push(hb_ep* e, const float* logits, int ld, int E, int renorm, int logits_bf16, const void* x_bf16, int ldx, int32_t* ids_out,
                     float* w_out, void* stream) {
  if (!e) return HB_ERR_INVALID;
  hb_ctx* ctx = e->ctx;
  HB_REQUIRE(ctx, logits && x_bf16 && ids_out && w_out && ldx >= e->H && ldx % 8 == 0 && hb_aligned(x_bf16, 16), HB_ERR_INVALID, "ep_route_push: bad arguments");
  HB_REQUIRE(ctx, E >= 1 && ld >= E && e->K <= 16 && e->K <= E, HB_ERR_INVALID, "ep_route_push: E=%d ld=%d K=%d", E, ld, e->K);
  const size_t smem = ((size_t)16 * E + 2 * (size_t)e->B * e->K) * 4;
  HB_REQUIRE(ctx, smem <= 48 * 1024, HB_ERR_UNSUPPORTED, "ep_route_push: E=%d too large for the fused router (route with hb_route_softmax_topk, then hb_ep_push_rows)", E);
  return hb_launch(ctx, "ep_route_push", true, ep_route_push_kernel, dim3(e->world), dim3(512), smem, reinterpret_cast<cudaStream_t>(stream), logits, ld, E,
                   e->K, renorm, logits_bf16, reinterpret_cast<const __nv_bfloat16*>(x_bf16), ldx, ids_out, w_out, e->B, e->H, e->rec_bytes, e->peers, e->rank,
                   (const uint32_t*)e->step_ctr);
}

int hb_ep_layer_local(hb_ep* e, const uint8_t* const* rec_tab, int li, int E, int I, float limit, const uint8_t* shared_rec, void* shared_out_bf16, void* ws,
                      void* stream) {
  if (!e) return HB_ERR_INVALID;
  hb_ctx* ctx = e->ctx;
  const int M = e->world * e->B;
  HB_REQUIRE(ctx, rec_tab && ws && hb_aligned(ws, 256) && E >= 1 && E <= HB_MAX_EXPERTS && li >= 0 && (!shared_rec || shared_out_bf16), HB_ERR_INVALID,
             "ep_layer_local: bad arguments");
  HB_REQUIRE(ctx, hbk_moe_decode_fast(e->H, I) && M * (e->K + 1) <= HB_MAX_PAIRS, HB_ERR_UNSUPPORTED, "ep_layer_local: H=%d I=%d, %d pairs", e->H, I, M * (e->K + 1));
  hbk_pair_src src;
  src.ids = reinterpret_cast<const int32_t*>(e->recv + (size_t)e->H * 2); src.w = reinterpret_cast<const float*>(e->recv + (size_t)e->H * 2 + (size_t)e->K * 4);
  src.ld_ids = e->rec_bytes / 4; src.M = M; src.K = e->K; src.tab = rec_tab; src.li = li; src.E = E; src.x_ld = e->rec_bytes / 2;
  src.shared_rec = shared_rec; src.sh_row0 = e->rank * e->B; src.sh_rows = shared_rec ? e->B : 0;
  src.wait_flags = e->ag_flag; src.wait_n = e->world; src.wait_step = e->step_ctr;
  hbk_ep_push push{};
  for (int p = 0; p < e->world; ++p) { push.rs[p] = e->peers.rs[p]; push.flag[p] = e->peers.rs_flag[p]; }
  push.B = e->B; push.rank = e->rank; push.world = e->world; push.step = e->step_ctr; push.done = e->done + kEpMaxRanks + 1;
  hbk_reduce red; red.ep = &push; red.shared_out = shared_rec ? shared_out_bf16 : nullptr;
  return hbk_moe_decode_run(ctx, src, e->recv, e->H, I, limit, red, ws, reinterpret_cast<cudaStream_t>(stream));
}

int hb_ep_wait_rows(hb_ep* e, void* stream) {
  if (!e) return HB_ERR_INVALID;
  return hb_launch(e->ctx, "ep_wait_rows", false, ep_wait_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), (const uint32_t*)e->ag_flag,
                   e->world, (const uint32_t*)e->step_ctr, e->ctx->dev_err, 0x40000u);
}

int hb_ep_push_partials(hb_ep* e, const float* part, void* stream) {
  if (!e) return HB_ERR_INVALID;
  hb_ctx* ctx = e->ctx;
  HB_REQUIRE(ctx, part && hb_aligned(part, 16) && (e->B * e->H) % 4 == 0, HB_ERR_INVALID, "ep_push_partials: bad arguments");
  int chunks = (e->B * e->H / 4 + 2047) / 2048;
  if (chunks > 16) chunks = 16;
  return hb_launch(ctx, "ep_push_partials", false, ep_push_partials_kernel, dim3(e->world, chunks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), part,
                   e->B, e->H, e->peers, e->rank, (const uint32_t*)e->step_ctr, e->done);
}

int hb_ep_combine(hb_ep* e, const void* shared_bf16, const float* lg, int ld, int col, void* out_bf16, void* stream) {
  if (!e) return HB_ERR_INVALID;
  hb_ctx* ctx = e->ctx;
  HB_REQUIRE(ctx, out_bf16 && (!lg || shared_bf16), HB_ERR_INVALID, "ep_combine: no output, or a gate without shared rows");
  const size_t n = (size_t)e->B * e->H;
  return hb_launch(ctx, "ep_combine", true, ep_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                   (const float*)e->rs, (const uint32_t*)e->rs_flag, e->world, e->B, e->H, reinterpret_cast<const __nv_bfloat16*>(shared_bf16), lg, ld, col,
                   reinterpret_cast<__nv_bfloat16*>(out_bf16), e->step_ctr, e->done + kEpMaxRanks, ctx->dev_err);
}

}  // extern "C"
