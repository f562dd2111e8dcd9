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

#include "hb_common.cuh"
#include "hb_kernels.h"

namespace hb {

constexpr int kEpMaxRanks = 8;
struct EpPeers {
  uint8_t* recv[kEpMaxRanks];        // peer p's gather buffer [G·B, rec_bytes]
  uint32_t* ag_flag[kEpMaxRanks];    // peer p's gather flags [G]
  float* rs[kEpMaxRanks];            // peer p's partial buffer [G, B, H]
  uint32_t* rs_flag[kEpMaxRanks];    // peer p's partial flags [G]
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// flag ≥ step (wrap-safe), polled at most ~2^24 times with back-off (seconds); false = gave up
__device__ __forceinline__ bool ep_wait_flag(const uint32_t* flag, uint32_t step, uint32_t* err, uint32_t site) {
  for (uint32_t it = 0; it < (1u << 24); ++it) {
    if ((int32_t)(ld_acquire_sys(flag) - step) >= 0) return true;
    if (it > 32) __nanosleep(it < 4096 ? 64 : 256);
    if ((it & 1023) == 1023 && *reinterpret_cast<volatile uint32_t*>(err)) return false;      // somebody already gave up
  }
  atomicOr(err, site);
  return false;
}

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
  return hb_launch(ctx, "ep_combine", false, ep_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                   (const float*)e->rs, (const uint32_t*)e->rs_flag, e->world, e->B, e->H, reinterpret_cast<const __nv_bfloat16*>(shared_bf16), lg, ld, col,
                   reinterpret_cast<__nv_bfloat16*>(out_bf16), e->step_ctr, e->done + kEpMaxRanks, ctx->dev_err);
}

}  // extern "C"
