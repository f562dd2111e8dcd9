// hb_moe_decode_routed_static: the routed decode operator for callers that cannot give it a workspace.
//
// Some hosts of this library may not allocate device memory at the point where they call it: an engine that hands out its
// whole memory budget at start-up and forbids cudaMalloc afterwards, a latency-critical decode loop where an allocation
// would synchronise the device, a plugin host that owns the allocator and exposes none to plugins.  For them the scratch
// the decode kernels need lives in this translation unit as a fixed device array that every GPU loading the library holds
// until the process exits; the caller passes only inputs and outputs.
//
// The array has one fixed size, so the entry point refuses problems whose scratch would not fit (see kStaticScratchBytes and
// hb_moe_decode_static_max_pairs).  All calls on a device share the array and it keeps whatever the last call left in it: the
// kernels re-initialise the parts that must start at zero (group list header, completion counters) on every call, but two
// calls whose kernels overlap on the GPU — different streams, or different contexts on one device — race on it.
#include "hb_common.cuh"
#include "hb_kernels.h"

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;             // 4 MiB per GPU
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the array, per device ordinal.  In host code `g_static_scratch` is only a handle for the runtime, not
// a device address: it must go through cudaGetSymbolAddress, with the right device current, before a kernel may use it.
// The cache is filled without a lock: two host threads making the FIRST call on a device at the same time both look the
// address up and both store the same value — harmless, and the only thing calls from different threads share on the host.
void* g_scratch_ptr[64] = {};

int scratch_for_current_device(hb_ctx* ctx, void** out) {
  int dev = -1;
  HB_CUDA(ctx, cudaGetDevice(&dev));
  HB_REQUIRE(ctx, dev >= 0 && dev < 64 && dev == ctx->device, HB_ERR_INVALID,
             "moe_decode_routed_static: current device %d is not the context's device %d", dev, ctx->device);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    HB_CUDA(ctx, cudaGetSymbolAddress(&p, g_static_scratch));
    HB_REQUIRE(ctx, p != nullptr && hb_aligned(p, 256), HB_ERR_CUDA, "moe_decode_routed_static: bad symbol address");
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return HB_OK;
}

}  // namespace

extern "C" {

int hb_moe_decode_static_max_pairs(int H, int I) {
  if (H <= 0 || I <= 0 || H % 32 || I % 32) return 0;
  int n = 0;
  while (n < HB_MAX_PAIRS && hbk_moe_decode_ws_stream_bytes(n + 1, H, I) <= kStaticScratchBytes) ++n;
  return n;
}

int hb_moe_decode_routed_static(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                                const void* x, int H, int I, float limit, const hb_pf_combine* cmb, void* stream) {
  if (!ctx) return HB_ERR_INVALID;
  if (M == 0) return HB_OK;
  HB_REQUIRE(ctx, ids && w && rec_tab && x && cmb && cmb->out, HB_ERR_INVALID, "moe_decode_routed_static: NULL argument");
  HB_REQUIRE(ctx, M > 0 && K > 0 && E > 0 && E <= HB_MAX_EXPERTS && li >= 0, HB_ERR_INVALID, "moe_decode_routed_static: M=%d K=%d E=%d li=%d", M, K, E, li);
  HB_REQUIRE(ctx, H > 0 && I > 0 && H % 32 == 0 && I % 32 == 0, HB_ERR_UNSUPPORTED, "moe_decode_routed_static: H=%d I=%d must be multiples of 32", H, I);
  HB_REQUIRE(ctx, hb_aligned(x, 16), HB_ERR_INVALID, "moe_decode_routed_static: x must be 16-byte aligned");
  const size_t need = hbk_moe_decode_ws_stream_bytes(M * K, H, I);    // this entry point always runs the streaming chain
  HB_REQUIRE(ctx, (long long)M * K <= HB_MAX_PAIRS && need <= kStaticScratchBytes, HB_ERR_UNSUPPORTED,
             "moe_decode_routed_static: %d pairs at H=%d I=%d need %zu bytes of scratch, the built-in array holds %zu (at most %d pairs at this shape); "
             "use hb_moe_decode_routed with a caller workspace",
             M * K, H, I, need, kStaticScratchBytes, hb_moe_decode_static_max_pairs(H, I));
  void* ws = nullptr;
  const int r = scratch_for_current_device(ctx, &ws);
  if (r) return r;
  hbk_pair_src src; src.ids = ids; src.w = w; src.M = M; src.K = K; src.tab = rec_tab; src.li = li; src.E = E;
  src.ws_stream_only = true;
  hbk_reduce red; red.shared = cmb->shared; red.lg = cmb->lg; red.ld = cmb->ld; red.col = cmb->col; red.out_bf16 = cmb->out;
  return hbk_moe_decode_run(ctx, src, x, H, I, limit, red, ws, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
