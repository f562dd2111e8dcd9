// Shared declarations of the library's translation units: the context, error plumbing, launch helpers and the small
// device-side toolbox (format decode, bf16/f16 helpers, mbarrier and bulk-copy wrappers for sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/hive_b200.h"

// Words of the context's 256-byte device block besides the error word [0]: [16] a counter the decode prep kernel owns, [17] the
// poll limit of waits on flags that other ranks set (hb_config.wait_polls), [18..19] counters of the prefill plan kernel.
constexpr int kErrWaitPolls = 17;
constexpr int kErrPlanMeet = 18;
constexpr int kErrBoundSite = 20;     // [20], [21]: first failed range check of a -DHB_BOUNDS build (site code, offending value)      // [18], [19]: the meeting counters of the prefill plan kernel

struct hb_ctx {
  int device = 0;
  int sm_count = 0;
  int max_ctas = 0;
  int flags = 0;
  int smem_optin = 0;            // cudaDevAttrMaxSharedMemoryPerBlockOptin
  uint32_t* dev_err = nullptr;   // device error word: 0 = fine; kernels OR a site code into it when a bounded wait gives up
  unsigned long long launches = 0;
  // tensor maps of the decode layer kernel (k_moe_dtc.cu): device array + the shape they were made for
  void* dtc_maps = nullptr;
  int dtc_H = 0, dtc_I = 0;
  // streaming down kernels (one per split-K width): whether the planned number of CTAs per SM is really resident, i.e. whether the
  // CTAs may meet inside the kernel (k_moe_decode.cu)
  const void* down_fn[8] = {nullptr}; bool down_meet[8] = {false};
  char err[512] = {0};
  // optional per-kernel timing (hb_profile_enable): a start/stop event pair around every launch, aggregated by hb_profile_read
  bool prof_on = false;
  int prof_n = 0;
  static constexpr int kProfMax = 8192;
  cudaEvent_t* prof_ev = nullptr;        // [2 * kProfMax], created on first enable
  const char** prof_name = nullptr;      // [kProfMax]
};

inline int hb_fail(hb_ctx* ctx, int code, const char* fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof ctx->err, fmt, ap);
    va_end(ap);
  }
  return code;
}

#define HB_CUDA(ctx, call)                                                                                  \
  do {                                                                                                      \
    cudaError_t e_ = (call);                                                                                \
    if (e_ != cudaSuccess) return hb_fail((ctx), HB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_));     \
  } while (0)

#define HB_REQUIRE(ctx, cond, code, ...) \
  do {                                   \
    if (!(cond)) return hb_fail((ctx), (code), __VA_ARGS__); \
  } while (0)

// Every kernel launch of the library goes through hb_launch: it counts the launch, converts a launch failure into a status
// with a message, optionally asks for programmatic dependent launch (the kernel then calls griddep_wait() before touching its
// inputs) and, when profiling is on, brackets the kernel with a CUDA event pair (PDL is then off so the pair times the kernel alone).
template <typename... KArgs, typename... Args>
inline int hb_launch(hb_ctx* ctx, const char* what, bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                     Args... args) {
  const bool prof = ctx->prof_on && ctx->prof_n < hb_ctx::kProfMax;
  if (prof) cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], st);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = (pdl && !ctx->prof_on && !(ctx->flags & HB_FLAG_NO_PDL)) ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (prof) { cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], st); ctx->prof_name[ctx->prof_n++] = what; }
  ctx->launches++;
  if (e != cudaSuccess) return hb_fail(ctx, HB_ERR_CUDA, "launch %s: %s", what, cudaGetErrorString(e));
  return HB_OK;
}

inline size_t hb_align256(size_t b) { return (b + 255) / 256 * 256; }
inline bool hb_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ------------------------------------------------------------------------------------------------ device toolbox
#ifdef __CUDACC__
namespace hb {

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// e4m3 → fp32, exact for every code (0x7F / 0xFF give NaN like the reference's decode)
__device__ __forceinline__ float e4m3_to_f32(uint32_t v) {
  const uint32_t e = (v >> 3) & 0xF, m = v & 7;
  float r;
  if (e == 0) r = (float)m * 0.001953125f;                                   // m · 2^-9
  else if (e == 15 && m == 7) r = __int_as_float(0x7fc00000);
  else r = __int_as_float(((e + 120u) << 23) | (m << 20));                   // (1 + m/8) · 2^(e-7)
  return (v & 0x80) ? -r : r;
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t nib) {
  const uint32_t c = nib & 7;
  // 0, .5, 1, 1.5, 2, 3, 4, 6
  const float t = c < 4 ? 0.5f * (float)c : (c == 4 ? 2.f : c == 5 ? 3.f : c == 6 ? 4.f : 6.f);
  return (nib & 8) ? -t : t;
}
__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16(x)); }

// Portable exp: Cody–Waite reduction + degree-5 polynomial with explicit fma, bit-identical on CPU and GPU
// (the form of the reference's engine/src/qwen/cpu/qwen_cpu_simd.h:23-41).
__device__ __forceinline__ float exp_portable(float x) {
  x = fminf(fmaxf(x, -87.0f), 88.0f);
  const float n = rintf(__fmul_rn(x, 1.44269504088896341f));
  float r = __fmaf_rn(n, -0.693359375f, x);
  r = __fmaf_rn(n, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = __fmaf_rn(p, r, 1.3981999507e-3f); p = __fmaf_rn(p, r, 8.3334519073e-3f); p = __fmaf_rn(p, r, 4.1665795894e-2f);
  p = __fmaf_rn(p, r, 1.6666665459e-1f); p = __fmaf_rn(p, r, 5.0000001201e-1f);
  const float rr = __fmul_rn(r, r);
  float y = __fmaf_rn(p, rr, r);
  y = __fadd_rn(y, 1.f);
  return __fmul_rn(y, __int_as_float(((int)n + 127) << 23));
}
__device__ __forceinline__ float sigmoid_portable(float x) { return __fdiv_rn(1.f, __fadd_rn(1.f, exp_portable(-x))); }
__device__ __forceinline__ float silu_portable(float x) { return __fdiv_rn(x, __fadd_rn(1.f, exp_portable(-x))); }

// ---- shared-memory barriers and bulk asynchronous copies (sm_90+ PTX, used here for sm_100a) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2^26 polls (seconds), ORs `site` into the error word and returns false.  Callers leave
// their loops when it fails, so a lost transaction ends the kernel instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* err, uint32_t site) {
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) __nanosleep(32);
  }
  if (err) atomicOr(err, site);
  return false;
}
// 1-D bulk copy global → shared, completion counted in bytes on `bar`.  dst, src 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Range checks of the debug build (compile with -DHB_BOUNDS: `python eke_hive_b200/build.py --bounds`).  HB_BOUND(err, cond, site, value)
// is `true` in the normal build.  In the debug build a failed check sets bit 31 of the context's error word, records the first
// failing site and value in the words behind it, and evaluates to false so that the caller skips the access: a wrong index becomes
// an HB_ERR_DEVICE_FLAG from hb_check_device instead of a memory fault.
#ifdef HB_BOUNDS
__device__ __forceinline__ bool hb_bound_check(uint32_t* err, bool ok, uint32_t site, long long value) {
  if (!ok && err) {
    atomicOr(err, 0x80000000u);
    if (atomicCAS(err + kErrBoundSite, 0u, site) == 0u) err[kErrBoundSite + 1] = (uint32_t)value;
  }
  return ok;
}
#define HB_BOUND(err, cond, site, value) (hb::hb_bound_check((err), (cond), (site), (long long)(value)))
#else
#define HB_BOUND(err, cond, site, value) (true)
#endif
__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

// two e2m1 codes (one byte: low nibble = first element) → half2, exact
__device__ __forceinline__ uint32_t cvt_e2m1x2_f16x2(uint32_t byte) {
  uint32_t out;
  asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %1;\n cvt.rn.f16x2.e2m1x2 %0, b0;\n}" : "=r"(out) : "r"(byte));
  return out;
}
// all four bytes of a word (eight e2m1 codes) → four half2
__device__ __forceinline__ void cvt_e2m1x8_f16x2(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
      " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(w));
}
// two e4m3 codes (low 16 bits) → half2, exact
__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint32_t two) {
  uint32_t out;
  asm("{\n .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %1;\n cvt.rn.f16x2.e4m3x2 %0, lo;\n}" : "=r"(out) : "r"(two));
  return out;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// D += A(16x16 f16, row) · B(16x8 f16, col), fp32 accumulate
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace hb
#endif
