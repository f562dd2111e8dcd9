/* hive_b200.h — C ABI of the B200 (sm_100a) quantized routed-expert path.
 *
 * One shared library, plain pointers and sizes, no C++ or framework types.  Every compute entry point is
 * stream-ordered and asynchronous: it takes DEVICE pointers, enqueues work on `stream` (a cudaStream_t passed as
 * void*; NULL = the legacy default stream) and returns without synchronising.  The caller owns every buffer,
 * including scratch (`ws`), whose size the matching *_ws_bytes function gives.  Nothing is allocated after
 * hb_create.  Return value: HB_OK (0) or a negative hb_status; hb_last_error() gives the message of the last failure
 * on that context.  No entry point throws, aborts or falls back to a CPU path.  Calls on one context must not overlap.
 *
 * Each declaration cites the operator of the reference engine it stands in for (paths inside the reference project).
 * The C++ engine's namespaces (hive::glm, hive::qwen, hive::q27::k) are mirrored over this ABI by
 * eke_hive_b200/csrc/hive_compat.hpp, so reference call sites compile unchanged against this library.
 */
#ifndef HIVE_B200_H
#define HIVE_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define HB_API
#else
#define HB_API __attribute__((visibility("default")))
#endif

typedef enum hb_status {
  HB_OK = 0,
  HB_ERR_INVALID = -1,      /* bad argument (null pointer, negative size, misaligned buffer) */
  HB_ERR_UNSUPPORTED = -2,  /* shape outside what the kernels accept (see hb_*_supported) */
  HB_ERR_CUDA = -3,         /* a CUDA runtime call failed; message holds cudaGetErrorString */
  HB_ERR_NO_DEVICE = -4,    /* no usable sm_100 device */
  HB_ERR_WORKSPACE = -5,    /* ws NULL or not 256-byte aligned */
  HB_ERR_DEVICE_FLAG = -6   /* a kernel gave up on a bounded wait and set the context's error word */
} hb_status;

typedef struct hb_ctx hb_ctx;

typedef struct hb_config {
  int device;       /* CUDA device ordinal */
  int max_ctas;     /* 0 = one CTA set per SM of the device; >0 caps the persistent grids (tests) */
  int flags;        /* HB_FLAG_* */
  unsigned wait_polls; /* how often a kernel polls a flag another rank sets before it gives up and sets the device error word
                          (hb_check_device then returns HB_ERR_DEVICE_FLAG); 0 = 2^24 polls with back-off, a few seconds */
} hb_config;
#define HB_FLAG_NO_PDL 1   /* launch every kernel fully serialised (no programmatic dependent launch) */
#define HB_FLAG_FUSED 2    /* decode: run gate/up, down and reduce as ONE persistent kernel (experimental; default: three kernels chained by PDL) */
#define HB_FLAG_DECODE_MMA_SYNC 8 /* decode: run the routed operators on the register-dequantisation (mma.sync) streaming kernels at every size */
#define HB_FLAG_DECODE_TC 16      /* same as HB_FLAG_DECODE_TC_GU (kept for callers that set it) */
#define HB_FLAG_DECODE_TC_GU 64   /* decode, routed operators: the gate/up pass runs on the tensor-memory kernel (exact digit planes of the activations,
                                     block-scaled FP4 MMAs) at every size, grouping and down pass on the streaming kernels.  With neither flag the
                                     library picks by the number of pairs of the call (40 or more: tensor memory); both engines meet the same
                                     tolerance, and a row's bits do not depend on its batch as long as the engine does not change — pin one
                                     with a flag where that matters */
#define HB_FLAG_DECODE_TC_DOWN 128 /* decode, routed operators on one GPU: where the gate/up pass runs on the tensor-memory kernel, the down pass does too
                                     (digit planes of y between the passes; the sums over a row's pairs in the kernel's tail) */
#define HB_FLAG_LAYER_A4 32       /* hb_moe_layer may run calls of more than 64 rows on the W4A4 grouped GEMM (activations quantised to NVFP4 — the
                                     reference's lossy opt-in, fn_moe_prefill_set_a4).  Without it hb_moe_layer keeps bf16 activations at every
                                     row count: the same numbers as the decode operators, never a silent change of arithmetic */
#define HB_FLAG_PREFILL_A16 4u /* hb_moe_prefill keeps bf16 activations (W4A16, the reference's default prefill arithmetic).  Calls of more than 64
                                  rows run a grouped GEMM on the tensor cores (kind::f16 MMAs over weight tiles dequantised exactly to bf16, fp32
                                  sums); calls of up to 64 rows run the decode kernels */
                               /* hb_moe_layer on such a context sends calls of more than 64 rows through the same GEMM (router → shared expert →
                                  routed experts with the fused combine); without it hb_moe_layer runs the decode kernels at every row count */
#define HB_FLAG_PREFILL_A16_ROWS 256u /* with HB_FLAG_PREFILL_A16: every call runs the decode kernels over sub-chunks of rows — bit-identical to
                                  hb_moe_decode_routed(_f32) on the same rows, but the expert records are streamed once per sub-chunk */

/* Expert record layout, byte-identical to hive::glm::ExpertRecLayout::make (engine/include/hive/glm/glm_moe.h:13-22):
 * [w1 gate e2m1 [I,H/2]][s1 e4m3 [I,H/16]][w3 up][s3][w2 down e2m1 [H,I/2]][s2 e4m3 [H,I/16]][g1 g3 g2 fp32], total 4096-aligned. */
typedef struct hb_rec_layout {
  uint64_t w1, s1, w3, s3, w2, s2, g, total;
} hb_rec_layout;

/* One (row, expert) pair — same ABI as hive::glm::MoePair (glm_moe.h:25): row at 0, rec at 8, w at 16, 24 bytes. */
typedef struct hb_moe_pair {
  int32_t row;
  const uint8_t* rec;
  float w;
} hb_moe_pair;

/* Shared-expert + gate combine of the routed operators — hive::qwen::FnPfCombine (engine/include/hive/qwen/fn_moe.h:59). */
typedef struct hb_pf_combine {
  const void* shared;  /* bf16 [M,H] */
  const float* lg;     /* gate logit of row m at lg[m*ld + col]; NULL = no gate: out = bf16(bf16(routed)+bf16(shared)) */
  int ld, col;
  void* out;           /* bf16 [M,H] */
} hb_pf_combine;

/* Dense weight matrix of the 27B-style decode GEMV — stands in for hive::q27::GMat (engine/include/hive/q27/q27_kernels.h:17-36). */
typedef enum hb_wfmt { HB_FMT_NVFP4 = 0, HB_FMT_LB3_G64 = 1, HB_FMT_LB2_G64 = 2 } hb_wfmt;
typedef struct hb_qmat {
  int fmt;            /* hb_wfmt */
  int N, K;           /* out × in */
  const uint8_t* w;   /* NVFP4: e2m1 [N,K/2].  LB2: codes [N,K/4] (4 per byte, low bits first).
                         LB3: low-two-bit plane [N,K/4] followed by the high-bit plane [N,K/8] (8 per byte, low bit first). */
  const void* s;      /* NVFP4: e4m3 [N,K/16].  LB*: fp16 [N,K/64] */
  const void* zp;     /* LB*: fp16 zero-points [N,K/64]; value = (q - zp) * s.  NVFP4: NULL */
  float g;            /* NVFP4 per-tensor scale (multiplies); LB*: ignored */
} hb_qmat;

/* ---- context (house style of the reference's C ABIs: engine/include/hive/qtts/qtts_capi.h:4-35) ---- */
HB_API int hb_create(const hb_config* cfg, hb_ctx** out);
HB_API void hb_destroy(hb_ctx* ctx);
HB_API const char* hb_last_error(const hb_ctx* ctx);
HB_API const char* hb_status_string(int status);
HB_API int hb_sm_count(const hb_ctx* ctx);
/* Reads (and clears) the device error word the kernels set when a bounded wait runs out.  Synchronises `stream`. */
HB_API int hb_check_device(hb_ctx* ctx, void* stream);
/* Number of kernels this library has launched on ctx since creation (the benchmark's launch count). */
HB_API uint64_t hb_launch_count(const hb_ctx* ctx);
/* Per-kernel device timing — the counterpart of the reference's HIVE_PROFILE event marks (engine/include/hive/glm/glm_experts.h:148-157).
 * While enabled, every kernel launch is bracketed by a CUDA event pair (and programmatic dependent launch is off, so a pair times
 * its kernel alone); hb_profile_read synchronises the device, sums the pairs by kernel name and clears the log (at most 8192
 * launches are kept between reads).  Enabling it the first time creates the events; do not enable it during stream capture. */
typedef struct hb_kernel_stat {
  char name[40];
  uint32_t launches;
  float total_ms;
} hb_kernel_stat;
HB_API int hb_profile_enable(hb_ctx* ctx, int on);
HB_API int hb_profile_read(hb_ctx* ctx, hb_kernel_stat* out, int max_out, int* n_out);

/* ---- formats ---- */
/* hive::glm::ExpertRecLayout::make — engine/include/hive/glm/glm_moe.h:15-21 */
HB_API int hb_rec_layout_make(int H, int I, hb_rec_layout* out);
/* hive::glm::nvfp4_dequant — engine/include/hive/glm/nvfp4.h:23, engine/src/glm/nvfp4.cu:65-74: out[n,k] = bf16(E2M1·(e4m3·g)) */
HB_API int hb_nvfp4_dequant(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, void* out_bf16, void* stream);
/* hive::glm::nvfp4_gemv / hive::q27::k::gemv — engine/include/hive/glm/nvfp4.h:21, engine/src/glm/nvfp4.cu:17-86:
 * y[m,n] = g·Σ_k x[m,k]·W[n,k], x bf16 [M,K] (row stride ldx), y fp32 [M,N] (row stride ldy), 1 ≤ M ≤ 16, K % 32 == 0. */
HB_API int hb_nvfp4_gemv(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, const void* x_bf16, int ldx, int M,
                         float* y, int ldy, void* stream);
/* hive::q27::k::requant_nvfp4's quantisation rule — engine/src/q27/q27_kernels.cu:2492-2542 — applied to an fp32 matrix:
 * g_mul[0] = amax/(448·6); scale = e4m3(m·gs/6); code = e2m1(v·gs/scale).  amax_scratch: 4 device bytes. */
HB_API int hb_nvfp4_quantize(hb_ctx* ctx, const float* w_f32, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax_scratch,
                             void* stream);
/* hive::q27::k::requant_nvfp4 — engine/include/hive/q27/q27_kernels.h:44-46, engine/src/q27/q27_kernels.cu:2492-2542: the NVFP4 copy of an
 * FP8 row-scaled matrix (w_fp8 e4m3 [N,K], value = fp8 · row_scale[n]): global scale from the largest magnitude, e4m3 scale per 16
 * values, e2m1 codes, round to nearest.  Unlike the reference's host function this one does not synchronise: the global scale is
 * left in g_mul[0] on the device (the reference returns it on the host).  amax_scratch: 4 device bytes. */
HB_API int hb_requant_nvfp4(hb_ctx* ctx, const uint8_t* w_fp8, const float* row_scale, int N, int K, uint8_t* q, uint8_t* s, float* g_mul,
                            float* amax_scratch, void* stream);
/* hive::qwen a4_quant_kernel — engine/src/qwen/fn_moe_pf.cu:456-502: per-row dynamic NVFP4 activation quantisation */
HB_API int hb_a4_quant(hb_ctx* ctx, const void* x_bf16, int ld, int n, int K, uint8_t* q, uint8_t* s, float* g, void* stream);

/* ---- routing ---- */
/* hive::qwen::router_softmax_topk — engine/include/hive/qwen/qwen_kernels.h:51-55, engine/src/qwen/qwen_kernels.cu:159-206.
 * logits fp32 [M,ld] (columns 0..E-1), optionally rounded to bf16 first; ties → smaller id; E ≤ 1024, k ≤ 16. */
HB_API int hb_route_softmax_topk(hb_ctx* ctx, const float* logits, int ld, int M, int E, int k, int renorm, int logits_bf16,
                                 int32_t* ids, float* w, void* stream);
/* hive::glm::router_topk — engine/include/hive/glm/glm_kernels.h:12-17, engine/src/glm/glm_kernels.cu:35-53 */
HB_API int hb_route_sigmoid_topk(hb_ctx* ctx, const float* logits, const float* bias, int M, int E, int k, float scale, int32_t* ids,
                                 float* w, void* stream);
/* hive::qwen::build_moe_pairs — engine/include/hive/qwen/qwen_kernels.h:63-66 */
HB_API int hb_build_moe_pairs(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                              hb_moe_pair* pairs, void* stream);
/* hive::qwen::moe_combine — engine/include/hive/qwen/qwen_kernels.h:58-59 (lg NULL: the GLM form without gate) */
HB_API int hb_moe_combine(hb_ctx* ctx, const float* routed, const void* shared_bf16, const float* lg, int ld, int col, int M, int H,
                          void* out_bf16, void* stream);

/* ---- routed-expert decode (1–16 tokens per expert: streaming split-K GEMV) ---- */
HB_API int hb_moe_decode_supported(int H, int I);
/* hive::glm::moe_decode_ws_bytes / hive::qwen::fn_moe_decode_ws_bytes — glm_moe.h:29, fn_moe.h:21 */
HB_API size_t hb_moe_decode_ws_bytes(int n_pairs, int H, int I);
/* hive::glm::moe_decode / hive::qwen::fn_moe_decode — engine/include/hive/glm/glm_moe.h:27-31, engine/include/hive/qwen/fn_moe.h:22-23:
 * out[row] += Σ_pairs w·expert(x[row]) (fp32, accumulated; per-row sum in pair order).  limit > 0 clamps (GLM), 0 = plain SiLU. */
HB_API int hb_moe_decode(hb_ctx* ctx, const hb_moe_pair* pairs, int n_pairs, const void* x_bf16, int H, int I, float limit,
                         float* out, void* ws, void* stream);
/* hive::qwen::fn_moe_decode_routed — engine/include/hive/qwen/fn_moe.h:25-31 (without the hybrid CPU/PCIe arguments):
 * out[m] = bf16( bf16(Σ_k w[m,k]·expert_ids[m,k](x[m])) + bf16( bf16(sigmoid(bf16(lg[m·ld+col]))) · shared[m] ) ).
 * Records come from rec_tab[li·E + id]; ids outside [0,E) and NULL records contribute nothing.  cmb->lg NULL = no gate. */
HB_API int hb_moe_decode_routed(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                                const void* x_bf16, int H, int I, float limit, const hb_pf_combine* cmb, void* ws, void* stream);
/* (No counterpart in the reference.)  hb_moe_decode_routed for callers that cannot allocate device memory when they call —
 * an engine that spends its whole memory budget at start-up and forbids cudaMalloc afterwards, a decode loop that must not
 * synchronise the device, a plugin host that keeps the allocator to itself.  Same arguments and result as
 * hb_moe_decode_routed without `ws`: the scratch is a fixed 4 MiB array built into the library (each GPU that loads the
 * library holds it until the process exits).  Limits and rules:
 *   - a call whose scratch would exceed the array fails with HB_ERR_UNSUPPORTED and a message naming the limit;
 *     hb_moe_decode_static_max_pairs(H, I) gives the largest M·K accepted at a shape (813 pairs at H 2048, I 512; 371 at H 4096, I 1536);
 *   - the first call on a device looks up the array's device address (with that device current); make that first call before
 *     any stream capture (two host threads that make that first call at the same time both look it up and store the same
 *     value: harmless).  No call allocates or frees memory;
 *   - every call on a device uses the same array and finds the previous call's contents in it (what must start at zero is
 *     cleared by the kernels themselves); calls that overlap on the GPU race on it — keep them on one stream;
 *   - it always runs the streaming kernels (its result is bit-identical to hb_moe_decode_routed on a context pinned with
 *     HB_FLAG_DECODE_MMA_SYNC, and within the common tolerance of what an unpinned context computes). */
HB_API int hb_moe_decode_static_max_pairs(int H, int I);
HB_API int hb_moe_decode_routed_static(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                                       const void* x_bf16, int H, int I, float limit, const hb_pf_combine* cmb, void* stream);
/* The routed sum alone, fp32, overwritten: out[m] = Σ_k w[m,k]·expert_ids[m,k](x[m]) in k order — the output contract of
 * hive::qwen::fn_moe_prefill without its combine (engine/include/hive/qwen/fn_moe.h:46-61) on the decode kernels.  Used by the
 * expert-parallel layer, where rec_tab holds NULL for experts that live on other GPUs (those pairs contribute nothing). */
HB_API int hb_moe_decode_routed_f32(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int li, int E,
                                    const void* x_bf16, int H, int I, float limit, float* out, void* ws, void* stream);
/* (No counterpart in the reference, which is single-GPU.)  One rank's share of an expert-parallel decode layer, in one pass:
 * routed_out[m] = Σ_k w[m,k]·expert_ids[m,k](x[m]) over the experts whose records this rank holds (NULL table entries = experts
 * held elsewhere, skipped), fp32 [M,H] overwritten — to be summed over ranks — and, when shared_rec is given, the always-on
 * shared expert on rows [sh_row0, sh_row0 + sh_rows) (this rank's own rows) → shared_out bf16 [sh_rows, H].  ids / w / x may be
 * strided views into a gathered exchange buffer: row m of ids / w starts at element m·ld_ids, row m of x at element m·ldx
 * (ldx a multiple of 8, x 16-byte aligned).  ws ≥ hb_moe_decode_ws_bytes(M·(K+1), H, I). */
HB_API int hb_moe_decode_ep_local(hb_ctx* ctx, const int32_t* ids, const float* w, int ld_ids, int M, int K, const uint8_t* const* rec_tab, int li,
                                  int E, const void* x_bf16, int ldx, int H, int I, float limit, const uint8_t* shared_rec, int sh_row0, int sh_rows,
                                  float* routed_out, void* shared_out_bf16, void* ws, void* stream);
/* (No counterpart in the reference.)  The two exchanges of an expert-parallel decode layer done by this library's own kernels over
 * NVLink peer memory instead of a collective library: rows are pushed into every rank's gather buffer, partial sums into the
 * owning rank's partial buffer, each followed by a step-number flag the receiver polls (bounded; a wait that gives up sets the
 * context's error word — hb_check_device reports it — and later waits return at once).
 *   hb_ep_rec_bytes(H, K)            bytes of one exchanged row record [bf16 row | int32 ids | fp32 weights], padded to 16
 *   hb_ep_export / import / close    share a device buffer between the ranks' processes (CUDA IPC): export gives a 64-byte handle and
 *                                    the buffer's offset inside its allocation; import (with the context's device current) maps it for
 *                                    this device's kernels and returns the buffer's address plus the base to close later
 *   hb_ep_create(...)                recv[p], ag_flag[p], rs[p], rs_flag[p] for p < world: addresses, valid on THIS device, of rank p's
 *                                    gather buffer [world·B·rec_bytes], gather flags [world] u32, partial buffer [world·B·H] f32
 *                                    and partial flags [world] u32 (the caller allocates its own, zero-filled, and maps its
 *                                    peers' through CUDA IPC or any other way); entry `rank` is the caller's own
 *   hb_ep_push_rows                  pack this rank's B rows and push them to every rank
 *   hb_ep_wait_rows                  returns (on the stream) when every rank's rows of this step are in the own gather buffer; then
 *                                    hb_moe_decode_ep_local reads them in place
 *   hb_ep_push_partials              part fp32 [world·B, H] (hb_moe_decode_ep_local's routed_out): rows of rank p → rank p
 *   hb_ep_combine                    waits for every rank's partials of the own rows, adds them in rank order, applies the
 *                                    shared-expert combine (hb_moe_combine's arithmetic) → out bf16 [B,H]; ends the step
 *   hb_ep_route_push                 softmax router (hb_route_softmax_topk's arithmetic; ids / w also returned) + hb_ep_push_rows in one launch
 *   hb_ep_layer_local                hb_ep_wait_rows + hb_moe_decode_ep_local on the gathered rows + hb_ep_push_partials as ONE chain of four
 *                                    kernels: the grouping kernel does the wait, the reduce kernel stores straight into the owners' buffers
 * A layer is then three calls: hb_ep_route_push, hb_ep_layer_local, hb_ep_combine.
 * All ranks must issue the same sequence of steps.  Calls of one hb_ep must not overlap. */
typedef struct hb_ep hb_ep;
HB_API size_t hb_ep_rec_bytes(int H, int K);
HB_API int hb_ep_export(hb_ctx* ctx, const void* ptr, void* handle64, size_t* offset);
HB_API int hb_ep_import(hb_ctx* ctx, const void* handle64, size_t offset, void** ptr, void** base);
HB_API int hb_ep_close(hb_ctx* ctx, void* base);
HB_API int hb_ep_create(hb_ctx* ctx, int rank, int world, int B, int H, int K, void* const* recv, void* const* ag_flag, void* const* rs,
                        void* const* rs_flag, hb_ep** out);
HB_API void hb_ep_destroy(hb_ep* ep);
HB_API int hb_ep_push_rows(hb_ep* ep, const void* x_bf16, int ldx, const int32_t* ids, const float* w, void* stream);
HB_API int hb_ep_route_push(hb_ep* ep, const float* logits, int ld, int E, int renorm, int logits_bf16, const void* x_bf16, int ldx,
                            int32_t* ids_out, float* w_out, void* stream);
HB_API int hb_ep_layer_local(hb_ep* ep, const uint8_t* const* rec_tab, int li, int E, int I, float limit, const uint8_t* shared_rec,
                             void* shared_out_bf16, void* ws, void* stream);
HB_API int hb_ep_wait_rows(hb_ep* ep, void* stream);
HB_API int hb_ep_push_partials(hb_ep* ep, const float* part, void* stream);
HB_API int hb_ep_combine(hb_ep* ep, const void* shared_bf16, const float* lg, int ld, int col, void* out_bf16, void* stream);
/* A whole decode MoE layer in one call: router (softmax when bias == NULL and sigmoid_scale == 0, else sigmoid+bias) → routed
 * experts → the always-on shared expert given as one more NVFP4 record (weight 1, every row; NULL = none) → combine.
 * Composition of the operators above in the order of engine/src/qwen/qwen_engine.cpp:818-878; ids_out / w_out [M,K] receive
 * the routing.  gate_col < 0: no shared-expert gate.  ws ≥ hb_moe_decode_ws_bytes(M·(K+1), H, I). */
HB_API int hb_moe_layer_decode(hb_ctx* ctx, const float* logits, int ld, int M, int E, int K, int renorm, int logits_bf16,
                               const float* bias, float sigmoid_scale, const uint8_t* const* rec_tab, int li,
                               const uint8_t* shared_rec, int gate_col, const void* x_bf16, int H, int I, float limit,
                               int32_t* ids_out, float* w_out, void* out_bf16, void* ws, void* stream);

/* ---- dense decode GEMV of the 27B-style MLP: NVFP4 and the 3-/2-bit group-64 formats (hb_qmat) ---- */
HB_API size_t hb_dense_gemv_ws_bytes(int fmt, int N, int K, int n_mats /* 1 = gemv, 2 = gemv_gu */);
/* hive::q27::k::gemv — engine/include/hive/q27/q27_kernels.h:48-50, engine/src/q27/q27_kernels.cu:2423-2449:
 * y[m,n] = Σ_k x[m,k]·W[n,k], fp32 accumulation, written as bf16 (yb) or fp32 (yf): exactly one non-NULL.  x bf16 [M,K] (row
 * stride ldx), M ≤ 16 (the reference takes ≤ 8; rows are processed 8 at a time with batch-independent arithmetic), K % 256 == 0. */
HB_API int hb_dense_gemv(hb_ctx* ctx, const hb_qmat* W, const void* x_bf16, int ldx, int M, void* yb_bf16, float* yf, int ldy, void* ws,
                         void* stream);
/* hive::q27::k::gemv_gu — engine/include/hive/q27/q27_kernels.h:62-64, engine/src/q27/q27_kernels.cu:258-289:
 * act[m,n] = bf16( bf16(silu(bf16 g)) · bf16 u ), g / u = rows n of the gate / up matrices (same K and format). */
HB_API int hb_dense_gemv_gu(hb_ctx* ctx, const hb_qmat* gate, const hb_qmat* up, const void* x_bf16, int ldx, int M, void* act_bf16, int lda,
                            void* ws, void* stream);
/* Dequantise a 3-/2-bit group-64 matrix to bf16 [N,K]: out = bf16((q − zp)·s) — the format's definition (no reference counterpart:
 * the reference ships no low-bit layout, only an error probe, tools/lowbit_probe.py:18-38). */
HB_API int hb_lb_dequant(hb_ctx* ctx, const hb_qmat* W, void* out_bf16, void* stream);

/* ---- routed-expert prefill: grouped W4A4 GEMM on the tcgen05 tensor cores ---- */
/* hive::qwen::fn_moe_prefill_supported — engine/include/hive/qwen/fn_moe.h:48.  Here: H and I multiples of 256. */
HB_API int hb_moe_prefill_supported(int H, int I);
/* hive::qwen::fn_moe_prefill_ws_bytes — engine/include/hive/qwen/fn_moe.h:56: scratch for sub-chunks of S rows. */
HB_API size_t hb_moe_prefill_ws_bytes(int S, int K, int E, int H, int I);
/* hive::qwen::fn_moe_prefill with NVFP4 activations (engine/include/hive/qwen/fn_moe.h:46-61, engine/src/qwen/fn_moe_pf.cu:439-446,
 * :858-941): for every row m, out[m] = Σ_k bf16(expert_{ids[m,k]}(x[m]))·w[m,k] (fp32, k order, overwritten), or with cmb the
 * fused combine → bf16 cmb->out and `out` may be NULL.  Inside an expert: x and y = bf16(silu(g)·u) are quantised per row to NVFP4
 * (hb_a4_quant's rule), both GEMMs run as block-scaled FP4 MMAs with fp32 accumulation, g, u, y and the down result are
 * rounded to bf16 where the decode kernels round them.  Records come from rec_tab[li·E + id]; ids outside [0,E) and NULL
 * records contribute nothing.  Rows are processed in sub-chunks of S; ws ≥ hb_moe_prefill_ws_bytes(S, K, E, H, I).  E ≤ 1024.
 * Block scales are read as unsigned e4m3 (the sign bit of a scale byte must be clear, as every NVFP4 writer leaves it).
 * With HB_FLAG_PREFILL_A16 in the context's flags the activations stay bf16 (W4A16: the decode operators' arithmetic and rounding
 * points).  Calls of more than 64 rows run the kind::f16 grouped GEMM (exact products, fp32 sums in the tensor core's order: the
 * decode operators' results up to summation order); calls of up to 64 rows, and every call with HB_FLAG_PREFILL_A16_ROWS, run the
 * decode kernels and are bit-identical to hb_moe_decode_routed(_f32) on the same rows. */
HB_API int hb_moe_prefill(hb_ctx* ctx, const uint8_t* const* rec_tab, int li, int E, const int32_t* ids, const float* w, int M, int K,
                          const void* x_bf16, int H, int I, float limit, float* out, void* ws, int S, void* stream, const hb_pf_combine* cmb);
/* The same GEMM on one dense NVFP4 matrix: y[m,n] = xg[m]·W.g·Σ_k xq[m,k]·xs[m,k/16]·W[n,k], fp32 [M, ldy].  xq / xs / xg as written by
 * hb_a4_quant.  N and K multiples of 256.  (No single counterpart in the reference; it is the building block hb_moe_prefill is
 * tested through.) */
HB_API int hb_nvfp4_gemm_a4(hb_ctx* ctx, const hb_qmat* W, const uint8_t* xq, const uint8_t* xs, const float* xg, int M, float* y, int ldy,
                            void* stream);
/* Measures the FP4 tensor-pipe ceiling of the device: every SM issues `rounds`×4 block-scaled 128×256×64 MMAs on operands held in
 * shared memory (no loads, no epilogue); *tflops = dense FP4 TFLOP/s.  Synchronises the device.  (No reference counterpart.) */
HB_API int hb_fp4_peak_probe(hb_ctx* ctx, int rounds, float* tflops);

/* ---- a whole MoE layer for any number of rows (the expert-dispatch scheduler) ---- */
/* router → routed experts → always-on shared expert (one more NVFP4 record, NULL = none) → combine, like hb_moe_layer_decode, for
 * any M.  By default every row count runs on the decode operators (bf16 activations, W4A16 — the reference's default arithmetic,
 * engine/include/hive/qwen/fn_moe.h:50-52), 64 rows at a time above 64 rows, so a row's result never depends on how many rows
 * the call has.  A context created with HB_FLAG_LAYER_A4 sends calls of more than 64 rows to the grouped tensor-core GEMM
 * (hb_moe_prefill with NVFP4 activations, W4A4) when the shape allows it (H, I multiples of 256) — the reference engine's own
 * switch (engine/src/qwen/qwen_engine.cpp:825, :873) with its opt-in arithmetic.
 * ws ≥ hb_moe_layer_ws_bytes(M, K, E, H, I). */
HB_API size_t hb_moe_layer_ws_bytes(int M, int K, int E, int H, int I);
HB_API int hb_moe_layer(hb_ctx* ctx, const float* logits, int ld, int M, int E, int K, int renorm, int logits_bf16, const float* bias,
                        float sigmoid_scale, const uint8_t* const* rec_tab, int li, const uint8_t* shared_rec, int gate_col,
                        const void* x_bf16, int H, int I, float limit, int32_t* ids_out, float* w_out, void* out_bf16, void* ws, void* stream);

/* ---- regime choice ---- */
/* What a caller needs to know before it runs a layer on M rows: how the (row, k) pairs fall on the experts and which operator
 * family takes them.  Host-side restatement of the classification the reference spreads over GlmExperts::decode_layer
 * (engine/src/glm/glm_experts.cpp:565-653: pairs grouped per expert, at most 8 rows per GEMV group as in
 * engine/include/hive/decode_handshake.h:26) and fn_moe_prefill's count / scan / tile rule (engine/src/qwen/fn_moe_pf.cu:39-75, :898).
 * ids: HOST int32 [M,K]; ids outside [0,E) are skipped.  counts (optional, [E]) receives the pairs per expert. */
typedef struct hb_plan {
  int regime;            /* 0 = decode operators (weight-streaming GEMV groups), 1 = prefill operator (grouped tensor-core GEMM) */
  int pairs;             /* valid (row, k) pairs */
  int distinct_experts;  /* experts with at least one pair: the records a decode call streams */
  int max_rows;          /* most pairs on one expert */
  int decode_groups;     /* Σ ceil(count / 8): work groups of the decode kernels */
  int prefill_tiles;     /* Σ ceil(count / 128): tiles of the grouped GEMM */
  double tile_fill;      /* pairs / (128 · prefill_tiles): how full the GEMM tiles would be */
  size_t ws_bytes;       /* workspace the chosen operator needs (0 when the shape is unsupported by it) */
} hb_plan;
HB_API int hb_dispatch_plan(const int32_t* ids_host, int M, int K, int E, int H, int I, int* counts, hb_plan* plan);

/* ---- record assembly: the step in front of the path (engine/src/glm/glm_experts.cpp:216-287, engine/include/hive/ckpt_quant.h:5-37) ----
 * hive::ckq::csf_decode on the device.  The e4m3 block-scale matrix [R, C] (C = K / 16) of a projection, stored compressed as
 * fixed u8 [R / 16, 16 + 8·C] (per 16 rows: 16 base code bytes, then 16·C 4-bit deltas row-major, even position = low nibble;
 * code = base + delta) and exception words u32 [n_exc] (code << 24 | flat index r·C + c; the stored delta there is 0), is expanded
 * into out [R, C].  A shape the format rules out (R % 16, the fixed shape, more than 2^24 scales) is refused on the host with
 * HB_ERR_INVALID, like the reference's `false`.  The data-dependent invariants are checked on the device; status (device int32[2])
 * receives {HB_CSF_* code, position} of the violation the reference's sequential decoder meets first (position = exception
 * ordinal for the exception checks, flat scale index for HB_CSF_CODE), {0, 0} when the tensor is sound.  out is unspecified
 * unless status[0] == 0.  All pointers are device-accessible (fixed 8-byte, exc 4-byte, out 16-byte aligned); the call enqueues on
 * `stream` and does not synchronise. */
enum { HB_CSF_OK = 0, HB_CSF_SHAPE = 2 /* record assembly only: the fixed tensor's shape does not fit the projection */, HB_CSF_EXC_INDEX = 4,
       HB_CSF_EXC_DELTA = 5, HB_CSF_EXC_VALUE = 6, HB_CSF_CODE = 7, HB_CSF_MISSING = 8 /* record assembly only: a NULL or misaligned tensor */ };
HB_API size_t hb_csf_ws_bytes(int R, int C);
HB_API int hb_csf_decode(hb_ctx* ctx, const uint8_t* fixed, int64_t fixed_rows, int64_t fixed_cols, const uint32_t* exc, uint64_t n_exc, int R, int C,
                         uint8_t* out, int32_t* status, void* ws, size_t ws_bytes, void* stream);
/* One projection of an expert as the checkpoint holds it: packed e2m1 bytes [rows, K/2], the fp32 global (`weight_scale_2`), and
 * either plain e4m3 scales [rows, K/16] or, with scale == NULL, the compressed pair. */
typedef struct hb_proj_src {
  const uint8_t* weight;
  const uint8_t* scale;
  const uint8_t* csf_fixed;
  const uint32_t* csf_exc;
  int64_t csf_fixed_rows, csf_fixed_cols;
  uint64_t n_exc;
  float global;
} hb_proj_src;
/* One expert: its three projections (gate, up, down) and where its record goes (16-byte aligned, hb_rec_layout(H, I).total bytes). */
typedef struct hb_record_job {
  hb_proj_src src[3];
  uint8_t* rec;
} hb_record_job;
/* GlmExperts::load_all on the device, for a batch of n experts in one go: jobs = DEVICE-accessible array [n]; every kernel of the
 * call runs once for the whole batch (job index in the grid), so a batch costs three launches however many records it holds (six when it has fewer tensors than the device has SMs; the
 * workspace is a few hundred bytes per record).
 * Weights are copied, scales copied or CSF-decoded straight into each record, the three globals written as g1 g3 g2; the bytes
 * after the globals up to `total` are left as they are.  status = device int32 [n][3][2]: one {HB_CSF_* code, position} per
 * projection ({0, 0} = sound; HB_CSF_SHAPE / HB_CSF_MISSING for what the reference's loader refuses by shape or dtype; the scales
 * of a projection whose status is not 0 are unspecified).  The reference aborts the load on the first violation; here the caller reads status
 * once per batch and decides.  Sources 16-byte aligned copy with 16-byte accesses, others byte by byte.
 * hb_record_pack is the same for one expert with the descriptor in host memory. */
HB_API size_t hb_record_pack_ws_bytes(int H, int I, int n);
HB_API int hb_record_pack_batch(hb_ctx* ctx, const hb_record_job* jobs, int n, int H, int I, int32_t* status, void* ws, size_t ws_bytes, void* stream);
HB_API int hb_record_pack(hb_ctx* ctx, const hb_proj_src* src, int H, int I, uint8_t* rec, int32_t* status, void* ws, size_t ws_bytes, void* stream);

/* ---- prefill helpers kept for callers that compose (engine/include/hive/glm/glm_moe.h:33-41) ---- */
/* hive::glm::expert_dequant — engine/include/hive/glm/glm_moe.h:32-33: one expert record → bf16 gu [2I, H] (gate rows then up rows) and
 * d [H, I].  The record's globals are read on the device: unlike the reference (engine/src/glm/glm_moe.cu:608-616) the call does not
 * synchronise the stream. */
HB_API int hb_expert_dequant(hb_ctx* ctx, const uint8_t* rec, int H, int I, void* gu_bf16, void* d_bf16, void* stream);
HB_API int hb_gather_rows(hb_ctx* ctx, const void* x_bf16, const int32_t* rows, int R, int H, void* out_bf16, void* stream);
HB_API int hb_swiglu_rows(hb_ctx* ctx, const void* gu_bf16, int R, int I, float limit, void* y_bf16, void* stream);
HB_API int hb_scatter_add_rows(hb_ctx* ctx, const void* e_bf16, const int32_t* rows, const float* w, int R, int H, float* out, void* stream);
HB_API int hb_add_f32(hb_ctx* ctx, float* a, const float* b, size_t n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HIVE_B200_H */
