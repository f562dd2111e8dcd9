/* TEST INFRASTRUCTURE — the CPU oracle of the quantized routed-expert path.
 *
 * A plain-C restatement of the reference engine's arithmetic for this path.  It is the checker used by tests/, by
 * __graft_entry__.smoke() and by bench.py's cpu_baseline leg; nothing in the shipped library links, imports or
 * calls it.  Each function names the reference file:line (paths inside the reference project) whose behaviour it
 * restates.  Parity status: pinned — tests/test_oracle_pins.py checks every function below against the reference's
 * own compiled CPU code (oracle/_ref/libhive_ref.so) and against the golden vectors in tests/golden/ generated from
 * it; the 3-/2-bit group-64 functions (ho_lb_*) have no reference counterpart: "parity unpinned" for those.
 */
#ifndef HIVE_ORACLE_H
#define HIVE_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- number formats: engine/include/hive/common.h:69-140, engine/cpu_shim/cuda_bf16.h:8-14 ---- */
float    ho_e2m1_to_f32(uint8_t nib);
float    ho_e4m3_to_f32(uint8_t v);
uint8_t  ho_f32_to_e4m3(float x);          /* RNE, saturating at ±448, NaN → 0x7F */
uint8_t  ho_f32_to_e2m1(float x);          /* RNE, ties to the even code */
uint16_t ho_f32_to_bf16(float x);          /* RNE */
float    ho_bf16_to_f32(uint16_t b);
float    ho_bf16r(float x);
/* engine/src/qwen/cpu/qwen_cpu_simd.h:23-41: Cody–Waite + degree-5 polynomial exp with explicit fma */
float    ho_exp_portable(float x);
float    ho_fp16_to_f32(uint16_t h);
uint16_t ho_f32_to_fp16(float x);          /* RNE */

/* ---- expert record: engine/include/hive/glm/glm_moe.h:13-22 — off = {w1,s1,w3,s3,w2,s2,g,total} ---- */
void ho_rec_layout(int H, int I, uint64_t off[8]);

/* ---- NVFP4 matrix ops ---- */
/* engine/src/glm/nvfp4.cu:65-74: out[n,k] = bf16( E2M1[nib] * (e4m3(s) * g) ) */
void ho_nvfp4_dequant_bf16(const uint8_t* w, const uint8_t* s, float g, int N, int K, uint16_t* out);
/* engine/src/cpu/expert_cpu_nvfp4.cpp:51-68: y[n] = g * Σ_b16 ( Σ_i a[k]·E2M1 ) · e4m3(s[n,b]) , fp32, k ascending */
void ho_gemv_nvfp4(const uint8_t* w, const uint8_t* s, float g, int N, int K, const float* a, int n0, int n1, float* y);
/* engine/src/cpu/expert_cpu_nvfp4.cpp:296-308.  silu_mode 0: x/(1+expf(-x)) (libm, the CPU expert kernel);
 * 1: the portable exp (the CPU-only daemon's silu_mul, qwen_cpu_simd.h:153-165).  tmp ≥ 3·I floats. */
void ho_expert_forward_nvfp4(const uint8_t* rec, const uint64_t* off, int H, int I, const float* a, float route_w, float limit,
                             int silu_mode, float* out, float* tmp);

/* ---- routers ---- */
/* Softmax top-k.  form 0 = the GPU operator (engine/src/qwen/qwen_kernels.cu:159-206): p = exp(l-max), weights
 * p·(1/Σp), optional ·(1/Σ_topk) in pick order; exp is the portable one so CPU and GPU agree to the bit.
 * form 1 = the CPU-only daemon (engine/src/qwen/cpu/qwen_cpu_engine.cpp:662-684): libm exp, p/Σp, p/Σ_topk.
 * Both: logits optionally rounded to bf16 first; k picks by (p desc, id asc).  E ≤ 1024, k ≤ 16. */
void ho_router_softmax_topk(const float* logits, int ld, int M, int E, int k, int renorm, int logits_bf16, int form,
                            int32_t* ids, float* w);
/* engine/src/glm/glm_kernels.cu:35-53 (GPU) and engine/src/glm/cpu/glm_cpu_engine.cpp:847-859 (CPU): s = 1/(1+exp(-l)),
 * pick k maxima of s+bias by a strict > scan, w = s/(Σs+1e-20)·scale, Σ in pick order.  form 0: portable exp, 1: libm exp. */
void ho_router_sigmoid_topk(const float* logits, const float* bias, int M, int E, int k, float scale, int form, int32_t* ids, float* w);

/* ---- MoE operators ---- */
/* engine/include/hive/glm/glm_moe.h:27-31 (moe_decode): out[row] += Σ_pairs w·expert(x[row]), pairs in the order given.
 * x holds bf16 values as fp32 [M,H]; recs[i] is pair i's record (NULL = skipped). */
void ho_moe_decode(const uint64_t* off, const int32_t* rows, const uint8_t* const* recs, const float* pw, int n_pairs,
                   const float* x, int H, int I, float limit, int silu_mode, float* out);
/* routed sum of a layer from ids/w: acc[m] = Σ_k w[m,k]·expert_{ids[m,k]}(x[m]) in k order (fp32, not rounded);
 * ids outside [0,E) or NULL records contribute nothing (engine/src/qwen/fn_moe.cu:298-305). */
void ho_moe_routed(const uint64_t* off, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int E,
                   const float* x, int H, int I, float limit, int silu_mode, float* acc);
/* engine/src/qwen/qwen_kernels.cu:208-216 (moe_combine):
 *   gate_logits != NULL: out = bf16( bf16(routed) + bf16( G · shared ) ), G = bf16(sigmoid(bf16(lg[m·ld+col]))) when round_gate
 *                        (the GPU operator) or sigmoid(lg) unrounded (the CPU daemon, qwen_cpu_engine.cpp:764-782);
 *   gate_logits == NULL: out = bf16( bf16(routed) + bf16(shared) )   (engine/src/glm/cpu/glm_cpu_engine.cpp:949).
 * shared holds bf16 values as fp32; out is written as bf16 bits. */
void ho_moe_combine(const float* routed, const float* shared, const float* gate_logits, int ld, int col, int round_gate, int M, int H,
                    uint16_t* out);

/* ---- quantizers ---- */
/* tools/q27_reencode.py:87-110 with search != 0 (five-factor per-block MSE search), or the device rule of
 * engine/src/q27/q27_kernels.cu:2506-2529 with search == 0.  g_mul = amax/(448·6) (the record's multiply convention). */
void ho_nvfp4_quantize(const float* w, int N, int K, int search, uint8_t* q, uint8_t* s, float* g_mul);
/* engine/src/qwen/fn_moe_pf.cu:456-502 (a4_quant_kernel): per-row dynamic NVFP4 activation quantization. x = bf16 values as fp32. */
void ho_a4_quant(const float* x, int ld, int n, int K, uint8_t* q, uint8_t* s, float* g);
/* one expert on one row with NVFP4 activations (the prefill path's W4A4 rounding points); out [H] = bf16 values, unweighted */
void ho_expert_forward_a4(const uint8_t* rec, const uint64_t* off, int H, int I, const float* x, float limit, float* out);

/* ---- 3-/2-bit group-64 dense matrices (layout defined by this project; no reference counterpart: parity unpinned) ----
 * bits = 2: w = [N, K/4] bytes, byte j of a row holds codes of columns 4j..4j+3, low bits first.
 * bits = 3: w = low plane [N, K/4] as above (low two bits) followed by high plane [N, K/8], byte j = bit 2 of columns 8j..8j+7.
 * s, zp: fp16 [N, K/64].  value = (q - zp) * s, the subtraction exact in fp32, one rounding in the product. */
size_t ho_lb_weight_bytes(int bits, int N, int K);
void ho_lb_quantize(const float* w, int N, int K, int bits, uint8_t* q, uint16_t* s, uint16_t* zp);
void ho_lb_dequant_bf16(const uint8_t* q, const uint16_t* s, const uint16_t* zp, int bits, int N, int K, uint16_t* out);
/* y[n] = Σ_groups s · ( Σ_k a[k]·q[k] − zp · Σ_k a[k] ), fp32, groups ascending */
void ho_lb_gemv(const uint8_t* q, const uint16_t* s, const uint16_t* zp, int bits, int N, int K, const float* a, int n0, int n1, float* y);
/* engine/src/q27/q27_kernels.cu:258-289 (gemv_gu): act[i] = bf16( bf16(silu(bf16 g)) · bf16 u ), silu through libm expf */
void ho_dense_act(const float* g, const float* u, int n, float* act);

/* ---- record assembly: compressed NVFP4 block scales ("CSF") ----
 * engine/include/hive/ckpt_quant.h:5-17 (format), engine/src/ckpt_quant.cpp:34-73 (csf_decode).  The e4m3 scale matrix [R, C] is
 * stored per group of 16 rows as 16 base code bytes + 16*C 4-bit deltas (row-major inside the group, even position = low nibble),
 * code = base + delta; each exception word (code << 24 | flat index) replaces one entry whose stored delta must be 0.
 * Returns 0 and fills out [R, C], or the number of the first violated invariant in the reference's order of checks
 * (HO_CSF_*; *where = exception ordinal for the exception checks, flat scale index for HO_CSF_CODE). */
enum { HO_CSF_OK = 0, HO_CSF_ROWS = 1, HO_CSF_SHAPE = 2, HO_CSF_TOO_MANY = 3, HO_CSF_EXC_INDEX = 4, HO_CSF_EXC_DELTA = 5, HO_CSF_EXC_VALUE = 6,
       HO_CSF_CODE = 7 };
int ho_csf_decode(const uint8_t* fixed, int64_t fixed_rows, int64_t fixed_cols, const uint32_t* exc, size_t n_exc, int R, int C, uint8_t* out,
                  int64_t* where);
/* engine/src/glm/glm_experts.cpp:216-287 (GlmExperts::load_all, one record): weights copied, scales copied or CSF-decoded straight
 * into the record, the three globals written as g1 g3 g2.  proj order: gate, up, down.  scale[j] == NULL selects the CSF pair.
 * Returns 0 or 10*(j+1) + HO_CSF_* of the first failing projection. */
int ho_record_pack(const uint64_t* off, int H, int I, const uint8_t* const weight[3], const uint8_t* const scale[3],
                   const uint8_t* const csf_fixed[3], const uint32_t* const csf_exc[3], const size_t n_exc[3], const float global[3],
                   uint8_t* rec);

#ifdef __cplusplus
}
#endif
#endif
