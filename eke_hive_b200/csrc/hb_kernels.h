// Internal launcher interface between the C-ABI translation unit (argument checks) and the kernel translation units.
// Every function enqueues on `st` and returns HB_OK or a negative hb_status with the context's message set.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/hive_b200.h"

int hbk_nvfp4_dequant(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, void* out, cudaStream_t st, const float* g_dev = nullptr);
int hbk_nvfp4_gemv(hb_ctx* ctx, const uint8_t* w, const uint8_t* s, float g, int N, int K, const void* x, int ldx, int M, float* y, int ldy,
                   cudaStream_t st);
int hbk_nvfp4_quantize(hb_ctx* ctx, const float* w, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax, cudaStream_t st);
int hbk_requant_nvfp4(hb_ctx* ctx, const uint8_t* w_fp8, const float* row_scale, int N, int K, uint8_t* q, uint8_t* s, float* g_mul, float* amax, cudaStream_t st);
int hbk_a4_quant(hb_ctx* ctx, const void* x, int ld, int n, int K, uint8_t* q, uint8_t* s, float* g, cudaStream_t st);
// the same quantisation with each row written to nd slots (dest[row·nd + j], negative = none) instead of its own; n_dev (optional):
// device word holding the number of rows to do when that is smaller than n
int hbk_quant_rows_scatter(hb_ctx* ctx, const void* x, int ld, int n, int K, const int* dest, int nd, uint8_t* q, uint8_t* s, float* g, cudaStream_t st,
                           const int* n_dev = nullptr);
int hbk_nvfp4_setup(hb_ctx* ctx);

int hbk_route_softmax_topk(hb_ctx* ctx, const float* logits, int ld, int M, int E, int k, int renorm, int logits_bf16, int32_t* ids, float* w,
                           cudaStream_t st, bool pdl);
int hbk_route_sigmoid_topk(hb_ctx* ctx, const float* logits, const float* bias, int M, int E, int k, float scale, int32_t* ids, float* w,
                           cudaStream_t st, bool pdl);
int hbk_build_pairs(hb_ctx* ctx, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* tab, int li, int E, hb_moe_pair* pairs,
                    cudaStream_t st, bool pdl);
int hbk_moe_combine(hb_ctx* ctx, const float* routed, const void* shared, const float* lg, int ld, int col, int M, int H, void* out, cudaStream_t st,
                    bool pdl);
int hbk_layer_prep(hb_ctx* ctx, const uint8_t** tab1, int32_t* ids1, float* w1, int M, const uint8_t* shared_rec, cudaStream_t st);
int hbk_f32_to_bf16(hb_ctx* ctx, const float* in, void* out, size_t n, cudaStream_t st);
int hbk_gather_rows(hb_ctx* ctx, const void* x, const int32_t* rows, int R, int H, void* out, cudaStream_t st);
int hbk_swiglu_rows(hb_ctx* ctx, const void* gu, int R, int I, float limit, void* y, cudaStream_t st);
int hbk_scatter_add_rows(hb_ctx* ctx, const void* e, const int32_t* rows, const float* w, int R, int H, float* out, cudaStream_t st);
int hbk_add_f32(hb_ctx* ctx, float* a, const float* b, size_t n, cudaStream_t st);

// ---- routed-expert decode ----
constexpr int HB_MAX_PAIRS = 4096;     // pairs per call (M·K plus the shared expert's M)
constexpr int HB_MAX_EXPERTS = 1024;
bool hbk_moe_decode_fast(int H, int I);                 // shapes the streaming tensor-core path takes
size_t hbk_moe_decode_ws_bytes(int n_pairs, int H, int I);          // what the public *_ws_bytes report: enough for either decode engine
size_t hbk_moe_decode_ws_stream_bytes(int n_pairs, int H, int I);   // the streaming chain alone
int hbk_moe_decode_setup(hb_ctx* ctx);                  // one-time kernel attributes (dynamic shared memory)
// Expert-parallel exchange hooks of a decode pass (k_ep.cu): wait for the gathered rows before grouping, push the routed sums to the
// owning ranks instead of storing them.
struct hbk_ep_push { float* rs[8]; uint32_t* flag[8]; int B, rank, world; const uint32_t* step; unsigned int* done; };
// Source of the pairs: either an explicit list, or router output (+ optionally the shared expert as M extra pairs of weight 1).
struct hbk_pair_src {
  const hb_moe_pair* pairs = nullptr; int n_pairs = 0;                       // list form
  const int32_t* ids = nullptr; const float* w = nullptr; int M = 0, K = 0;  // routed form
  const uint8_t* const* tab = nullptr; int li = 0, E = 0;
  const uint8_t* shared_rec = nullptr;
  int ld_ids = 0;                                                            // row pitch of ids / w in elements (0 = K)
  int x_ld = 0;                                                              // row pitch of x in elements (0 = H; other values: streaming path only)
  int sh_row0 = 0, sh_rows = -1;                                             // rows that get the shared expert's pair (-1 = all M)
  const uint32_t* wait_flags = nullptr; int wait_n = 0; const uint32_t* wait_step = nullptr;   // grouping first waits until wait_flags[0..n) ≥ *wait_step + 1
  // routed form, optional: route inside the grouping kernel (ids / w are then outputs written before they are grouped)
  int route = 0;                                                             // 0 = ids / w given, 1 = softmax, 2 = sigmoid + bias
  const float* logits = nullptr; int ld = 0, renorm = 0, logits_bf16 = 0;
  const float* bias = nullptr; float sig_scale = 1.f;
  int pairs_hint = 0;                                                        // pairs of the enclosing call when this one is a sub-chunk of it: the engine is picked as for the whole
  bool ws_stream_only = false;                                               // ws holds hbk_moe_decode_ws_stream_bytes only: the streaming chain must run
};
// What the last kernel does with the per-pair outputs.
struct hbk_reduce {
  float* out_accum = nullptr;                 // list form: out[row] += Σ in pair order (fp32)
  const void* shared = nullptr;               // routed form: external shared rows bf16 [M,H] (or the shared record's pairs when null)
  const float* lg = nullptr; int ld = 0, col = 0;
  void* out_bf16 = nullptr;                   // routed form with combine
  float* out_f32 = nullptr;                   // routed form without combine: overwritten with Σ_k w·expert
  void* shared_out = nullptr;                 // with out_f32 and a shared record: the shared expert's rows bf16 [sh_rows, H], written apart
  const hbk_ep_push* ep = nullptr;            // routed sums go to the owning ranks' partial buffers (row m belongs to rank m / B) instead of out_f32
};
int hbk_moe_decode_run(hb_ctx* ctx, const hbk_pair_src& src, const void* x, int H, int I, float limit, const hbk_reduce& red, void* ws,
                       cudaStream_t st);

// decode layer on the block-scaled tensor cores (k_moe_dtc.cu): routed form only, H and I multiples of 256
bool hbk_moe_dtc_supported(int H, int I);
bool hbk_moe_dtc_gu_fits(const hb_ctx* ctx, int n_pairs, int E, int H, int I);
size_t hbk_moe_dtc_ws_extra(int n_pairs, int H, int I);      // bytes it needs after the streaming path's workspace
int hbk_moe_dtc_setup(hb_ctx* ctx);
// gate/up pass alone on the tensor cores, between the streaming path's grouping kernel and its down kernel
int hbk_moe_dtc_gu_run(hb_ctx* ctx, const void* x, int x_ld, int M, const uint8_t* const* tab, int n_tab, const uint8_t* shared_rec, int P, int H, int I,
                       float limit, void* ws, const uint32_t* wait_flags, int wait_n, const uint32_t* wait_step, cudaStream_t st);
// down pass on the tensor cores behind it (digit planes of y, 128-row tiles of w2); with `red` it sums the rows' pairs itself
namespace hb { struct ReduceArgs; }
bool hbk_moe_dtc_down_fits(const hb_ctx* ctx, int n_pairs, int E, int H, int I);
int hbk_moe_dtc_down_run(hb_ctx* ctx, int P, int H, int I, void* ws, const hb::ReduceArgs* red, unsigned int* fin, cudaStream_t st);

// the anchored weight maps of both passes (made on first use per shape), for kernels that stream raw code boxes of the records
int hbk_moe_dtc_maps(hb_ctx* ctx, const uint8_t* const* tab, int n_tab, const uint8_t* shared_rec, int H, int I, cudaStream_t st);
void hbk_moe_dtc_map_set(const hb_ctx* ctx, int kind, const void** maps, const unsigned long long** anchor);   // kind 0: w1/w3 (pitch H/2), 1: w2 (pitch I/2)
int hbk_moe_dtc_vmax();

// dense GEMV (k_dense.cu)
int hbk_dense_setup(hb_ctx* ctx);
int hbk_moe_prefill_setup(hb_ctx* ctx);
