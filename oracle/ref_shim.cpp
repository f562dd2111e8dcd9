// TEST INFRASTRUCTURE — not part of the shipped library.
//
// extern "C" window onto the reference engine's own CPU code for the quantized routed-expert path.  The reference
// sources are compiled where they lie (see oracle/Makefile); nothing of them is copied here.  This file only
// forwards to the reference's public functions and, for the whole-layer runner, strings the reference's public
// CPU-backend calls (make_mat / matmul_multi / simd helpers) together in the order its CPU-only daemon does.
//
// Reference entry points bound here (paths inside the reference project):
//   engine/include/hive/common.h:69-140            e4m3 / e2m1 decode + encode, bf16 helpers
//   engine/include/hive/expert_cpu.h:78-106         gemv_nvfp4_rows*, expert_forward_nvfp4
//   engine/include/hive/cpu/cpu_backend.h:23-108    Pool, make_mat, matmul_multi, bf16r
//   engine/src/qwen/cpu/qwen_cpu_simd.h:17-41,153-165  portable exp / sigmoid / silu, silu_mul
//   engine/src/qwen/cpu/qwen_cpu_engine.cpp:655-783 order of operations of the CPU MoE layer (followed by ref_moe_layer_*)
//   engine/include/hive/ckpt_quant.h:35-37          csf_decode (compressed NVFP4 block scales of a checkpoint projection)
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <algorithm>
#include <vector>

#include <string>

#include "hive/ckpt_quant.h"
#include "hive/common.h"
#include "hive/cpu/cpu_backend.h"
#include "hive/expert_cpu.h"
#include "src/qwen/cpu/qwen_cpu_simd.h"

using namespace hive;
namespace simd = hive::qwen::cpu::simd;

extern "C" {

float ref_e4m3_to_f32(uint8_t v) { return e4m3_to_f32(v); }
float ref_e2m1_to_f32(uint8_t v) { return e2m1_to_f32(v); }
uint8_t ref_f32_to_e4m3(float x) { return f32_to_e4m3_host(x); }
uint8_t ref_f32_to_e2m1(float x) { return f32_to_e2m1(x); }
float ref_bf16r(float x) { return hive::cpu::bf16r(x); }
float ref_exp_portable(float x) { return simd::exp_s(x); }
float ref_sigm_portable(float x) { return simd::sigm_s(x); }
float ref_silu_portable(float x) { return simd::silu_s(x); }

void ref_gemv_nvfp4_rows_scalar(const uint8_t* W, const uint8_t* s, float g, int N, int K, const float* a, int n0, int n1, float* y) {
  hive::cpu::gemv_nvfp4_rows_scalar(W, s, g, N, K, a, n0, n1, y);
}
void ref_gemv_nvfp4_rows(const uint8_t* W, const uint8_t* s, float g, int N, int K, const float* a, int n0, int n1, float* y) {
  hive::cpu::gemv_nvfp4_rows(W, s, g, N, K, a, n0, n1, y);
}
// One expert on one activation row (bf16 values held as fp32).  rec points at an expert record laid out as
// [w1][s1][w3][s3][w2][s2][g1 g3 g2]; offsets are passed by the caller so this file needs no GPU header.
void ref_expert_forward_nvfp4(const uint8_t* rec, const uint64_t* off /*w1,s1,w3,s3,w2,s2,g*/, int H, int I, const float* a, float route_w,
                              float limit, float* out, float* tmp) {
  hive::cpu::ExpertDescNvfp4 e;
  e.dim = H; e.inter = I;
  e.w1 = rec + off[0]; e.s1 = rec + off[1]; e.w3 = rec + off[2]; e.s3 = rec + off[3]; e.w2 = rec + off[4]; e.s2 = rec + off[5];
  float g[3];
  std::memcpy(g, rec + off[6], 12);
  e.g1 = g[0]; e.g3 = g[1]; e.g2 = g[2];
  hive::cpu::expert_forward_nvfp4(e, a, route_w, limit, out, tmp);
}

int ref_pool_threads() { return hive::cpu::Pool::get().threads(); }
int ref_pool_nodes() { return hive::cpu::Pool::get().nodes(); }

// ---- the CPU-only daemon's MoE layer on the reference's CPU backend -------------------------------------------------------
// Weights of one layer as the CPU engine stacks them: gu = [gates of every expert ; ups of every expert] (2·E·I rows of H),
// d = [first half-rows of every expert's down ; second half-rows] (2·E·H/2 rows of I) — qwen_cpu_engine.cpp:731-753.
struct RefLayer {
  int H, I, E;
  hive::cpu::Mat gu, d;
  std::vector<float> g_gate, g_up, g_down;
};

void* ref_layer_create(int H, int I, int E, const uint8_t* const* recs, const uint64_t* off) {
  auto* L = new RefLayer{H, I, E, {}, {}, {}, {}, {}};
  const size_t wgu = (size_t)I * H / 2, sgu = (size_t)I * H / 16, hh = (size_t)H / 2;
  std::vector<uint8_t> w((size_t)2 * E * wgu), s((size_t)2 * E * sgu);
  for (int e = 0; e < E; ++e) {
    std::memcpy(w.data() + (size_t)e * wgu, recs[e] + off[0], wgu);
    std::memcpy(s.data() + (size_t)e * sgu, recs[e] + off[1], sgu);
    std::memcpy(w.data() + (size_t)(E + e) * wgu, recs[e] + off[2], wgu);
    std::memcpy(s.data() + (size_t)(E + e) * sgu, recs[e] + off[3], sgu);
  }
  // per-expert globals are applied after the matmul (silu_mul's sa / sb, the bf16(D·g) pass), so the Mat carries 1
  L->gu = hive::cpu::make_mat(hive::cpu::WType::NVFP4, 2 * E * I, H, w.data(), s.data(), hive::cpu::SType::E4M3, 1.f);
  std::vector<uint8_t> wd((size_t)E * H * I / 2), sd((size_t)E * H * I / 16);
  const size_t rw = (size_t)I / 2, rs = (size_t)I / 16;
  for (int e = 0; e < E; ++e) {
    std::memcpy(wd.data() + ((size_t)e * hh) * rw, recs[e] + off[4], hh * rw);
    std::memcpy(sd.data() + ((size_t)e * hh) * rs, recs[e] + off[5], hh * rs);
    std::memcpy(wd.data() + ((size_t)(E + e) * hh) * rw, recs[e] + off[4] + hh * rw, hh * rw);
    std::memcpy(sd.data() + ((size_t)(E + e) * hh) * rs, recs[e] + off[5] + hh * rs, hh * rs);
  }
  L->d = hive::cpu::make_mat(hive::cpu::WType::NVFP4, E * H, I, wd.data(), sd.data(), hive::cpu::SType::E4M3, 1.f);
  L->g_gate.resize(E); L->g_up.resize(E); L->g_down.resize(E);
  for (int e = 0; e < E; ++e) {
    float g[3];
    std::memcpy(g, recs[e] + off[6], 12);
    L->g_gate[e] = g[0]; L->g_up[e] = g[1]; L->g_down[e] = g[2];
  }
  return L;
}
void ref_layer_destroy(void* p) {
  auto* L = (RefLayer*)p;
  if (!L) return;
  hive::cpu::free_mat(L->gu); hive::cpu::free_mat(L->d);
  delete L;
}

// Routed part of a layer for given ids / weights: pair_out-style weighted sum in k order, fp32 acc [M, H] (not rounded).
// ids < 0 or ≥ E contribute nothing.  limit > 0 selects the clamped activation (GLM), else plain SiLU through the portable exp.
void ref_layer_routed(void* p, int M, int K, const int32_t* ids, const float* wts, const float* x, float limit, float* acc) {
  using hive::cpu::MatJob; using hive::cpu::MatView; using hive::cpu::bf16r;
  RefLayer& L = *(RefLayer*)p;
  const int H = L.H, I = L.I, E = L.E, hh = H / 2;
  std::vector<int> cnt(E, 0), off(E + 1, 0), prow, pslot, pexp;
  int P = 0;
  for (int i = 0; i < M * K; ++i) if (ids[i] >= 0 && ids[i] < E) { ++cnt[ids[i]]; ++P; }
  for (int e = 0; e < E; ++e) off[e + 1] = off[e] + cnt[e];
  prow.resize(P); pslot.resize(P); pexp.resize(P);
  {
    std::vector<int> fill(off.begin(), off.end() - 1);
    for (int m = 0; m < M; ++m)
      for (int k = 0; k < K; ++k) {
        const int e = ids[(size_t)m * K + k];
        if (e < 0 || e >= E) continue;
        const int q = fill[e]++;
        prow[q] = m; pslot[q] = k; pexp[q] = e;
      }
  }
  std::vector<float> Xe((size_t)P * H), G((size_t)P * I), U((size_t)P * I), Y((size_t)P * I), D2((size_t)P * H);
  for (int q = 0; q < P; ++q) std::memcpy(Xe.data() + (size_t)q * H, x + (size_t)prow[q] * H, (size_t)H * 4);
  std::vector<MatJob> jobs;
  for (int e = 0; e < E; ++e) {
    if (!cnt[e]) continue;
    const int r = off[e];
    jobs.push_back(MatJob{MatView{&L.gu, e * I, (e + 1) * I}, G.data() + (size_t)r * I, I, Xe.data() + (size_t)r * H, cnt[e], H});
    jobs.push_back(MatJob{MatView{&L.gu, E * I + e * I, E * I + (e + 1) * I}, U.data() + (size_t)r * I, I, Xe.data() + (size_t)r * H, cnt[e], H});
  }
  if (!jobs.empty()) hive::cpu::matmul_multi(jobs.data(), (int)jobs.size(), nullptr, 0, 0);
  for (int r = 0; r < P; ++r) {
    const int e = pexp[r];
    if (limit > 0.f) {
      for (int i = 0; i < I; ++i) {
        float g = bf16r(G[(size_t)r * I + i] * L.g_gate[e]), u = bf16r(U[(size_t)r * I + i] * L.g_up[e]);
        u = std::fmin(std::fmax(u, -limit), limit); g = std::fmin(g, limit);
        Y[(size_t)r * I + i] = bf16r(g / (1.f + std::exp(-g)) * u);
      }
    } else {
      simd::silu_mul_v(G.data() + (size_t)r * I, U.data() + (size_t)r * I, I, L.g_gate[e], L.g_up[e], Y.data() + (size_t)r * I);
    }
  }
  jobs.clear();
  for (int e = 0; e < E; ++e) {
    if (!cnt[e]) continue;
    const int r = off[e];
    jobs.push_back(MatJob{MatView{&L.d, e * hh, (e + 1) * hh}, D2.data() + (size_t)r * H, H, Y.data() + (size_t)r * I, cnt[e], I});
    jobs.push_back(MatJob{MatView{&L.d, E * hh + e * hh, E * hh + (e + 1) * hh}, D2.data() + (size_t)r * H + hh, H, Y.data() + (size_t)r * I, cnt[e], I});
  }
  if (!jobs.empty()) hive::cpu::matmul_multi(jobs.data(), (int)jobs.size(), nullptr, 0, 0);
  std::vector<int> slot((size_t)M * K, -1);
  for (int q = 0; q < P; ++q) slot[(size_t)prow[q] * K + pslot[q]] = q;
  for (int m = 0; m < M; ++m)
    for (int d = 0; d < H; ++d) {
      float a = 0.f;
      for (int k = 0; k < K; ++k) {
        const int q = slot[(size_t)m * K + k];
        if (q < 0) continue;
        a = a + wts[(size_t)m * K + k] * bf16r(D2[(size_t)q * H + d] * L.g_down[pexp[q]]);
      }
      acc[(size_t)m * H + d] = a;
    }
}

// 1 = decoded, 0 = refused (the reference's message is copied into err, NUL-terminated, when err_len > 0)
int ref_csf_decode(const uint8_t* fixed, int64_t fixed_rows, int64_t fixed_cols, const uint32_t* exc, size_t n_exc, int R, int C, uint8_t* out,
                   char* err, int err_len) {
  std::string e;
  const bool ok = hive::ckq::csf_decode(fixed, fixed_rows, fixed_cols, exc, n_exc, R, C, out, &e);
  if (err && err_len > 0) { std::strncpy(err, e.c_str(), (size_t)err_len - 1); err[err_len - 1] = 0; }
  return ok ? 1 : 0;
}

}
