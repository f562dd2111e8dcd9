/* TEST INFRASTRUCTURE — CPU oracle of the quantized routed-expert path (see hive_oracle.h for the contract and the
 * reference file:line each function restates).  Plain C, scalar, single-threaded; compiled with -ffp-contract=off so every
 * rounding below is the one written.  Never linked into, imported by or called from the shipped library. */
#include "hive_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------------ formats */
static const float kE2M1[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

float ho_e2m1_to_f32(uint8_t nib) { return kE2M1[nib & 15]; }

/* engine/include/hive/common.h:69-80 */
float ho_e4m3_to_f32(uint8_t v) {
  const uint32_t s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
  float r;
  if (e == 0) r = ldexpf((float)m, -9);
  else if (e == 15 && m == 7) r = nanf("");
  else r = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
  return s ? -r : r;
}

/* engine/include/hive/common.h:88-113 (round to nearest even, saturate to ±448) */
uint8_t ho_f32_to_e4m3(float x) {
  if (isnan(x)) return 0x7F;
  uint32_t bits;
  memcpy(&bits, &x, 4);
  const uint8_t sign = (uint8_t)(bits >> 31);
  float a = fabsf(x);
  if (a > 448.0f) a = 448.0f;
  if (a < ldexpf(1.0f, -10)) return (uint8_t)(sign << 7);
  if (a < ldexpf(1.0f, -6)) {
    const float r = nearbyintf(a * 512.0f);
    const uint8_t m = (uint8_t)r;
    if (m == 8) return (uint8_t)((sign << 7) | (1 << 3));
    return (uint8_t)((sign << 7) | m);
  }
  int e;
  const float f = frexpf(a, &e);
  int E = e - 1 + 7;
  float r = nearbyintf((f * 2.0f - 1.0f) * 8.0f);
  if (r == 8.0f) { r = 0; E += 1; }
  if (E > 15 || (E == 15 && r >= 7)) return (uint8_t)((sign << 7) | 0x7E);
  return (uint8_t)((sign << 7) | (E << 3) | (uint8_t)r);
}

/* engine/include/hive/common.h:124-136 */
uint8_t ho_f32_to_e2m1(float v) {
  const float a = fabsf(v);
  uint8_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  else c = 7;
  return (uint8_t)(c | (v < 0 ? 8 : 0));
}

/* engine/include/hive/cpu/cpu_backend.h:103-108 */
float ho_bf16r(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return x;
  u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
  float r;
  memcpy(&r, &u, 4);
  return r;
}
uint16_t ho_f32_to_bf16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) return (uint16_t)((u >> 16) | ((u & 0x007fffffu) ? 0x40 : 0));   /* inf / quiet NaN */
  u = u + 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float ho_bf16_to_f32(uint16_t b) {
  const uint32_t u = (uint32_t)b << 16;
  float r;
  memcpy(&r, &u, 4);
  return r;
}

float ho_fp16_to_f32(uint16_t h) {
  const uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023;
  float r;
  if (e == 0) r = ldexpf((float)m, -24);
  else if (e == 31) r = m ? nanf("") : INFINITY;
  else r = ldexpf(1.0f + (float)m / 1024.0f, (int)e - 15);
  uint32_t u;
  memcpy(&u, &r, 4);
  u |= s;
  memcpy(&r, &u, 4);
  return r;
}
uint16_t ho_f32_to_fp16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000);
  const float a = fabsf(x);
  if (isnan(x)) return (uint16_t)(sign | 0x7e00);
  if (a >= 65520.0f) return (uint16_t)(sign | 0x7c00);
  if (a < ldexpf(1.0f, -14)) {                       /* subnormal: multiples of 2^-24 */
    const float q = nearbyintf(a * 16777216.0f);
    return (uint16_t)(sign | (uint16_t)q);           /* q == 1024 carries into the smallest normal */
  }
  int e;
  const float f = frexpf(a, &e);                     /* a = f·2^e, f in [0.5,1) */
  float m = nearbyintf((f * 2.0f - 1.0f) * 1024.0f);
  int E = e - 1 + 15;
  if (m == 1024.0f) { m = 0; E += 1; }
  if (E >= 31) return (uint16_t)(sign | 0x7c00);
  return (uint16_t)(sign | (E << 10) | (uint16_t)m);
}

/* engine/src/qwen/cpu/qwen_cpu_simd.h:23-41 */
float ho_exp_portable(float x) {
  const float kExpHi = 88.0f, kExpLo = -87.0f, kLog2e = 1.44269504088896341f, kLn2Hi = 0.693359375f, kLn2Lo = -2.12194440e-4f;
  const float kP0 = 1.9875691500e-4f, kP1 = 1.3981999507e-3f, kP2 = 8.3334519073e-3f, kP3 = 4.1665795894e-2f,
              kP4 = 1.6666665459e-1f, kP5 = 5.0000001201e-1f;
  x = fminf(fmaxf(x, kExpLo), kExpHi);
  const float n = nearbyintf(x * kLog2e);
  float r = fmaf(n, -kLn2Hi, x);
  r = fmaf(n, -kLn2Lo, r);
  float p = kP0;
  p = fmaf(p, r, kP1); p = fmaf(p, r, kP2); p = fmaf(p, r, kP3); p = fmaf(p, r, kP4); p = fmaf(p, r, kP5);
  const float rr = r * r;
  float y = fmaf(p, rr, r);
  y = y + 1.f;
  const uint32_t e = (uint32_t)((int32_t)n + 127) << 23;
  float s;
  memcpy(&s, &e, 4);
  return y * s;
}
static float silu_by_mode(float x, int mode) { return mode ? x / (1.f + ho_exp_portable(-x)) : x / (1.f + expf(-x)); }

/* ------------------------------------------------------------------------------------------------ record */
void ho_rec_layout(int H, int I, uint64_t off[8]) {
  const uint64_t wgu = (uint64_t)I * H / 2, sgu = (uint64_t)I * H / 16, wd = (uint64_t)H * I / 2, sd = (uint64_t)H * I / 16;
  off[0] = 0; off[1] = wgu; off[2] = off[1] + sgu; off[3] = off[2] + wgu; off[4] = off[3] + sgu; off[5] = off[4] + wd;
  off[6] = off[5] + sd;
  off[7] = (off[6] + 16 + 4095) / 4096 * 4096;
}

/* ------------------------------------------------------------------------------------------------ NVFP4 ops */
void ho_nvfp4_dequant_bf16(const uint8_t* w, const uint8_t* s, float g, int N, int K, uint16_t* out) {
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const float sc = ho_e4m3_to_f32(s[(size_t)n * (K / 16) + k / 16]) * g;
      const uint8_t b = w[(size_t)n * (K / 2) + k / 2];
      out[(size_t)n * K + k] = ho_f32_to_bf16(kE2M1[(k & 1) ? (b >> 4) : (b & 15)] * sc);
    }
}

void ho_gemv_nvfp4(const uint8_t* w, const uint8_t* s, float g, int N, int K, const float* a, int n0, int n1, float* y) {
  (void)N;
  float lut[256];
  for (int i = 0; i < 256; ++i) lut[i] = ho_e4m3_to_f32((uint8_t)i);
  for (int n = n0; n < n1; ++n) {
    const uint8_t* wr = w + (size_t)n * (K / 2);
    const uint8_t* sr = s + (size_t)n * (K / 16);
    float acc = 0.f;
    for (int b = 0; b < K / 16; ++b) {
      float d = 0.f;
      for (int i = 0; i < 16; ++i) {
        const int k = b * 16 + i;
        const uint8_t byte = wr[k / 2];
        d += a[k] * kE2M1[(k & 1) ? (byte >> 4) : (byte & 15)];
      }
      acc += d * lut[sr[b]];
    }
    y[n] = acc * g;
  }
}

void ho_expert_forward_nvfp4(const uint8_t* rec, const uint64_t* off, int H, int I, const float* a, float route_w, float limit,
                             int silu_mode, float* out, float* tmp) {
  float g[3];
  memcpy(g, rec + off[6], 12);
  float* gate = tmp; float* up = gate + I; float* y = up + I;
  ho_gemv_nvfp4(rec + off[0], rec + off[1], g[0], I, H, a, 0, I, gate);
  ho_gemv_nvfp4(rec + off[2], rec + off[3], g[1], I, H, a, 0, I, up);
  for (int i = 0; i < I; ++i) {
    float gv = ho_bf16r(gate[i]), uv = ho_bf16r(up[i]);
    if (limit > 0.f) { uv = fminf(fmaxf(uv, -limit), limit); gv = fminf(gv, limit); }
    y[i] = ho_bf16r(silu_by_mode(gv, silu_mode) * uv);
  }
  ho_gemv_nvfp4(rec + off[4], rec + off[5], g[2], H, I, y, 0, H, out);
  for (int k = 0; k < H; ++k) out[k] = ho_bf16r(out[k]) * route_w;
}

/* ------------------------------------------------------------------------------------------------ routers */
void ho_router_softmax_topk(const float* logits, int ld, int M, int E, int k, int renorm, int logits_bf16, int form,
                            int32_t* ids, float* w) {
  float* p = (float*)malloc(sizeof(float) * (size_t)E);
  for (int m = 0; m < M; ++m) {
    const float* lr = logits + (size_t)m * ld;
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) { p[e] = logits_bf16 ? ho_bf16r(lr[e]) : lr[e]; mx = fmaxf(mx, p[e]); }
    if (form == 0) {
      /* the GPU operator sums per lane (e = lane + 32·j, j ascending) and then by a 16,8,4,2,1 butterfly */
      float lane_sum[32];
      for (int l = 0; l < 32; ++l) lane_sum[l] = 0.f;
      for (int e = 0; e < E; ++e) p[e] = ho_exp_portable(p[e] - mx);
      for (int l = 0; l < 32; ++l) for (int e = l; e < E; e += 32) lane_sum[l] += p[e];
      for (int o = 16; o > 0; o >>= 1) { float t[32]; for (int l = 0; l < 32; ++l) t[l] = lane_sum[l] + lane_sum[l ^ o]; memcpy(lane_sum, t, sizeof t); }
      const float inv = 1.f / lane_sum[0];
      float tot = 0.f, pw[16];
      for (int r = 0; r < k; ++r) {
        float best = -1.f; int bid = 0x7fffffff;
        for (int e = 0; e < E; ++e) if (p[e] >= 0.f && (p[e] > best || (p[e] == best && e < bid))) { best = p[e]; bid = e; }
        const float sw = best * inv;
        tot += sw;
        ids[(size_t)m * k + r] = bid; pw[r] = sw;
        if (bid != 0x7fffffff) p[bid] = -1.f;
      }
      const float sc = renorm ? 1.f / tot : 1.f;
      for (int r = 0; r < k; ++r) w[(size_t)m * k + r] = pw[r] * sc;
    } else {
      float sum = 0.f;
      for (int e = 0; e < E; ++e) { p[e] = expf(p[e] - mx); sum += p[e]; }
      for (int e = 0; e < E; ++e) p[e] /= sum;
      float tot = 0.f; int sel[16];
      for (int r = 0; r < k; ++r) {
        int bid = -1;
        for (int e = 0; e < E; ++e) {
          int taken = 0;
          for (int q = 0; q < r; ++q) taken |= sel[q] == e;
          if (taken) continue;
          if (bid < 0 || p[e] > p[bid]) bid = e;      /* ascending scan with strict > : the smaller id wins ties */
        }
        sel[r] = bid; tot += p[bid];
      }
      for (int r = 0; r < k; ++r) { ids[(size_t)m * k + r] = sel[r]; w[(size_t)m * k + r] = renorm ? p[sel[r]] / tot : p[sel[r]]; }
    }
  }
  free(p);
}

void ho_router_sigmoid_topk(const float* logits, const float* bias, int M, int E, int k, float scale, int form, int32_t* ids, float* w) {
  float* s = (float*)malloc(sizeof(float) * (size_t)E * 2);
  float* c = s + E;
  for (int m = 0; m < M; ++m) {
    const float* lr = logits + (size_t)m * E;
    for (int e = 0; e < E; ++e) {
      const float v = 1.f / (1.f + (form ? expf(-lr[e]) : ho_exp_portable(-lr[e])));
      s[e] = v; c[e] = v + (bias ? bias[e] : 0.f);
    }
    float sum = 0.f; int sel[16];
    for (int j = 0; j < k; ++j) {
      int best = -1; float bv = -INFINITY;
      for (int e = 0; e < E; ++e) if (c[e] > bv) { bv = c[e]; best = e; }
      sel[j] = best; c[best] = -INFINITY; sum += s[best];
    }
    const float inv = 1.f / (sum + 1e-20f);
    for (int j = 0; j < k; ++j) { ids[(size_t)m * k + j] = sel[j]; w[(size_t)m * k + j] = s[sel[j]] * inv * scale; }
  }
  free(s);
}

/* ------------------------------------------------------------------------------------------------ MoE operators */
void ho_moe_decode(const uint64_t* off, const int32_t* rows, const uint8_t* const* recs, const float* pw, int n_pairs,
                   const float* x, int H, int I, float limit, int silu_mode, float* out) {
  float* e = (float*)malloc(sizeof(float) * ((size_t)H + 3 * (size_t)I));
  float* tmp = e + H;
  for (int i = 0; i < n_pairs; ++i) {
    if (!recs[i]) continue;
    ho_expert_forward_nvfp4(recs[i], off, H, I, x + (size_t)rows[i] * H, pw[i], limit, silu_mode, e, tmp);
    float* o = out + (size_t)rows[i] * H;
    for (int d = 0; d < H; ++d) o[d] += e[d];
  }
  free(e);
}

void ho_moe_routed(const uint64_t* off, const int32_t* ids, const float* w, int M, int K, const uint8_t* const* rec_tab, int E,
                   const float* x, int H, int I, float limit, int silu_mode, float* acc) {
  float* e = (float*)malloc(sizeof(float) * ((size_t)H + 3 * (size_t)I));
  float* tmp = e + H;
  for (int m = 0; m < M; ++m) {
    float* a = acc + (size_t)m * H;
    for (int d = 0; d < H; ++d) a[d] = 0.f;
    for (int k = 0; k < K; ++k) {
      const int id = ids[(size_t)m * K + k];
      if (id < 0 || id >= E || !rec_tab[id]) continue;
      ho_expert_forward_nvfp4(rec_tab[id], off, H, I, x + (size_t)m * H, 1.f, limit, silu_mode, e, tmp);
      const float wv = w[(size_t)m * K + k];
      for (int d = 0; d < H; ++d) a[d] = a[d] + wv * e[d];
    }
  }
  free(e);
}

void ho_moe_combine(const float* routed, const float* shared, const float* gate_logits, int ld, int col, int round_gate, int M, int H,
                    uint16_t* out) {
  for (int m = 0; m < M; ++m) {
    float g = 1.f;
    if (gate_logits) {
      const float l = gate_logits[(size_t)m * ld + col];
      if (round_gate) g = ho_bf16r(1.f / (1.f + ho_exp_portable(-ho_bf16r(l))));
      else g = 1.f / (1.f + ho_exp_portable(-l));
    }
    for (int d = 0; d < H; ++d) {
      const size_t i = (size_t)m * H + d;
      const float sh = gate_logits ? ho_bf16r(g * shared[i]) : ho_bf16r(shared[i]);
      out[i] = ho_f32_to_bf16(ho_bf16r(routed[i]) + sh);
    }
  }
}

/* ------------------------------------------------------------------------------------------------ quantizers */
static int nearest_code(double a, const double* tab, int n) {       /* tools/q27_reencode.py:68-76 */
  if (a > tab[n - 1]) a = tab[n - 1];
  int hi = 0;
  while (hi < n && tab[hi] < a) ++hi;                                /* searchsorted(..., side="left") */
  if (hi < 1) hi = 1;
  if (hi > n - 1) hi = n - 1;
  const int lo = hi - 1;
  const double dlo = a - tab[lo], dhi = tab[hi] - a;
  return (dhi < dlo || (dhi == dlo && hi % 2 == 0)) ? hi : lo;
}

void ho_nvfp4_quantize(const float* w, int N, int K, int search, uint8_t* q, uint8_t* s, float* g_mul) {
  static const double kFactors[5] = {1.0, 0.95, 0.9, 0.85, 1.05};
  static const double kE2[8] = {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0};
  double e4[127];
  for (int c = 0; c < 127; ++c) e4[c] = (double)ho_e4m3_to_f32((uint8_t)c);
  float amaxf = 0.f;
  for (size_t i = 0; i < (size_t)N * K; ++i) amaxf = fmaxf(amaxf, fabsf(w[i]));
  const double amax = (double)amaxf;
  *g_mul = amaxf > 0.f ? amaxf / (448.f * 6.f) : 1.f;                 /* fp32 division, as the device kernel does */
  /* search: np.float32(448*6/amax) (a double division rounded once); device rule: 448.f*6.f / amax in fp32 */
  const float g = amaxf > 0.f ? (search ? (float)(448.0 * 6.0 / amax) : 448.f * 6.f / amaxf) : 1.f;
  for (int n = 0; n < N; ++n)
    for (int b = 0; b < K / 16; ++b) {
      const float* wb = w + (size_t)n * K + (size_t)b * 16;
      uint8_t code[16];
      uint8_t sc_out = 0;
      if (search) {
        float blk[16], bmax = 0.f;
        for (int i = 0; i < 16; ++i) { blk[i] = wb[i] * g; bmax = fmaxf(bmax, fabsf(blk[i])); }
        double best_err = 0;
        for (int f = 0; f < 5; ++f) {
          const float t = (bmax / 6.0f) * (float)kFactors[f];
          const int sc = nearest_code((double)t, e4, 127);
          const double sv = e4[sc];
          double err = 0;
          uint8_t c[16];
          for (int i = 0; i < 16; ++i) {
            const double y = sv > 0 ? (double)blk[i] / sv : 0.0;
            const int ci = nearest_code(fabs(y), kE2, 8);
            const double rec = (y > 0 ? 1.0 : y < 0 ? -1.0 : 0.0) * kE2[ci] * sv;
            err += (rec - (double)blk[i]) * (rec - (double)blk[i]);
            c[i] = (uint8_t)(ci | (signbit(blk[i]) ? 8 : 0));
          }
          if (f == 0 || err < best_err) { best_err = err; sc_out = (uint8_t)sc; memcpy(code, c, 16); }
        }
      } else {                                                       /* engine/src/q27/q27_kernels.cu:2506-2529 */
        float m = 0.f;
        for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(wb[i]));
        sc_out = ho_f32_to_e4m3(m * g / 6.f);
        const float sd = ho_e4m3_to_f32(sc_out);
        for (int i = 0; i < 16; ++i) code[i] = sd > 0.f ? ho_f32_to_e2m1(wb[i] * g / sd) : 0;
      }
      s[(size_t)n * (K / 16) + b] = sc_out;
      for (int i = 0; i < 8; ++i) q[(size_t)n * (K / 2) + (size_t)b * 8 + i] = (uint8_t)((code[2 * i] & 15) | (code[2 * i + 1] << 4));
    }
}

void ho_a4_quant(const float* x, int ld, int n, int K, uint8_t* q, uint8_t* s, float* g) {
  for (int r = 0; r < n; ++r) {
    const float* xr = x + (size_t)r * ld;
    float a = 0.f;
    for (int k = 0; k < K; ++k) a = fmaxf(a, fabsf(xr[k]));
    const float gx = a > 0.f ? a / (6.f * 448.f) : 1.f, inv = 1.f / gx;
    g[r] = gx;
    for (int b = 0; b < K / 16; ++b) {
      float ab = 0.f;
      for (int j = 0; j < 16; ++j) ab = fmaxf(ab, fabsf(xr[b * 16 + j]));
      const uint8_t se = ho_f32_to_e4m3(ab / 6.f * inv);
      const float sv = ho_e4m3_to_f32(se);
      const float f = sv > 0.f ? inv / sv : 0.f;
      for (int j = 0; j < 8; ++j) {
        const uint8_t lo = ho_f32_to_e2m1(xr[b * 16 + 2 * j] * f), hi = ho_f32_to_e2m1(xr[b * 16 + 2 * j + 1] * f);
        q[(size_t)r * (K / 2) + (size_t)b * 8 + j] = (uint8_t)((lo & 15) | (hi << 4));
      }
      s[(size_t)r * (K / 16) + b] = se;
    }
  }
}

/* W4A4 GEMV of one quantised activation row (codes aq, scales as, global ag) against an NVFP4 matrix: what the block-scaled
 * tensor-core GEMM of the prefill path computes (engine/src/qwen/fn_moe_pf.cu:439-446): per 16-value block the integer-valued
 * dot product of the two code vectors (exact) times both block scales, summed in fp32 (double here: the hardware's summation
 * order is not specified, so the oracle keeps the sum exact and rounds once). */
static void gemv_a4(const uint8_t* wq, const uint8_t* wsc, int N, int K, const uint8_t* aq, const uint8_t* as, double* y) {
  for (int n = 0; n < N; ++n) {
    double acc = 0.0;
    for (int b = 0; b < K / 16; ++b) {
      float dot = 0.f;
      for (int j = 0; j < 8; ++j) {
        const uint8_t wb = wq[(size_t)n * (K / 2) + (size_t)b * 8 + j], ab = aq[(size_t)b * 8 + j];
        dot += ho_e2m1_to_f32(wb & 15) * ho_e2m1_to_f32(ab & 15) + ho_e2m1_to_f32(wb >> 4) * ho_e2m1_to_f32(ab >> 4);
      }
      acc += (double)dot * (double)ho_e4m3_to_f32(wsc[(size_t)n * (K / 16) + b]) * (double)ho_e4m3_to_f32(as[b]);
    }
    y[n] = acc;
  }
}

/* One expert on one row with NVFP4 activations: x → a4 quant → gate, up; g = bf16(acc·gx·g1), u = bf16(acc·gx·g3),
 * y = bf16(silu(g)·u) → a4 quant → down; out = bf16(acc·(gy·g2)) (fn_moe_pf.cu:636-660, :903-908).  out is not multiplied by a
 * routing weight: the prefill reduce does that. */
void ho_expert_forward_a4(const uint8_t* rec, const uint64_t* off, int H, int I, const float* x, float limit, float* out) {
  float g[3];
  memcpy(g, rec + off[6], 12);
  const int Kmax = H > I ? H : I;
  uint8_t* q = (uint8_t*)malloc((size_t)Kmax / 2 + (size_t)Kmax / 16);
  uint8_t* sc = q + Kmax / 2;
  double* acc = (double*)malloc(sizeof(double) * (size_t)(2 * I > H ? 2 * I : H));
  float* y = (float*)malloc(sizeof(float) * (size_t)I);
  float gx;
  ho_a4_quant(x, H, 1, H, q, sc, &gx);
  gemv_a4(rec + off[0], rec + off[1], I, H, q, sc, acc);
  gemv_a4(rec + off[2], rec + off[3], I, H, q, sc, acc + I);
  for (int i = 0; i < I; ++i) {
    float gv = ho_bf16r((float)acc[i] * gx * g[0]), uv = ho_bf16r((float)acc[I + i] * gx * g[1]);
    if (limit > 0.f) { uv = fminf(fmaxf(uv, -limit), limit); gv = fminf(gv, limit); }
    y[i] = ho_bf16r(gv / (1.f + expf(-gv)) * uv);
  }
  float gy;
  ho_a4_quant(y, I, 1, I, q, sc, &gy);
  gemv_a4(rec + off[4], rec + off[5], H, I, q, sc, acc);
  for (int d = 0; d < H; ++d) out[d] = ho_bf16r((float)acc[d] * (gy * g[2]));
  free(y); free(acc); free(q);
}

/* ------------------------------------------------------------------------------------------------ 3-/2-bit group-64 */
size_t ho_lb_weight_bytes(int bits, int N, int K) { return bits == 2 ? (size_t)N * K / 4 : (size_t)N * K / 4 + (size_t)N * K / 8; }

static int lb_code(const uint8_t* q, int bits, int N, int K, int n, int k) {
  int c = (q[(size_t)n * (K / 4) + k / 4] >> (2 * (k & 3))) & 3;
  if (bits == 3) c |= ((q[(size_t)N * (K / 4) + (size_t)n * (K / 8) + k / 8] >> (k & 7)) & 1) << 2;
  return c;
}

void ho_lb_quantize(const float* w, int N, int K, int bits, uint8_t* q, uint16_t* s, uint16_t* zp) {
  const int qmax = (1 << bits) - 1;
  memset(q, 0, ho_lb_weight_bytes(bits, N, K));
  for (int n = 0; n < N; ++n)
    for (int gidx = 0; gidx < K / 64; ++gidx) {
      const float* wg = w + (size_t)n * K + (size_t)gidx * 64;
      float mn = wg[0], mx = wg[0];
      for (int i = 1; i < 64; ++i) { mn = fminf(mn, wg[i]); mx = fmaxf(mx, wg[i]); }
      uint16_t sh = ho_f32_to_fp16((mx - mn) / (float)qmax);
      if (ho_fp16_to_f32(sh) <= 0.f) sh = ho_f32_to_fp16(1.f);
      const float sf = ho_fp16_to_f32(sh);
      const uint16_t zh = ho_f32_to_fp16(-mn / sf);
      const float zf = ho_fp16_to_f32(zh);
      s[(size_t)n * (K / 64) + gidx] = sh; zp[(size_t)n * (K / 64) + gidx] = zh;
      for (int i = 0; i < 64; ++i) {
        float c = nearbyintf(wg[i] / sf + zf);
        if (c < 0.f) c = 0.f;
        if (c > (float)qmax) c = (float)qmax;
        const int ci = (int)c, k = gidx * 64 + i;
        q[(size_t)n * (K / 4) + k / 4] |= (uint8_t)((ci & 3) << (2 * (k & 3)));
        if (bits == 3) q[(size_t)N * (K / 4) + (size_t)n * (K / 8) + k / 8] |= (uint8_t)(((ci >> 2) & 1) << (k & 7));
      }
    }
}

void ho_lb_dequant_bf16(const uint8_t* q, const uint16_t* s, const uint16_t* zp, int bits, int N, int K, uint16_t* out) {
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const float sf = ho_fp16_to_f32(s[(size_t)n * (K / 64) + k / 64]), zf = ho_fp16_to_f32(zp[(size_t)n * (K / 64) + k / 64]);
      out[(size_t)n * K + k] = ho_f32_to_bf16(((float)lb_code(q, bits, N, K, n, k) - zf) * sf);
    }
}

void ho_lb_gemv(const uint8_t* q, const uint16_t* s, const uint16_t* zp, int bits, int N, int K, const float* a, int n0, int n1, float* y) {
  for (int n = n0; n < n1; ++n) {
    float acc = 0.f;
    for (int gidx = 0; gidx < K / 64; ++gidx) {
      float d = 0.f, sx = 0.f;
      for (int i = 0; i < 64; ++i) {
        const int k = gidx * 64 + i;
        d += a[k] * (float)lb_code(q, bits, N, K, n, k);
        sx += a[k];
      }
      const float sf = ho_fp16_to_f32(s[(size_t)n * (K / 64) + gidx]), zf = ho_fp16_to_f32(zp[(size_t)n * (K / 64) + gidx]);
      acc += (d - zf * sx) * sf;
    }
    y[n] = acc;
  }
}

void ho_dense_act(const float* g, const float* u, int n, float* act) {
  for (int i = 0; i < n; ++i) {
    const float gv = ho_bf16r(g[i]), uv = ho_bf16r(u[i]);
    act[i] = ho_bf16r(ho_bf16r(gv / (1.f + expf(-gv))) * uv);
  }
}

/* ================================================================================================ record assembly
 * Compressed block scales, engine/src/ckpt_quant.cpp:34-73.  Position n of a group = 16 rows x C columns row-major; delta n sits in
 * body[n / 2], low nibble when n is even. */
static int csf_delta(const uint8_t* grp, size_t n) { return (grp[16 + (n >> 1)] >> ((n & 1) * 4)) & 15; }

int ho_csf_decode(const uint8_t* fixed, int64_t fixed_rows, int64_t fixed_cols, const uint32_t* exc, size_t n_exc, int R, int C, uint8_t* out,
                  int64_t* where) {
  if (where) *where = 0;
  if (R <= 0 || C <= 0 || R % 16 != 0) return HO_CSF_ROWS;
  if (fixed_rows != R / 16 || fixed_cols != 16 + 8 * (int64_t)C) return HO_CSF_SHAPE;
  const int64_t total = (int64_t)R * C, per_group = 16 * (int64_t)C;
  if (total > ((int64_t)1 << 24)) return HO_CSF_TOO_MANY;
  for (int64_t i = 0; i < total; ++i) {                   /* flat index i = group * 16C + position inside the group */
    const uint8_t* grp = fixed + (size_t)(i / per_group) * (size_t)fixed_cols;
    const int64_t n = i % per_group;
    const int code = grp[n / C] + csf_delta(grp, (size_t)n);
    out[i] = code > 0x7E ? 0xFF : (uint8_t)code;         /* 0xFF = not a scale unless an exception replaces it */
  }
  for (size_t k = 0; k < n_exc; ++k) {
    const int64_t i = exc[k] & 0xFFFFFF;
    const unsigned v = exc[k] >> 24;
    if (where) *where = (int64_t)k;
    if (i >= total) return HO_CSF_EXC_INDEX;
    if (csf_delta(fixed + (size_t)(i / per_group) * (size_t)fixed_cols, (size_t)(i % per_group)) != 0) return HO_CSF_EXC_DELTA;
    if (v > 0x7E) return HO_CSF_EXC_VALUE;
    out[i] = (uint8_t)v;                                  /* a later exception for the same index wins */
  }
  for (int64_t i = 0; i < total; ++i)
    if (out[i] > 0x7E) { if (where) *where = i; return HO_CSF_CODE; }
  if (where) *where = 0;
  return HO_CSF_OK;
}

int ho_record_pack(const uint64_t* off, int H, int I, const uint8_t* const weight[3], const uint8_t* const scale[3],
                   const uint8_t* const csf_fixed[3], const uint32_t* const csf_exc[3], const size_t n_exc[3], const float global[3],
                   uint8_t* rec) {
  const uint64_t w_off[3] = {off[0], off[2], off[4]}, s_off[3] = {off[1], off[3], off[5]};
  const int rows[3] = {I, I, H}, cols[3] = {H, H, I};
  for (int j = 0; j < 3; ++j) {
    const size_t nw = (size_t)rows[j] * cols[j] / 2, ns = (size_t)rows[j] * cols[j] / 16;
    memcpy(rec + w_off[j], weight[j], nw);
    if (scale[j]) memcpy(rec + s_off[j], scale[j], ns);
    else {
      const int C = cols[j] / 16;
      const int r = ho_csf_decode(csf_fixed[j], rows[j] / 16, 16 + 8 * (int64_t)C, csf_exc[j], n_exc[j], rows[j], C, rec + s_off[j], NULL);
      if (r) return 10 * (j + 1) + r;
    }
    memcpy(rec + off[6] + 4 * j, &global[j], 4);
  }
  return 0;
}

