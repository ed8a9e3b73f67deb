/*
 * Plain-C restatement of the integer / index part of the MoE layer (TEST INFRASTRUCTURE: only
 * tests and the build check compile or call it; the library never does).
 *
 * Follows, in the MoE-Gen project:
 *   scoring + top-k   moe_gen/models/deepseek/deepseekv2/modeling_deepseek_v2.py:493-533
 *                     moe_gen/models/deepseek/deepseekv3/modeling_deepseek_v3.py:509-561
 *   histogram + sort  modeling_deepseek_v3.py:630-635
 *   FP8 de-quantise   moe_gen/models/Wrapper.py:109-138
 * Canonical choices where the reference leaves the result open (topk(sorted=False), argsort
 * without stable=True): score descending with ties to the lower expert id; experts ascending
 * with tokens ascending inside an expert.
 * Pinned by tests/test_oracle_golden.py against the fixtures recorded from the reference.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GATE_SOFTMAX_GREEDY 0
#define GATE_SOFTMAX_GROUP_MAX 1
#define GATE_SIGMOID_NOAUX_TC 2
#define GATE_SOFTMAX_TOPK_RENORM 3

/* picks the k best of v[0..n) (value descending, ties -> lower index) into out[] */
static void topk_lower_id(const float* v, int n, int k, int* out, unsigned char* taken) {
  memset(taken, 0, (size_t)n);
  for (int r = 0; r < k; ++r) {
    int best = -1;
    for (int i = 0; i < n; ++i)
      if (!taken[i] && (best < 0 || v[i] > v[best])) best = i;
    taken[best] = 1;
    out[r] = best;
  }
}

int mgo_route(const float* logits, const float* bias, int64_t T, int E, int k, int n_group, int topk_group,
              int gating, int norm, float scale, int32_t* idx_out, float* w_out) {
  float* s = (float*)malloc(sizeof(float) * (size_t)E);
  float* c = (float*)malloc(sizeof(float) * (size_t)E);
  float* gs = (float*)malloc(sizeof(float) * (size_t)(n_group > 0 ? n_group : 1));
  int* pick = (int*)malloc(sizeof(int) * (size_t)(E > n_group ? E : n_group));
  unsigned char* taken = (unsigned char*)malloc((size_t)E);
  if (!s || !c || !gs || !pick || !taken) return -1;
  for (int64_t t = 0; t < T; ++t) {
    const float* lg = logits + t * E;
    if (gating == GATE_SIGMOID_NOAUX_TC) {
      for (int e = 0; e < E; ++e) {
        s[e] = 1.0f / (1.0f + expf(-lg[e]));
        c[e] = s[e] + bias[e];
      }
    } else {
      float m = lg[0], sum = 0.f;
      for (int e = 1; e < E; ++e) m = lg[e] > m ? lg[e] : m;
      for (int e = 0; e < E; ++e) { s[e] = expf(lg[e] - m); sum += s[e]; }
      for (int e = 0; e < E; ++e) { s[e] = s[e] / sum; c[e] = s[e]; }
    }
    if (gating == GATE_SOFTMAX_GROUP_MAX || gating == GATE_SIGMOID_NOAUX_TC) {
      const int gsz = E / n_group;
      for (int g = 0; g < n_group; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
        for (int i = 0; i < gsz; ++i) {
          float v = c[g * gsz + i];
          if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
        }
        gs[g] = gating == GATE_SIGMOID_NOAUX_TC ? b1 + b2 : b1;   /* top-2 sum / max */
      }
      topk_lower_id(gs, n_group, topk_group, pick, taken);
      unsigned keep = 0;
      for (int r = 0; r < topk_group; ++r) keep |= 1u << pick[r];
      for (int e = 0; e < E; ++e)
        if (!((keep >> (e / gsz)) & 1u)) c[e] = 0.0f;             /* masked with 0.0, not -inf */
    }
    topk_lower_id(c, E, k, pick, taken);
    float denom = 0.f;
    for (int r = 0; r < k; ++r) {
      idx_out[t * k + r] = pick[r];
      w_out[t * k + r] = gating == GATE_SIGMOID_NOAUX_TC ? s[pick[r]] : c[pick[r]];
      denom += w_out[t * k + r];
    }
    for (int r = 0; r < k; ++r) {
      float w = w_out[t * k + r];
      if (gating == GATE_SOFTMAX_TOPK_RENORM) w = w / denom;
      else if (gating == GATE_SIGMOID_NOAUX_TC) { if (k > 1 && norm) w = w / (denom + 1e-20f); w = w * scale; }
      else { if (k > 1 && norm) w = w / (denom + 1e-20f); else w = w * scale; }
      w_out[t * k + r] = w;
    }
  }
  free(s); free(c); free(gs); free(pick); free(taken);
  return 0;
}

/* counts[E], offsets[E+1], order[T*k]: order[p] = flattened (token*k+slot) index of sorted row p */
int mgo_permute_plan(const int32_t* idx, int64_t T, int k, int E, int32_t* counts, int32_t* offsets,
                     int32_t* order) {
  memset(counts, 0, sizeof(int32_t) * (size_t)E);
  for (int64_t i = 0; i < T * k; ++i) counts[idx[i]]++;
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
  int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * (size_t)E);
  if (!cur) return -1;
  memcpy(cur, offsets, sizeof(int32_t) * (size_t)E);
  for (int64_t i = 0; i < T * k; ++i) order[cur[idx[i]]++] = (int32_t)i;   /* stable counting sort */
  free(cur);
  return 0;
}

static float e4m3_to_float(uint8_t b) {
  const int sign = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
  float v;
  if (e == 0) v = ldexpf((float)m, -9);                 /* subnormal: m * 2^-9 */
  else if (e == 15 && m == 7) v = NAN;                  /* the only NaN of e4m3fn */
  else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  return sign ? -v : v;
}

static uint16_t float_to_bf16_rn(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);   /* NaN */
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* out = bf16(float(q) * scale[r/128][c/128]) */
int mgo_dequant_fp8(const uint8_t* q, const float* scale, int64_t rows, int64_t cols, uint16_t* out) {
  const int64_t bcols = (cols + 127) / 128;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      out[r * cols + c] = float_to_bf16_rn(e4m3_to_float(q[r * cols + c]) * scale[(r / 128) * bcols + c / 128]);
  return 0;
}
