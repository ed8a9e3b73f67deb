// Routing (scoring + top-k), permute plan (histogram, prefix sums, stable placement),
// row scatter and weighted combine.  All HBM-bound index/byte work: one warp per token,
// 128-bit vector accesses on rows.
#include <mutex>

#include "common.cuh"

namespace mg {

// ---------------------------------------------------------------------------------------
// scoring + top-k: one warp per token, lane l owns experts [l*P, l*P+P)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  v = v + 0.0f;  // -0.0 -> +0.0 so that equal values have equal keys
  uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
// larger key = better pick: score descending, then index ascending
__device__ __forceinline__ unsigned long long make_key(float v, uint32_t index) {
  return (static_cast<unsigned long long>(ordered_bits(v)) << 32) | (0xFFFFFFFFu - index);
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long k) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, k, o);
    k = other > k ? other : k;
  }
  return k;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
// fixed-order sum: the same pairing on every launch, so results are reproducible
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// Routing of one token by one warp, with the detection of near-ties for the fix-up (fix != nullptr).
//
// The tensor-core router product accumulates H/16 partial sums in fp32 with truncation: its error grows
// with H and with the size of the sums.  Measured on random inputs: 1.2e-5 * max|logit| at H = 7168; the
// bound assumed below is 4x that (the tests hold the measured error under half of it).  With a logit
// error of at most dl, a sigmoid score moves by at most dl/4 (a group score, the sum of two, by dl/2) and a
// softmax score p by at most 2*p*dl.  A token is "close" when its last kept group or expert leads the
// best rejected one by less than twice that; only then can the pick differ from that of exact logits.
// For a close token the experts that can change the outcome ("in play") are listed as (token, expert)
// pairs, their logits are recomputed exactly, and the token is routed again:
//   * group selection close: in-play groups are those within the error of the kept/rejected boundary;
//     of each, the experts that can be among the values its score is made of;
//   * top-k: with U_min / U_max the groups kept in every / in some admissible outcome and v_lo / v_hi
//     the k-th best value over them, the experts of U_max between v_lo - 2*de and v_hi + 2*de (anything
//     above is picked and anything below is not, whatever the errors do).
// Every other logit keeps its tensor-core value: it cannot change a pick, and it moves a routing weight by
// no more than it does for a token that is not close.
// fix layout (int32): [0] tokens to route again, [1] of which with whole rows to recompute, [2] pairs
// asked for (may exceed the capacity), [3] unused; tokens [4, 4+T); row tokens [4+T, 4+2T); pairs from
// 4+2T, rp.pair_cap of them.  A token whose pairs do not fit, or whose groups are not runs of lanes,
// has its whole row recomputed instead.
__host__ __device__ inline float route_fix_err(int hidden) { return 6.0e-9f * hidden + 4.0e-6f; }
__device__ __forceinline__ float from_ordered_bits(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

struct RouteParams {
  int E, k, n_group, topk_group, gating, norm;
  float scale;
  float fix_err;
  int pair_cap;
  int64_t T;
};

// k-th best selection value when only the groups in `groups` compete (others count as 0.0, as in the
// selection itself); -inf when fewer than k experts exist.
template <int P>
__device__ __forceinline__ float kth_best_value(const float (&c0)[P], uint32_t groups, bool grouped, int gsz,
                                                int E, int k, int lane) {
  uint32_t taken = 0, best = 0;
  for (int r = 0; r < k; ++r) {
    uint32_t bkey = 0u;
    int bslot = 0;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      const int e = lane * P + i;
      const float v = (!grouped || ((groups >> (e / gsz)) & 1u)) ? c0[i] : 0.0f;
      const uint32_t key = (e < E && !((taken >> i) & 1u)) ? ordered_bits(v) : 0u;
      if (key > bkey) { bkey = key; bslot = i; }
    }
    best = __reduce_max_sync(0xFFFFFFFFu, bkey);
    if (best == 0u) return __int_as_float(0xff800000);
    const uint32_t e_win = __reduce_min_sync(0xFFFFFFFFu, bkey == best ? static_cast<uint32_t>(lane * P + bslot) : 0xFFFFFFFFu);
    if (lane == static_cast<int>(e_win) / P) taken |= 1u << bslot;
  }
  return from_ordered_bits(best);
}

template <int P>
__device__ __forceinline__ void route_token(const float* __restrict__ logits, const float* __restrict__ bias,
                                            int64_t t, const RouteParams& rp, int32_t* __restrict__ out_idx,
                                            float* __restrict__ out_w, int32_t* __restrict__ fix) {
  const int lane = threadIdx.x & 31;
  const int E = rp.E;
  const float NEG_INF = __int_as_float(0xff800000);
  float group_margin = __int_as_float(0x7f800000), group_kept_min = 0.f, group_open_max = NEG_INF;
  float grp_b1 = NEG_INF, grp_b2 = NEG_INF;      // the two best values of this lane's group (groups that are lane runs)
  bool lane_groups = false;
  uint32_t kept_groups = 0;
  float lane_gs = NEG_INF;                       // score of the group this lane reports
  int lane_g = -1;

  float lg[P];   // logits
  float s[P];    // scores (softmax or sigmoid)
  float c[P];    // selection values
  const float* row = logits + t * E;
#pragma unroll
  for (int i = 0; i < P; ++i) {
    int e = lane * P + i;
    lg[i] = e < E ? row[e] : NEG_INF;
  }
  if (rp.gating == MG_GATE_SIGMOID_NOAUX_TC) {
#pragma unroll
    for (int i = 0; i < P; ++i) {
      int e = lane * P + i;
      s[i] = 1.0f / (1.0f + expf(-lg[i]));
      c[i] = e < E ? __fadd_rn(s[i], bias[e]) : NEG_INF;
    }
  } else {
    float m = NEG_INF;
#pragma unroll
    for (int i = 0; i < P; ++i) m = fmaxf(m, lg[i]);
    m = warp_max_f(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      s[i] = (lane * P + i) < E ? expf(lg[i] - m) : 0.f;
      sum = __fadd_rn(sum, s[i]);
    }
    sum = warp_sum_f(sum);
#pragma unroll
    for (int i = 0; i < P; ++i) {
      s[i] = __fdiv_rn(s[i], sum);
      c[i] = (lane * P + i) < E ? s[i] : NEG_INF;
    }
  }

  float c0[P];   // selection values before the group mask
#pragma unroll
  for (int i = 0; i < P; ++i) c0[i] = c[i];

  // group-limited selection: keep topk_group groups, others compete with value 0.0
  if (rp.gating == MG_GATE_SOFTMAX_GROUP_MAX || rp.gating == MG_GATE_SIGMOID_NOAUX_TC) {
    const int G = rp.n_group, gsz = E / G;
    float my_gs = NEG_INF;   // score of the group this lane reports (one lane per group)
    int my_g = -1;
    const int lanes_per_group = gsz / P;
    if (gsz % P == 0 && (lanes_per_group & (lanes_per_group - 1)) == 0 && lanes_per_group <= 32) {
      // a lane's experts all lie in one group and a group is a power-of-two run of lanes:
      // all groups reduce at once with xor shuffles inside the run
      float b1 = NEG_INF, b2 = NEG_INF;
#pragma unroll
      for (int i = 0; i < P; ++i) {
        float v = c[i];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
      }
      for (int o = lanes_per_group >> 1; o > 0; o >>= 1) {
        float o1 = __shfl_xor_sync(0xFFFFFFFFu, b1, o);
        float o2 = __shfl_xor_sync(0xFFFFFFFFu, b2, o);
        float hi = fmaxf(b1, o1), lo = fminf(b1, o1);
        b2 = fmaxf(lo, fmaxf(b2, o2));
        b1 = hi;
      }
      grp_b1 = b1; grp_b2 = b2;
      lane_groups = true;
      const int g = (lane * P) / gsz;
      if (lane * P < E && (lane & (lanes_per_group - 1)) == 0) {
        my_g = g;
        my_gs = rp.gating == MG_GATE_SIGMOID_NOAUX_TC ? __fadd_rn(b1, b2) : b1;
      }
    } else {
      for (int g = 0; g < G; ++g) {
        float b1 = NEG_INF, b2 = NEG_INF;  // two largest values of group g seen by this lane
#pragma unroll
        for (int i = 0; i < P; ++i) {
          int e = lane * P + i;
          if (e < E && e / gsz == g) {
            float v = c[i];
            if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          float o1 = __shfl_xor_sync(0xFFFFFFFFu, b1, o);
          float o2 = __shfl_xor_sync(0xFFFFFFFFu, b2, o);
          float hi = fmaxf(b1, o1), lo = fminf(b1, o1);
          b2 = fmaxf(lo, fmaxf(b2, o2));
          b1 = hi;
        }
        if (lane == g) {
          my_g = g;
          my_gs = rp.gating == MG_GATE_SIGMOID_NOAUX_TC ? __fadd_rn(b1, b2) : b1;
        }
      }
    }
    // topk_group rounds: best score first, equal scores -> lower group id
    uint32_t gmask = 0;
    const uint32_t gkey = ordered_bits(my_gs);
    for (int r = 0; r < rp.topk_group; ++r) {
      const bool open = my_g >= 0 && !((gmask >> my_g) & 1u);
      const uint32_t best = __reduce_max_sync(0xFFFFFFFFu, open ? gkey : 0u);
      const uint32_t win = __reduce_min_sync(0xFFFFFFFFu, (open && gkey == best) ? static_cast<uint32_t>(my_g) : 0xFFFFFFFFu);
      gmask |= 1u << win;
    }
    if (fix != nullptr) {
      const bool kept = my_g >= 0 && ((gmask >> my_g) & 1u);
      group_kept_min = -warp_max_f(kept ? -my_gs : NEG_INF);
      group_open_max = warp_max_f(my_g >= 0 && !kept ? my_gs : NEG_INF);
      group_margin = group_kept_min - group_open_max;
      kept_groups = gmask;
      lane_gs = my_gs;
      lane_g = my_g;
    }
#pragma unroll
    for (int i = 0; i < P; ++i) {
      int e = lane * P + i;
      if (e < E && !((gmask >> (e / gsz)) & 1u)) c[i] = 0.0f;
    }
  }

  // k rounds of warp arg-max: score descending, equal scores -> lower expert id
  uint32_t taken = 0;
  int my_idx = 0, last_owner = 0;
  float my_w = 0.f, last_c = 0.f;
  for (int r = 0; r < rp.k; ++r) {
    uint32_t bkey = 0u;
    int bslot = 0;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      const uint32_t key = ((lane * P + i) < E && !((taken >> i) & 1u)) ? ordered_bits(c[i]) : 0u;
      if (key > bkey) { bkey = key; bslot = i; }          // strict: the lowest index among equals stays
    }
    const uint32_t best = __reduce_max_sync(0xFFFFFFFFu, bkey);
    const uint32_t e_win = __reduce_min_sync(0xFFFFFFFFu, (bkey == best && bkey != 0u) ? static_cast<uint32_t>(lane * P + bslot) : 0xFFFFFFFFu);
    const int owner = static_cast<int>(e_win) / P;
    float wv = 0.f;
    if (lane == owner) {
      taken |= 1u << bslot;
#pragma unroll
      for (int i = 0; i < P; ++i)
        if (i == bslot) { wv = rp.gating == MG_GATE_SIGMOID_NOAUX_TC ? s[i] : c[i]; last_c = c[i]; }
    }
    wv = __shfl_sync(0xFFFFFFFFu, wv, owner);
    last_owner = owner;
    if (lane == r) { my_idx = static_cast<int>(e_win); my_w = wv; }
  }
  if (fix != nullptr) {
    last_c = __shfl_sync(0xFFFFFFFFu, last_c, last_owner);
    float next_c = NEG_INF, amax = 0.f;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      if ((lane * P + i) < E) {
        amax = fmaxf(amax, fabsf(lg[i]));
        if (!((taken >> i) & 1u)) next_c = fmaxf(next_c, c[i]);
      }
    }
    next_c = warp_max_f(next_c);
    amax = warp_max_f(amax);
    const float dl = rp.fix_err * fmaxf(1.0f, amax);
    const bool sig = rp.gating == MG_GATE_SIGMOID_NOAUX_TC;
    const bool grouped = sig || rp.gating == MG_GATE_SOFTMAX_GROUP_MAX;
    const int gsz = grouped ? E / rp.n_group : E;
    const float dg = sig ? 0.5f * dl : 2.0f * fabsf(group_kept_min) * dl;
    const bool g_close = grouped && group_margin < 2.0f * dg;
    const bool e_close = (last_c - next_c) < 2.0f * (sig ? 0.25f * dl : 2.0f * fabsf(last_c) * dl);
    if (g_close || e_close) {                       // the same for the whole warp
      bool whole_row = g_close && !lane_groups;
      if (!whole_row) {
        uint32_t in_play = 0;                        // bit i: this lane's expert i
        if (!g_close) {
          const float de = sig ? 0.25f * dl : 2.0f * fabsf(last_c) * dl;
          const float lo = next_c - 2.0f * de, hi = last_c + 2.0f * de;
#pragma unroll
          for (int i = 0; i < P; ++i) {
            const int e = lane * P + i;
            const bool open = e < E && (!grouped || ((kept_groups >> (e / gsz)) & 1u));
            if (open && c0[i] >= lo && c0[i] <= hi) in_play |= 1u << i;
          }
        } else {
          const bool near = lane_g >= 0 && lane_gs >= group_open_max - 2.0f * dg && lane_gs <= group_kept_min + 2.0f * dg;
          const uint32_t play_groups = __reduce_or_sync(0xFFFFFFFFu, near ? 1u << lane_g : 0u);
          const uint32_t u_max = kept_groups | play_groups, u_min = kept_groups & ~play_groups;
          const float v_hi = kth_best_value<P>(c0, u_max, true, gsz, E, rp.k, lane);
          const float v_lo = kth_best_value<P>(c0, u_min, true, gsz, E, rp.k, lane);
          const float de = sig ? 0.25f * dl : 2.0f * fmaxf(fabsf(v_hi), fabsf(last_c)) * dl;
          const float de_g = sig ? 0.25f * dl : 2.0f * fabsf(grp_b1) * dl;
          const float contender = (sig ? grp_b2 : grp_b1) - 2.0f * de_g;
#pragma unroll
          for (int i = 0; i < P; ++i) {
            const int e = lane * P + i;
            if (e >= E) continue;
            const int g = e / gsz;
            if (!((u_max >> g) & 1u)) continue;
            const bool band = c0[i] >= v_lo - 2.0f * de && c0[i] <= v_hi + 2.0f * de;
            const bool scores = ((play_groups >> g) & 1u) && c0[i] >= contender;
            if (band || scores) in_play |= 1u << i;
          }
        }
        bool full = false;
        int32_t* pairs = fix + 4 + 2 * rp.T;
#pragma unroll
        for (int i = 0; i < P; ++i) {
          if ((in_play >> i) & 1u) {
            const int pos = atomicAdd(fix + 2, 1);
            if (pos < rp.pair_cap) {
              pairs[2 * pos] = static_cast<int32_t>(t);
              pairs[2 * pos + 1] = lane * P + i;
            } else {
              full = true;
            }
          }
        }
        whole_row = __any_sync(0xFFFFFFFFu, full);
      }
      if (lane == 0) {
        fix[4 + atomicAdd(fix, 1)] = static_cast<int32_t>(t);
        if (whole_row) fix[4 + rp.T + atomicAdd(fix + 1, 1)] = static_cast<int32_t>(t);
      }
    }
  }

  // normalise / scale
  float denom = 0.f;
  for (int r = 0; r < rp.k; ++r) denom = __fadd_rn(denom, __shfl_sync(0xFFFFFFFFu, my_w, r));
  if (rp.gating == MG_GATE_SOFTMAX_TOPK_RENORM) {
    my_w = __fdiv_rn(my_w, denom);
  } else if (rp.gating == MG_GATE_SIGMOID_NOAUX_TC) {
    if (rp.k > 1 && rp.norm) my_w = __fdiv_rn(my_w, __fadd_rn(denom, 1e-20f));
    my_w = __fmul_rn(my_w, rp.scale);
  } else {
    if (rp.k > 1 && rp.norm) my_w = __fdiv_rn(my_w, __fadd_rn(denom, 1e-20f));
    else my_w = __fmul_rn(my_w, rp.scale);
  }
  if (lane < rp.k) {
    out_idx[t * rp.k + lane] = my_idx;
    out_w[t * rp.k + lane] = my_w;
  }
}

template <int P>
__global__ void __launch_bounds__(256) route_topk_kernel(const float* __restrict__ logits,
                                                         const float* __restrict__ bias,
                                                         int64_t T, RouteParams rp,
                                                         int32_t* __restrict__ out_idx,
                                                         float* __restrict__ out_w, int32_t* __restrict__ fix) {
  const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  route_token<P>(logits, bias, t, rp, out_idx, out_w, fix);
}

// The close tokens once more, now that their in-play logits are exact.
template <int P>
__global__ void __launch_bounds__(256) route_topk_list_kernel(const float* __restrict__ logits,
                                                              const float* __restrict__ bias, RouteParams rp,
                                                              int32_t* __restrict__ out_idx, float* __restrict__ out_w,
                                                              const int32_t* __restrict__ fix) {
  const int n = fix[0];
  const int warps = gridDim.x * (blockDim.x >> 5);
  for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += warps)
    route_token<P>(logits, bias, fix[4 + i], rp, out_idx, out_w, nullptr);
}

// Whole logits rows of the listed tokens, recomputed as the rounded exact sum: the products of two bf16
// values are exact in fp64 and the 64-bit accumulation leaves an error far below half an fp32 ulp, so
// the stored value is the correctly rounded logit whatever the summation order.  A block takes a batch
// of kFixTokens tokens (their x rows in shared memory) and a slice of kFixSlice experts; each warp holds
// a kFixWarpExperts x kFixTokens tile of fp64 sums, lanes across H, so that an operand is widened to
// fp64 once per 4 or 8 multiply-adds.
constexpr int kFixTokens = 4;
constexpr int kFixWarpExperts = 8;
constexpr int kFixSlice = 8 * kFixWarpExperts;     // 8 warps per block
__device__ __forceinline__ double bf16_lo_f64(uint32_t pair) { return static_cast<double>(__uint_as_float(pair << 16)); }
__device__ __forceinline__ double bf16_hi_f64(uint32_t pair) { return static_cast<double>(__uint_as_float(pair & 0xffff0000u)); }
__global__ void __launch_bounds__(256) route_fix_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ gate_w, int H, int E,
                                                               const int32_t* __restrict__ fix, int64_t T,
                                                               float* __restrict__ logits) {
  extern __shared__ __align__(16) unsigned char fix_smem[];
  uint4* xs = reinterpret_cast<uint4*>(fix_smem);            // [kFixTokens][H/8]
  const int n = fix[1];
  const int32_t* list = fix + 4 + T;
  const int vecs = H >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_slices = (E + kFixSlice - 1) / kFixSlice;
  const int n_batches = (n + kFixTokens - 1) / kFixTokens;
  int loaded = -1;
  for (int item = blockIdx.x; item < n_batches * n_slices; item += gridDim.x) {
    const int b = item / n_slices, slice = item - b * n_slices;
    int tok[kFixTokens];
#pragma unroll
    for (int j = 0; j < kFixTokens; ++j) {
      const int i = b * kFixTokens + j;
      tok[j] = list[i < n ? i : n - 1];                      // a short batch repeats its last token
    }
    if (b != loaded) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < kFixTokens; ++j) {
        const uint4* row = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(tok[j]) * H);
        for (int v = threadIdx.x; v < vecs; v += blockDim.x) xs[j * vecs + v] = row[v];
      }
      __syncthreads();
      loaded = b;
    }
    const int e0 = slice * kFixSlice + warp * kFixWarpExperts;
    if (e0 >= E) continue;                                    // warp-uniform; no barrier below in this item
    const uint4* wrow[kFixWarpExperts];
#pragma unroll
    for (int i = 0; i < kFixWarpExperts; ++i) {
      const int e = e0 + i < E ? e0 + i : E - 1;
      wrow[i] = reinterpret_cast<const uint4*>(gate_w + static_cast<int64_t>(e) * H);
    }
    double acc[kFixWarpExperts][kFixTokens];
#pragma unroll
    for (int i = 0; i < kFixWarpExperts; ++i)
#pragma unroll
      for (int j = 0; j < kFixTokens; ++j) acc[i][j] = 0.0;
    for (int v = lane; v < vecs; v += 32) {
      uint4 wv[kFixWarpExperts], xv[kFixTokens];
#pragma unroll
      for (int i = 0; i < kFixWarpExperts; ++i) wv[i] = wrow[i][v];
#pragma unroll
      for (int j = 0; j < kFixTokens; ++j) xv[j] = xs[j * vecs + v];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        double xl[kFixTokens], xh[kFixTokens];
#pragma unroll
        for (int j = 0; j < kFixTokens; ++j) {
          const uint32_t pair = q == 0 ? xv[j].x : q == 1 ? xv[j].y : q == 2 ? xv[j].z : xv[j].w;
          xl[j] = bf16_lo_f64(pair);
          xh[j] = bf16_hi_f64(pair);
        }
#pragma unroll
        for (int i = 0; i < kFixWarpExperts; ++i) {
          const uint32_t pair = q == 0 ? wv[i].x : q == 1 ? wv[i].y : q == 2 ? wv[i].z : wv[i].w;
          const double wl = bf16_lo_f64(pair), wh = bf16_hi_f64(pair);
#pragma unroll
          for (int j = 0; j < kFixTokens; ++j) {
            acc[i][j] = fma(xl[j], wl, acc[i][j]);
            acc[i][j] = fma(xh[j], wh, acc[i][j]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kFixWarpExperts; ++i) {
#pragma unroll
      for (int j = 0; j < kFixTokens; ++j) {
        double a = acc[i][j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
        if (lane == 0 && e0 + i < E && b * kFixTokens + j < n)
          logits[static_cast<int64_t>(tok[j]) * E + e0 + i] = static_cast<float>(a);
      }
    }
  }
}

// Single logits, the same way: one warp per (token, expert) pair, lanes across H.
__global__ void __launch_bounds__(256) route_fix_pairs_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const __nv_bfloat16* __restrict__ gate_w, int H, int E,
                                                              const int32_t* __restrict__ fix, int64_t T, int pair_cap,
                                                              float* __restrict__ logits) {
  const int n = fix[2] < pair_cap ? fix[2] : pair_cap;
  const int32_t* pairs = fix + 4 + 2 * T;
  const int vecs = H >> 3;
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  for (int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < n; i += warps) {
    const int64_t t = pairs[2 * i];
    const int e = pairs[2 * i + 1];
    const uint4* xr = reinterpret_cast<const uint4*>(x + t * H);
    const uint4* wr = reinterpret_cast<const uint4*>(gate_w + static_cast<int64_t>(e) * H);
    double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
    for (int v = lane; v < vecs; v += 32) {
      const uint4 xv = xr[v], wv = wr[v];
      a0 = fma(bf16_lo_f64(xv.x), bf16_lo_f64(wv.x), a0);
      a1 = fma(bf16_hi_f64(xv.x), bf16_hi_f64(wv.x), a1);
      a2 = fma(bf16_lo_f64(xv.y), bf16_lo_f64(wv.y), a2);
      a3 = fma(bf16_hi_f64(xv.y), bf16_hi_f64(wv.y), a3);
      a0 = fma(bf16_lo_f64(xv.z), bf16_lo_f64(wv.z), a0);
      a1 = fma(bf16_hi_f64(xv.z), bf16_hi_f64(wv.z), a1);
      a2 = fma(bf16_lo_f64(xv.w), bf16_lo_f64(wv.w), a2);
      a3 = fma(bf16_hi_f64(xv.w), bf16_hi_f64(wv.w), a3);
    }
    double a = (a0 + a1) + (a2 + a3);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
    if (lane == 0) logits[t * E + e] = static_cast<float>(a);
  }
}

static int route_P(int n_experts) {
  const int P = (n_experts + 31) / 32;
  return P <= 1 ? 1 : P <= 2 ? 2 : P <= 4 ? 4 : P <= 5 ? 5 : P <= 8 ? 8 : P <= 16 ? 16 : 0;
}

static int64_t route_pair_cap(int64_t T) { return 8 * T + 64; }
size_t route_fix_bytes(int64_t T) { return static_cast<size_t>(4 + 2 * T + 2 * route_pair_cap(T)) * 4; }

// Routing from the tensor-core router product with the near-tie fix-up: routes every token, lists the
// close tokens and the logits that decide them, recomputes those exactly (single logits, or whole rows
// where the pairs could not be listed) and routes the close tokens again.  The selection equals that of
// correctly rounded fp32 logits.  fix: route_fix_bytes(T) of scratch, laid out as described above.
int launch_route_topk_fixup(const Handle* h, const void* x, const void* gate_w, float* logits, const float* bias,
                            int64_t T, int32_t* idx, float* w, int32_t* fix, cudaStream_t st, int* launches) {
  if (T == 0) return MG_OK;
  const mg_layer_desc& d = h->d;
  if (T > (0x7fffffff - 64) / 8) { set_error("token count beyond the fix-up list's index range"); return MG_ERR_SHAPE; }
  RouteParams rp{d.n_experts, d.top_k, d.n_group, d.topk_group, d.gating, d.norm_topk_prob,
                 d.routed_scale, route_fix_err(d.hidden), static_cast<int>(route_pair_cap(T)), T};
  const int P = route_P(d.n_experts);
  if (P == 0) { set_error("n_experts %d > 512 unsupported by the top-k kernel", d.n_experts); return MG_ERR_SHAPE; }
  MG_CUDA(cudaMemsetAsync(fix, 0, 16, st));
  const int warps = 8;
  dim3 grid(static_cast<unsigned>((T + warps - 1) / warps)), block(warps * 32);
  const int sms = h->sm_count > 0 ? h->sm_count : 148;
  const size_t smem = static_cast<size_t>(kFixTokens) * d.hidden * 2;
  static bool done[64];
  if (smem > 48 * 1024 && !(h->device >= 0 && h->device < 64 && done[h->device])) {
    MG_CUDA(cudaFuncSetAttribute(route_fix_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)));
    if (h->device >= 0 && h->device < 64) done[h->device] = true;
  }
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wb = static_cast<const __nv_bfloat16*>(gate_w);
#define MG_ROUTE_CASE(PP)                                                                              \
  case PP:                                                                                             \
    route_topk_kernel<PP><<<grid, block, 0, st>>>(logits, bias, T, rp, idx, w, fix);                   \
    route_fix_logits_kernel<<<sms, 256, smem, st>>>(xb, wb, d.hidden, d.n_experts, fix, T, logits);    \
    route_fix_pairs_kernel<<<4 * sms, 256, 0, st>>>(xb, wb, d.hidden, d.n_experts, fix, T, rp.pair_cap, logits); \
    route_topk_list_kernel<PP><<<sms, block, 0, st>>>(logits, bias, rp, idx, w, fix);                  \
    break
  switch (P) {
    MG_ROUTE_CASE(1); MG_ROUTE_CASE(2); MG_ROUTE_CASE(4); MG_ROUTE_CASE(5); MG_ROUTE_CASE(8); MG_ROUTE_CASE(16);
  }
#undef MG_ROUTE_CASE
  MG_CUDA(cudaGetLastError());
  if (launches) *launches += 4;
  return MG_OK;
}

int launch_route_topk(const Handle* h, const float* logits, const float* bias, int64_t T,
                      int32_t* idx, float* w, cudaStream_t st) {
  if (T == 0) return MG_OK;
  const mg_layer_desc& d = h->d;
  RouteParams rp{d.n_experts, d.top_k, d.n_group, d.topk_group, d.gating, d.norm_topk_prob,
                 d.routed_scale, 0.f, 0, T};
  const int warps = 8;
  dim3 grid(static_cast<unsigned>((T + warps - 1) / warps)), block(warps * 32);
  const int P = (d.n_experts + 31) / 32;
#define MG_ROUTE_CASE(PP)                                                             \
  route_topk_kernel<PP><<<grid, block, 0, st>>>(logits, bias, T, rp, idx, w, nullptr)
  if (P <= 1) MG_ROUTE_CASE(1);
  else if (P <= 2) MG_ROUTE_CASE(2);
  else if (P <= 4) MG_ROUTE_CASE(4);
  else if (P <= 5) MG_ROUTE_CASE(5);
  else if (P <= 8) MG_ROUTE_CASE(8);
  else if (P <= 16) MG_ROUTE_CASE(16);
  else { set_error("n_experts %d > 512 unsupported by the top-k kernel", d.n_experts); return MG_ERR_SHAPE; }
#undef MG_ROUTE_CASE
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

// ---------------------------------------------------------------------------------------
// permute plan
// ---------------------------------------------------------------------------------------
constexpr int kPlanTokens = 256;  // tokens per block (one per thread)

__global__ void __launch_bounds__(kPlanTokens) plan_count_kernel(const int32_t* __restrict__ idx,
                                                                 int64_t T, int k, int lo, int n,
                                                                 int32_t* __restrict__ block_counts) {
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < n; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  int64_t t = static_cast<int64_t>(blockIdx.x) * kPlanTokens + threadIdx.x;
  if (t < T) {
    for (int j = 0; j < k; ++j) {
      int e = idx[t * k + j] - lo;
      if (e >= 0 && e < n) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n; e += blockDim.x)
    block_counts[static_cast<int64_t>(blockIdx.x) * n + e] = hist[e];
}

// one warp per expert: turns block_counts[:, e] into an exclusive prefix over the blocks (32 blocks
// per step, warp scan) and writes the expert's total
__global__ void __launch_bounds__(256) plan_scan_kernel(int32_t* __restrict__ block_counts, int nblk, int n,
                                                        int32_t* __restrict__ counts) {
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= n) return;
  int32_t run = 0;
  for (int b0 = 0; b0 < nblk; b0 += 32) {
    const int b = b0 + lane;
    const int32_t c = b < nblk ? block_counts[static_cast<int64_t>(b) * n + e] : 0;
    int32_t inc = c;                                   // inclusive scan over the 32 lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += v;
    }
    if (b < nblk) block_counts[static_cast<int64_t>(b) * n + e] = run + inc - c;
    run += __shfl_sync(0xFFFFFFFFu, inc, 31);
  }
  if (lane == 0) counts[e] = run;
}

// one block: offsets = exclusive scan of counts, pad_offsets = the same over counts rounded up to
// whole 128-row tiles (n <= kMaxExperts = 512 = one value per thread)
__global__ void __launch_bounds__(kMaxExperts) plan_offsets_kernel(const int32_t* __restrict__ counts, int n,
                                                                   int32_t* __restrict__ offsets,
                                                                   int32_t* __restrict__ pad_offsets) {
  __shared__ int32_t warp_o[kMaxExperts / 32], warp_p[kMaxExperts / 32];
  const int e = threadIdx.x, lane = e & 31, w = e >> 5;
  const int32_t c = e < n ? counts[e] : 0;
  const int32_t cp = (c + kTileM - 1) / kTileM * kTileM;
  int32_t io = c, ip = cp;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int32_t vo = __shfl_up_sync(0xFFFFFFFFu, io, o), vp = __shfl_up_sync(0xFFFFFFFFu, ip, o);
    if (lane >= o) { io += vo; ip += vp; }
  }
  if (lane == 31) { warp_o[w] = io; warp_p[w] = ip; }
  __syncthreads();
  int32_t bo = 0, bp = 0;
  for (int i = 0; i < w; ++i) { bo += warp_o[i]; bp += warp_p[i]; }
  if (e < n) {
    offsets[e] = bo + io - c;
    pad_offsets[e] = bp + ip - cp;
    if (e == n - 1) { offsets[n] = bo + io; pad_offsets[n] = bp + ip; }
  }
}

__global__ void __launch_bounds__(kPlanTokens) plan_place_kernel(const int32_t* __restrict__ idx,
                                                                 int64_t T, int k, int lo, int n,
                                                                 const int32_t* __restrict__ block_base,
                                                                 const int32_t* __restrict__ pad_offsets,
                                                                 int32_t* __restrict__ dst_row) {
  extern __shared__ int32_t sm[];
  constexpr int W = kPlanTokens / 32;
  uint32_t* bm = reinterpret_cast<uint32_t*>(sm);  // [W][n] lanes of warp w that picked e
  int32_t* wbase = sm + W * n;                     // [W][n] first row for warp w, expert e
  for (int i = threadIdx.x; i < W * n; i += blockDim.x) bm[i] = 0u;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t t = static_cast<int64_t>(blockIdx.x) * kPlanTokens + threadIdx.x;
  if (t < T) {
    for (int j = 0; j < k; ++j) {
      int e = idx[t * k + j] - lo;
      if (e >= 0 && e < n) atomicOr(&bm[warp * n + e], 1u << lane);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    int32_t run = pad_offsets[e] + block_base[static_cast<int64_t>(blockIdx.x) * n + e];
    for (int w = 0; w < W; ++w) {
      wbase[w * n + e] = run;
      run += __popc(bm[w * n + e]);
    }
  }
  __syncthreads();
  if (t < T) {
    const uint32_t lt = (1u << lane) - 1u;
    for (int j = 0; j < k; ++j) {
      int e = idx[t * k + j] - lo;
      int32_t dst = -1;
      if (e >= 0 && e < n) dst = wbase[warp * n + e] + __popc(bm[warp * n + e] & lt);
      dst_row[t * k + j] = dst;
    }
  }
}

size_t plan_ws_bytes(const Handle* h, int64_t T) {
  int64_t nblk = (T + kPlanTokens - 1) / kPlanTokens;
  if (nblk < 1) nblk = 1;
  // per-block counts, then 2*(E+1) ints used by the expert-parallel entry points
  return (static_cast<size_t>(nblk) * h->d.n_experts + 2 * (h->d.n_experts + 1)) * sizeof(int32_t);
}

int launch_permute_plan(const Handle* h, const int32_t* idx, int64_t T, int expert_lo, int n_exp,
                        int32_t* counts, int32_t* offsets, int32_t* pad_offsets, int32_t* dst_row,
                        void* ws, cudaStream_t st, int* launches) {
  const int k = h->d.top_k;
  int nblk = static_cast<int>((T + kPlanTokens - 1) / kPlanTokens);
  int32_t* bc = static_cast<int32_t*>(ws);
  if (nblk > 0) {
    plan_count_kernel<<<nblk, kPlanTokens, n_exp * sizeof(int32_t), st>>>(idx, T, k, expert_lo,
                                                                          n_exp, bc);
    MG_CUDA(cudaGetLastError());
  }
  plan_scan_kernel<<<(n_exp + 7) / 8, 256, 0, st>>>(bc, nblk, n_exp, counts);
  MG_CUDA(cudaGetLastError());
  plan_offsets_kernel<<<1, kMaxExperts, 0, st>>>(counts, n_exp, offsets, pad_offsets);
  MG_CUDA(cudaGetLastError());
  if (nblk > 0) {
    size_t smem = static_cast<size_t>(2) * (kPlanTokens / 32) * n_exp * sizeof(int32_t);
    plan_place_kernel<<<nblk, kPlanTokens, smem, st>>>(idx, T, k, expert_lo, n_exp, bc,
                                                       pad_offsets, dst_row);
    MG_CUDA(cudaGetLastError());
  }
  if (launches) *launches += nblk > 0 ? 4 : 2;
  return MG_OK;
}

// ---------------------------------------------------------------------------------------
// permute plan without any allocation: the scratch lives in the library image
// ---------------------------------------------------------------------------------------
// Per-block expert counts for up to kStaticPlanBlocks * kStaticPlanExperts entries (65536
// tokens at 512 experts; more tokens when there are fewer experts) plus the two small offset
// arrays.  Every GPU that loads this library carries these ~516 KiB until the process exits.
constexpr int kStaticPlanBlocks = 256;
constexpr int kStaticPlanExperts = 512;
constexpr int kStaticPlanInts = kStaticPlanBlocks * kStaticPlanExperts + 2 * (kStaticPlanExperts + 1);
static __device__ __align__(256) int32_t g_plan_scratch[kStaticPlanInts];

// In host code `g_plan_scratch` is only a stand-in for the symbol; the address a kernel can use
// is looked up once per device, with that device current.
static int static_plan_scratch(int device, int32_t** out) {
  static std::mutex mu;
  static int32_t* addr[64] = {nullptr};
  MG_REQUIRE(device >= 0 && device < 64, MG_ERR_LIMIT, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[device] == nullptr) {
    void* p = nullptr;
    MG_CUDA(cudaGetSymbolAddress(&p, g_plan_scratch));
    addr[device] = static_cast<int32_t*>(p);
  }
  *out = addr[device];
  return MG_OK;
}

int launch_permute_plan_static(const Handle* h, const int32_t* idx, int64_t T, int expert_lo, int n_exp,
                               int32_t* counts, int32_t* offsets, int32_t* pad_offsets, int32_t* dst_row,
                               cudaStream_t st) {
  const int64_t nblk = (T + kPlanTokens - 1) / kPlanTokens;
  const int64_t need = nblk * h->d.n_experts + 2 * (h->d.n_experts + 1);
  MG_REQUIRE(need <= kStaticPlanInts, MG_ERR_LIMIT,
             "mg_permute_plan_static: %lld tokens x %d experts need %lld scratch words, the built-in scratch holds "
             "%d (at most %d tokens at %d experts); use mg_permute_plan with caller-provided scratch",
             static_cast<long long>(T), h->d.n_experts, static_cast<long long>(need), kStaticPlanInts,
             kStaticPlanBlocks * kPlanTokens, kStaticPlanExperts);
  int dev = -1;
  MG_CUDA(cudaGetDevice(&dev));
  MG_REQUIRE(dev == h->device, MG_ERR_STATE, "current device %d is not the handle's device %d", dev, h->device);
  int32_t* scratch = nullptr;
  int rc = static_plan_scratch(dev, &scratch);
  if (rc != MG_OK) return rc;
  // Nothing here needs a cleared scratch: the count kernel writes every per-block entry the scan
  // and placement kernels read, so whatever the previous call left behind is overwritten first.
  return launch_permute_plan(h, idx, T, expert_lo, n_exp, counts, offsets, pad_offsets, dst_row, scratch, st,
                             nullptr);
}

// ---------------------------------------------------------------------------------------
// row scatter: one warp per token, x row read once, written to each destination row
// ---------------------------------------------------------------------------------------
// PEER: dst_row packs (destination rank << kPeerShift | row) and rows are written to that
// rank's buffer through its peer mapping (plain stores over NVLink).
// DEDUP: when several picks of a token go to the same rank, only the first one's row travels; for
// the others the kernel writes, into the destination rank's duplicate table at the pick's row, the
// row of that first pick, and the owner copies the row locally (fill_duplicate_rows_kernel).
// BACK: every pick also leaves, in the destination rank's return table at the pick's row, where the
// expert's output for that row has to go: source rank << kPeerShift | (token * k + slot).
template <bool PEER, bool DEDUP, bool BACK>
__global__ void __launch_bounds__(256) permute_rows_kernel(const uint4* __restrict__ x,
                                                           const int32_t* __restrict__ dst_row,
                                                           int64_t T, int k, int vec_per_row,
                                                           PeerPtrs bufs, PeerPtrs dups, PeerPtrs backs, int my_rank,
                                                           Guard guard) {
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  int32_t my_dst = lane < k ? dst_row[t * k + lane] : -1;
  if (my_dst >= 0 && !MG_GUARD((PEER ? (my_dst & kPeerRowMask) : my_dst) < guard.rows_bound &&
                               (!PEER || (my_dst >> kPeerShift) < guard.n_peers), guard, 103))
    my_dst = -1;
  if (BACK && my_dst >= 0)
    static_cast<int32_t*>(backs.p[my_dst >> kPeerShift])[my_dst & kPeerRowMask] =
        (my_rank << kPeerShift) | static_cast<int32_t>(t * k + lane);
  uint32_t skip = 0;                           // bit j: pick j's row is copied on its owner
  if (DEDUP) {
    int my_first = -1;                         // earliest pick of this token with my destination rank
    for (int j = 0; j < k; ++j) {
      const int32_t d = __shfl_sync(0xFFFFFFFFu, my_dst, j);
      if (my_first < 0 && j < lane && d >= 0 && my_dst >= 0 && (d >> kPeerShift) == (my_dst >> kPeerShift))
        my_first = j;
    }
    const int32_t first_dst = __shfl_sync(0xFFFFFFFFu, my_dst, my_first < 0 ? 0 : my_first);
    if (my_first >= 0)
      static_cast<int32_t*>(dups.p[my_dst >> kPeerShift])[my_dst & kPeerRowMask] = first_dst & kPeerRowMask;
    skip = __ballot_sync(0xFFFFFFFFu, my_first >= 0);
  }
  const uint4* src = x + t * vec_per_row;
  for (int v0 = 0; v0 < vec_per_row; v0 += 128) {
    uint4 val[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int v = v0 + u * 32 + lane;
      if (v < vec_per_row) val[u] = __ldg(src + v);
    }
    for (int j = 0; j < k; ++j) {
      int32_t d = __shfl_sync(0xFFFFFFFFu, my_dst, j);
      if (d < 0 || ((skip >> j) & 1u)) continue;
      uint4* dst = static_cast<uint4*>(PEER ? bufs.p[d >> kPeerShift] : bufs.p[0]) +
                   static_cast<int64_t>(PEER ? (d & kPeerRowMask) : d) * vec_per_row;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int v = v0 + u * 32 + lane;
        if (v < vec_per_row) dst[v] = val[u];
      }
    }
  }
}

// Owner side of the de-duplicated dispatch: row r with dup[r] >= 0 becomes a copy of row dup[r]
// (both in this rank's receive buffer).  Rows without an entry keep the -1 the owner wrote before
// the dispatch.
__global__ void __launch_bounds__(256) fill_duplicate_rows_kernel(uint4* __restrict__ rows,
                                                                  const int32_t* __restrict__ dup,
                                                                  int64_t n_rows, int vec_per_row, Guard guard) {
  const int lane = threadIdx.x & 31;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int32_t s = dup[r];
  if (s < 0) return;
  if (!MG_GUARD(s < n_rows, guard, 105)) return;
  const uint4* src = rows + static_cast<int64_t>(s) * vec_per_row;
  uint4* dst = rows + r * vec_per_row;
  for (int v0 = 0; v0 < vec_per_row; v0 += 128) {
    uint4 val[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int v = v0 + u * 32 + lane;
      if (v < vec_per_row) val[u] = src[v];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int v = v0 + u * 32 + lane;
      if (v < vec_per_row) dst[v] = val[u];
    }
  }
}

int launch_permute_rows(const Handle* h, const void* x, const int32_t* dst_row, int64_t T,
                        void* perm_x, cudaStream_t st) {
  if (T == 0) return MG_OK;
  const int warps = 8;
  dim3 grid(static_cast<unsigned>((T + warps - 1) / warps)), block(warps * 32);
  PeerPtrs bufs{};
  bufs.p[0] = perm_x;
  permute_rows_kernel<false, false, false><<<grid, block, 0, st>>>(static_cast<const uint4*>(x), dst_row, T,
                                                                   h->d.top_k, h->d.hidden / 8, bufs, bufs, bufs, 0,
                                                                   Guard{h->d_status, h->guard_rows, 1});
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

int launch_dispatch_rows(const Handle* h, const void* x, const int32_t* dst, int64_t T,
                         const PeerPtrs& peers, const PeerPtrs* dups, const PeerPtrs* backs, cudaStream_t st) {
  if (T == 0) return MG_OK;
  const int warps = 8;
  dim3 grid(static_cast<unsigned>((T + warps - 1) / warps)), block(warps * 32);
  const uint4* xs = static_cast<const uint4*>(x);
  const int k = h->d.top_k, vpr = h->d.hidden / 8, me = h->d.ep_rank;
  const PeerPtrs& d = dups ? *dups : peers;
  const PeerPtrs& b = backs ? *backs : peers;
  const Guard guard{h->d_status, h->guard_rows, h->d.ep_size};
  if (dups != nullptr && backs != nullptr)
    permute_rows_kernel<true, true, true><<<grid, block, 0, st>>>(xs, dst, T, k, vpr, peers, d, b, me, guard);
  else if (dups != nullptr)
    permute_rows_kernel<true, true, false><<<grid, block, 0, st>>>(xs, dst, T, k, vpr, peers, d, b, me, guard);
  else if (backs != nullptr)
    permute_rows_kernel<true, false, true><<<grid, block, 0, st>>>(xs, dst, T, k, vpr, peers, d, b, me, guard);
  else
    permute_rows_kernel<true, false, false><<<grid, block, 0, st>>>(xs, dst, T, k, vpr, peers, d, b, me, guard);
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

// Owner side of the return: the output rows of local experts [e_lo, e_lo + e_n) go to the ranks their
// tokens came from, each into row (token * k + slot) of that rank's return buffer, as the return table
// says (rows without an entry are padding; rows of this rank's own tokens stay where they are).  Plain 128-bit stores through the peer mappings; a warp per
// row, rows taken in a grid-stride loop because their number is only known on the device.
__global__ void __launch_bounds__(256) return_rows_kernel(const uint4* __restrict__ out_rows,
                                                          const int32_t* __restrict__ back,
                                                          const int32_t* __restrict__ pad, int e_lo, int e_n,
                                                          int vec_per_row, PeerPtrs rets, int my_rank, Guard guard) {
  const int lane = threadIdx.x & 31;
  const int64_t row0 = pad[e_lo], row1 = pad[e_lo + e_n];
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t r = row0 + static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < row1; r += warps) {
    const int32_t b = back[r];
    if (b < 0 || (b >> kPeerShift) == my_rank) continue;     // padding, or a token of this rank: it reads the row in place
    if (!MG_GUARD((b >> kPeerShift) < guard.n_peers, guard, 106)) continue;
    const uint4* src = out_rows + r * vec_per_row;
    uint4* dst = static_cast<uint4*>(rets.p[b >> kPeerShift]) + static_cast<int64_t>(b & kPeerRowMask) * vec_per_row;
    for (int v0 = 0; v0 < vec_per_row; v0 += 128) {
      uint4 val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int v = v0 + u * 32 + lane;
        if (v < vec_per_row) val[u] = src[v];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        int v = v0 + u * 32 + lane;
        if (v < vec_per_row) dst[v] = val[u];
      }
    }
  }
}

int launch_return_rows(const Handle* h, const void* out_rows, const int32_t* back, const int32_t* pad, int e_lo,
                       int e_n, const PeerPtrs& rets, cudaStream_t st) {
  if (e_n <= 0) return MG_OK;
  return_rows_kernel<<<h->sm_count * 2, 256, 0, st>>>(static_cast<const uint4*>(out_rows), back, pad, e_lo, e_n,
                                                      h->d.hidden / 8, rets, h->d.ep_rank,
                                                      Guard{h->d_status, h->guard_rows, h->d.ep_size});
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

int launch_fill_duplicates(const Handle* h, void* rows, const int32_t* dup, int64_t n_rows, cudaStream_t st) {
  if (n_rows == 0) return MG_OK;
  const int warps = 8;
  dim3 grid(static_cast<unsigned>((n_rows + warps - 1) / warps)), block(warps * 32);
  fill_duplicate_rows_kernel<<<grid, block, 0, st>>>(static_cast<uint4*>(rows), dup, n_rows, h->d.hidden / 8,
                                                     Guard{h->d_status, n_rows, h->d.ep_size});
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

// ---------------------------------------------------------------------------------------
// combine: y[t] = sum_j w[t,j] * out_rows[dst_row[t,j]] (+ shared[t])
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ float round_bf16(float f) {
  return __bfloat162float(__float2bfloat16_rn(f));
}

// by_slot = rank + 1 (expert-parallel pushed return): a pick whose owner is another rank lies at row
// (token * k + slot) of this rank's return buffer (bufs.p[owner] all point at it), a pick of this rank's own
// experts is read in place from its out_rows (bufs.p[rank]); 0 = rows as dst_row says.
template <int MODE, bool PEER>
__global__ void __launch_bounds__(256) combine_kernel(PeerPtrs bufs,
                                                      const int32_t* __restrict__ dst_row,
                                                      const int32_t* __restrict__ topk_idx,
                                                      const float* __restrict__ topk_w,
                                                      const uint4* __restrict__ shared,
                                                      const uint4* residual,
                                                      int64_t T, int k, int vec_per_row, int v_chunk,
                                                      uint4* y, int by_slot, const int32_t* __restrict__ delta,
                                                      Guard guard) {
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  int32_t my_dst = -1, my_e = 0x7fffffff;
  float my_w = 0.f;
  if (lane < k) {
    my_dst = dst_row[t * k + lane];
    if (my_dst >= 0 && !MG_GUARD((PEER ? (my_dst & kPeerRowMask) : my_dst) < guard.rows_bound &&
                                 (!PEER || (my_dst >> kPeerShift) < guard.n_peers), guard, 104))
      my_dst = -1;
    if (by_slot > 0 && my_dst >= 0 && (my_dst >> kPeerShift) != by_slot - 1)
      my_dst = (my_dst & ~kPeerRowMask) | static_cast<int32_t>(t * k + lane);
    // mirror of the owners' rows in this rank's own expert-sorted order (bufs.p[0]): row in the owner's
    // buffer + the expert's offset between the two layouts
    if (delta != nullptr && my_dst >= 0) my_dst = (my_dst & kPeerRowMask) + delta[topk_idx[t * k + lane]];
    my_w = topk_w[t * k + lane];
    if (MODE == MG_COMBINE_BF16_SEQ) my_e = topk_idx[t * k + lane];
    if (MODE != MG_COMBINE_FP32) my_w = round_bf16(my_w);
  }
  // BF16_SEQ adds in ascending expert order: rank of my slot among the k picks
  int order_src = lane;  // slot visited at step `lane`
  if (MODE == MG_COMBINE_BF16_SEQ) {
    int rank = 0;
    for (int j = 0; j < k; ++j) {
      int32_t ej = __shfl_sync(0xFFFFFFFFu, my_e, j);
      if (lane < k && (ej < my_e || (ej == my_e && j < lane))) ++rank;
    }
    // step r visits the slot whose rank is r
    order_src = 0;
    for (int j = 0; j < k; ++j) {
      int rj = __shfl_sync(0xFFFFFFFFu, rank, j);
      if (rj == lane) order_src = j;
    }
  }
  // per pick: weight and the address of its row (nullptr = skipped pick), in the order of the adds
  const uint4* base[kMaxTopK];
  float wj[kMaxTopK];
#pragma unroll
  for (int s = 0; s < kMaxTopK; ++s) {
    const int j = (MODE == MG_COMBINE_BF16_SEQ ? __shfl_sync(0xFFFFFFFFu, order_src, s & 31) : s) & 31;
    const int32_t d = __shfl_sync(0xFFFFFFFFu, my_dst, j);
    const float w = __shfl_sync(0xFFFFFFFFu, my_w, j);
    const bool use = s < k && d >= 0;
    wj[s] = use ? w : 0.f;
    const uint4* rows = static_cast<const uint4*>(PEER ? bufs.p[use ? (d >> kPeerShift) : 0] : bufs.p[0]);
    base[s] = use ? rows + static_cast<int64_t>(PEER ? (d & kPeerRowMask) : d) * vec_per_row : nullptr;
  }
  // blockIdx.y: the slice of the row this block's warps cover (small batches are spread over more
  // warps than tokens so that the gather is not one latency chain per token)
  const int v_begin = blockIdx.y * v_chunk;
  const int v_end = min(vec_per_row, v_begin + v_chunk);
  for (int v = v_begin + lane; v < v_end; v += 32) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
    for (int s0 = 0; s0 < kMaxTopK; s0 += 4) {
      if (s0 < k) {
        // four row loads in flight before the first is consumed
        uint4 val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          val[u] = make_uint4(0u, 0u, 0u, 0u);
          // peer rows are written by another GPU during this forward: plain (coherent) loads
          if (base[s0 + u] != nullptr) val[u] = PEER ? base[s0 + u][v] : __ldg(base[s0 + u] + v);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float f[8];
          unpack8(val[u], f);
          const float w = wj[s0 + u];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            // a skipped pick contributes w = 0 and f = 0: adding 0 changes nothing in any mode
            float p = __fmul_rn(f[i], w);
            if (MODE == MG_COMBINE_FP32) acc[i] = __fadd_rn(acc[i], p);
            else if (MODE == MG_COMBINE_BF16_PROD) acc[i] = __fadd_rn(acc[i], round_bf16(p));
            else acc[i] = round_bf16(__fadd_rn(acc[i], round_bf16(p)));
          }
        }
      }
    }
    if (shared != nullptr) {
      float f[8];
      unpack8(__ldg(shared + t * vec_per_row + v), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(round_bf16(acc[i]), f[i]);
    }
    if (residual != nullptr) {
      // decoder-layer glue: the block's bf16 output is added to the bf16 residual stream (y may alias it)
      float f[8];
      unpack8(residual[t * vec_per_row + v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(round_bf16(acc[i]), f[i]);
    }
    y[t * vec_per_row + v] = pack8(acc);
  }
}

template <bool PEER>
static int launch_combine_impl(const Handle* h, const PeerPtrs& bufs, const int32_t* dst_row,
                               const int32_t* idx, const float* w, const void* shared, const void* residual,
                               int64_t T, void* y, cudaStream_t st, int by_slot = 0,
                               const int32_t* delta = nullptr) {
  if (T == 0) return MG_OK;
  const int warps = 8;
  const int k = h->d.top_k, vpr = h->d.hidden / 8;
  // at least ~16 warps per SM: with few tokens every row is cut into slices of whole 32-vector steps
  const int steps = (vpr + 31) / 32;
  int64_t slices = (static_cast<int64_t>(h->sm_count) * 16 + T - 1) / T;
  if (slices > steps) slices = steps;
  if (slices < 1) slices = 1;
  const int v_chunk = static_cast<int>((steps + slices - 1) / slices) * 32;
  dim3 grid(static_cast<unsigned>((T + warps - 1) / warps), static_cast<unsigned>((vpr + v_chunk - 1) / v_chunk));
  dim3 block(warps * 32);
#define MG_COMBINE_CASE(M)                                                                       \
  combine_kernel<M, PEER><<<grid, block, 0, st>>>(bufs, dst_row, idx, w,                          \
                                                  static_cast<const uint4*>(shared),              \
                                                  static_cast<const uint4*>(residual), T, k, vpr, \
                                                  v_chunk, static_cast<uint4*>(y), by_slot, delta,              \
                                                  Guard{h->d_status, h->guard_rows, PEER ? h->d.ep_size : 1})
  switch (h->d.combine_mode) {
    case MG_COMBINE_FP32: MG_COMBINE_CASE(MG_COMBINE_FP32); break;
    case MG_COMBINE_BF16_PROD: MG_COMBINE_CASE(MG_COMBINE_BF16_PROD); break;
    case MG_COMBINE_BF16_SEQ: MG_COMBINE_CASE(MG_COMBINE_BF16_SEQ); break;
    default: set_error("bad combine_mode"); return MG_ERR_CONFIG;
  }
#undef MG_COMBINE_CASE
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

int launch_combine(const Handle* h, const void* out_rows, const int32_t* dst_row,
                   const int32_t* idx, const float* w, const void* shared, const void* residual, int64_t T,
                   void* y, cudaStream_t st) {
  PeerPtrs bufs{};
  bufs.p[0] = const_cast<void*>(out_rows);
  return launch_combine_impl<false>(h, bufs, dst_row, idx, w, shared, residual, T, y, st);
}

int launch_combine_slots(const Handle* h, const void* ret_rows, const void* own_out_rows, const int32_t* dst,
                         const int32_t* idx, const float* w, const void* shared, int64_t T, void* y, cudaStream_t st) {
  PeerPtrs bufs{};
  for (int r = 0; r < h->d.ep_size && r < kMaxPeers; ++r) bufs.p[r] = const_cast<void*>(ret_rows);
  bufs.p[h->d.ep_rank] = const_cast<void*>(own_out_rows);
  return launch_combine_impl<true>(h, bufs, dst, idx, w, shared, nullptr, T, y, st, h->d.ep_rank + 1);
}

int launch_combine_mirror(const Handle* h, const void* mirror, const int32_t* dst, const int32_t* delta,
                          const int32_t* idx, const float* w, const void* shared, int64_t T, void* y, cudaStream_t st) {
  PeerPtrs bufs{};
  for (int r = 0; r < h->d.ep_size && r < kMaxPeers; ++r) bufs.p[r] = const_cast<void*>(mirror);
  return launch_combine_impl<true>(h, bufs, dst, idx, w, shared, nullptr, T, y, st, 0, delta);
}

// delta[e] = (first row of expert e in this rank's own expert-sorted order, unpadded)
//          - (first row of this rank's rows of expert e in the owner's buffer):
// what turns a row number of the owner's layout (ep_layout_kernel) into a row of this rank's mirror.
__global__ void __launch_bounds__(512) ep_mirror_delta_kernel(const int32_t* __restrict__ counts_all, int n_ranks,
                                                              int rank, int E, int e_local,
                                                              int32_t* __restrict__ delta) {
  __shared__ int32_t tot[kMaxExperts];
  __shared__ int32_t before[kMaxExperts];
  __shared__ int32_t pad[kMaxExperts];
  __shared__ int32_t own[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int32_t t = 0, b = 0;
    for (int s = 0; s < n_ranks; ++s) {
      const int32_t c = counts_all[s * E + e];
      if (s < rank) b += c;
      t += c;
    }
    tot[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < n_ranks) {
    const int d = threadIdx.x;
    int32_t p = 0;
    for (int j = 0; j < e_local; ++j) {
      pad[d * e_local + j] = p;
      p += (tot[d * e_local + j] + kTileM - 1) / kTileM * kTileM;
    }
  }
  if (threadIdx.x == 32) {
    int32_t p = 0;
    for (int e = 0; e < E; ++e) {
      own[e] = p;
      p += counts_all[rank * E + e];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) delta[e] = own[e] - pad[e] - before[e];
}

int launch_mirror_delta(const Handle* h, const int32_t* counts_all, int32_t* delta, cudaStream_t st) {
  ep_mirror_delta_kernel<<<1, 512, 0, st>>>(counts_all, h->d.ep_size, h->d.ep_rank, h->d.n_experts, h->e_local, delta);
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

int launch_combine_peers(const Handle* h, const PeerPtrs& peers, const int32_t* dst,
                         const int32_t* idx, const float* w, const void* shared, int64_t T, void* y,
                         cudaStream_t st) {
  return launch_combine_impl<true>(h, peers, dst, idx, w, shared, nullptr, T, y, st);
}

// ---------------------------------------------------------------------------------------
// RMSNorm in front of the block: out = w * bf16(x * rsqrt(mean(x^2) + eps)), one CTA per row.
// fp32 statistics, the normalised value rounded to bf16 before the bf16 weight multiplies it
// (DeepseekV3RMSNorm.forward, modeling_deepseek_v3.py:125-150).  Division and square root are the
// IEEE ones, as on the host.
// ---------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormCached = 4;     // 16-byte vectors of the row a thread keeps in registers

__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const uint4* __restrict__ x,
                                                               const uint4* __restrict__ weight, float eps,
                                                               int vec_per_row, uint4* __restrict__ out) {
  __shared__ float partial[kNormThreads / 32];
  __shared__ float s_scale;
  const int64_t row = blockIdx.x;
  const uint4* src = x + row * vec_per_row;
  uint4 keep[kNormCached];
  float sum = 0.f;
  int n = 0;
  for (int v = threadIdx.x; v < vec_per_row; v += kNormThreads, ++n) {
    const uint4 q = __ldg(src + v);
    if (n < kNormCached) keep[n] = q;
    float f[8];
    unpack8(q, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) sum = fmaf(f[i], f[i], sum);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < kNormThreads / 32; ++i) tot += partial[i];
    s_scale = 1.0f / sqrtf(tot / static_cast<float>(vec_per_row * 8) + eps);
  }
  __syncthreads();
  const float scale = s_scale;
  n = 0;
  for (int v = threadIdx.x; v < vec_per_row; v += kNormThreads, ++n) {
    const uint4 q = n < kNormCached ? keep[n] : __ldg(src + v);
    float f[8], w[8];
    unpack8(q, f);
    unpack8(__ldg(weight + v), w);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __fmul_rn(w[i], round_bf16(__fmul_rn(f[i], scale)));
    out[row * vec_per_row + v] = pack8(f);
  }
}

int launch_rmsnorm(const Handle* h, const void* x, const void* weight, float eps, int64_t T, void* out,
                   cudaStream_t st) {
  if (T == 0) return MG_OK;
  rmsnorm_kernel<<<static_cast<unsigned>(T), kNormThreads, 0, st>>>(
      static_cast<const uint4*>(x), static_cast<const uint4*>(weight), eps, h->d.hidden / 8,
      static_cast<uint4*>(out));
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

// ---------------------------------------------------------------------------------------
// expert-parallel layout: where this rank's rows go in every owner's expert-sorted buffer
// ---------------------------------------------------------------------------------------
// counts_all[s][e]: picks of expert e among rank s's tokens.  Owner of e is e / e_local.  In the
// owner's buffer expert segments start on 128-row boundaries, and inside a segment the rows of
// source rank 0 come first, then rank 1, ... (tokens ascending within a source rank).
//   send_base[e]   = owner << kPeerShift | first row of this rank's rows of expert e
//   recv_counts[j] = rows of local expert j over all sources; recv_pad[j] their padded offsets
// If an owner would need more than cap_rows rows, its send_base entries become negative (the
// scatter and combine kernels skip negative destinations) and the status word is set.
__global__ void __launch_bounds__(512) ep_layout_kernel(const int32_t* __restrict__ counts_all, int n_ranks,
                                                        int rank, int E, int e_local, int cap_rows,
                                                        int32_t* __restrict__ send_base,
                                                        int32_t* __restrict__ recv_counts,
                                                        int32_t* __restrict__ recv_pad,
                                                        int32_t* __restrict__ status) {
  __shared__ int32_t tot[kMaxExperts];
  __shared__ int32_t before[kMaxExperts];
  __shared__ int32_t pad[kMaxExperts];
  __shared__ int32_t over[kMaxPeers];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int32_t t = 0, b = 0;
    for (int s = 0; s < n_ranks; ++s) {
      int32_t c = counts_all[s * E + e];
      if (s < rank) b += c;
      t += c;
    }
    tot[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < n_ranks) {
    const int d = threadIdx.x;
    int32_t p = 0;
    for (int j = 0; j < e_local; ++j) {
      pad[d * e_local + j] = p;
      p += (tot[d * e_local + j] + kTileM - 1) / kTileM * kTileM;
    }
    over[d] = p > cap_rows;
    if (d == rank) recv_pad[e_local] = p > cap_rows ? 0 : p;
    if (p > cap_rows && atomicCAS(status, MG_DEV_OK, MG_DEV_CAPACITY) == MG_DEV_OK) status[1] = d;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = e / e_local;
    send_base[e] = over[d] ? kSkipRow : ((d << kPeerShift) | (pad[e] + before[e]));
    if (d == rank) {
      const int j = e - d * e_local;
      recv_counts[j] = over[d] ? 0 : tot[e];
      recv_pad[j] = over[d] ? 0 : pad[e];
    }
  }
}

int launch_ep_count(const Handle* h, const int32_t* idx, int64_t T, int32_t* counts, void* ws,
                    cudaStream_t st) {
  const int E = h->d.n_experts, k = h->d.top_k;
  int nblk = static_cast<int>((T + kPlanTokens - 1) / kPlanTokens);
  int32_t* bc = static_cast<int32_t*>(ws);
  if (nblk > 0) {
    plan_count_kernel<<<nblk, kPlanTokens, E * sizeof(int32_t), st>>>(idx, T, k, 0, E, bc);
    MG_CUDA(cudaGetLastError());
  }
  plan_scan_kernel<<<(E + 7) / 8, 256, 0, st>>>(bc, nblk, E, counts);
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

int launch_ep_place(const Handle* h, const int32_t* idx, int64_t T, const int32_t* counts_all,
                    int cap_rows, void* ws, int32_t* recv_counts, int32_t* recv_pad, int32_t* dst,
                    cudaStream_t st) {
  const int E = h->d.n_experts, k = h->d.top_k;
  int nblk = static_cast<int>((T + kPlanTokens - 1) / kPlanTokens);
  int32_t* bc = static_cast<int32_t*>(ws);
  int32_t* send_base = bc + static_cast<size_t>(nblk > 0 ? nblk : 1) * E;
  ep_layout_kernel<<<1, 512, 0, st>>>(counts_all, h->d.ep_size, h->d.ep_rank, E, h->e_local, cap_rows,
                                      send_base, recv_counts, recv_pad, h->d_status);
  MG_CUDA(cudaGetLastError());
  if (nblk > 0) {
    size_t smem = static_cast<size_t>(2) * (kPlanTokens / 32) * E * sizeof(int32_t);
    plan_place_kernel<<<nblk, kPlanTokens, smem, st>>>(idx, T, k, 0, E, bc, send_base, dst);
    MG_CUDA(cudaGetLastError());
  }
  return MG_OK;
}

}  // namespace mg
