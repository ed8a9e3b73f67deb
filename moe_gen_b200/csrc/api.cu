// extern "C" surface: handle, sizes, stage entry points and the whole-layer forward.
#include <stdarg.h>
#include <string.h>

#include <new>

#include <nvtx3/nvToolsExt.h>
#include <stdlib.h>

#include "common.cuh"

namespace mg {

static thread_local char g_err[512] = "";

static bool log_calls() {
  static const bool on = [] { const char* v = getenv("MG_LOG"); return v != nullptr && v[0] == '1'; }();
  return on;
}
CallTrace::CallTrace(const char* name, long long n) {
  nvtxRangePushA(name);
  if (log_calls()) fprintf(stderr, "[moegen_b200] %s n=%lld\n", name, n);
}
CallTrace::~CallTrace() { nvtxRangePop(); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return static_cast<int>(e);
}

static Handle* check(mg_handle hh) {
  Handle* h = reinterpret_cast<Handle*>(hh);
  if (h == nullptr || h->magic != kMagic) { set_error("invalid handle"); return nullptr; }
  return h;
}

Handle* check_handle(mg_handle hh) { return check(hh); }

static int64_t padded_rows(const Handle* h, int64_t rows) {
  return ((rows + kTileM - 1) / kTileM + h->e_local) * kTileM;
}

// workspace carving ---------------------------------------------------------------------
enum { WS_LOGITS, WS_IDX, WS_W, WS_COUNTS, WS_OFFSETS, WS_PAD, WS_DST, WS_PERM, WS_H, WS_OUT, WS_PLAN,
       WS_HS, WS_SHARED, WS_DEQ, WS_FIX, WS_N };
struct WsLayout { size_t off[WS_N]; size_t total; };

static size_t dequant_ws(const Handle* h) {
  if (h->d.weight_format != MG_WEIGHT_FP8_BLOCK128) return 0;
  return static_cast<size_t>(h->e_local) * 3 * h->d.inter * h->d.hidden * 2;
}

// How an FP8 layer's grouped GEMMs get bf16 operands (MG_OPT_FP8_MODE):
//   in-kernel   every CTA converts the weight tiles of its own row tiles in shared memory: no scratch, but
//               a weight is converted once per 128 or 256 rows that use it;
//   pre-dequant a bf16 copy of all expert weights in scratch, written by a separate pass on a side stream;
//   ring        the GEMM kernel's own CTAs convert every weight once per expert and share the bf16 copy
//               through a ring of a few tens of MB (gemm.cu: grouped_gemm_ring_kernel): 58 MB of scratch
//               instead of 2 bytes per weight.
// AUTO: converting in the kernel re-does the work for every row tile of an expert; de-quantising first
// moves every weight through HBM three more times.  On the DeepSeek-V3 shape the two cost the same near
// 1024 rows per expert (256-row tiles), measured; below that converting wins by up to 2.7x, above it
// de-quantising first by up to 12 %.  The ring was built to take the large batches without the HBM round
// trip of the bf16 copy, but L2 does not hold it (measured at the benchmark size: 21.6 GB written to and
// 35.2 GB read from DRAM by the gate/up launch, i.e. the ring goes through HBM like the separate pass's
// copy does), and it ends 5 % behind pre-dequantise there; it is chosen only on request.
constexpr int64_t kRingMaxRows = 1ll << 24;          // rows the ring's counters are sized for
static int fp8_mode_for(const Handle* h, int64_t rows) {
  if (h->d.weight_format != MG_WEIGHT_FP8_BLOCK128) return MG_FP8_IN_KERNEL;
  if (h->opt_fp8_mode != MG_FP8_AUTO) return h->opt_fp8_mode;
  if (h->opt_batch_tokens * h->d.top_k > rows) rows = h->opt_batch_tokens * h->d.top_k;
  return rows >= static_cast<int64_t>(1024) * h->d.n_experts ? MG_FP8_PREDEQUANT : MG_FP8_IN_KERNEL;
}

struct RingWs { size_t ring_bytes; int64_t counter_ints; size_t total; };
static RingWs ring_ws(const Handle* h) {
  const mg_layer_desc& d = h->d;
  const RingPlan a = ring_plan(2 * d.inter, d.hidden, kRingMaxRows, h->e_local, h->opt_ring_bytes);
  const RingPlan b = ring_plan(d.hidden, d.inter, kRingMaxRows, h->e_local, h->opt_ring_bytes);
  RingWs w;
  w.ring_bytes = (a.ring_bytes > b.ring_bytes ? a.ring_bytes : b.ring_bytes);
  w.ring_bytes = (w.ring_bytes + 255) / 256 * 256;
  w.counter_ints = 2 * (a.max_granules > b.max_granules ? a.max_granules : b.max_granules);
  w.total = w.ring_bytes + static_cast<size_t>(w.counter_ints) * 4;
  return w;
}

// scratch the FP8 mode of a call over `rows` routed rows needs
static size_t fp8_scratch_bytes(const Handle* h, int64_t rows) {
  switch (fp8_mode_for(h, rows)) {
    case MG_FP8_PREDEQUANT: return dequant_ws(h);
    case MG_FP8_RING: return ring_ws(h).total;
    default: return 0;
  }
}

static bool fp8_predequant(const Handle* h, int64_t T) {
  return fp8_mode_for(h, T * h->d.top_k) == MG_FP8_PREDEQUANT;
}

static WsLayout ws_layout(const Handle* h, int64_t T, int64_t R) {
  const mg_layer_desc& d = h->d;
  if (R <= 0) R = T * d.top_k;
  const size_t Rp = static_cast<size_t>(padded_rows(h, R));
  WsLayout L;
  size_t off = 0;
  auto take = [&](int which, size_t bytes) { L.off[which] = off; off += (bytes + 255) / 256 * 256; };
  // first, so that its address does not depend on T: calls with different token counts on one
  // workspace can then share the de-quantised copy (MG_OPT_KEEP_DEQUANT)
  take(WS_DEQ, fp8_scratch_bytes(h, T * d.top_k));
  take(WS_LOGITS, static_cast<size_t>(T) * d.n_experts * 4);
  take(WS_IDX, static_cast<size_t>(T) * d.top_k * 4);
  take(WS_W, static_cast<size_t>(T) * d.top_k * 4);
  take(WS_COUNTS, static_cast<size_t>(d.n_experts) * 4);
  take(WS_OFFSETS, static_cast<size_t>(d.n_experts + 1) * 4);
  take(WS_PAD, static_cast<size_t>(d.n_experts + 1) * 4);
  take(WS_DST, static_cast<size_t>(T) * d.top_k * 4);
  take(WS_PERM, Rp * d.hidden * 2);
  take(WS_H, Rp * d.inter * 2);
  take(WS_OUT, Rp * d.hidden * 2);
  take(WS_PLAN, plan_ws_bytes(h, T));
  take(WS_HS, static_cast<size_t>(T) * d.inter_shared * 2);
  take(WS_SHARED, d.inter_shared ? static_cast<size_t>(T) * d.hidden * 2 : 0);
  take(WS_FIX, route_fix_bytes(T));
  L.total = off;
  return L;
}

}  // namespace mg

using namespace mg;

extern "C" {

const char* mg_last_error(void) { return g_err; }

int mg_create(const mg_layer_desc* desc, mg_handle* out) {
  MG_REQUIRE(desc && out, MG_ERR_NULL, "mg_create: null argument");
  MG_REQUIRE(desc->struct_bytes == static_cast<int32_t>(sizeof(mg_layer_desc)), MG_ERR_CONFIG,
             "mg_layer_desc.struct_bytes=%d, library expects %d", desc->struct_bytes,
             static_cast<int>(sizeof(mg_layer_desc)));
  const mg_layer_desc& d = *desc;
  MG_REQUIRE(d.hidden > 0 && d.hidden % 256 == 0, MG_ERR_SHAPE, "hidden=%d must be a positive multiple of 256", d.hidden);
  MG_REQUIRE(d.inter > 0 && d.inter % 128 == 0, MG_ERR_SHAPE, "inter=%d must be a positive multiple of 128", d.inter);
  MG_REQUIRE(d.inter_shared >= 0 && d.inter_shared % 128 == 0, MG_ERR_SHAPE,
             "inter_shared=%d must be a multiple of 128", d.inter_shared);
  MG_REQUIRE(d.n_experts >= 1 && d.n_experts <= kMaxExperts && d.n_experts % 4 == 0, MG_ERR_SHAPE,
             "n_experts=%d must be a multiple of 4 in [4,%d]", d.n_experts, kMaxExperts);
  MG_REQUIRE(d.top_k >= 1 && d.top_k <= kMaxTopK && d.top_k <= d.n_experts, MG_ERR_SHAPE,
             "top_k=%d must be in [1,min(%d,n_experts)]", d.top_k, kMaxTopK);
  MG_REQUIRE(d.gating >= 0 && d.gating <= 3, MG_ERR_CONFIG, "unknown gating mode %d", d.gating);
  MG_REQUIRE(d.combine_mode >= 0 && d.combine_mode <= 2, MG_ERR_CONFIG, "unknown combine mode %d", d.combine_mode);
  MG_REQUIRE(d.weight_format == MG_WEIGHT_BF16 || d.weight_format == MG_WEIGHT_FP8_BLOCK128, MG_ERR_CONFIG,
             "unknown weight format %d", d.weight_format);
  if (d.gating == MG_GATE_SOFTMAX_GROUP_MAX || d.gating == MG_GATE_SIGMOID_NOAUX_TC) {
    MG_REQUIRE(d.n_group >= 1 && d.n_group <= 32 && d.n_experts % d.n_group == 0, MG_ERR_CONFIG,
               "n_group=%d must divide n_experts and be <= 32", d.n_group);
    MG_REQUIRE(d.topk_group >= 1 && d.topk_group <= d.n_group, MG_ERR_CONFIG, "topk_group=%d must be in [1,n_group]",
               d.topk_group);
    MG_REQUIRE(d.n_experts / d.n_group >= (d.gating == MG_GATE_SIGMOID_NOAUX_TC ? 2 : 1), MG_ERR_CONFIG,
               "groups too small for the group score");
  }
  MG_REQUIRE(d.ep_size >= 1 && d.ep_rank >= 0 && d.ep_rank < d.ep_size && d.n_experts % d.ep_size == 0, MG_ERR_CONFIG,
             "ep_rank=%d / ep_size=%d invalid for %d experts", d.ep_rank, d.ep_size, d.n_experts);
  Handle* h = new (std::nothrow) Handle();
  MG_REQUIRE(h != nullptr, MG_ERR_STATE, "out of host memory");
  h->magic = kMagic;
  h->d = d;
  h->e_local = d.n_experts / d.ep_size;
  h->last_launches = 0;
  h->stage_timing = false;
  h->opt_fp8_mode = MG_FP8_AUTO;
  h->opt_pair_gemm = false;
  h->opt_fp8_m256 = 1;
  h->opt_shared_early = 2;
  h->opt_batch_tokens = 0;
  h->opt_keep_dequant = false;
  h->opt_ring_bytes = static_cast<size_t>(56) << 20;
  h->opt_ring_persist = 0;
  h->guard_rows = 0x7fffffffffffffffll;
  h->deq_valid = false;
  h->deq_inflight = false;
  h->deq_scratch = nullptr;
  h->deq_packed = nullptr;
  h->deq_stream = nullptr;
  h->side = nullptr;
  h->ret_streams_used = false;
  h->ev_entry = nullptr;
  for (int i = 0; i < kDequantChunks; ++i) h->ev_w13[i] = h->ev_w2[i] = nullptr;
  h->stage_calls = 0;
  for (int s = 0; s < kStageSlots; ++s)
    for (int i = 0; i <= MG_STAGE_COUNT; ++i) h->stage_ev[s][i] = nullptr;
  cudaError_t e = cudaGetDevice(&h->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, h->device);
  int major = 0;
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, h->device);
  if (e == cudaSuccess && major != 10) {
    delete h;
    set_error("device compute capability %d.x: this library contains sm_100a code only", major);
    return MG_ERR_STATE;
  }
  if (e == cudaSuccess) e = cudaMalloc(&h->d_status, 2 * sizeof(int32_t));
  if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, 2 * sizeof(int32_t));
  if (e != cudaSuccess) { delete h; return cuda_fail(e, "mg_create"); }
  *out = reinterpret_cast<mg_handle>(h);
  return MG_OK;
}

int mg_destroy(mg_handle hh) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  cudaFree(h->d_status);
  for (int s = 0; s < kStageSlots; ++s)
    for (int i = 0; i <= MG_STAGE_COUNT; ++i)
      if (h->stage_ev[s][i]) cudaEventDestroy(h->stage_ev[s][i]);
  if (h->side) cudaStreamDestroy(h->side);
  if (h->copy_in) {
    cudaStreamDestroy(h->copy_in);
    cudaStreamDestroy(h->copy_out);
    for (int i = 0; i < 2; ++i) { cudaEventDestroy(h->ev_in[i]); cudaEventDestroy(h->ev_done[i]); cudaEventDestroy(h->ev_out[i]); }
    cudaEventDestroy(h->ev_host);
  }
  if (h->side2) cudaStreamDestroy(h->side2);
  if (h->side3) {
    cudaStreamDestroy(h->side3);
    for (int i = 0; i < kDequantChunks; ++i) cudaEventDestroy(h->ev_part[i]);
    cudaEventDestroy(h->ev_ret);
    for (int i = 0; i < kMaxPeers; ++i) {
      cudaStreamDestroy(h->ret_streams[i]);
      cudaEventDestroy(h->ev_rets[i]);
    }
  }
  if (h->ev_shared_in) cudaEventDestroy(h->ev_shared_in);
  if (h->ev_shared_out) cudaEventDestroy(h->ev_shared_out);
  if (h->ev_entry) cudaEventDestroy(h->ev_entry);
  for (int i = 0; i < kDequantChunks; ++i) {
    if (h->ev_w13[i]) cudaEventDestroy(h->ev_w13[i]);
    if (h->ev_w2[i]) cudaEventDestroy(h->ev_w2[i]);
  }
  h->magic = 0;
  delete h;
  return MG_OK;
}

int mg_device_status(mg_handle hh, int32_t* code, int32_t* detail) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  int32_t v[2] = {0, 0};
  MG_CUDA(cudaMemcpy(v, h->d_status, sizeof(v), cudaMemcpyDeviceToHost));
  if (v[0] != 0) MG_CUDA(cudaMemset(h->d_status, 0, sizeof(v)));
  if (code) *code = v[0];
  if (detail) *detail = v[1];
  return MG_OK;
}

int mg_device_status_async(mg_handle hh, int32_t* host_words, void* stream) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(host_words, MG_ERR_NULL, "null argument");
  MG_CUDA(cudaMemcpyAsync(host_words, h->d_status, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost,
                          static_cast<cudaStream_t>(stream)));
  return MG_OK;
}

int mg_l2_set_aside(size_t bytes, size_t* granted) {
  MG_CUDA(cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, bytes));
  size_t got = 0;
  MG_CUDA(cudaDeviceGetLimit(&got, cudaLimitPersistingL2CacheSize));
  if (granted) *granted = got;
  return MG_OK;
}

int mg_packed_weight_bytes(mg_handle hh, size_t* bytes) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(bytes, MG_ERR_NULL, "null argument");
  *bytes = packed_layout(h).total;
  return MG_OK;
}

int mg_workspace_bytes(mg_handle hh, int64_t max_tokens, int64_t max_rows, size_t* bytes) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(bytes, MG_ERR_NULL, "null argument");
  MG_REQUIRE(max_tokens >= 0 && max_rows >= 0, MG_ERR_SHAPE, "negative size");
  MG_REQUIRE(max_tokens * h->d.top_k < (1ll << 31) - 65536, MG_ERR_LIMIT, "tokens*top_k exceeds 32-bit row indices");
  *bytes = ws_layout(h, max_tokens, max_rows).total;
  return MG_OK;
}

int mg_padded_rows(mg_handle hh, int64_t n_rows, int64_t* padded) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(padded, MG_ERR_NULL, "null argument");
  *padded = padded_rows(h, n_rows);
  return MG_OK;
}

int mg_pack_expert(mg_handle hh, int32_t local_expert, const void* d_gate, const void* d_up, const void* d_down,
                   const float* gs, const float* us, const float* ds, void* d_packed, void* stream) {
  MG_TRACE("mg_pack_expert", local_expert);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_gate && d_up && d_down && d_packed, MG_ERR_NULL, "mg_pack_expert: null pointer");
  h->deq_valid = false;
  h->deq_inflight = false;
  return launch_pack_expert(h, local_expert, d_gate, d_up, d_down, gs, us, ds, d_packed,
                            static_cast<cudaStream_t>(stream));
}

int mg_dequant_fp8_block128(const void* d_q, const float* d_scale_inv, int64_t rows, int64_t cols, void* d_out,
                            void* stream) {
  MG_TRACE("mg_dequant_fp8_block128", rows);
  MG_REQUIRE(d_q && d_scale_inv && d_out, MG_ERR_NULL, "mg_dequant_fp8_block128: null pointer");
  MG_REQUIRE(rows >= 0 && cols >= 0, MG_ERR_SHAPE, "negative size");
  return launch_dequant(d_q, d_scale_inv, rows, cols, d_out, static_cast<cudaStream_t>(stream));
}

int mg_gate_logits(mg_handle hh, const void* d_x, const void* d_gate_w, int64_t T, float* d_logits, void* stream) {
  MG_TRACE("mg_gate_logits", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_x && d_gate_w && d_logits, MG_ERR_NULL, "mg_gate_logits: null pointer");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  MG_REQUIRE(h->d.n_experts <= 256, MG_ERR_SHAPE, "router GEMM supports at most 256 experts");
  GemmProblem p{};
  p.a = d_x; p.a_rows = T; p.b = d_gate_w; p.n_groups = 1; p.n_per_group = h->d.n_experts; p.K = h->d.hidden;
  p.pad_offsets = nullptr; p.counts = nullptr; p.dense_rows = T; p.out = d_logits; p.ldo = h->d.n_experts;
  p.epilogue = h->d.gating == MG_GATE_SOFTMAX_TOPK_RENORM ? EPI_ROUND_BF16_F32 : EPI_PLAIN_F32;
  return launch_grouped_gemm(h, p, static_cast<cudaStream_t>(stream));
}

// The fix-up recomputes fp32 logits; the bf16 router of MG_GATE_SOFTMAX_TOPK_RENORM rounds its logits to
// bf16, where near-ties are exact ties that both sides break by the lower index.
static bool route_fixup_applies(const Handle* h) {
  return h->opt_route_fixup && h->d.gating != MG_GATE_SOFTMAX_TOPK_RENORM;
}

int mg_gate_route_topk(mg_handle hh, const void* d_x, const void* d_gate_w, const float* d_bias, int64_t T,
                       float* d_logits, int32_t* d_idx, float* d_w, int32_t* d_fix, void* stream) {
  MG_TRACE("mg_gate_route_topk", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_x && d_gate_w && d_logits && d_idx && d_w && d_fix, MG_ERR_NULL, "mg_gate_route_topk: null pointer");
  MG_REQUIRE(h->d.gating != MG_GATE_SIGMOID_NOAUX_TC || d_bias, MG_ERR_NULL, "noaux_tc gating needs the correction bias");
  int rc = mg_gate_logits(hh, d_x, d_gate_w, T, d_logits, stream);
  if (rc != MG_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!route_fixup_applies(h)) {
    if (T > 0) MG_CUDA(cudaMemsetAsync(d_fix, 0, 16, st));
    return launch_route_topk(h, d_logits, d_bias, T, d_idx, d_w, st);
  }
  return launch_route_topk_fixup(h, d_x, d_gate_w, d_logits, d_bias, T, d_idx, d_w, d_fix, st, nullptr);
}

int mg_route_fix_bytes(int64_t T, size_t* bytes) {
  MG_REQUIRE(bytes, MG_ERR_NULL, "mg_route_fix_bytes: null pointer");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  *bytes = route_fix_bytes(T);
  return MG_OK;
}

int mg_route_topk(mg_handle hh, const float* d_logits, const float* d_bias, int64_t T, int32_t* d_idx, float* d_w,
                  void* stream) {
  MG_TRACE("mg_route_topk", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_logits && d_idx && d_w, MG_ERR_NULL, "mg_route_topk: null pointer");
  MG_REQUIRE(h->d.gating != MG_GATE_SIGMOID_NOAUX_TC || d_bias != nullptr, MG_ERR_NULL,
             "noaux_tc gating needs e_score_correction_bias");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  return launch_route_topk(h, d_logits, d_bias, T, d_idx, d_w, static_cast<cudaStream_t>(stream));
}

int mg_plan_ws_bytes(mg_handle hh, int64_t T, size_t* bytes) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(bytes, MG_ERR_NULL, "null argument");
  *bytes = plan_ws_bytes(h, T);
  return MG_OK;
}

int mg_permute_plan(mg_handle hh, const int32_t* d_idx, int64_t T, int32_t expert_lo, int32_t n_plan,
                    int32_t* d_counts, int32_t* d_offsets, int32_t* d_pad, int32_t* d_dst, void* d_ws, void* stream) {
  MG_TRACE("mg_permute_plan", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_idx && d_counts && d_offsets && d_pad && d_dst && d_ws, MG_ERR_NULL, "mg_permute_plan: null pointer");
  MG_REQUIRE(T >= 0 && expert_lo >= 0 && n_plan >= 1 && expert_lo + n_plan <= h->d.n_experts, MG_ERR_SHAPE,
             "expert range [%d,%d) outside [0,%d)", expert_lo, expert_lo + n_plan, h->d.n_experts);
  return launch_permute_plan(h, d_idx, T, expert_lo, n_plan, d_counts, d_offsets, d_pad, d_dst, d_ws,
                             static_cast<cudaStream_t>(stream), nullptr);
}

int mg_permute_plan_static(mg_handle hh, const int32_t* d_idx, int64_t T, int32_t expert_lo, int32_t n_plan,
                           int32_t* d_counts, int32_t* d_offsets, int32_t* d_pad, int32_t* d_dst, void* stream) {
  MG_TRACE("mg_permute_plan_static", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_idx && d_counts && d_offsets && d_pad && d_dst, MG_ERR_NULL, "mg_permute_plan_static: null pointer");
  MG_REQUIRE(T >= 0 && expert_lo >= 0 && n_plan >= 1 && expert_lo + n_plan <= h->d.n_experts, MG_ERR_SHAPE,
             "expert range [%d,%d) outside [0,%d)", expert_lo, expert_lo + n_plan, h->d.n_experts);
  return launch_permute_plan_static(h, d_idx, T, expert_lo, n_plan, d_counts, d_offsets, d_pad, d_dst,
                                    static_cast<cudaStream_t>(stream));
}

int mg_permute_rows(mg_handle hh, const void* d_x, const int32_t* d_dst, int64_t T, void* d_perm, void* stream) {
  MG_TRACE("mg_permute_rows", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_x && d_dst && d_perm, MG_ERR_NULL, "mg_permute_rows: null pointer");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  return launch_permute_rows(h, d_x, d_dst, T, d_perm, static_cast<cudaStream_t>(stream));
}

int mg_dequant_ws_bytes(mg_handle hh, size_t* bytes) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(bytes, MG_ERR_NULL, "null argument");
  // what mg_expert_ffn may use of d_dequant_ws under the current MG_OPT_FP8_MODE (AUTO: the bf16 copy)
  *bytes = h->d.weight_format != MG_WEIGHT_FP8_BLOCK128 || h->opt_fp8_mode == MG_FP8_IN_KERNEL ? 0
           : h->opt_fp8_mode == MG_FP8_RING ? ring_ws(h).total : dequant_ws(h);
  return MG_OK;
}

// records the event that ends `stage` (and every skipped stage before it) when timing is on
static void mark(Handle* h, int stage, cudaStream_t st) {
  if (h->stage_timing) cudaEventRecord(h->stage_ev[h->stage_calls % kStageSlots][stage + 1], st);
}

static int ensure_side_stream(Handle* h) {
  if (h->side) return MG_OK;
  MG_CUDA(cudaStreamCreateWithFlags(&h->side, cudaStreamNonBlocking));
  MG_CUDA(cudaEventCreateWithFlags(&h->ev_entry, cudaEventDisableTiming));
  for (int i = 0; i < kDequantChunks; ++i) {
    MG_CUDA(cudaEventCreateWithFlags(&h->ev_w13[i], cudaEventDisableTiming));
    MG_CUDA(cudaEventCreateWithFlags(&h->ev_w2[i], cudaEventDisableTiming));
  }
  return MG_OK;
}

// Launches the chunked de-quantisation of all local experts on the side stream (ordered after
// what is already on `st`) and remembers that it is in flight for this packed buffer / scratch.
static int start_dequant(Handle* h, const void* packed, void* deq, cudaStream_t st, int* launches) {
  int rc = ensure_side_stream(h);
  if (rc != MG_OK) return rc;
  const int E = h->e_local;
  const int n_chunks = E < kDequantChunks ? E : kDequantChunks;
  const int per = (E + n_chunks - 1) / n_chunks;
  MG_CUDA(cudaEventRecord(h->ev_entry, st));
  MG_CUDA(cudaStreamWaitEvent(h->side, h->ev_entry, 0));
  for (int which = 0; which < 2; ++which) {
    for (int c = 0; c < n_chunks; ++c) {
      const int lo = c * per, n = (lo + per <= E ? per : E - lo);
      rc = launch_dequant_packed(h, packed, deq, which, lo, n, h->side);
      if (rc != MG_OK) return rc;
      MG_CUDA(cudaEventRecord(which == 0 ? h->ev_w13[c] : h->ev_w2[c], h->side));
    }
  }
  if (launches) *launches += 2 * n_chunks;
  h->deq_inflight = true;
  h->deq_valid = false;
  h->deq_scratch = deq;
  h->deq_packed = packed;
  h->deq_stream = st;
  return MG_OK;
}

static int ensure_return_stream(Handle* h) {
  if (h->side3) return MG_OK;
  MG_CUDA(cudaStreamCreateWithFlags(&h->side3, cudaStreamNonBlocking));
  for (int i = 0; i < kDequantChunks; ++i) MG_CUDA(cudaEventCreateWithFlags(&h->ev_part[i], cudaEventDisableTiming));
  MG_CUDA(cudaEventCreateWithFlags(&h->ev_ret, cudaEventDisableTiming));
  for (int i = 0; i < kMaxPeers; ++i) {
    MG_CUDA(cudaStreamCreateWithFlags(&h->ret_streams[i], cudaStreamNonBlocking));
    MG_CUDA(cudaEventCreateWithFlags(&h->ev_rets[i], cudaEventDisableTiming));
  }
  return MG_OK;
}

// Copy-engine return of the local experts [lo, lo + n): for every expert and source rank one copy of that
// rank's rows (contiguous in out_rows: ep_layout_kernel's order) to where the source rank's own expert-sorted
// order puts them in its buffer.  All sizes come from the gathered counts in host memory.
static int copy_part(Handle* h, const ReturnHook* hook, const void* out_rows, int lo, int n, cudaEvent_t ready) {
  const int N = h->d.ep_size, E = h->d.n_experts, El = h->e_local, me = h->d.ep_rank;
  for (int s = 0; s < N; ++s) MG_CUDA(cudaStreamWaitEvent(h->ret_streams[s], ready, 0));
  h->ret_streams_used = true;
  const int32_t* cnt = hook->host_counts;
  const size_t row_bytes = static_cast<size_t>(h->d.hidden) * 2;
  // padded offsets of this rank's experts up to lo, and whether the layout kernel dropped this owner's rows
  int64_t pad_e = 0, pad_all = 0;
  for (int j = 0; j < El; ++j) {
    int64_t tot = 0;
    for (int s = 0; s < N; ++s) tot += cnt[static_cast<size_t>(s) * E + me * El + j];
    if (j < lo) pad_e += (tot + kTileM - 1) / kTileM * kTileM;
    pad_all += (tot + kTileM - 1) / kTileM * kTileM;
  }
  if (pad_all > hook->cap_rows) return MG_OK;              // overflow: nothing was dispatched here (status word set)
  for (int j = lo; j < lo + n; ++j) {
    const int e = me * El + j;
    int64_t seg = pad_e, tot = 0;
    for (int s = 0; s < N; ++s) {
      const int64_t rows = cnt[static_cast<size_t>(s) * E + e];
      if (rows > 0) {
        int64_t own = 0;                                    // first row of expert e in rank s's own order
        for (int e2 = 0; e2 < e; ++e2) own += cnt[static_cast<size_t>(s) * E + e2];
        MG_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(hook->rets.p[s]) + own * row_bytes,
                                static_cast<const uint8_t*>(out_rows) + seg * row_bytes, rows * row_bytes,
                                cudaMemcpyDeviceToDevice, h->ret_streams[s]));
      }
      seg += rows;
      tot += rows;
    }
    pad_e += (tot + kTileM - 1) / kTileM * kTileM;
  }
  return MG_OK;
}

// the output rows of local experts [lo, lo + n) are complete on `st`: send them home beside what `st` does next
static int push_part(Handle* h, const ReturnHook* hook, const void* out_rows, const int32_t* pad, int lo, int n,
                     int part, cudaStream_t st) {
  cudaEvent_t ev = h->ev_part[part % kDequantChunks];
  MG_CUDA(cudaEventRecord(ev, st));
  if (hook->host_counts != nullptr) return copy_part(h, hook, out_rows, lo, n, ev);
  MG_CUDA(cudaStreamWaitEvent(h->side3, ev, 0));
  return launch_return_rows(h, out_rows, hook->back, pad, lo, n, hook->rets, h->side3);
}

static int join_return(Handle* h, cudaStream_t st) {
  if (h->ret_streams_used) {
    for (int s = 0; s < h->d.ep_size; ++s) {
      MG_CUDA(cudaEventRecord(h->ev_rets[s], h->ret_streams[s]));
      MG_CUDA(cudaStreamWaitEvent(st, h->ev_rets[s], 0));
    }
    h->ret_streams_used = false;
    return MG_OK;
  }
  MG_CUDA(cudaEventRecord(h->ev_ret, h->side3));
  MG_CUDA(cudaStreamWaitEvent(st, h->ev_ret, 0));
  return MG_OK;
}

static int expert_ffn(Handle* h, const void* perm_x, const int32_t* pad, const int32_t* counts, int64_t rows_padded,
                      const void* packed, void* h_buf, void* out_rows, void* deq, cudaStream_t st, int* launches,
                      bool timed = false, const ReturnHook* hook = nullptr) {
  if (hook != nullptr) {
    int rc0 = ensure_return_stream(h);
    if (rc0 != MG_OK) return rc0;
  }
  const mg_layer_desc& d = h->d;
  const PackedLayout L = packed_layout(h);
  const uint8_t* base = static_cast<const uint8_t*>(packed);
  const bool fp8 = d.weight_format == MG_WEIGHT_FP8_BLOCK128;
  const int E = h->e_local;
  GemmProblem p{};
  p.a_rows = rows_padded;
  // a caller that hands in scratch has chosen a scratch mode: the ring if that is the option, else the bf16 copy
  const int mode = !fp8 || deq == nullptr ? MG_FP8_IN_KERNEL
                   : h->opt_fp8_mode == MG_FP8_RING ? MG_FP8_RING : MG_FP8_PREDEQUANT;
  if (mode != MG_FP8_PREDEQUANT) {
    // bf16 weights, FP8 tiles converted inside the GEMM kernels, or FP8 weights converted once into the
    // L2-resident ring by the GEMM kernel itself: two launches over all experts
    if (mode == MG_FP8_RING) {
      MG_REQUIRE(rows_padded <= kRingMaxRows, MG_ERR_LIMIT, "ring mode handles up to %lld rows per call",
                 static_cast<long long>(kRingMaxRows));
      const RingWs rw = ring_ws(h);
      p.ring = deq;
      p.ring_bytes = rw.ring_bytes;
      p.ring_counters = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(deq) + rw.ring_bytes);
      p.ring_counter_ints = rw.counter_ints;
    }
    if (timed) mark(h, MG_STAGE_DEQUANT, st);
    p.a = perm_x; p.b = base + L.w13; p.n_groups = E; p.n_per_group = 2 * d.inter; p.K = d.hidden;
    p.pad_offsets = pad; p.counts = counts; p.out = h_buf; p.ldo = d.inter; p.epilogue = EPI_SWIGLU_BF16;
    p.b_fp8 = fp8;
    p.scales = fp8 ? reinterpret_cast<const float*>(base + L.s13) : nullptr;
    int rc = launch_grouped_gemm(h, p, st);
    if (rc != MG_OK) return rc;
    if (timed) mark(h, MG_STAGE_EXPERT_GEMM1, st);
    p.a = h_buf; p.b = base + L.w2; p.n_per_group = d.hidden; p.K = d.inter; p.out = out_rows; p.ldo = d.hidden;
    p.epilogue = EPI_PLAIN_BF16;
    p.scales = fp8 ? reinterpret_cast<const float*>(base + L.s2) : nullptr;
    if (hook != nullptr && mode != MG_FP8_RING) {
      // the down projection in parts of experts, each part's rows sent home while the next part computes
      const int parts = hook->n_parts < 1 ? 1 : hook->n_parts > E ? E : hook->n_parts > kDequantChunks ? kDequantChunks : hook->n_parts;
      const int per = (E + parts - 1) / parts;
      const size_t w2_expert = static_cast<size_t>(d.hidden) * d.inter * L.w_elem;
      const size_t s2_expert = static_cast<size_t>(d.hidden / 128) * (d.inter / 128);
      for (int c = 0, lo = 0; lo < E; ++c, lo += per) {
        const int n = lo + per <= E ? per : E - lo;
        p.n_groups = n; p.pad_offsets = pad + lo; p.counts = counts + lo;
        p.b = base + L.w2 + lo * w2_expert;
        p.scales = fp8 ? reinterpret_cast<const float*>(base + L.s2) + lo * s2_expert : nullptr;
        rc = launch_grouped_gemm(h, p, st);
        if (rc != MG_OK) return rc;
        rc = push_part(h, hook, out_rows, pad, lo, n, c, st);
        if (rc != MG_OK) return rc;
        if (launches) *launches += 2;
      }
      rc = join_return(h, st);
    } else {
      rc = launch_grouped_gemm(h, p, st);
      if (rc == MG_OK && hook != nullptr) {
        rc = push_part(h, hook, out_rows, pad, 0, E, 0, st);
        if (rc == MG_OK) rc = join_return(h, st);
      }
    }
    if (timed) mark(h, MG_STAGE_EXPERT_GEMM2, st);
    if (launches) *launches += mode == MG_FP8_RING ? 4 : 2;      // ring: a counter reset in front of each GEMM
    return rc;
  }
  // FP8 weights de-quantised into `deq` one chunk of experts ahead of the bf16 GEMMs: the
  // conversion is HBM-bound and runs on a side stream while the tensor cores work on the
  // previous chunk, so only the first chunk is exposed
  int rc = ensure_side_stream(h);
  if (rc != MG_OK) return rc;
  const int n_chunks = E < kDequantChunks ? E : kDequantChunks;
  const int per = (E + n_chunks - 1) / n_chunks;
  // MG_OPT_KEEP_DEQUANT: the copy made by the previous call (same packed buffer, same scratch,
  // same stream) is still current, e.g. between the token chunks of one host-buffer forward
  // keep-dequant level 2: the caller orders the streams itself (expert-parallel micro-batches)
  const bool same = h->deq_scratch == deq && h->deq_packed == packed &&
                    (h->deq_stream == st || h->opt_keep_dequant == 2);
  const bool reuse = h->opt_keep_dequant && h->deq_valid && same;
  if (!reuse && !(h->deq_inflight && same)) {       // not started ahead of time by start_dequant
    rc = start_dequant(h, packed, deq, st, launches);
    if (rc != MG_OK) return rc;
  }
  h->deq_inflight = false;
  if (timed) mark(h, MG_STAGE_DEQUANT, st);
  const __nv_bfloat16* w13 = static_cast<const __nv_bfloat16*>(deq);
  const __nv_bfloat16* w2 = w13 + static_cast<size_t>(E) * 2 * d.inter * d.hidden;
  for (int which = 0; which < 2; ++which) {
    for (int c = 0; c < n_chunks; ++c) {
      const int lo = c * per, n = (lo + per <= E ? per : E - lo);
      if (n <= 0) continue;
      if (!reuse) MG_CUDA(cudaStreamWaitEvent(st, which == 0 ? h->ev_w13[c] : h->ev_w2[c], 0));
      p.n_groups = n; p.pad_offsets = pad + lo; p.counts = counts + lo; p.b_fp8 = false; p.scales = nullptr;
      if (which == 0) {
        p.a = perm_x; p.b = w13 + static_cast<size_t>(lo) * 2 * d.inter * d.hidden; p.n_per_group = 2 * d.inter;
        p.K = d.hidden; p.out = h_buf; p.ldo = d.inter; p.epilogue = EPI_SWIGLU_BF16;
      } else {
        p.a = h_buf; p.b = w2 + static_cast<size_t>(lo) * d.hidden * d.inter; p.n_per_group = d.hidden;
        p.K = d.inter; p.out = out_rows; p.ldo = d.hidden; p.epilogue = EPI_PLAIN_BF16;
      }
      rc = launch_grouped_gemm(h, p, st);
      if (rc != MG_OK) return rc;
      if (which == 1 && hook != nullptr) {
        rc = push_part(h, hook, out_rows, pad, lo, n, c, st);
        if (rc != MG_OK) return rc;
      }
    }
    if (which == 1 && hook != nullptr) {
      rc = join_return(h, st);
      if (rc != MG_OK) return rc;
    }
    if (timed) mark(h, which == 0 ? MG_STAGE_EXPERT_GEMM1 : MG_STAGE_EXPERT_GEMM2, st);
  }
  if (launches) *launches += 2 * n_chunks;
  h->deq_valid = true;
  h->deq_scratch = deq;
  h->deq_packed = packed;
  h->deq_stream = st;
  return MG_OK;
}

}  // extern "C"
namespace mg {
int expert_ffn_return(Handle* h, const void* perm_x, const int32_t* pad, const int32_t* counts, int64_t rows_padded,
                      const void* packed, void* h_buf, void* out_rows, void* deq, const ReturnHook& hook,
                      cudaStream_t st) {
  return expert_ffn(h, perm_x, pad, counts, rows_padded, packed, h_buf, out_rows, deq, st, nullptr, false, &hook);
}
}  // namespace mg
extern "C" {

int mg_dequant_start(mg_handle hh, const void* d_packed, void* d_dequant_ws, void* stream) {
  MG_TRACE("mg_dequant_start", 0);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_packed && d_dequant_ws, MG_ERR_NULL, "mg_dequant_start: null pointer");
  MG_REQUIRE(h->d.weight_format == MG_WEIGHT_FP8_BLOCK128, MG_ERR_CONFIG, "layer has no FP8 weights");
  if (h->opt_fp8_mode == MG_FP8_RING || h->opt_fp8_mode == MG_FP8_IN_KERNEL) return MG_OK;   // converted inside mg_expert_ffn
  return start_dequant(h, d_packed, d_dequant_ws, static_cast<cudaStream_t>(stream), nullptr);
}

int mg_expert_ffn(mg_handle hh, const void* d_perm_x, const int32_t* d_pad, const int32_t* d_counts,
                  int64_t n_rows_padded, const void* d_packed, void* d_h_buf, void* d_out_rows, void* d_deq,
                  void* stream) {
  MG_TRACE("mg_expert_ffn", n_rows_padded);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_perm_x && d_pad && d_counts && d_packed && d_h_buf && d_out_rows, MG_ERR_NULL,
             "mg_expert_ffn: null pointer");
  MG_REQUIRE(n_rows_padded >= 0 && n_rows_padded % kTileM == 0, MG_ERR_SHAPE,
             "n_rows_padded=%lld must be a multiple of %d", static_cast<long long>(n_rows_padded), kTileM);
  return expert_ffn(h, d_perm_x, d_pad, d_counts, n_rows_padded, d_packed, d_h_buf, d_out_rows, d_deq,
                    static_cast<cudaStream_t>(stream), nullptr);
}

static int shared_ffn(Handle* h, const void* x, int64_t T, const void* packed, void* hs, void* out, cudaStream_t st,
                      bool timed = false) {
  const mg_layer_desc& d = h->d;
  MG_REQUIRE(d.inter_shared > 0, MG_ERR_CONFIG, "layer has no shared expert");
  const PackedLayout L = packed_layout(h);
  const uint8_t* base = static_cast<const uint8_t*>(packed);
  GemmProblem p{};
  p.a = x; p.a_rows = T; p.b = base + L.sh13; p.n_groups = 1; p.n_per_group = 2 * d.inter_shared; p.K = d.hidden;
  p.dense_rows = T; p.out = hs; p.ldo = d.inter_shared; p.epilogue = EPI_SWIGLU_BF16;
  int rc = launch_grouped_gemm(h, p, st);
  if (rc != MG_OK) return rc;
  if (timed) mark(h, MG_STAGE_SHARED_GEMM1, st);
  p.a = hs; p.b = base + L.sh2; p.n_per_group = d.hidden; p.K = d.inter_shared; p.out = out; p.ldo = d.hidden;
  p.epilogue = EPI_PLAIN_BF16;
  return launch_grouped_gemm(h, p, st);
}

int mg_shared_ffn(mg_handle hh, const void* d_x, int64_t T, const void* d_packed, void* d_hs, void* d_out,
                  void* stream) {
  MG_TRACE("mg_shared_ffn", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_x && d_packed && d_hs && d_out, MG_ERR_NULL, "mg_shared_ffn: null pointer");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  return shared_ffn(h, d_x, T, d_packed, d_hs, d_out, static_cast<cudaStream_t>(stream));
}

int mg_combine(mg_handle hh, const void* d_out_rows, const int32_t* d_dst, const int32_t* d_idx, const float* d_w,
               const void* d_shared, int64_t T, void* d_y, void* stream) {
  MG_TRACE("mg_combine", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_out_rows && d_dst && d_idx && d_w && d_y, MG_ERR_NULL, "mg_combine: null pointer");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  return launch_combine(h, d_out_rows, d_dst, d_idx, d_w, d_shared, nullptr, T, d_y, static_cast<cudaStream_t>(stream));
}

int mg_workspace_ptr(mg_handle hh, void* d_ws, int64_t max_tokens, int64_t max_rows, int32_t which, void** ptr) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_ws && ptr, MG_ERR_NULL, "null argument");
  MG_REQUIRE(which >= 0 && which < WS_N, MG_ERR_SHAPE, "which=%d out of range", which);
  *ptr = static_cast<uint8_t*>(d_ws) + ws_layout(h, max_tokens, max_rows).off[which];
  return MG_OK;
}

// d_residual: nullptr, or [T,H] bf16 added to the block's bf16 output in the combine (may be d_y)
// d_logits_in: nullptr, or caller-computed fp32 router logits [T,E] used in place of the router GEMM
static int moe_forward_impl(mg_handle hh, const void* d_x, int64_t T, const void* d_gate_w, const float* d_bias,
                            const void* d_packed, void* d_ws, size_t ws_bytes, const void* d_residual, void* d_y,
                            void* stream, const float* d_logits_in = nullptr) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) { h->last_launches = 0; return MG_OK; }   // empty batch: nothing to read or write
  MG_REQUIRE(d_x && (d_gate_w || d_logits_in) && d_packed && d_ws && d_y, MG_ERR_NULL, "mg_moe_forward: null pointer");
  MG_REQUIRE(h->d.ep_size == 1, MG_ERR_CONFIG, "mg_moe_forward is the single-GPU path (ep_size == 1)");
  MG_REQUIRE(h->d.gating != MG_GATE_SIGMOID_NOAUX_TC || d_bias != nullptr, MG_ERR_NULL,
             "noaux_tc gating needs e_score_correction_bias");
  const mg_layer_desc& d = h->d;
  const WsLayout L = ws_layout(h, T, 0);
  MG_REQUIRE(ws_bytes >= L.total, MG_ERR_WORKSPACE, "workspace %zu bytes < %zu needed for %lld tokens", ws_bytes,
             L.total, static_cast<long long>(T));
  h->last_launches = 0;
  if (T == 0) return MG_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(d_ws);
  float* logits = reinterpret_cast<float*>(ws + L.off[WS_LOGITS]);
  int32_t* idx = reinterpret_cast<int32_t*>(ws + L.off[WS_IDX]);
  float* w = reinterpret_cast<float*>(ws + L.off[WS_W]);
  int32_t* counts = reinterpret_cast<int32_t*>(ws + L.off[WS_COUNTS]);
  int32_t* offsets = reinterpret_cast<int32_t*>(ws + L.off[WS_OFFSETS]);
  int32_t* pad = reinterpret_cast<int32_t*>(ws + L.off[WS_PAD]);
  int32_t* dst = reinterpret_cast<int32_t*>(ws + L.off[WS_DST]);
  void* perm = ws + L.off[WS_PERM];
  void* hbuf = ws + L.off[WS_H];
  void* orow = ws + L.off[WS_OUT];
  void* plan = ws + L.off[WS_PLAN];
  void* hs = ws + L.off[WS_HS];
  void* sh = d.inter_shared ? ws + L.off[WS_SHARED] : nullptr;
  void* deq = fp8_scratch_bytes(h, T * d.top_k) > 0 ? ws + L.off[WS_DEQ] : nullptr;
  int launches = 0;
  const long long guard_keep = h->guard_rows;
  h->guard_rows = padded_rows(h, T * d.top_k);     // what this call's dst_row entries may address
  struct RestoreGuard { Handle* h; long long v; ~RestoreGuard() { h->guard_rows = v; } } restore_guard{h, guard_keep};
  if (h->stage_timing) MG_CUDA(cudaEventRecord(h->stage_ev[h->stage_calls % kStageSlots][0], st));
  int rc;
  const bool deq_same = h->deq_scratch == deq && h->deq_packed == d_packed && h->deq_stream == st;
  if (deq != nullptr && fp8_predequant(h, T) && !(h->opt_keep_dequant && h->deq_valid && deq_same) &&
      !(h->deq_inflight && deq_same)) {
    // the weights do not depend on the routing: their de-quantisation starts now, beside the
    // router, plan and scatter kernels
    rc = start_dequant(h, d_packed, deq, st, &launches);
    if (rc != MG_OK) return rc;
  }
  if (d_logits_in != nullptr) {
    logits = const_cast<float*>(d_logits_in);      // only read from here on
  } else {
    rc = mg_gate_logits(hh, d_x, d_gate_w, T, logits, stream);
    if (rc != MG_OK) return rc;
    launches += 1;
  }
  mark(h, MG_STAGE_GATE_LOGITS, st);
  // The shared expert needs only x: its GEMMs (tensor-bound) run on a second stream beside the
  // top-k, plan and scatter kernels (HBM- and latency-bound) instead of after the routed experts.
  // pays only while the kernels are short (measured: V2-Lite at 2048 tokens 0.428 -> 0.383 ms; at
  // 32768 / 65536 tokens of V2-236B / V3 the step got 1-2 % slower), hence the automatic setting
  const bool shared_early = d.inter_shared && (h->opt_shared_early == 1 || (h->opt_shared_early == 2 && T <= 4096));
  if (shared_early) {
    if (!h->side2) {
      MG_CUDA(cudaStreamCreateWithFlags(&h->side2, cudaStreamNonBlocking));
      MG_CUDA(cudaEventCreateWithFlags(&h->ev_shared_in, cudaEventDisableTiming));
      MG_CUDA(cudaEventCreateWithFlags(&h->ev_shared_out, cudaEventDisableTiming));
    }
    MG_CUDA(cudaEventRecord(h->ev_shared_in, st));
    MG_CUDA(cudaStreamWaitEvent(h->side2, h->ev_shared_in, 0));
    rc = shared_ffn(h, d_x, T, d_packed, hs, sh, h->side2, false);
    if (rc != MG_OK) return rc;
    MG_CUDA(cudaEventRecord(h->ev_shared_out, h->side2));
    launches += 2;
  }
  if (d_logits_in == nullptr && route_fixup_applies(h)) {
    // logits from the tensor-core product: tokens whose pick its rounding could have changed are re-routed
    // from exactly recomputed logits, so the routing is that of correctly rounded fp32 logits
    rc = launch_route_topk_fixup(h, d_x, d_gate_w, logits, d_bias, T, idx, w,
                                 reinterpret_cast<int32_t*>(ws + L.off[WS_FIX]), st, &launches);
  } else {
    rc = launch_route_topk(h, logits, d_bias, T, idx, w, st);
    launches += 1;
  }
  if (rc != MG_OK) return rc;
  mark(h, MG_STAGE_ROUTE_TOPK, st);
  rc = launch_permute_plan(h, idx, T, 0, d.n_experts, counts, offsets, pad, dst, plan, st, &launches);
  if (rc != MG_OK) return rc;
  mark(h, MG_STAGE_PERMUTE_PLAN, st);
  rc = launch_permute_rows(h, d_x, dst, T, perm, st);
  if (rc != MG_OK) return rc;
  mark(h, MG_STAGE_PERMUTE_ROWS, st);
  launches += 1;
  rc = expert_ffn(h, perm, pad, counts, padded_rows(h, T * d.top_k), d_packed, hbuf, orow, deq, st, &launches, true);
  if (rc != MG_OK) return rc;
  if (shared_early) {
    MG_CUDA(cudaStreamWaitEvent(st, h->ev_shared_out, 0));
    mark(h, MG_STAGE_SHARED_GEMM1, st);
  } else if (d.inter_shared) {
    rc = shared_ffn(h, d_x, T, d_packed, hs, sh, st, true);
    if (rc != MG_OK) return rc;
    launches += 2;
  } else {
    mark(h, MG_STAGE_SHARED_GEMM1, st);
  }
  mark(h, MG_STAGE_SHARED_GEMM2, st);
  rc = launch_combine(h, orow, dst, idx, w, sh, d_residual, T, d_y, st);
  if (rc != MG_OK) return rc;
  mark(h, MG_STAGE_COMBINE, st);
  launches += 1;
  h->last_launches = launches;
  if (h->stage_timing) ++h->stage_calls;
  return MG_OK;
}

int mg_moe_forward(mg_handle hh, const void* d_x, int64_t T, const void* d_gate_w, const float* d_bias,
                   const void* d_packed, void* d_ws, size_t ws_bytes, void* d_y, void* stream) {
  MG_TRACE("mg_moe_forward", T);
  return moe_forward_impl(hh, d_x, T, d_gate_w, d_bias, d_packed, d_ws, ws_bytes, nullptr, d_y, stream);
}

int mg_moe_forward_from_logits(mg_handle hh, const void* d_x, int64_t T, const float* d_logits, const float* d_bias,
                               const void* d_packed, void* d_ws, size_t ws_bytes, void* d_y, void* stream) {
  MG_TRACE("mg_moe_forward_from_logits", T);
  MG_REQUIRE(d_logits != nullptr || T == 0, MG_ERR_NULL, "mg_moe_forward_from_logits: null logits");
  return moe_forward_impl(hh, d_x, T, nullptr, d_bias, d_packed, d_ws, ws_bytes, nullptr, d_y, stream, d_logits);
}

// ---- host-buffer forward: chunk pipeline behind the C ABI ------------------------------------------
// Chunk sizes: the copy-in of the first chunk and the copy-out of the last one cannot overlap with
// compute, so those two are half a chunk; the ones between them are one and a half, because every
// chunk streams all expert weights once.
static int host_chunk_plan(int64_t T, int64_t chunk, int64_t* sizes, int max_n) {
  int n = 0;
  if (T <= 0) return 0;
  const int64_t c = chunk < 1 ? 1 : chunk;
  auto put = [&](int64_t v) { if (n < max_n) sizes[n] = v; ++n; };
  if (T <= 2 * c) {
    for (int64_t t0 = 0; t0 < T; t0 += c) put(T - t0 < c ? T - t0 : c);
    return n;
  }
  const int64_t edge = c / 2 > 128 ? c / 2 : 128;
  int64_t rest = T - 2 * edge;
  const int64_t mid = c + c / 2;
  const int64_t n_mid = (rest + mid - 1) / mid > 1 ? (rest + mid - 1) / mid : 1;
  int64_t base = (rest + n_mid - 1) / n_mid;
  base = (base + 127) / 128 * 128;
  put(edge);
  while (rest > 0) {
    const int64_t v = base < rest ? base : rest;
    put(v);
    rest -= v;
  }
  put(edge);
  return n;
}
constexpr int kMaxHostChunks = 1024;

struct HostWs { size_t stage_bytes, fwd_off, fwd_bytes, total; int64_t cs; };
static HostWs host_ws(Handle* h, int64_t T, int64_t chunk) {
  int64_t sizes[kMaxHostChunks];
  const int n = host_chunk_plan(T, chunk, sizes, kMaxHostChunks);
  int64_t cs = 1;
  for (int i = 0; i < n && i < kMaxHostChunks; ++i) cs = sizes[i] > cs ? sizes[i] : cs;
  HostWs w;
  w.cs = cs;
  w.stage_bytes = (static_cast<size_t>(cs) * h->d.hidden * 2 + 255) / 256 * 256;     // one of 4: x in [2], y out [2]
  w.fwd_off = 4 * w.stage_bytes;
  // the FP8 mode is chosen for the whole batch, not per chunk
  const int64_t keep = h->opt_batch_tokens;
  if (h->d.weight_format == MG_WEIGHT_FP8_BLOCK128 && T > cs) h->opt_batch_tokens = T;
  w.fwd_bytes = ws_layout(h, cs, 0).total;
  h->opt_batch_tokens = keep;
  w.total = w.fwd_off + w.fwd_bytes;
  return w;
}

static int ensure_host_streams(Handle* h) {
  if (h->copy_in) return MG_OK;
  MG_CUDA(cudaStreamCreateWithFlags(&h->copy_in, cudaStreamNonBlocking));
  MG_CUDA(cudaStreamCreateWithFlags(&h->copy_out, cudaStreamNonBlocking));
  for (int i = 0; i < 2; ++i) {
    MG_CUDA(cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming));
    MG_CUDA(cudaEventCreateWithFlags(&h->ev_done[i], cudaEventDisableTiming));
    MG_CUDA(cudaEventCreateWithFlags(&h->ev_out[i], cudaEventDisableTiming));
  }
  MG_CUDA(cudaEventCreateWithFlags(&h->ev_host, cudaEventDisableTiming));
  return MG_OK;
}

int mg_host_chunk_plan(int64_t n_tokens, int64_t chunk_tokens, int64_t* sizes, int32_t max_chunks, int32_t* n_chunks) {
  MG_REQUIRE(n_chunks && (sizes || max_chunks == 0), MG_ERR_NULL, "mg_host_chunk_plan: null argument");
  MG_REQUIRE(n_tokens >= 0 && chunk_tokens >= 1 && max_chunks >= 0, MG_ERR_SHAPE, "mg_host_chunk_plan: bad size");
  *n_chunks = host_chunk_plan(n_tokens, chunk_tokens, sizes, max_chunks);
  return MG_OK;
}

int mg_host_workspace_bytes(mg_handle hh, int64_t n_tokens, int64_t chunk_tokens, size_t* bytes) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(bytes, MG_ERR_NULL, "null argument");
  MG_REQUIRE(n_tokens >= 0 && chunk_tokens >= 1, MG_ERR_SHAPE, "mg_host_workspace_bytes: bad size");
  *bytes = host_ws(h, n_tokens, chunk_tokens).total;
  return MG_OK;
}

int mg_moe_forward_host(mg_handle hh, const void* x_host, int64_t T, const void* d_gate_w, const float* d_bias,
                        const void* d_packed, void* d_ws, size_t ws_bytes, void* y_host, int64_t chunk_tokens,
                        void* stream) {
  MG_TRACE("mg_moe_forward_host", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0 && chunk_tokens >= 1, MG_ERR_SHAPE, "mg_moe_forward_host: bad size");
  if (T == 0) { h->last_launches = 0; return MG_OK; }
  MG_REQUIRE(x_host && y_host && d_gate_w && d_packed && d_ws, MG_ERR_NULL, "mg_moe_forward_host: null pointer");
  int64_t sizes[kMaxHostChunks];
  const int n = host_chunk_plan(T, chunk_tokens, sizes, kMaxHostChunks);
  MG_REQUIRE(n <= kMaxHostChunks, MG_ERR_LIMIT, "more than %d chunks: raise chunk_tokens", kMaxHostChunks);
  const HostWs W = host_ws(h, T, chunk_tokens);
  MG_REQUIRE(ws_bytes >= W.total, MG_ERR_WORKSPACE, "workspace %zu bytes < %zu needed (mg_host_workspace_bytes)", ws_bytes,
             W.total);
  int rc = ensure_host_streams(h);
  if (rc != MG_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(d_ws);
  uint8_t* xin[2] = {ws, ws + W.stage_bytes};
  uint8_t* yout[2] = {ws + 2 * W.stage_bytes, ws + 3 * W.stage_bytes};
  const size_t row = static_cast<size_t>(h->d.hidden) * 2;
  // the copy streams start after whatever the caller's stream holds
  MG_CUDA(cudaEventRecord(h->ev_host, st));
  MG_CUDA(cudaStreamWaitEvent(h->copy_in, h->ev_host, 0));
  MG_CUDA(cudaStreamWaitEvent(h->copy_out, h->ev_host, 0));
  // one de-quantisation (pre-dequantise mode) serves every chunk of this batch
  const int64_t keep_batch = h->opt_batch_tokens;
  const int keep_deq = h->opt_keep_dequant;
  if (h->d.weight_format == MG_WEIGHT_FP8_BLOCK128 && T > W.cs) h->opt_batch_tokens = T;
  h->opt_keep_dequant = 1;
  h->deq_valid = false;
  h->deq_inflight = false;
  int launches = 0;
  if (fp8_predequant(h, W.cs)) {
    // the weights do not depend on the input: their de-quantisation starts now, beside the first copy-in
    const WsLayout L = ws_layout(h, W.cs, 0);
    rc = start_dequant(h, d_packed, ws + W.fwd_off + L.off[WS_DEQ], st, &launches);
    if (rc != MG_OK) return rc;
  }
  int64_t t0 = 0;
  for (int c = 0; c < n && rc == MG_OK; ++c) {
    const int b = c & 1;
    const int64_t m = sizes[c];
    if (c >= 2) MG_CUDA(cudaStreamWaitEvent(h->copy_in, h->ev_done[b], 0));      // chunk c-2 has consumed this buffer
    MG_CUDA(cudaMemcpyAsync(xin[b], static_cast<const uint8_t*>(x_host) + t0 * row, m * row, cudaMemcpyHostToDevice,
                            h->copy_in));
    MG_CUDA(cudaEventRecord(h->ev_in[b], h->copy_in));
    MG_CUDA(cudaStreamWaitEvent(st, h->ev_in[b], 0));
    if (c >= 2) MG_CUDA(cudaStreamWaitEvent(st, h->ev_out[b], 0));               // chunk c-2's result has left
    rc = moe_forward_impl(hh, xin[b], m, d_gate_w, d_bias, d_packed, ws + W.fwd_off, W.fwd_bytes, nullptr, yout[b], stream);
    launches += h->last_launches;
    if (rc != MG_OK) break;
    MG_CUDA(cudaEventRecord(h->ev_done[b], st));
    MG_CUDA(cudaStreamWaitEvent(h->copy_out, h->ev_done[b], 0));
    MG_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(y_host) + t0 * row, yout[b], m * row, cudaMemcpyDeviceToHost,
                            h->copy_out));
    MG_CUDA(cudaEventRecord(h->ev_out[b], h->copy_out));
    t0 += m;
  }
  h->opt_batch_tokens = keep_batch;
  h->opt_keep_dequant = keep_deq;
  h->deq_valid = false;
  if (rc != MG_OK) return rc;
  // the caller's stream ends after the last copies: synchronising it means y_host is complete
  MG_CUDA(cudaStreamWaitEvent(st, h->ev_out[(n - 1) & 1], 0));
  if (n >= 2) MG_CUDA(cudaStreamWaitEvent(st, h->ev_out[(n - 2) & 1], 0));
  h->last_launches = launches;
  return MG_OK;
}

int mg_rmsnorm(mg_handle hh, const void* d_x, const void* d_weight, float eps, int64_t T, void* d_out,
               void* stream) {
  MG_TRACE("mg_rmsnorm", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) return MG_OK;
  MG_REQUIRE(d_x && d_weight && d_out, MG_ERR_NULL, "mg_rmsnorm: null pointer");
  MG_REQUIRE(eps >= 0.f, MG_ERR_CONFIG, "mg_rmsnorm: negative eps");
  return launch_rmsnorm(h, d_x, d_weight, eps, T, d_out, static_cast<cudaStream_t>(stream));
}

int mg_moe_block_forward(mg_handle hh, const void* d_hidden, const void* d_norm_weight, float eps, int64_t T,
                         const void* d_gate_w, const float* d_bias, const void* d_packed, void* d_xnorm,
                         void* d_ws, size_t ws_bytes, void* d_out, void* stream) {
  MG_TRACE("mg_moe_block_forward", T);
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) { h->last_launches = 0; return MG_OK; }
  MG_REQUIRE(d_hidden && d_norm_weight && d_xnorm && d_out, MG_ERR_NULL, "mg_moe_block_forward: null pointer");
  MG_REQUIRE(d_xnorm != d_hidden && d_xnorm != d_out, MG_ERR_CONFIG,
             "mg_moe_block_forward: the normalised rows need a buffer of their own");
  int rc = mg_rmsnorm(hh, d_hidden, d_norm_weight, eps, T, d_xnorm, stream);
  if (rc != MG_OK) return rc;
  rc = moe_forward_impl(hh, d_xnorm, T, d_gate_w, d_bias, d_packed, d_ws, ws_bytes, d_hidden, d_out, stream);
  if (rc == MG_OK) h->last_launches += 1;
  return rc;
}

int mg_set_option(mg_handle hh, int32_t option, int32_t value) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  switch (option) {
    case MG_OPT_FP8_MODE:
      MG_REQUIRE(value >= MG_FP8_AUTO && value <= MG_FP8_RING, MG_ERR_CONFIG, "bad FP8 mode %d", value);
      h->opt_fp8_mode = value;
      return MG_OK;
    case MG_OPT_PAIR_GEMM: h->opt_pair_gemm = value != 0; return MG_OK;
    case MG_OPT_SHARED_EARLY:
      MG_REQUIRE(value >= 0 && value <= 2, MG_ERR_CONFIG, "bad value %d", value);
      h->opt_shared_early = value;
      return MG_OK;
    case MG_OPT_BATCH_TOKENS:
      MG_REQUIRE(value >= 0, MG_ERR_CONFIG, "bad value %d", value);
      h->opt_batch_tokens = value;
      return MG_OK;
    case MG_OPT_FP8_M256:
      MG_REQUIRE(value >= 0 && value <= 2, MG_ERR_CONFIG, "bad value %d", value);
      h->opt_fp8_m256 = value;
      return MG_OK;
    case MG_OPT_ROWS_BOUND:
      MG_REQUIRE(value >= 0, MG_ERR_CONFIG, "bad value %d", value);
      h->guard_rows = value > 0 ? value : 0x7fffffffffffffffll;
      return MG_OK;
    case MG_OPT_RING_PERSIST: h->opt_ring_persist = value != 0; return MG_OK;
    case MG_OPT_ROUTE_FIXUP: h->opt_route_fixup = value != 0; return MG_OK;
    case MG_OPT_RING_BYTES:
      MG_REQUIRE(value >= 1, MG_ERR_CONFIG, "bad ring size %d MiB", value);
      h->opt_ring_bytes = static_cast<size_t>(value) << 20;
      return MG_OK;
    case MG_OPT_KEEP_DEQUANT:
      MG_REQUIRE(value >= 0 && value <= 2, MG_ERR_CONFIG, "bad keep-dequant level %d", value);
      h->opt_keep_dequant = value;
      h->deq_valid = false;          // switching it on or off never trusts an older copy
      return MG_OK;
    default: set_error("unknown option %d", option); return MG_ERR_CONFIG;
  }
}

int mg_set_stage_timing(mg_handle hh, int32_t enable) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  if (enable) {
    for (int s = 0; s < kStageSlots; ++s)
      for (int i = 0; i <= MG_STAGE_COUNT; ++i)
        if (!h->stage_ev[s][i]) MG_CUDA(cudaEventCreate(&h->stage_ev[s][i]));
    h->stage_calls = 0;
  }
  h->stage_timing = enable != 0;
  return MG_OK;
}

int mg_stage_times(mg_handle hh, float* ms, int32_t n) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(ms && n >= MG_STAGE_COUNT, MG_ERR_NULL, "mg_stage_times: need room for %d values", MG_STAGE_COUNT);
  MG_REQUIRE(h->stage_calls > 0, MG_ERR_STATE, "no timed forward has completed on this handle");
  const int n_sets = h->stage_calls < kStageSlots ? h->stage_calls : kStageSlots;
  for (int i = 0; i < MG_STAGE_COUNT; ++i) ms[i] = 0.f;
  for (int s = 0; s < n_sets; ++s) {
    for (int i = 0; i < MG_STAGE_COUNT; ++i) {
      float t = 0.f;
      MG_CUDA(cudaEventElapsedTime(&t, h->stage_ev[s][i], h->stage_ev[s][i + 1]));
      ms[i] += t / n_sets;
    }
  }
  return MG_OK;
}

int mg_selftest_wait_timeout(mg_handle hh, int32_t limit_ms, void* stream) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, MG_ERR_LIMIT, "limit_ms=%d must be in [1,1000]", limit_ms);
  return launch_wait_probe(h, limit_ms, static_cast<cudaStream_t>(stream));
}

int mg_last_launch_count(mg_handle hh, int32_t* launches) {
  Handle* h = check(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(launches, MG_ERR_NULL, "null argument");
  *launches = h->last_launches;
  return MG_OK;
}

}  // extern "C"
