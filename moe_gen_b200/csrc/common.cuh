// Internal declarations shared by the translation units of libmoegen_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/moegen_b200.h"

namespace mg {

constexpr int kTileM = 128;          // rows per GEMM tile == expert segment alignment
constexpr int kMaxExperts = 512;     // plan and top-k kernels keep per-expert state on chip
constexpr int kMaxTopK = 16;
constexpr int kMaxPeers = 8;         // ranks of one NVSwitch domain
constexpr int kPeerShift = 24;       // expert-parallel destinations: rank << 24 | row
constexpr int kPeerRowMask = (1 << kPeerShift) - 1;
constexpr int kSkipRow = -(1 << 30); // stays negative after the in-segment rank is added
constexpr int kDequantChunks = 8;    // expert chunks of the overlapped FP8 de-quantisation
constexpr int kStageSlots = 32;      // forwards whose per-stage times are kept for averaging

// thread-local error text -------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);   // records text, returns (int)e

#define MG_CUDA(call)                                                    \
  do {                                                                   \
    cudaError_t _e = (call);                                             \
    if (_e != cudaSuccess) return ::mg::cuda_fail(_e, #call);            \
  } while (0)

#define MG_REQUIRE(cond, code, ...)                                      \
  do {                                                                   \
    if (!(cond)) { ::mg::set_error(__VA_ARGS__); return (code); }        \
  } while (0)

// encoded TMA descriptors of the (pointer, shape, box) combinations a handle has launched with
struct TensorMapCache {
  static constexpr int kEntries = 96;
  struct Entry {
    const void* base;
    uint64_t rows, cols;
    uint32_t box_rows, kind;
    CUtensorMap map;
  };
  Entry e[kEntries];
  int used = 0, next = 0;
};

// Call tracing: an NVTX range around every entry point that does device work (visible to a profiler
// that attaches; without one the calls cost a branch), and, when the environment variable MG_LOG is 1,
// one line per call on stderr: name and the call's leading size.
struct CallTrace {
  CallTrace(const char* name, long long n);
  ~CallTrace();
};
#define MG_TRACE(name, n) ::mg::CallTrace _mg_trace(name, static_cast<long long>(n))

struct Handle {
  uint32_t magic;
  mg_layer_desc d;
  int device;
  int sm_count;
  int e_local;            // experts owned by this rank
  int32_t* d_status;      // [2]: code, detail
  int last_launches;
  int opt_keep_dequant;   // 1/2: reuse the de-quantised copy of the previous call while nothing changed
  bool deq_valid;
  bool deq_inflight;      // start_dequant ran for (deq_packed, deq_scratch, deq_stream); expert_ffn only waits
  const void* deq_scratch;
  const void* deq_packed;
  cudaStream_t deq_stream;
  int64_t opt_batch_tokens;  // total tokens of a batch fed in chunks (0 = unknown), for the AUTO rule
  int opt_fp8_m256;       // in-kernel FP8: 0 = 128-row tiles, 1 = 256-row tiles when experts are big, 2 = always
  bool opt_pair_gemm;     // bf16 expert GEMMs on SM pairs (tcgen05 cta_group::2)
  int opt_fp8_mode;       // MG_FP8_AUTO / MG_FP8_PREDEQUANT / MG_FP8_IN_KERNEL / MG_FP8_RING
  long long guard_rows;   // bound the row-moving kernels check table entries against in a -DMG_BOUNDS_CHECK build
  size_t opt_ring_bytes;  // budget of the bf16 ring of MG_FP8_RING (it should stay resident in L2)
  bool opt_route_fixup = true;   // MG_OPT_ROUTE_FIXUP
  int opt_ring_persist;          // ring accesses carry the L2 evict_last policy (needs an L2 set-aside, mg_l2_set_aside)
  cudaStream_t side;      // de-quantisation runs here, one chunk of experts ahead of the GEMMs
  cudaEvent_t ev_entry, ev_w13[kDequantChunks], ev_w2[kDequantChunks];
  cudaStream_t copy_in, copy_out;   // host-buffer forward: copies of the chunks either side of the compute
  cudaEvent_t ev_in[2], ev_done[2], ev_out[2], ev_host;
  cudaStream_t side3;     // expert-parallel return: pushes of finished expert parts run here beside the GEMMs
  cudaEvent_t ev_part[kDequantChunks], ev_ret;
  // copy-engine return: one stream per destination rank, so that the copies to different peers run on
  // different engines at once (one stream of 4 MB copies reaches about 300 GB/s)
  cudaStream_t ret_streams[8];
  cudaEvent_t ev_rets[8];
  bool ret_streams_used;
  cudaStream_t side2;     // the shared expert's GEMMs run here beside the routing and scatter kernels
  cudaEvent_t ev_shared_in, ev_shared_out;
  int opt_shared_early;
  bool stage_timing;      // record an event after every stage of mg_moe_forward
  int stage_calls;        // forwards recorded since timing was enabled
  cudaEvent_t stage_ev[kStageSlots][MG_STAGE_COUNT + 1];   // ring of event sets, one per forward
  mutable TensorMapCache tmaps;
};
constexpr uint32_t kMagic = 0x4d474232u;  // "MGB2"

static inline int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// packed weight buffer offsets (bytes) ------------------------------------------------
struct PackedLayout {
  size_t w13, w2, s13, s2, sh13, sh2, total;
  size_t w_elem;          // bytes per routed weight element
};
PackedLayout packed_layout(const Handle* h);

// routing / permute / combine launchers (route.cu) -------------------------------------
int launch_route_topk(const Handle* h, const float* logits, const float* bias, int64_t T,
                      int32_t* idx, float* w, cudaStream_t st);
size_t route_fix_bytes(int64_t T);
int launch_route_topk_fixup(const Handle* h, const void* x, const void* gate_w, float* logits, const float* bias,
                            int64_t T, int32_t* idx, float* w, int32_t* fix, cudaStream_t st, int* launches);
size_t plan_ws_bytes(const Handle* h, int64_t T);
int launch_permute_plan(const Handle* h, const int32_t* idx, int64_t T, int expert_lo, int n_exp,
                        int32_t* counts, int32_t* offsets, int32_t* pad_offsets, int32_t* dst_row,
                        void* ws, cudaStream_t st, int* launches);
int launch_permute_plan_static(const Handle* h, const int32_t* idx, int64_t T, int expert_lo, int n_exp,
                               int32_t* counts, int32_t* offsets, int32_t* pad_offsets, int32_t* dst_row,
                               cudaStream_t st);
int launch_permute_rows(const Handle* h, const void* x, const int32_t* dst_row, int64_t T,
                        void* perm_x, cudaStream_t st);
int launch_combine(const Handle* h, const void* out_rows, const int32_t* dst_row,
                   const int32_t* idx, const float* w, const void* shared, const void* residual, int64_t T,
                   void* y, cudaStream_t st);
int launch_rmsnorm(const Handle* h, const void* x, const void* weight, float eps, int64_t T, void* out,
                   cudaStream_t st);

struct PeerPtrs { void* p[kMaxPeers]; };

// Index guard of the row-moving kernels.  In a build with -DMG_BOUNDS_CHECK (the stand-in for a memory
// checker on machines where none can run) every row index taken from a table is compared with the
// bound the host knows; the first violation is recorded in the status word (MG_DEV_BOUNDS, detail =
// which kernel) and the access is skipped, never trapped.  Other builds carry the struct and ignore it.
struct Guard {
  int32_t* status;
  long long rows_bound;   // rows of the buffer the indices point into (LLONG_MAX = not declared)
  int n_peers;
};
#ifdef MG_BOUNDS_CHECK
#define MG_GUARD(ok, g, where) \
  ((ok) ? true : ((atomicCAS((g).status, MG_DEV_OK, MG_DEV_BOUNDS) == MG_DEV_OK ? ((g).status[1] = (where)) : 0), false))
#else
#define MG_GUARD(ok, g, where) (true)
#endif
// expert-parallel return pushed from inside the expert FFN: after the down projection of each part of the
// local experts, their output rows travel to the token owners' return buffers on a side stream
struct ReturnHook {
  const int32_t* back;    // this rank's return table [cap_rows] (pushed by a kernel)
  PeerPtrs rets;          // every rank's return buffer as mapped here
  int n_parts;            // parts the down projection is cut into (when it is not chunked already)
  // copied by the copy engines instead (back == nullptr): the gathered counts [ep_size][E] in HOST memory;
  // every (expert, source rank) segment of out_rows goes to the source rank's buffer at the place the
  // source rank's own expert-sorted order gives it
  const int32_t* host_counts;
  int64_t cap_rows;
};
int launch_dispatch_rows(const Handle* h, const void* x, const int32_t* dst, int64_t T,
                         const PeerPtrs& peers, const PeerPtrs* dups, const PeerPtrs* backs, cudaStream_t st);
int launch_return_rows(const Handle* h, const void* out_rows, const int32_t* back, const int32_t* pad, int e_lo,
                       int e_n, const PeerPtrs& rets, cudaStream_t st);
int launch_combine_slots(const Handle* h, const void* ret_rows, const void* own_out_rows, const int32_t* dst,
                         const int32_t* idx, const float* w, const void* shared, int64_t T, void* y, cudaStream_t st);
int launch_mirror_delta(const Handle* h, const int32_t* counts_all, int32_t* delta, cudaStream_t st);
int launch_combine_mirror(const Handle* h, const void* mirror, const int32_t* dst, const int32_t* delta,
                          const int32_t* idx, const float* w, const void* shared, int64_t T, void* y, cudaStream_t st);
int launch_fill_duplicates(const Handle* h, void* rows, const int32_t* dup, int64_t n_rows, cudaStream_t st);
int launch_combine_peers(const Handle* h, const PeerPtrs& peers, const int32_t* dst,
                         const int32_t* idx, const float* w, const void* shared, int64_t T, void* y,
                         cudaStream_t st);
int launch_ep_count(const Handle* h, const int32_t* idx, int64_t T, int32_t* counts, void* ws,
                    cudaStream_t st);
int launch_ep_place(const Handle* h, const int32_t* idx, int64_t T, const int32_t* counts_all,
                    int cap_rows, void* ws, int32_t* recv_counts, int32_t* recv_pad, int32_t* dst,
                    cudaStream_t st);

// weights (pack.cu) --------------------------------------------------------------------
int launch_pack_expert(const Handle* h, int local_expert, const void* g, const void* u,
                       const void* dn, const float* gs, const float* us, const float* ds,
                       void* packed, cudaStream_t st);
int launch_dequant(const void* q, const float* s, int64_t rows, int64_t cols, void* out,
                   cudaStream_t st);
// de-quantise every routed expert of a packed FP8 buffer into a bf16 buffer of the same
// layout (w13 then w2)
int launch_dequant_packed(const Handle* h, const void* packed, void* bf16_out, int which, int e_lo, int e_n,
                          cudaStream_t st);

// grouped GEMM (gemm.cu) ---------------------------------------------------------------
enum GemmEpilogue { EPI_SWIGLU_BF16 = 0, EPI_PLAIN_BF16 = 1, EPI_PLAIN_F32 = 2, EPI_ROUND_BF16_F32 = 3 };

struct GemmProblem {
  const void* a;          // [a_rows, K] bf16 row-major
  int64_t a_rows;
  const void* b;          // [n_groups * n_per_group, K] row-major ("N x K, K-major"), bf16 or FP8 e4m3
  bool b_fp8;             // B holds e4m3 bytes; `scales` holds fp32 [rows/128][K/128]
  const float* scales;
  int n_groups;
  int n_per_group;        // rows of B per group (2I for SwiGLU, H for down, E for the gate)
  int K;
  const int32_t* pad_offsets;  // [n_groups+1] device, or nullptr = dense (one group, rows = dense_rows)
  const int32_t* counts;       // [n_groups] device
  int64_t dense_rows;
  void* out;              // bf16 or fp32
  int64_t ldo;            // elements between output rows
  int epilogue;
  // W8A16 through the L2-resident ring (grouped FP8 weights only): scratch for the bf16 ring and its
  // 2 x max_granules counters, sized with ring_plan(); nullptr = not this path
  void* ring;
  size_t ring_bytes;
  int32_t* ring_counters;
  int64_t ring_counter_ints;
};
// how a grouped FP8 GEMM of this shape uses a ring of at most budget_bytes
struct RingPlan {
  int pg;                 // N tiles per granule
  int slots;              // granules in the ring
  size_t granule_bytes, ring_bytes;
  int64_t max_granules;   // upper bound of granules for a_rows padded rows in n_groups experts
};
RingPlan ring_plan(int n_per_group, int K, int64_t a_rows, int n_groups, size_t budget_bytes);
int launch_grouped_gemm(const Handle* h, const GemmProblem& p, cudaStream_t st);
int launch_wait_probe(const Handle* h, int limit_ms, cudaStream_t st);

// the expert FFN with the expert-parallel return pushed from inside it (api.cu)
int expert_ffn_return(Handle* h, const void* perm_x, const int32_t* pad, const int32_t* counts, int64_t rows_padded,
                      const void* packed, void* h_buf, void* out_rows, void* deq, const ReturnHook& hook,
                      cudaStream_t st);

}  // namespace mg
