// Expert-parallel entry points: symmetric device buffers shared between the ranks of one
// NVSwitch domain (CUDA IPC), and the dispatch / return steps that move rows with plain
// stores and loads through the peer mappings.  No TMA and no multicast touches peer memory.
#include <string.h>

#include "common.cuh"

using namespace mg;

namespace mg {
Handle* check_handle(mg_handle hh);
}

extern "C" {

int mg_ep_alloc(size_t bytes, void** d_ptr) {
  MG_REQUIRE(d_ptr && bytes > 0, MG_ERR_NULL, "mg_ep_alloc: null argument or zero size");
  MG_CUDA(cudaMalloc(d_ptr, bytes));
  return MG_OK;
}

int mg_ep_free(void* d_ptr) {
  if (d_ptr) MG_CUDA(cudaFree(d_ptr));
  return MG_OK;
}

int mg_ep_export(void* d_ptr, void* handle64) {
  MG_REQUIRE(d_ptr && handle64, MG_ERR_NULL, "mg_ep_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t hd;
  MG_CUDA(cudaIpcGetMemHandle(&hd, d_ptr));
  memcpy(handle64, &hd, 64);
  return MG_OK;
}

int mg_ep_import(const void* handle64, void** d_ptr) {
  MG_REQUIRE(handle64 && d_ptr, MG_ERR_NULL, "mg_ep_import: null argument");
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle64, 64);
  MG_CUDA(cudaIpcOpenMemHandle(d_ptr, hd, cudaIpcMemLazyEnablePeerAccess));
  return MG_OK;
}

int mg_ep_unimport(void* d_ptr) {
  if (d_ptr) MG_CUDA(cudaIpcCloseMemHandle(d_ptr));
  return MG_OK;
}

int mg_ep_count(mg_handle hh, const int32_t* d_topk_idx, int64_t T, int32_t* d_counts, void* d_plan_ws,
                void* stream) {
  MG_TRACE("mg_ep_count", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_counts && d_plan_ws && (T == 0 || d_topk_idx), MG_ERR_NULL, "mg_ep_count: null pointer");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  return launch_ep_count(h, d_topk_idx, T, d_counts, d_plan_ws, static_cast<cudaStream_t>(stream));
}

int mg_ep_place(mg_handle hh, const int32_t* d_topk_idx, int64_t T, const int32_t* d_counts_all, int64_t cap_rows,
                void* d_plan_ws, int32_t* d_recv_counts, int32_t* d_recv_pad, int32_t* d_dst, void* stream) {
  MG_TRACE("mg_ep_place", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_counts_all && d_plan_ws && d_recv_counts && d_recv_pad && (T == 0 || (d_topk_idx && d_dst)),
             MG_ERR_NULL, "mg_ep_place: null pointer");
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  MG_REQUIRE(h->d.ep_size <= kMaxPeers, MG_ERR_LIMIT, "ep_size %d > %d", h->d.ep_size, kMaxPeers);
  MG_REQUIRE(cap_rows > 0 && cap_rows % kTileM == 0 && cap_rows <= kPeerRowMask, MG_ERR_LIMIT,
             "cap_rows=%lld must be a positive multiple of %d below 2^%d", static_cast<long long>(cap_rows), kTileM,
             kPeerShift);
  return launch_ep_place(h, d_topk_idx, T, d_counts_all, static_cast<int>(cap_rows), d_plan_ws, d_recv_counts,
                         d_recv_pad, d_dst, static_cast<cudaStream_t>(stream));
}

static int gather_peers(const Handle* h, void* const* ptrs, PeerPtrs* out) {
  MG_REQUIRE(ptrs != nullptr, MG_ERR_NULL, "null peer pointer table");
  MG_REQUIRE(h->d.ep_size <= kMaxPeers, MG_ERR_LIMIT, "ep_size %d > %d", h->d.ep_size, kMaxPeers);
  for (int i = 0; i < kMaxPeers; ++i) out->p[i] = nullptr;
  for (int i = 0; i < h->d.ep_size; ++i) {
    MG_REQUIRE(ptrs[i] != nullptr, MG_ERR_NULL, "peer pointer %d is null", i);
    out->p[i] = ptrs[i];
  }
  return MG_OK;
}

int mg_ep_dispatch(mg_handle hh, const void* d_x, const int32_t* d_dst, int64_t T, void* const* peer_recv,
                   void* stream) {
  MG_TRACE("mg_ep_dispatch", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) return MG_OK;
  MG_REQUIRE(d_x && d_dst, MG_ERR_NULL, "mg_ep_dispatch: null pointer");
  PeerPtrs peers;
  int rc = gather_peers(h, peer_recv, &peers);
  if (rc != MG_OK) return rc;
  return launch_dispatch_rows(h, d_x, d_dst, T, peers, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

int mg_ep_dispatch_dedup(mg_handle hh, const void* d_x, const int32_t* d_dst, int64_t T, void* const* peer_recv,
                         void* const* peer_dup, void* stream) {
  MG_TRACE("mg_ep_dispatch_dedup", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) return MG_OK;
  MG_REQUIRE(d_x && d_dst, MG_ERR_NULL, "mg_ep_dispatch_dedup: null pointer");
  PeerPtrs peers, dups;
  int rc = gather_peers(h, peer_recv, &peers);
  if (rc != MG_OK) return rc;
  rc = gather_peers(h, peer_dup, &dups);
  if (rc != MG_OK) return rc;
  return launch_dispatch_rows(h, d_x, d_dst, T, peers, &dups, nullptr, static_cast<cudaStream_t>(stream));
}

int mg_ep_dispatch_back(mg_handle hh, const void* d_x, const int32_t* d_dst, int64_t T, void* const* peer_recv,
                        void* const* peer_dup, void* const* peer_back, void* stream) {
  MG_TRACE("mg_ep_dispatch_back", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) return MG_OK;
  MG_REQUIRE(d_x && d_dst && peer_back, MG_ERR_NULL, "mg_ep_dispatch_back: null pointer");
  MG_REQUIRE(T * h->d.top_k <= kPeerRowMask, MG_ERR_LIMIT, "tokens * top_k exceeds 2^%d picks per rank", kPeerShift);
  PeerPtrs peers, dups, backs;
  int rc = gather_peers(h, peer_recv, &peers);
  if (rc != MG_OK) return rc;
  rc = gather_peers(h, peer_back, &backs);
  if (rc != MG_OK) return rc;
  if (peer_dup != nullptr) {
    rc = gather_peers(h, peer_dup, &dups);
    if (rc != MG_OK) return rc;
  }
  return launch_dispatch_rows(h, d_x, d_dst, T, peers, peer_dup ? &dups : nullptr, &backs,
                              static_cast<cudaStream_t>(stream));
}

int mg_ep_expert_ffn_return(mg_handle hh, const void* d_recv_x, const int32_t* d_recv_pad, const int32_t* d_recv_counts,
                            int64_t cap_rows, const void* d_packed, void* d_h_buf, void* d_out_rows, void* d_dequant_ws,
                            const int32_t* d_back, void* const* peer_ret, int32_t n_parts, void* stream) {
  MG_TRACE("mg_ep_expert_ffn_return", cap_rows);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_recv_x && d_recv_pad && d_recv_counts && d_packed && d_h_buf && d_out_rows && d_back, MG_ERR_NULL,
             "mg_ep_expert_ffn_return: null pointer");
  MG_REQUIRE(cap_rows >= 0 && cap_rows % kTileM == 0, MG_ERR_SHAPE, "cap_rows=%lld must be a multiple of %d",
             static_cast<long long>(cap_rows), kTileM);
  ReturnHook hook{};
  hook.back = d_back;
  hook.n_parts = n_parts;
  int rc = gather_peers(h, peer_ret, &hook.rets);
  if (rc != MG_OK) return rc;
  return expert_ffn_return(h, d_recv_x, d_recv_pad, d_recv_counts, cap_rows, d_packed, d_h_buf, d_out_rows, d_dequant_ws,
                           hook, static_cast<cudaStream_t>(stream));
}

int mg_ep_expert_ffn_copy_return(mg_handle hh, const void* d_recv_x, const int32_t* d_recv_pad,
                                 const int32_t* d_recv_counts, int64_t cap_rows, const void* d_packed, void* d_h_buf,
                                 void* d_out_rows, void* d_dequant_ws, const int32_t* h_counts_all,
                                 void* const* peer_ret, int32_t n_parts, void* stream) {
  MG_TRACE("mg_ep_expert_ffn_copy_return", cap_rows);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_recv_x && d_recv_pad && d_recv_counts && d_packed && d_h_buf && d_out_rows && h_counts_all, MG_ERR_NULL,
             "mg_ep_expert_ffn_copy_return: null pointer");
  MG_REQUIRE(cap_rows >= 0 && cap_rows % kTileM == 0, MG_ERR_SHAPE, "cap_rows=%lld must be a multiple of %d",
             static_cast<long long>(cap_rows), kTileM);
  const int64_t n = static_cast<int64_t>(h->d.ep_size) * h->d.n_experts;
  for (int64_t i = 0; i < n; ++i)
    MG_REQUIRE(h_counts_all[i] >= 0 && h_counts_all[i] <= kPeerRowMask, MG_ERR_SHAPE,
               "mg_ep_expert_ffn_copy_return: count %d at %lld is not a row count", h_counts_all[i], static_cast<long long>(i));
  ReturnHook hook{};
  hook.back = nullptr;
  hook.n_parts = n_parts;
  hook.host_counts = h_counts_all;
  hook.cap_rows = cap_rows;
  int rc = gather_peers(h, peer_ret, &hook.rets);
  if (rc != MG_OK) return rc;
  return expert_ffn_return(h, d_recv_x, d_recv_pad, d_recv_counts, cap_rows, d_packed, d_h_buf, d_out_rows, d_dequant_ws,
                           hook, static_cast<cudaStream_t>(stream));
}

int mg_ep_mirror_delta(mg_handle hh, const int32_t* d_counts_all, int32_t* d_delta, void* stream) {
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_counts_all && d_delta, MG_ERR_NULL, "mg_ep_mirror_delta: null pointer");
  return launch_mirror_delta(h, d_counts_all, d_delta, static_cast<cudaStream_t>(stream));
}

int mg_ep_combine_mirror(mg_handle hh, const void* d_mirror, const int32_t* d_dst, const int32_t* d_delta,
                         const int32_t* d_topk_idx, const float* d_topk_w, const void* d_shared_out, int64_t T,
                         void* d_y, void* stream) {
  MG_TRACE("mg_ep_combine_mirror", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) return MG_OK;
  MG_REQUIRE(d_mirror && d_dst && d_delta && d_topk_idx && d_topk_w && d_y, MG_ERR_NULL, "mg_ep_combine_mirror: null pointer");
  return launch_combine_mirror(h, d_mirror, d_dst, d_delta, d_topk_idx, d_topk_w, d_shared_out, T, d_y,
                               static_cast<cudaStream_t>(stream));
}

int mg_ep_combine_slots(mg_handle hh, const void* d_ret, const void* d_out_rows, const int32_t* d_dst,
                        const int32_t* d_topk_idx, const float* d_topk_w, const void* d_shared_out, int64_t T, void* d_y,
                        void* stream) {
  MG_TRACE("mg_ep_combine_slots", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) return MG_OK;
  MG_REQUIRE(d_ret && d_out_rows && d_dst && d_topk_idx && d_topk_w && d_y, MG_ERR_NULL, "mg_ep_combine_slots: null pointer");
  MG_REQUIRE(h->d.ep_size <= kMaxPeers, MG_ERR_LIMIT, "ep_size %d > %d", h->d.ep_size, kMaxPeers);
  return launch_combine_slots(h, d_ret, d_out_rows, d_dst, d_topk_idx, d_topk_w, d_shared_out, T, d_y,
                              static_cast<cudaStream_t>(stream));
}

int mg_ep_clear_duplicates(mg_handle hh, void* d_dup, int64_t cap_rows, void* stream) {
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_dup && cap_rows >= 0, MG_ERR_NULL, "mg_ep_clear_duplicates: bad argument");
  MG_CUDA(cudaMemsetAsync(d_dup, 0xFF, static_cast<size_t>(cap_rows) * 4, static_cast<cudaStream_t>(stream)));
  return MG_OK;
}

int mg_ep_fill_duplicates(mg_handle hh, void* d_recv_x, const void* d_dup, int64_t cap_rows, void* stream) {
  MG_TRACE("mg_ep_fill_duplicates", cap_rows);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(d_recv_x && d_dup && cap_rows >= 0, MG_ERR_NULL, "mg_ep_fill_duplicates: bad argument");
  return launch_fill_duplicates(h, d_recv_x, static_cast<const int32_t*>(d_dup), cap_rows,
                                static_cast<cudaStream_t>(stream));
}

int mg_ep_combine(mg_handle hh, void* const* peer_out, const int32_t* d_dst, const int32_t* d_topk_idx,
                  const float* d_topk_w, const void* d_shared_out, int64_t T, void* d_y, void* stream) {
  MG_TRACE("mg_ep_combine", T);
  Handle* h = check_handle(hh);
  if (!h) return MG_ERR_STATE;
  MG_REQUIRE(T >= 0, MG_ERR_SHAPE, "negative token count");
  if (T == 0) return MG_OK;
  MG_REQUIRE(d_dst && d_topk_idx && d_topk_w && d_y, MG_ERR_NULL, "mg_ep_combine: null pointer");
  PeerPtrs peers;
  int rc = gather_peers(h, peer_out, &peers);
  if (rc != MG_OK) return rc;
  return launch_combine_peers(h, peers, d_dst, d_topk_idx, d_topk_w, d_shared_out, T, d_y,
                              static_cast<cudaStream_t>(stream));
}

}  // extern "C"
