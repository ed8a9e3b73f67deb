/*
 * moegen_b200 — C ABI of the B200 (sm_100a) MoE-layer library.
 *
 * This is the boundary that replaces, for the MoE layer only, what the
 * reference reaches through its op_builder-compiled pybind module
 * (core/MoE_Gen_Binding.cpp:44-87: get_weights / free_weights_buffer /
 * clear_expert_buffer) plus the PyTorch arithmetic of
 * moe_gen/models/deepseek/deepseekv2/modeling_deepseek_v2.py (MoEGate,
 * DeepseekV2MoE) and .../deepseekv3/modeling_deepseek_v3.py (MoEGate,
 * DeepseekV3MoE) and of transformers' MixtralSparseMoeBlock.
 *
 * Conventions
 *  - plain C symbols, no torch / pybind types; every pointer named d_* is a
 *    raw DEVICE address on the device the handle was created on, `stream` is a
 *    cudaStream_t passed as void*;
 *  - every call returns an int: 0 = OK, negative = argument / shape / state
 *    error detected on the host before any launch, positive = CUDA runtime or
 *    driver error (cudaError_t value).  Nothing throws, exits or traps.
 *    mg_last_error() returns a text for the last non-zero return on the calling
 *    thread.  Problems found on the device (a bounded wait that ran out) are
 *    written to a status word that mg_device_status() reads after the caller
 *    has synchronised the stream;
 *  - calls are asynchronous on `stream`; the caller owns all memory (inputs,
 *    outputs, workspace, packed weights).  The library owns only the handle;
 *  - one handle is bound to one device and used by one thread at a time.
 */
#ifndef MOEGEN_B200_H
#define MOEGEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* gating modes */
#define MG_GATE_SOFTMAX_GREEDY      0  /* modeling_deepseek_v2.py:493-504  */
#define MG_GATE_SOFTMAX_GROUP_MAX   1  /* modeling_deepseek_v2.py:505-526  */
#define MG_GATE_SIGMOID_NOAUX_TC    2  /* modeling_deepseek_v3.py:509-547  */
#define MG_GATE_SOFTMAX_TOPK_RENORM 3  /* MixtralSparseMoeBlock router     */

/* combine modes */
#define MG_COMBINE_FP32       0  /* modeling_deepseek_v3.py:702-710: fp32 products, fp32 sum */
#define MG_COMBINE_BF16_PROD  1  /* modeling_deepseek_v2.py:744-757: bf16 weight, bf16 products */
#define MG_COMBINE_BF16_SEQ   2  /* Mixtral: bf16 products added one by one, experts ascending */

/* expert weight formats */
#define MG_WEIGHT_BF16          0
#define MG_WEIGHT_FP8_BLOCK128  1  /* e4m3 + fp32 scale per 128x128 block (Wrapper.py:109-138) */

/* error codes (negative: host-side argument/state errors) */
#define MG_OK                 0
#define MG_ERR_NULL          -1
#define MG_ERR_SHAPE         -2  /* unsupported or inconsistent shape */
#define MG_ERR_CONFIG        -3  /* unsupported combination in mg_layer_desc */
#define MG_ERR_WORKSPACE     -4  /* workspace too small */
#define MG_ERR_STATE         -5  /* handle not usable (wrong device, destroyed) */
#define MG_ERR_DRIVER        -6  /* CUDA driver entry point unavailable */
#define MG_ERR_LIMIT         -7  /* size beyond a documented maximum */

/* device status word values (mg_device_status) */
#define MG_DEV_OK             0
#define MG_DEV_WAIT_TIMEOUT   1  /* a bounded mbarrier wait ran out; results invalid */
#define MG_DEV_CAPACITY       2  /* expert-parallel receive buffer too small; detail = rank */
#define MG_DEV_BOUNDS         3  /* checked build (-DMG_BOUNDS_CHECK) only: a row index read from a table lay outside
                                    its buffer; the access was skipped; detail = 103 scatter, 104 combine,
                                    105 duplicate fill, 106 pushed return */

/* stages of mg_moe_forward, in launch order (mg_stage_times) */
#define MG_STAGE_GATE_LOGITS   0
#define MG_STAGE_ROUTE_TOPK    1
#define MG_STAGE_PERMUTE_PLAN  2
#define MG_STAGE_PERMUTE_ROWS  3
#define MG_STAGE_DEQUANT       4
#define MG_STAGE_EXPERT_GEMM1  5  /* gate/up projections + SiLU*mul */
#define MG_STAGE_EXPERT_GEMM2  6  /* down projection */
#define MG_STAGE_SHARED_GEMM1  7
#define MG_STAGE_SHARED_GEMM2  8
#define MG_STAGE_COMBINE       9
#define MG_STAGE_COUNT        10

typedef struct mg_layer_desc {
  int32_t struct_bytes;    /* = sizeof(mg_layer_desc), for versioning */
  int32_t hidden;          /* H:  config.hidden_size */
  int32_t inter;           /* I:  config.moe_intermediate_size (Mixtral: intermediate_size) */
  int32_t inter_shared;    /* I_s = n_shared_experts * I, 0 = no shared expert */
  int32_t n_experts;       /* E:  config.n_routed_experts (global) */
  int32_t top_k;           /* k:  config.num_experts_per_tok */
  int32_t n_group;         /* config.n_group   (1 when ungrouped) */
  int32_t topk_group;      /* config.topk_group */
  int32_t gating;          /* MG_GATE_* */
  int32_t norm_topk_prob;  /* config.norm_topk_prob */
  float   routed_scale;    /* config.routed_scaling_factor */
  int32_t weight_format;   /* MG_WEIGHT_* */
  int32_t combine_mode;    /* MG_COMBINE_* */
  int32_t ep_rank;         /* this rank owns experts [ep_rank*E/ep_size, (ep_rank+1)*E/ep_size) */
  int32_t ep_size;         /* (modeling_deepseek_v3.py:586-587) */
} mg_layer_desc;

typedef struct mg_handle_s* mg_handle;

/* ---- handle ------------------------------------------------------------- */

/* Validates the description and binds a handle to the current CUDA device.
 * Replaces: the config reads of DeepseekV3MoE.__init__ / MoEGate.__init__
 * (modeling_deepseek_v3.py:470-492,564-611). */
int mg_create(const mg_layer_desc* desc, mg_handle* out);
int mg_destroy(mg_handle h);

/* Text of the last error returned on this thread ("" if none). */
const char* mg_last_error(void);

/* Reads (and clears) the device status word; the caller must have synchronised
 * the streams it used.  *code gets MG_DEV_*; *detail a kernel-specific value. */
int mg_device_status(mg_handle h, int32_t* code, int32_t* detail);

/* The same two words copied to host_words[2] (pinned host memory) by an asynchronous copy on `stream`:
 * no host synchronisation and no clearing.  A caller that cannot afford a synchronising read after every
 * forward (the expert-parallel layer) enqueues this behind its kernels and looks at the words once an
 * event recorded after it has completed; a non-zero code is then fetched and cleared with
 * mg_device_status.  No counterpart in the reference. */
int mg_device_status_async(mg_handle h, int32_t* host_words, void* stream);

/* Sets aside `bytes` of the current device's L2 for accesses with the "evict last" policy
 * (cudaLimitPersistingL2CacheSize: a limit of this process's context, gone when the process ends);
 * *granted receives what the device allows.  The set-aside serves normal accesses too while no such
 * lines occupy it.  No counterpart in the reference. */
int mg_l2_set_aside(size_t bytes, size_t* granted);

/* ---- sizes -------------------------------------------------------------- */

/* Bytes of the packed weight buffer for the experts this rank owns (+ shared
 * expert).  Replaces the per-expert slots of GPU_Weight_Buffer
 * (core/GPU_Weight_Buffer/GPU_Weight_Buffer.cpp:64-101). */
int mg_packed_weight_bytes(mg_handle h, size_t* bytes);

/* Bytes of workspace mg_moe_forward needs for up to max_tokens local tokens and
 * up to max_rows rows routed to this rank's experts (max_rows = 0 means
 * max_tokens * top_k, the single-GPU bound). */
int mg_workspace_bytes(mg_handle h, int64_t max_tokens, int64_t max_rows, size_t* bytes);

/* Rows of the expert-sorted buffers for n_rows routed rows: every expert's
 * segment starts on a 128-row boundary, so up to 127 pad rows per expert. */
int mg_padded_rows(mg_handle h, int64_t n_rows, int64_t* padded);

/* ---- weights ------------------------------------------------------------ */

/* Copies one expert's three matrices ([I,H] gate_proj, [I,H] up_proj, [H,I]
 * down_proj, row-major, as nn.Linear stores them: modeling_deepseek_v3.py:439-467;
 * Mixtral: w1, w3, w2) into the packed buffer.  local_expert in [0, E/ep_size),
 * or -1 for the shared expert ([I_s,H],[I_s,H],[H,I_s]).  For
 * MG_WEIGHT_FP8_BLOCK128 the matrices are e4m3 bytes and d_*_scale are the fp32
 * [ceil(rows/128), ceil(cols/128)] weight_scale_inv tensors; for MG_WEIGHT_BF16
 * the scale pointers are ignored.  The shared expert is always bf16.
 * Replaces HtoD copy into a slot + Expert_Wrapper's per-call parameter binding
 * (moe_gen/models/Wrapper.py:470-491). */
int mg_pack_expert(mg_handle h, int32_t local_expert,
                   const void* d_gate, const void* d_up, const void* d_down,
                   const float* d_gate_scale, const float* d_up_scale, const float* d_down_scale,
                   void* d_packed, void* stream);

/* De-quantises an e4m3 [rows,cols] matrix with 128x128 block scales to bf16:
 * bf16(float(q) * scale[r/128][c/128]).  Replaces deepseek_v3_dequantization
 * (moe_gen/models/Wrapper.py:109-138). */
int mg_dequant_fp8_block128(const void* d_q, const float* d_scale_inv, int64_t rows, int64_t cols,
                            void* d_out_bf16, void* stream);

/* ---- stages ------------------------------------------------------------- */

/* logits[T,E] (fp32) = x[T,H] (bf16) . gate_w[E,H]^T (bf16), fp32 accumulation
 * on the tensor cores.  For MG_GATE_SOFTMAX_TOPK_RENORM the logits are rounded to
 * bf16 (the Mixtral router is a bf16 nn.Linear) and stored widened to fp32.
 * Replaces F.linear(x.float(), W.float()) (modeling_deepseek_v3.py:503-508). */
int mg_gate_logits(mg_handle h, const void* d_x, const void* d_gate_w, int64_t n_tokens,
                   float* d_logits, void* stream);

/* Scoring + top-k from fp32 logits: topk_idx[T,k] (int32, global expert ids,
 * slot order = selection score descending, equal scores -> lower id) and
 * topk_w[T,k] (fp32).  d_bias[E] (fp32) only for MG_GATE_SIGMOID_NOAUX_TC.
 * Replaces MoEGate.forward after the logits (modeling_deepseek_v2.py:493-533,
 * modeling_deepseek_v3.py:509-561). */
int mg_route_topk(mg_handle h, const float* d_logits, const float* d_bias, int64_t n_tokens,
                  int32_t* d_topk_idx, float* d_topk_w, void* stream);

/* Router product and top-k in one call, with the near-tie fix-up: mg_gate_logits, mg_route_topk, then
 * every token whose pick the tensor-core product's rounding could have changed (its last kept expert or
 * group leads the best rejected one by less than a logits error of (6e-9 * H + 4e-6) * max(1, max|logit|)
 * allows, four times the error measured for the product) has the logits that can decide it recomputed as
 * the rounded exact sum (bf16 products accumulated in fp64) and is routed again.  The selection is that
 * of correctly rounded fp32 logits, the value F.linear(x.float(), W.float()) approximates
 * (modeling_deepseek_v3.py:503-508); mg_moe_forward routes this way unless MG_OPT_ROUTE_FIXUP is 0.
 * d_logits[T,E]: scratch, holds the logits afterwards (recomputed entries included).
 * d_fix: scratch of mg_route_fix_bytes(T) bytes, int32; afterwards [0] = tokens routed again, [1] = of
 * which with their whole row recomputed, [2] = single logits asked for; the tokens from [4], the
 * row tokens from [4+T], the (token, expert) pairs from [4+2T] (8T+64 pairs at most; a token whose pairs
 * do not fit has its row recomputed).  For MG_GATE_SOFTMAX_TOPK_RENORM (bf16-rounded logits, where
 * near-ties are exact ties) the call is mg_gate_logits + mg_route_topk and the counts are 0. */
int mg_gate_route_topk(mg_handle h, const void* d_x, const void* d_gate_w, const float* d_bias, int64_t n_tokens,
                       float* d_logits, int32_t* d_topk_idx, float* d_topk_w, int32_t* d_fix, void* stream);
int mg_route_fix_bytes(int64_t n_tokens, size_t* bytes);

/* Histogram + prefix sums + stable placement over experts [expert_lo,
 * expert_lo + n_plan_experts): picks outside that range are skipped (dst_row=-1).
 *   counts[n]        rows per expert
 *   offsets[n+1]     exclusive scan of counts (the reference's row order)
 *   pad_offsets[n+1] the same with every expert starting on a 128-row boundary
 *   dst_row[T*k]     row of (token, slot) in the padded expert-sorted buffers;
 *                    tokens ascend inside an expert (stable sort)
 * d_plan_ws: scratch of mg_plan_ws_bytes() bytes.
 * Replaces cnts.scatter_/sum, argsort (modeling_deepseek_v3.py:630-635). */
int mg_plan_ws_bytes(mg_handle h, int64_t n_tokens, size_t* bytes);
int mg_permute_plan(mg_handle h, const int32_t* d_topk_idx, int64_t n_tokens,
                    int32_t expert_lo, int32_t n_plan_experts,
                    int32_t* d_counts, int32_t* d_offsets, int32_t* d_pad_offsets,
                    int32_t* d_dst_row, void* d_plan_ws, void* stream);

/* mg_permute_plan for callers that must not allocate device memory and have no scratch
 * buffer to hand in.  It has no counterpart in the reference.  Such callers exist around this
 * library: an engine that sized its weight and KV buffers from all the memory that was free at
 * start-up has nothing left to cudaMalloc later, and inside a decode loop a cudaMalloc would
 * stall every stream of the device.  The arguments and results are those of mg_permute_plan
 * without d_plan_ws: the scratch is a fixed array inside the library image (about 516 KiB,
 * present on every GPU that loads the library, for the life of the process).
 *  - limit: ceil(n_tokens/256) * n_experts + 2*(n_experts+1) <= 132098 words, i.e. up to 65536
 *    tokens at 512 experts (more tokens with fewer experts).  Larger requests return
 *    MG_ERR_LIMIT with a text saying so; use mg_permute_plan then;
 *  - the call makes no cudaMalloc / cudaFree and calls no allocating routine;
 *  - the first call on a device looks up the device address of the array (one
 *    cudaGetSymbolAddress, with the handle's device current); make that first call before any
 *    stream capture begins;
 *  - all calls on a device share the one array and it keeps the previous call's contents.  The
 *    kernels overwrite every word before reading it, so nothing has to be cleared, but two
 *    calls that overlap on the GPU (different streams, no ordering between them) race on it. */
int mg_permute_plan_static(mg_handle h, const int32_t* d_topk_idx, int64_t n_tokens,
                           int32_t expert_lo, int32_t n_plan_experts,
                           int32_t* d_counts, int32_t* d_offsets, int32_t* d_pad_offsets,
                           int32_t* d_dst_row, void* stream);

/* perm_x[dst_row[t*k+j], :] = x[t, :] for every pick with dst_row >= 0.
 * Replaces sorted_tokens = x[idxs // k] (modeling_deepseek_v3.py:634). */
int mg_permute_rows(mg_handle h, const void* d_x, const int32_t* d_dst_row, int64_t n_tokens,
                    void* d_perm_x, void* stream);

/* Grouped SwiGLU experts over the padded expert-sorted rows:
 *   h_buf[r, :]   = silu(perm_x[r] . Wg_e^T) * (perm_x[r] . Wu_e^T)   (bf16)
 *   out_rows[r,:] = h_buf[r] . Wd_e^T                                  (bf16)
 * for r in [pad_offsets[e], pad_offsets[e]+counts[e]).  n_rows_padded bounds the
 * buffers (rows of perm_x / h_buf / out_rows).  For FP8 layers d_dequant_ws may be NULL
 * (the kernels convert weight tiles on the fly in shared memory) or a scratch of
 * mg_dequant_ws_bytes() bytes, whose size and use follow MG_OPT_FP8_MODE (a bf16 copy of all
 * expert weights, or the ring of MG_FP8_RING); results are identical.
 * Replaces the expert loop (modeling_deepseek_v3.py:675-691) and
 * DeepseekV3MLP.forward (modeling_deepseek_v3.py:463-467). */
int mg_dequant_ws_bytes(mg_handle h, size_t* bytes);
/* Optional: starts the de-quantisation into d_dequant_ws now (on the handle's side stream,
 * ordered after what `stream` holds), so that it overlaps whatever the caller enqueues before
 * the mg_expert_ffn call with the same packed buffer, scratch and stream, which then only
 * waits for it.  No counterpart in the reference. */
int mg_dequant_start(mg_handle h, const void* d_packed, void* d_dequant_ws, void* stream);
int mg_expert_ffn(mg_handle h, const void* d_perm_x, const int32_t* d_pad_offsets,
                  const int32_t* d_counts, int64_t n_rows_padded, const void* d_packed,
                  void* d_h_buf, void* d_out_rows, void* d_dequant_ws, void* stream);

/* Shared expert on the un-permuted tokens: shared_out = MLP_shared(x).
 * hs_buf: [T, I_s] bf16 scratch.  Replaces self.shared_experts(identity)
 * (modeling_deepseek_v3.py:624-625). */
int mg_shared_ffn(mg_handle h, const void* d_x, int64_t n_tokens, const void* d_packed,
                  void* d_hs_buf, void* d_shared_out, void* stream);

/* y[t] = sum_j topk_w[t,j] * out_rows[dst_row[t*k+j]]  (+ shared_out[t] when
 * d_shared_out != NULL), arithmetic per combine_mode.  Picks with dst_row < 0
 * contribute nothing.  Replaces new_x[idxs] = outs and the weighted sum
 * (modeling_deepseek_v3.py:702-711) and y + shared (…:624-625). */
int mg_combine(mg_handle h, const void* d_out_rows, const int32_t* d_dst_row,
               const int32_t* d_topk_idx, const float* d_topk_w, const void* d_shared_out,
               int64_t n_tokens, void* d_y, void* stream);

/* ---- whole layer on one GPU (ep_size == 1) ------------------------------- */

/* y[T,H] = MoE(x[T,H]); bf16 in and out.  d_bias may be NULL unless the gating
 * needs it.  No host synchronisation.  Replaces DeepseekV3MoE.forward /
 * DeepseekV2MoE.forward / MixtralSparseMoeBlock.forward
 * (modeling_deepseek_v3.py:614-626, modeling_deepseek_v2.py:642-668). */
int mg_moe_forward(mg_handle h, const void* d_x, int64_t n_tokens,
                   const void* d_gate_w, const float* d_bias, const void* d_packed,
                   void* d_workspace, size_t workspace_bytes, void* d_y, void* stream);

/* The layer on HOST buffers: x_host / y_host are [n_tokens, H] bf16 in host memory (pinned, for the copies
 * to overlap).  Tokens are independent, so the batch goes through in chunks: chunk c+1 is copied in and
 * chunk c-1 copied out on the library's copy streams while chunk c computes on `stream`; the first and
 * last chunk are half of chunk_tokens (their copies are exposed), the ones between one and a half.  FP8
 * layers in pre-dequantise mode de-quantise once for all chunks.  d_workspace holds the staging buffers
 * and the forward's workspace: mg_host_workspace_bytes(h, n_tokens, chunk_tokens).  The call returns once
 * everything is enqueued; `stream` is ordered after the last copy, so y_host is complete when the caller
 * has synchronised it.  mg_host_chunk_plan gives the chunk sizes (no device needed).
 * Replaces the host side the reference reaches through its engine: hidden states staged to the device,
 * DeepseekV3MoE.forward, results staged back (moe_gen/engine.py:708-763 around modeling_deepseek_v3.py:614-626). */
int mg_host_chunk_plan(int64_t n_tokens, int64_t chunk_tokens, int64_t* sizes, int32_t max_chunks, int32_t* n_chunks);
int mg_host_workspace_bytes(mg_handle h, int64_t n_tokens, int64_t chunk_tokens, size_t* bytes);
int mg_moe_forward_host(mg_handle h, const void* x_host, int64_t n_tokens, const void* d_gate_w, const float* d_bias,
                        const void* d_packed, void* d_workspace, size_t workspace_bytes, void* y_host,
                        int64_t chunk_tokens, void* stream);

/* The same layer on router logits the caller computed: logits[T,E] fp32 replace the library's
 * router product, everything after it is mg_moe_forward.  The reference computes its logits with an
 * fp32 matrix product (F.linear(x.float(), W.float()), modeling_deepseek_v3.py:503-508); the
 * library's own router product accumulates on the tensor cores, whose rounding can differ in the
 * last bits and flip a selection between two experts whose scores are within about 1e-4 of each
 * other.  A caller that needs the selection of its own fp32 logits bit for bit passes them here:
 * scoring, top-k and every later stage are exact functions of these logits. */
int mg_moe_forward_from_logits(mg_handle h, const void* d_x, int64_t n_tokens, const float* d_logits,
                               const float* d_bias, const void* d_packed, void* d_workspace,
                               size_t workspace_bytes, void* d_y, void* stream);

/* ---- expert parallelism (ep_size > 1): one process per GPU ------------------- */
/* The reference's expert-parallel branch (modeling_deepseek_v3.py:636-672,692-700) exchanges
 * counts with all_to_all_single, rows with two all_to_all calls and regroups on the host.
 * Here every rank owns two buffers that all ranks map (CUDA IPC over NVLink):
 *   recv_x   [cap_rows, H]  rows routed to this rank's experts, expert-sorted and 128-padded
 *   out_rows [cap_rows, H]  the experts' outputs for those rows
 * A rank writes its tokens straight into the owners' recv_x (dispatch = the permute scatter
 * with peer destinations) and later reads the owners' out_rows (return = the combine gather
 * with peer sources).  Between the steps the ranks need a barrier (any stream-ordered
 * collective, e.g. a one-element NCCL all-reduce): after dispatch before the experts run, and
 * after the experts before combine.  Sequence per forward on each rank:
 *   mg_gate_route_topk (or mg_gate_logits + mg_route_topk), mg_ep_count -> all-gather counts -> mg_ep_place,
 *   mg_ep_dispatch, [mg_shared_ffn], barrier, mg_expert_ffn, barrier, mg_ep_combine. */

/* Device memory that can be shared with the other ranks / its 64-byte IPC handle / mapping
 * a peer's handle / unmapping.  The importing process must run on a GPU with peer access. */
int mg_ep_alloc(size_t bytes, void** d_ptr);
int mg_ep_free(void* d_ptr);
int mg_ep_export(void* d_ptr, void* handle64);
int mg_ep_import(const void* handle64, void** d_ptr);
int mg_ep_unimport(void* d_ptr);

/* counts[E]: picks per global expert among this rank's n_tokens tokens.  d_plan_ws
 * (mg_plan_ws_bytes) must stay untouched until mg_ep_place.  Replaces the histogram of
 * modeling_deepseek_v3.py:630-632. */
int mg_ep_count(mg_handle h, const int32_t* d_topk_idx, int64_t n_tokens, int32_t* d_counts,
                void* d_plan_ws, void* stream);

/* From the all-gathered counts [ep_size][E] (row s = rank s): recv_counts[E/ep_size] and
 * recv_pad[E/ep_size+1] of this rank's experts (inputs of mg_expert_ffn), and dst[T*k] =
 * owner_rank << 24 | row in the owner's buffers.  Inside an expert's segment the rows of rank
 * 0 come first, then rank 1, ..., tokens ascending.  If a rank would receive more than
 * cap_rows rows, picks sent to it are dropped (dst < 0) and the device status becomes
 * MG_DEV_CAPACITY.  Replaces all_to_all_single + host split computation + numpy argsort
 * (modeling_deepseek_v3.py:636-671). */
int mg_ep_place(mg_handle h, const int32_t* d_topk_idx, int64_t n_tokens, const int32_t* d_counts_all,
                int64_t cap_rows, void* d_plan_ws, int32_t* d_recv_counts, int32_t* d_recv_pad,
                int32_t* d_dst, void* stream);

/* peer_recv[ep_size]: every rank's recv_x as mapped in this process (own buffer at own rank).
 * Replaces dist.all_to_all of the sorted rows (modeling_deepseek_v3.py:656-659). */
int mg_ep_dispatch(mg_handle h, const void* d_x, const int32_t* d_dst, int64_t n_tokens,
                   void* const* peer_recv, void* stream);

/* The same dispatch with one row per (token, destination rank) on the wire instead of one per
 * (token, expert): with group-limited routing several of a token's experts live on the same rank
 * (DeepSeek-V3 on 8 ranks: 8 picks on at most 4 ranks).  Every rank owns a duplicate table of
 * cap_rows int32 next to its recv_x (peer_dup[ep_size], mapped like peer_recv):
 *   1. the owner sets its table to -1 (mg_ep_clear_duplicates) before the ranks exchange counts,
 *   2. mg_ep_dispatch_dedup sends the row of a token's first pick on a rank and, for its later
 *      picks on that rank, writes the first pick's row number into the owner's table,
 *   3. after the barrier that follows the dispatch the owner copies those rows inside its own
 *      recv_x (mg_ep_fill_duplicates), then runs mg_expert_ffn.
 * recv_x ends up bit-identical to what mg_ep_dispatch leaves.  No reference counterpart: its
 * all_to_all sends every (token, expert) row (modeling_deepseek_v3.py:656-659). */
int mg_ep_clear_duplicates(mg_handle h, void* d_dup, int64_t cap_rows, void* stream);
int mg_ep_dispatch_dedup(mg_handle h, const void* d_x, const int32_t* d_dst, int64_t n_tokens,
                         void* const* peer_recv, void* const* peer_dup, void* stream);
int mg_ep_fill_duplicates(mg_handle h, void* d_recv_x, const void* d_dup, int64_t cap_rows, void* stream);

/* The return as a push that overlaps the experts (no counterpart in the reference, whose return is a third
 * all_to_all after the expert loop, modeling_deepseek_v3.py:692-700).  Every rank owns two more shared
 * buffers: a return table back[cap_rows] (int32, set to -1 with mg_ep_clear_duplicates before the ranks
 * exchange counts) and a return buffer ret[T_local * k, H] (bf16).
 *   1. mg_ep_dispatch_back is mg_ep_dispatch / mg_ep_dispatch_dedup (peer_dup NULL / given) that also
 *      writes, into the owner's return table at every pick's row, rank << 24 | (token * k + slot);
 *   2. mg_ep_expert_ffn_return is mg_expert_ffn whose down projection runs in n_parts parts of experts
 *      (the chunks of pre-dequantise mode when that is on): as soon as a part is done, its output rows are
 *      stored into the token owners' return buffers on a side stream while the next part computes
 *      (rows of this rank's own tokens stay in d_out_rows); the call returns with `stream` ordered
 *      after the last store;
 *   3. after a barrier among the ranks, mg_ep_combine_slots sums a token's k rows from its own rank's
 *      return buffer, or from this rank's d_out_rows for picks of its own experts (d_dst tells which
 *      is which and which picks were dropped): local, HBM-speed. */
int mg_ep_dispatch_back(mg_handle h, const void* d_x, const int32_t* d_dst, int64_t n_tokens,
                        void* const* peer_recv, void* const* peer_dup, void* const* peer_back, void* stream);
int mg_ep_expert_ffn_return(mg_handle h, const void* d_recv_x, const int32_t* d_recv_pad,
                            const int32_t* d_recv_counts, int64_t cap_rows, const void* d_packed, void* d_h_buf,
                            void* d_out_rows, void* d_dequant_ws, const int32_t* d_back, void* const* peer_ret,
                            int32_t n_parts, void* stream);
int mg_ep_combine_slots(mg_handle h, const void* d_ret, const void* d_out_rows, const int32_t* d_dst,
                        const int32_t* d_topk_idx, const float* d_topk_w, const void* d_shared_out, int64_t n_tokens,
                        void* d_y, void* stream);

/* The return through the copy engines (no counterpart in the reference either).  The rows this rank's
 * experts computed for one source rank and one expert are contiguous in d_out_rows, and that source rank
 * wants them contiguous too, at the place its own expert-sorted order gives expert e.  So the return is
 * one device-to-device copy per (expert, source rank), issued on a side stream as soon as the part of the
 * down projection that holds the expert is done, into the source rank's return buffer ret[T_local * k, H]
 * (its own rank included): no SM stores a remote row.  The sizes are the gathered counts, which this call
 * needs in HOST memory: h_counts_all[ep_size][n_experts], i.e. the caller reads them back after the
 * all-gather (one synchronising 4 * ep_size * n_experts byte copy per forward).
 *   mg_ep_mirror_delta   d_delta[e] = what turns a row number of the owner's layout (d_dst) into a row of
 *                        this rank's return buffer, from the gathered counts on the device;
 *   mg_ep_combine_mirror the combine over the return buffer alone (local, HBM speed), after the barrier
 *                        that follows the experts.
 * Bit-identical to the other two returns. */
int mg_ep_expert_ffn_copy_return(mg_handle h, const void* d_recv_x, const int32_t* d_recv_pad,
                                 const int32_t* d_recv_counts, int64_t cap_rows, const void* d_packed, void* d_h_buf,
                                 void* d_out_rows, void* d_dequant_ws, const int32_t* h_counts_all,
                                 void* const* peer_ret, int32_t n_parts, void* stream);
int mg_ep_mirror_delta(mg_handle h, const int32_t* d_counts_all, int32_t* d_delta, void* stream);
int mg_ep_combine_mirror(mg_handle h, const void* d_mirror, const int32_t* d_dst, const int32_t* d_delta,
                         const int32_t* d_topk_idx, const float* d_topk_w, const void* d_shared_out,
                         int64_t n_tokens, void* d_y, void* stream);

/* peer_out[ep_size]: every rank's out_rows.  Replaces the return all_to_all and the
 * weighted sum (modeling_deepseek_v3.py:692-710). */
int mg_ep_combine(mg_handle h, void* const* peer_out, const int32_t* d_dst, const int32_t* d_topk_idx,
                  const float* d_topk_w, const void* d_shared_out, int64_t n_tokens, void* d_y,
                  void* stream);

/* ---- decoder-layer glue either side of the block -------------------------------------
 * The caller of the MoE block normalises the residual stream in front of it and adds the block's
 * output back (modeling_deepseek_v3.py:1361-1365: residual = h; h = post_attention_layernorm(h);
 * h = mlp(h); h = residual + h).
 *
 * mg_rmsnorm: out[T,H] = weight * bf16(x * rsqrt(mean(x^2) + eps)); x, weight [H], out bf16;
 * fp32 statistics (DeepseekV3RMSNorm.forward, modeling_deepseek_v3.py:125-150, with the bf16
 * weight the model holds after model.to(bfloat16)).
 *
 * mg_moe_block_forward: out = hidden + moe(rmsnorm(hidden)).  The normalised rows go to d_xnorm
 * ([T,H] bf16, caller's scratch, distinct from hidden and out); the residual add happens in the
 * combine kernel (the block's output is rounded to bf16 first, as the reference's bf16 module
 * output is), so d_out may be d_hidden.  Workspace as for mg_moe_forward. */
int mg_rmsnorm(mg_handle h, const void* d_x, const void* d_weight, float eps, int64_t n_tokens,
               void* d_out, void* stream);
int mg_moe_block_forward(mg_handle h, const void* d_hidden, const void* d_norm_weight, float eps,
                         int64_t n_tokens, const void* d_gate_w, const float* d_bias, const void* d_packed,
                         void* d_xnorm, void* d_workspace, size_t workspace_bytes, void* d_out, void* stream);

/* Pointers into a workspace laid out by mg_moe_forward, for tests and tools:
 * which = 0 logits, 1 topk_idx, 2 topk_w, 3 counts, 4 offsets, 5 pad_offsets,
 * 6 dst_row, 7 perm_x, 8 h_buf, 9 out_rows. */
int mg_workspace_ptr(mg_handle h, void* d_workspace, int64_t max_tokens, int64_t max_rows,
                     int32_t which, void** ptr);

/* Self-test of the failure path (no counterpart in the reference, whose get_weights polls
 * forever: core/GPU_Weight_Buffer/GPU_Weight_Buffer.cpp:171-221): launches one thread that
 * waits, with the GEMM kernels' bounded-wait helper and a limit of limit_ms (1..1000), on a
 * barrier nothing completes.  After synchronising, mg_device_status must report
 * MG_DEV_WAIT_TIMEOUT with detail 99 and the context must still be usable. */
int mg_selftest_wait_timeout(mg_handle h, int32_t limit_ms, void* stream);

/* Number of kernel launches the last mg_moe_forward on this handle issued. */
int mg_last_launch_count(mg_handle h, int32_t* launches);

/* Options (no counterpart in the reference).
 * MG_OPT_FP8_MODE, for MG_WEIGHT_FP8_BLOCK128 layers: where the grouped GEMMs get their bf16 operands
 * (the reference de-quantises every expert's matrices on every expert call, moe_gen/models/Wrapper.py:481-491):
 *   MG_FP8_IN_KERNEL   every CTA converts the FP8 weight tiles of its own row tiles in shared memory; no
 *                      scratch; a weight is converted once per 128 or 256 rows that use it;
 *   MG_FP8_PREDEQUANT  a bf16 copy of all local expert weights in scratch (2 bytes per weight), written by
 *                      a separate pass on a side stream one chunk of experts ahead of the bf16 GEMMs;
 *   MG_FP8_RING        the GEMM kernel's CTAs convert every weight once per expert into a bf16 ring of
 *                      MG_OPT_RING_BYTES and fetch their B tiles from it by TMA: no bf16 copy of the weights,
 *                      58 MB of scratch; measured 5 % slower than MG_FP8_PREDEQUANT at 65536 tokens of the
 *                      DeepSeek-V3 layer (the ring does not stay in L2), so only on request;
 *   MG_FP8_AUTO        (default) in-kernel while an expert sees fewer than 1024 rows on average
 *                      (measured cross-over on the DeepSeek-V3 shape), else pre-dequantise.
 * All give bit-identical results.  Set before asking mg_workspace_bytes / mg_dequant_ws_bytes. */
#define MG_OPT_FP8_MODE    1
#define MG_FP8_AUTO        0
#define MG_FP8_PREDEQUANT  1
#define MG_FP8_IN_KERNEL   2
#define MG_FP8_RING        3
/* MG_OPT_RING_BYTES: size of the ring of MG_FP8_RING in MiB (default 56: it has to fit in the 126 MB L2
 * next to the activations in flight).  Set before asking mg_workspace_bytes / mg_dequant_ws_bytes. */
#define MG_OPT_RING_BYTES  7
/* MG_OPT_RING_PERSIST: 1 = the ring's stores and loads carry the L2 "evict last" policy, so that the ring
 * outlives the streaming traffic beside it; it takes effect inside the part of L2 that the process has
 * set aside for such accesses (mg_l2_set_aside).  0 (default) = ordinary accesses. */
#define MG_OPT_RING_PERSIST 8
/* MG_OPT_ROWS_BOUND: rows of the expert-sorted buffers the caller hands to the stage-level entry points
 * (mg_permute_rows, mg_combine, the expert-parallel dispatch and combine calls); 0 = not declared.  Only a
 * library built with -DMG_BOUNDS_CHECK looks at it: its row-moving kernels then compare every row index they
 * read from a table with this bound and report MG_DEV_BOUNDS instead of touching memory outside the buffer.
 * mg_moe_forward sets its own bound. */
#define MG_OPT_ROWS_BOUND 9
/* MG_OPT_ROUTE_FIXUP: 1 (default) = mg_moe_forward re-routes near-tie tokens from exactly recomputed logits
 * (see mg_gate_route_topk); 0 = it routes every token from the tensor-core product as it is. */
#define MG_OPT_ROUTE_FIXUP 10
/* MG_OPT_PAIR_GEMM: 1 = the bf16 expert GEMMs run on SM pairs (clusters of two CTAs,
 * tcgen05 cta_group::2, 256x256 tiles); 0 = one CTA per SM, 128x256 tiles. */
#define MG_OPT_PAIR_GEMM   2
/* MG_OPT_FP8_M256: tile height of the convert-in-the-GEMM kernels: 0 = 128 rows, 1 (default) =
 * 256 rows (one converted weight tile feeds two MMAs) when experts average at least 120 rows,
 * 2 = always 256. */
#define MG_OPT_FP8_M256    4
/* MG_OPT_BATCH_TOKENS: a caller that feeds one batch through mg_moe_forward in chunks sets the
 * batch's total token count here (0 = off, the default); MG_FP8_AUTO then decides on the larger
 * of this and the call's T, because the de-quantised copy can serve every chunk
 * (MG_OPT_KEEP_DEQUANT).  Set before asking mg_workspace_bytes. */
#define MG_OPT_BATCH_TOKENS 5
/* MG_OPT_SHARED_EARLY: 1 = mg_moe_forward runs the shared expert's two GEMMs on a library
 * stream beside the top-k, plan and scatter kernels (ordered after the router GEMM by an event,
 * joined before the combine); 0 = on the caller's stream after the routed experts; 2 (default) = 1 for
 * calls of at most 4096 tokens, where the kernels are short enough to gain from running side by
 * side, else 0.  When the shared expert runs early the
 * stage times of the shared expert (mg_stage_times) read as the wait at the join, not as its GEMMs. */
#define MG_OPT_SHARED_EARLY 6
/* MG_OPT_KEEP_DEQUANT: 1 = in pre-dequantise mode, a call may reuse the bf16 copy the previous
 * call on this handle left in the same scratch, if the packed buffer and the stream are the
 * same and no expert was re-packed in between.  Meant for the token chunks of ONE logical
 * forward (MoELayer.forward_host sets it around its chunk loop and clears it afterwards), so
 * that the weights are de-quantised once per forward, not once per chunk.  The caller must
 * not touch the scratch in between.  2 = the same, and the calls may be on different streams
 * whose ordering the caller guarantees (the expert-parallel micro-batches do). */
#define MG_OPT_KEEP_DEQUANT 3
int mg_set_option(mg_handle h, int32_t option, int32_t value);

/* Per-stage device times of mg_moe_forward (no counterpart in the reference, whose
 * timers are commented out: moe_gen/models/Wrapper.py:112-137).  When enabled, the
 * forward records a CUDA event on `stream` after every stage; after the caller has
 * synchronised, mg_stage_times() returns the milliseconds per MG_STAGE_* (0 for stages
 * the layer does not have), averaged over the forwards since timing was enabled (the
 * last 32 if there were more). */
int mg_set_stage_timing(mg_handle h, int32_t enable);
int mg_stage_times(mg_handle h, float* ms, int32_t n);

#ifdef __cplusplus
}
#endif
#endif /* MOEGEN_B200_H */
