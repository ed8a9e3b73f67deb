// Grouped GEMM for sm_100a: C[rows, N] = A[rows, K] . B_e[N, K]^T per expert segment,
// bf16 operands, fp32 accumulation in tensor memory.
//
//   * persistent kernel, one CTA per SM, 6 warps: warp 0 = TMA producer, warp 1 = MMA
//     issuer + TMEM owner, warps 2-5 = epilogue (one TMEM lane quarter each);
//   * operands arrive by TMA (cp.async.bulk.tensor, no multicast) into a 4-stage ring of
//     128B-swizzled K-major tiles (A 128x64, B 256x64) guarded by mbarriers;
//   * tcgen05.mma cta_group::1 kind::f16, M=128, N<=256, K=16 per instruction, accumulating
//     into one of two 256-column TMEM buffers so the epilogue of tile i overlaps the MMAs of
//     tile i+1;
//   * epilogue reads TMEM with tcgen05.ld (one row per thread) and applies SiLU(gate)*up,
//     or stores plain bf16 / fp32;
//   * the tile list is derived on the device from the padded expert offsets (every expert
//     starts on a 128-row boundary, so a tile never straddles two experts) — no host sync;
//   * W8A16 variant (F8B): the B tile arrives as FP8 e4m3 bytes; eight converter warps turn it
//     into the bf16 operand tile in shared memory, bf16(float(q) * scale[row/128][k/128]) —
//     bit-identical to de-quantising the whole matrix first — in the same 128B-swizzled
//     layout TMA would have produced, then hand it to the MMA warp through an mbarrier;
//   * every mbarrier wait is bounded; on expiry the kernel records MG_DEV_WAIT_TIMEOUT, all
//     roles leave their loops, TMEM is freed and the kernel returns.
#include <cuda_fp8.h>

#include "common.cuh"

namespace mg {

constexpr int BM = 128;
constexpr int BK = 64;                       // 64 bf16 = 128 bytes = one swizzle row
constexpr int BN_MAX = 256;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;         // 16 KiB
constexpr int B_BYTES = BN_MAX * BK * 2;     // 32 KiB
constexpr int B8_BYTES = BN_MAX * BK;         // 16 KiB: the same tile as FP8 bytes
constexpr int B_SLOTS = 3;                   // converted bf16 B tiles in flight (W8A16 variant)
constexpr int GEMM_THREADS = 192;
constexpr int CONVERT_THREADS = 256;
constexpr int NUM_BARS = 2 * STAGES + 4 + 2 * B_SLOTS;

template <bool F8B>
struct Cfg {
  static constexpr int STAGE_BYTES = A_BYTES + (F8B ? B8_BYTES : B_BYTES);
  static constexpr int NS = F8B ? 3 : STAGES;       // W8A16: a stage less, a converted-tile slot more
  static constexpr int RING_BYTES = NS * STAGE_BYTES + (F8B ? B_SLOTS * B_BYTES : 0);
  static constexpr int THREADS = GEMM_THREADS + (F8B ? CONVERT_THREADS : 0);
};
constexpr int TMEM_COLS = 512;
constexpr int ACC_COLS = 256;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct GemmArgs {
  const int32_t* pad_offsets;   // nullptr => dense
  const int32_t* counts;
  int n_groups;
  int dense_rows;
  int n_tiles;                  // tiles along N per group
  int bn;                       // UMMA N
  int n_per_group;              // rows of B per group
  int k_blocks;
  int group_m;
  uint32_t idesc;
  const float* scales;          // W8A16: [rows of B / 128][K / 128] fp32
  int scale_cols;               // K / 128
  void* out;
  long long ldo;
  int32_t* status;
};

constexpr size_t SMEM_CTRL_BYTES = 8 * NUM_BARS + 16 + 4 * (2 * kMaxExperts + 2);
template <bool F8B>
constexpr size_t gemm_smem_bytes() { return 1024 + Cfg<F8B>::RING_BYTES + SMEM_CTRL_BYTES + 1024 + 4 * 2 * 2048; }

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// nanoseconds; the two halves are read separately and the high half checked, so that a carry of the low
// half between the reads cannot produce a value that is off by 2^32 ns
__device__ __forceinline__ unsigned long long global_timer() {
  uint32_t hi, lo, hi2;
  do {
    asm volatile("mov.u32 %0, %%globaltimer_hi;" : "=r"(hi));
    asm volatile("mov.u32 %0, %%globaltimer_lo;" : "=r"(lo));
    asm volatile("mov.u32 %0, %%globaltimer_hi;" : "=r"(hi2));
  } while (hi != hi2);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}
// The limit of a bounded wait has run out.  The 64-bit timer is read as two halves; a read that straddles
// a carry of the low half can come out far too small or too large, so the difference is taken as a
// signed number (a reading below t0 never counts) and an expiry must be seen by two readings in a row.
__device__ __forceinline__ bool timed_out(unsigned long long t0, unsigned long long limit_ns) {
  const long long d1 = static_cast<long long>(global_timer() - t0);
  if (d1 <= static_cast<long long>(limit_ns)) return false;
  const long long d2 = static_cast<long long>(global_timer() - t0);
  return d2 > static_cast<long long>(limit_ns) && d2 >= d1;
}
// Bounded wait.  Returns false if the wait ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status, int where,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (timed_out(t0, limit_ns)) {
        *abort_flag = 1;
        if (atomicCAS(status, MG_DEV_OK, MG_DEV_WAIT_TIMEOUT) == MG_DEV_OK) status[1] = where;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// L2 residency hints for data that is written once and read many times before it is overwritten
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar,
                                                 uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void st_global_hint16(void* ptr, const uint4& v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(ptr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w), "l"(pol)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 128B-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);        // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                        // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                        // SWIZZLE_128B
  return d;
}

// ---- tile scheduler -------------------------------------------------------------------
struct Tile {
  int row0;        // first row of A / C
  int valid_rows;  // rows of the tile that belong to the expert
  int b_row;       // first row of B
  int n_idx;       // tile index along N
};

__device__ __forceinline__ Tile locate_tile(int tile, const int* s_pad, const int* s_cnt,
                                            int n_groups, int n_tiles, int n_per_group, int bn,
                                            int group_m) {
  // greatest e with prefix(e) <= tile, prefix(e) = (s_pad[e]-s_pad[0])/BM*n_tiles (the offsets
  // may be a slice of a longer table, so they need not start at 0)
  const int base0 = s_pad[0];
  int lo = 0, hi = n_groups;  // answer in [lo, hi)
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (((s_pad[mid] - base0) / BM) * n_tiles <= tile) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int local = tile - ((s_pad[e] - base0) / BM) * n_tiles;
  const int m_e = (s_pad[e + 1] - s_pad[e]) / BM;
  const int per_group = group_m * n_tiles;
  const int grp = local / per_group;
  const int rem = local - grp * per_group;
  const int gm = min(group_m, m_e - grp * group_m);
  const int n = rem / gm;
  const int m = grp * group_m + (rem - n * gm);
  Tile t;
  t.row0 = s_pad[e] + m * BM;
  t.valid_rows = min(BM, s_cnt[e] - m * BM);
  t.b_row = e * n_per_group + n * bn;
  t.n_idx = n;
  return t;
}

__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// 16 FP8 values -> 16 bf16 (two 16-byte chunks), each bf16(float(q) * s)
__device__ __forceinline__ void convert16(const uint4& q, float s, uint4& lo, uint4& hi) {
  const __nv_fp8x2_storage_t* p = reinterpret_cast<const __nv_fp8x2_storage_t*>(&q);
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p[i], __NV_E4M3);
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
    __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(f.x, s), __fmul_rn(f.y, s));
    o[i] = *reinterpret_cast<uint32_t*>(&b);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// ---- epilogue ---------------------------------------------------------------------------
// bf16 outputs leave through shared memory: each epilogue warp owns 32 rows, writes a 32-row x
// 32-column piece (2 KiB) into one of its two staging buffers and one lane hands it to TMA
// (cp.async.bulk.tensor store), so the global writes are full lines issued asynchronously
// instead of 64-byte runs per thread.  Rows of a piece that lie in an expert's padding are
// written too (they belong to nobody); rows beyond the tensor are clipped by TMA.
constexpr int EPI_PIECE_BYTES = 32 * 64;                 // 32 rows x 32 bf16

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0),
               "r"(c1), "r"(src)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

struct EpiWarp {
  uint8_t* stage;      // this warp's staging buffers
  uint32_t pieces;     // pieces issued so far (selects the buffer)
  int lane;
  int nbuf;            // 2 staging buffers, or 1 where shared memory is short
};

// stores 32 bf16 (packed[16]) of this thread's row as one row of the warp's piece and sends it
__device__ __forceinline__ void send_piece(EpiWarp& w, const CUtensorMap* tmC, const uint32_t* packed, int col0,
                                           int row_first, bool warp_live) {
  if (!warp_live) return;                                // uniform per warp
  uint8_t* buf = w.stage + (w.nbuf == 2 ? (w.pieces & 1u) : 0u) * EPI_PIECE_BYTES;
  // the store that last used this buffer has finished reading it
  if (w.lane == 0) {
    if (w.nbuf == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  __syncwarp();
  // the piece is laid out as TMA's SWIZZLE_64B expects it (16-byte chunk index XOR bits 7-8 of the
  // offset = (row / 2) mod 4), which also spreads a quarter-warp's stores over all banks
  uint4* dst = reinterpret_cast<uint4*>(buf + w.lane * 64);
  const int sw = (w.lane >> 1) & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    dst[i ^ sw] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (w.lane == 0) tma_store_2d(tmC, col0, row_first, smem_u32(buf));
  ++w.pieces;
}

// One thread = one accumulator row (TMEM lane): read it in 32-column pieces, apply the epilogue.
// `row` is this thread's global row, `row_first` the first row of its warp, `live` whether the
// row belongs to the expert, `warp_live` whether any row of the warp does.
template <int EPI>
__device__ __forceinline__ void epilogue_rows(uint32_t taddr, const GemmArgs& g, const CUtensorMap* tmC, EpiWarp& w,
                                              long long row, int row_first, int n_idx, bool live, bool warp_live) {
  if (EPI == EPI_SWIGLU_BF16) {
    const int half = g.bn >> 1;
    for (int c = 0; c < half; c += 32) {
      uint32_t gr[32], ur[32];
      tc_ld32(taddr + c, gr);
      tc_ld32(taddr + half + c, ur);
      tc_ld_wait();
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float h0 = silu_f(__uint_as_float(gr[2 * i])) * __uint_as_float(ur[2 * i]);
        float h1 = silu_f(__uint_as_float(gr[2 * i + 1])) * __uint_as_float(ur[2 * i + 1]);
        __nv_bfloat162 b2 = __floats2bfloat162_rn(h0, h1);
        packed[i] = *reinterpret_cast<uint32_t*>(&b2);
      }
      send_piece(w, tmC, packed, n_idx * half + c, row_first, warp_live);
    }
  } else if (EPI == EPI_PLAIN_BF16) {
    for (int c = 0; c < g.bn; c += 32) {
      uint32_t r[32];
      tc_ld32(taddr + c, r);
      tc_ld_wait();
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        packed[i] = *reinterpret_cast<uint32_t*>(&b2);
      }
      send_piece(w, tmC, packed, n_idx * g.bn + c, row_first, warp_live);
    }
  } else {
    // fp32 output, N = n_per_group columns in one tile (the router logits): direct stores
    float* orow = static_cast<float*>(g.out) + row * g.ldo;
    for (int c = 0; c < g.n_per_group; c += 32) {
      uint32_t r[32];
      tc_ld32(taddr + c, r);
      tc_ld_wait();
      if (live) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          if (c + i < g.n_per_group) {
            float4 v;
            v.x = __uint_as_float(r[i]); v.y = __uint_as_float(r[i + 1]);
            v.z = __uint_as_float(r[i + 2]); v.w = __uint_as_float(r[i + 3]);
            if (EPI == EPI_ROUND_BF16_F32) {
              v.x = __bfloat162float(__float2bfloat16_rn(v.x)); v.y = __bfloat162float(__float2bfloat16_rn(v.y));
              v.z = __bfloat162float(__float2bfloat16_rn(v.z)); v.w = __bfloat162float(__float2bfloat16_rn(v.w));
            }
            *reinterpret_cast<float4*>(orow + c + i) = v;
          }
        }
      }
    }
  }
}

// all stores of this warp have left shared memory and reached global memory
__device__ __forceinline__ void epilogue_drain(const EpiWarp& w) {
  if (w.lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __syncwarp();
}

// The scales of one 128-row block of B for a whole tile (one per 128 columns of K, at most 128 of
// them) are fetched once per tile, spread over the lanes of a warp, and handed out by shuffle: a
// global load per k-block would put an L2 round trip on every k-block's critical path.
struct TileScales {
  float v[4];
  __device__ __forceinline__ void load(const float* row, int n_cols, int lane) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (i * 32 + lane) < n_cols ? __ldg(row + i * 32 + lane) : 0.f;
  }
  __device__ __forceinline__ float get(int col) const {
    float x = v[0];
    if (col >= 32) x = v[1];
    if (col >= 64) x = v[2];
    if (col >= 96) x = v[3];
    return __shfl_sync(0xFFFFFFFFu, x, col & 31);
  }
};

template <int EPI, bool F8B>
__global__ void __launch_bounds__(Cfg<F8B>::THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmArgs g) {
  constexpr int STAGE_BYTES = Cfg<F8B>::STAGE_BYTES;
  constexpr int NS = Cfg<F8B>::NS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg<F8B>::RING_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint64_t* bready = bars + 2 * STAGES + 4;            // converted B tile ready (W8A16)
  uint64_t* bfree = bars + 2 * STAGES + 4 + B_SLOTS;   // converted B tile consumed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_pad = reinterpret_cast<int*>(tmem_slot + 4);
  int* s_cnt = s_pad + kMaxExperts + 1;
  uint8_t* epi_stage = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem + Cfg<F8B>::RING_BYTES + SMEM_CTRL_BYTES) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull[a]), 1); mbar_init(smem_u32(&tempty[a]), 4); }
    for (int j = 0; j < B_SLOTS; ++j) { mbar_init(smem_u32(&bready[j]), CONVERT_THREADS / 64); mbar_init(smem_u32(&bfree[j]), 1); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (g.pad_offsets != nullptr) {
    for (int i = threadIdx.x; i <= g.n_groups; i += blockDim.x) s_pad[i] = g.pad_offsets[i];
    for (int i = threadIdx.x; i < g.n_groups; i += blockDim.x) s_cnt[i] = g.counts[i];
  } else if (threadIdx.x == 0) {
    s_pad[0] = 0;
    s_pad[1] = (g.dense_rows + BM - 1) / BM * BM;
    s_cnt[0] = g.dense_rows;
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = ((s_pad[g.n_groups] - s_pad[0]) / BM) * g.n_tiles;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bslot_base = smem_base + NS * STAGE_BYTES;   // W8A16: converted B tiles

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      const uint32_t tx_bytes = A_BYTES + static_cast<uint32_t>(g.bn) * BK * (F8B ? 1 : 2);
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const Tile t = locate_tile(tile, s_pad, s_cnt, g.n_groups, g.n_tiles, g.n_per_group, g.bn, g.group_m);
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % NS, ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, abort_flag, g.status, 1)) break;
          const uint32_t fb = smem_u32(&full[s]);
          mbar_expect_tx(fb, tx_bytes);
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          tma_load_2d(sa, &tmA, kb * BK, t.row0, fb);
          tma_load_2d(sa + A_BYTES, &tmB, kb * BK, t.b_row, fb);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&tempty[acc]), acc_ph ^ 1u, abort_flag, g.status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        bool ok = true;
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % NS, ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&full[s]), ph, abort_flag, g.status, 3)) { ok = false; break; }
          const uint32_t j = it % B_SLOTS, jph = (it / B_SLOTS) & 1u;
          if (F8B && !mbar_wait(smem_u32(&bready[j]), jph, abort_flag, g.status, 5)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(F8B ? bslot_base + j * B_BYTES : sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 bf16 = 32 bytes = 2 sixteen-byte units further along K inside the swizzle row
            tc_mma_bf16(d_tmem, da + 2 * k, db + 2 * k, g.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(smem_u32(&empty[s]));   // frees the stage once these MMAs have read it
          if (F8B) tc_commit(smem_u32(&bfree[j]));
        }
        if (!ok) break;
        tc_commit(smem_u32(&tfull[acc]));   // accumulator complete
      }
    }
  } else if (F8B && warp >= 6) {
    // ---------------- FP8 -> bf16 converter (W8A16) ----------------
    // Two groups of 4 warps take alternate k-blocks, so each thread pays the per-k-block hand-off
    // (barrier waits, proxy fence, arrive) half as often; one lane per warp polls the barriers.
    const int cw = warp - GEMM_THREADS / 32;              // 0..7
    const uint32_t grp = cw & 1;
    const int ct = (cw >> 1) * 32 + lane;                 // 0..127 inside the group
    const int units = g.bn * (BK / 16);                   // 16-byte units of the FP8 tile
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
      const Tile t = locate_tile(tile, s_pad, s_cnt, g.n_groups, g.n_tiles, g.n_per_group, g.bn, g.group_m);
      const float* srow = g.scales + static_cast<long long>(t.b_row >> 7) * g.scale_cols;
      // one scale per 128 rows x 128 columns: rows [0,128) and [128,256) of the tile
      bool ok = true;
      for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
        if ((it & 1u) != grp) continue;
        const uint32_t s = it % NS, ph = (it / NS) & 1u;
        const uint32_t j = it % B_SLOTS, jph = (it / B_SLOTS) & 1u;
        const float s0 = __ldg(srow + (kb >> 1));
        const float s1 = g.bn > 128 ? __ldg(srow + g.scale_cols + (kb >> 1)) : s0;
        int good = 1;
        if (lane == 0)
          good = mbar_wait(smem_u32(&full[s]), ph, abort_flag, g.status, 6) &&
                 mbar_wait(smem_u32(&bfree[j]), jph ^ 1u, abort_flag, g.status, 7);
        good = __shfl_sync(0xFFFFFFFFu, good, 0);         // also orders the other lanes after the wait
        if (!good) { ok = false; break; }
        const uint8_t* src = smem + s * STAGE_BYTES + A_BYTES;
        uint8_t* dst = smem + NS * STAGE_BYTES + j * B_BYTES;
#pragma unroll
        for (int u = ct; u < units; u += CONVERT_THREADS / 2) {
          const int r = u >> 2, c = u & 3;                // row of the tile, 16-byte chunk of its 64 bytes
          const uint4 q = *reinterpret_cast<const uint4*>(src + u * 16);
          uint4 lo, hi;
          convert16(q, r < 128 ? s0 : s1, lo, hi);
          // 128-byte bf16 row, 16-byte chunks XOR-swizzled by (row mod 8), as TMA SWIZZLE_128B lays them out
          uint8_t* drow = dst + r * 128;
          *reinterpret_cast<uint4*>(drow + (((2 * c) ^ (r & 7)) << 4)) = lo;
          *reinterpret_cast<uint4*>(drow + (((2 * c + 1) ^ (r & 7)) << 4)) = hi;
        }
        // make the generic-proxy writes visible to the tensor core's shared-memory reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bready[j]));
      }
      if (!ok) break;
    }
  } else if (warp >= 2 && warp < 6) {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;             // TMEM lanes [32*quarter, 32*quarter+32)
    const int row_in_tile = quarter * 32 + lane;
    EpiWarp ew{epi_stage + quarter * 2 * EPI_PIECE_BYTES, 0u, lane, 2};
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
      const Tile t = locate_tile(tile, s_pad, s_cnt, g.n_groups, g.n_tiles, g.n_per_group, g.bn, g.group_m);
      const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
      if (!mbar_wait(smem_u32(&tfull[acc]), acc_ph, abort_flag, g.status, 4)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool live = row_in_tile < t.valid_rows;
      const long long row = static_cast<long long>(t.row0) + row_in_tile;
      epilogue_rows<EPI>(taddr, g, &tmC, ew, row, t.row0 + quarter * 32, t.n_idx, live, quarter * 32 < t.valid_rows);
      // hand the accumulator back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty[acc]));
    }
    epilogue_drain(ew);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}


// =======================================================================================
// 2-CTA variant: a cluster of two CTAs (one SM pair) computes a 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128 of the 256
// B rows, so every SM moves half the B bytes per FLOP of the 1-CTA kernel; the accumulator
// halves live in each CTA's own TMEM.  CTA rank 0 ("leader") issues the MMAs.  Barriers:
//   full[s]    leader only; both CTAs' TMA loads complete their bytes on it
//   empty[s]   one copy per CTA; the leader's commit arrives on both (commit multicast, which
//              signals barriers and moves no data)
//   tfull[a]   one copy per CTA, same mechanism, tells each epilogue its half is complete
//   tempty[a]  leader only; the 4 epilogue warps of both CTAs arrive on it (remote arrive)
// TMA loads are plain 2-D tile loads (no multicast) of this GPU's own memory.
// =======================================================================================
// W8A16 on SM pairs (F8B): each CTA receives its B half as FP8 bytes and its 8 converter warps
// write the bf16 half tile; both CTAs' converters arrive on the leader's bready[j]; full[s] is
// then local to each CTA (its own A and FP8 bytes), because its converters must wait on it.
constexpr int STAGES2_MAX = 6;                          // bf16: 6 stages of 32 KiB; W8A16: 5 of 24 KiB
constexpr int B2_BYTES = 128 * BK * 2;                  // this CTA's half of the B tile, bf16
constexpr int B2F8_BYTES = 128 * BK;                    // the same half as FP8 bytes
constexpr int B2_SLOTS = 5;                             // converted half tiles in flight: the hand-off
                                                        // crosses the SM pair, so it needs depth
constexpr int NUM_BARS2 = 2 * STAGES2_MAX + 4 + 2 * B2_SLOTS;
template <bool F8B>
struct Cfg2 {
  static constexpr int STAGE_BYTES = A_BYTES + (F8B ? B2F8_BYTES : B2_BYTES);      // 24 / 32 KiB
  static constexpr int STAGES = F8B ? 5 : 6;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES + (F8B ? B2_SLOTS * B2_BYTES : 0);
  static constexpr int THREADS = GEMM_THREADS + (F8B ? CONVERT_THREADS : 0);
};
constexpr size_t SMEM2_CTRL_BYTES = 8 * NUM_BARS2 + 16 + 4 * (3 * kMaxExperts + 3);
template <bool F8B>
constexpr size_t gemm2_smem_bytes() { return 1024 + Cfg2<F8B>::RING_BYTES + SMEM2_CTRL_BYTES + 1024 + 4 * 2 * 2048; }

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// both CTAs of the pair issue it; the completion bytes are counted on the leader's barrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar & 0xFEFFFFFFu), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(static_cast<uint16_t>(3))
      : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct Tile2 {
  int row0;       // first of the pair's 256 rows
  int rows_left;  // rows of the expert from row0 on (may exceed 256)
  int b_row;      // first of the 256 B rows
  int n_idx;
};

// A tile of SUB row tiles (SUB x 128 rows).  s_pp[e] = number of such tiles (per N tile) of the
// experts before e; tiles that cover 2048 rows form one L2 reuse group (N-major inside it).
template <int SUB>
__device__ __forceinline__ Tile2 locate_tile_sub(int tile, const int* s_pad, const int* s_cnt, const int* s_pp,
                                                 int n_groups, int n_tiles, int n_per_group) {
  constexpr int GROUP = 2048 / (SUB * BM);
  int lo = 0, hi = n_groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (s_pp[mid] * n_tiles <= tile) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int local = tile - s_pp[e] * n_tiles;
  const int mp_e = s_pp[e + 1] - s_pp[e];
  const int per_group = GROUP * n_tiles;
  const int grp = local / per_group;
  const int rem = local - grp * per_group;
  const int gm = min(GROUP, mp_e - grp * GROUP);
  const int n = rem / gm;
  const int mp = grp * GROUP + (rem - n * gm);
  Tile2 t;
  t.row0 = s_pad[e] + mp * SUB * BM;
  t.rows_left = s_cnt[e] - mp * SUB * BM;
  t.b_row = e * n_per_group + n * BN_MAX;
  t.n_idx = n;
  return t;
}
__device__ __forceinline__ Tile2 locate_tile2(int tile, const int* s_pad, const int* s_cnt, const int* s_pp,
                                              int n_groups, int n_tiles, int n_per_group) {
  return locate_tile_sub<2>(tile, s_pad, s_cnt, s_pp, n_groups, n_tiles, n_per_group);
}

template <int EPI, bool F8B>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg2<F8B>::THREADS, 1)
grouped_gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, const GemmArgs g) {
  constexpr int STAGE2_BYTES = Cfg2<F8B>::STAGE_BYTES;
  constexpr int STAGES2 = Cfg2<F8B>::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg2<F8B>::RING_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES2_MAX;
  uint64_t* tfull = bars + 2 * STAGES2_MAX;
  uint64_t* tempty = bars + 2 * STAGES2_MAX + 2;
  uint64_t* bready = bars + 2 * STAGES2_MAX + 4;               // leader: both CTAs' converters arrive
  uint64_t* bfree = bars + 2 * STAGES2_MAX + 4 + B2_SLOTS;     // per CTA, via the leader's commit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_pad = reinterpret_cast<int*>(tmem_slot + 4);
  int* s_cnt = s_pad + kMaxExperts + 1;
  int* s_pp = s_cnt + kMaxExperts + 1;
  uint8_t* epi_stage = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem + Cfg2<F8B>::RING_BYTES + SMEM2_CTRL_BYTES) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull[a]), 1); mbar_init(smem_u32(&tempty[a]), 8); }
    for (int j = 0; j < B2_SLOTS; ++j) {
      mbar_init(smem_u32(&bready[j]), 2 * (CONVERT_THREADS / 64));   // 4 warps of the k-block's group, both CTAs
      mbar_init(smem_u32(&bfree[j]), 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (g.pad_offsets != nullptr) {
    for (int i = threadIdx.x; i <= g.n_groups; i += blockDim.x) s_pad[i] = g.pad_offsets[i];
    for (int i = threadIdx.x; i < g.n_groups; i += blockDim.x) s_cnt[i] = g.counts[i];
  } else if (threadIdx.x == 0) {
    s_pad[0] = 0;
    s_pad[1] = (g.dense_rows + BM - 1) / BM * BM;
    s_cnt[0] = g.dense_rows;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < g.n_groups; ++e) {
      s_pp[e] = acc;
      acc += ((s_pad[e + 1] - s_pad[e]) / BM + 1) / 2;
    }
    s_pp[g.n_groups] = acc;
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();      // barriers of both CTAs initialised, TMEM allocated on both SMs
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = s_pp[g.n_groups] * g.n_tiles;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bslot_base = smem_base + STAGES2 * STAGE2_BYTES;   // W8A16: converted half tiles

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs) {
        const Tile2 t = locate_tile2(tile, s_pad, s_cnt, s_pp, g.n_groups, g.n_tiles, g.n_per_group);
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES2, ph = (it / STAGES2) & 1u;
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, abort_flag, g.status, 11)) break;
          const uint32_t fb = smem_u32(&full[s]);
          const uint32_t sa = smem_base + s * STAGE2_BYTES;
          if (F8B) {
            mbar_expect_tx(fb, STAGE2_BYTES);                      // this CTA's A and FP8 half, own barrier
            tma_load_2d(sa, &tmA, kb * BK, t.row0 + static_cast<int>(rank) * BM, fb);
            tma_load_2d(sa + A_BYTES, &tmB, kb * BK, t.b_row + static_cast<int>(rank) * 128, fb);
          } else {
            if (rank == 0) mbar_expect_tx(fb, 2 * STAGE2_BYTES);   // both CTAs' A and B halves
            tma_load_2d_pair(sa, &tmA, kb * BK, t.row0 + static_cast<int>(rank) * BM, fb);
            tma_load_2d_pair(sa + A_BYTES, &tmB, kb * BK, t.b_row + static_cast<int>(rank) * 128, fb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs, ++tcount) {
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&tempty[acc]), acc_ph ^ 1u, abort_flag, g.status, 12)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        bool ok = true;
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES2, ph = (it / STAGES2) & 1u;
          if (!mbar_wait(smem_u32(&full[s]), ph, abort_flag, g.status, 13)) { ok = false; break; }
          const uint32_t j = it % B2_SLOTS, jph = (it / B2_SLOTS) & 1u;
          if (F8B && !mbar_wait(smem_u32(&bready[j]), jph, abort_flag, g.status, 15)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE2_BYTES;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(F8B ? bslot_base + j * B2_BYTES : sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc_mma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, g.idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit_pair(smem_u32(&empty[s]));
          if (F8B) tc_commit_pair(smem_u32(&bfree[j]));
        }
        if (!ok) break;
        tc_commit_pair(smem_u32(&tfull[acc]));
      }
    }
  } else if (F8B && warp >= 6) {
    // ---------------- FP8 -> bf16 converter (both CTAs, own half of B) ----------------
    // two groups of 4 warps take alternate k-blocks; one lane per warp polls the barriers
    const int cw = warp - GEMM_THREADS / 32;
    const uint32_t grp = cw & 1;
    const int ct = (cw >> 1) * 32 + lane;
    uint32_t it = 0;
    for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs) {
      const Tile2 t = locate_tile2(tile, s_pad, s_cnt, s_pp, g.n_groups, g.n_tiles, g.n_per_group);
      // the half tile is 128 rows = one scale block row
      const float* srow = g.scales + static_cast<long long>((t.b_row >> 7) + static_cast<int>(rank)) * g.scale_cols;
      TileScales scs;
      scs.load(srow, g.scale_cols, lane);
      bool ok = true;
      for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
        if ((it & 1u) != grp) continue;
        const uint32_t s = it % STAGES2, ph = (it / STAGES2) & 1u;
        const uint32_t j = it % B2_SLOTS, jph = (it / B2_SLOTS) & 1u;
        const float sc = scs.get(kb >> 1);
        int good = 1;
        if (lane == 0)
          good = mbar_wait(smem_u32(&full[s]), ph, abort_flag, g.status, 16) &&
                 mbar_wait(smem_u32(&bfree[j]), jph ^ 1u, abort_flag, g.status, 17);
        good = __shfl_sync(0xFFFFFFFFu, good, 0);
        if (!good) { ok = false; break; }
        const uint8_t* src = smem + s * STAGE2_BYTES + A_BYTES;
        uint8_t* dst = smem + STAGES2 * STAGE2_BYTES + j * B2_BYTES;
#pragma unroll
        for (int u = ct; u < 128 * (BK / 16); u += CONVERT_THREADS / 2) {
          const int r = u >> 2, c = u & 3;
          const uint4 q = *reinterpret_cast<const uint4*>(src + u * 16);
          uint4 lo, hi;
          convert16(q, sc, lo, hi);
          uint8_t* drow = dst + r * 128;
          *reinterpret_cast<uint4*>(drow + (((2 * c) ^ (r & 7)) << 4)) = lo;
          *reinterpret_cast<uint4*>(drow + (((2 * c + 1) ^ (r & 7)) << 4)) = hi;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bready[j]), 0));
      }
      if (!ok) break;
    }
  } else if (warp >= 2 && warp < 6) {
    // ---------------- epilogue (both CTAs, own 128 rows) ----------------
    const int quarter = warp & 3;
    const int row_in_half = quarter * 32 + lane;
    EpiWarp ew{epi_stage + quarter * 2 * EPI_PIECE_BYTES, 0u, lane, 2};
    uint32_t tcount = 0;
    for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs, ++tcount) {
      const Tile2 t = locate_tile2(tile, s_pad, s_cnt, s_pp, g.n_groups, g.n_tiles, g.n_per_group);
      const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
      if (!mbar_wait(smem_u32(&tfull[acc]), acc_ph, abort_flag, g.status, 14)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
      const int my_rows = t.rows_left - static_cast<int>(rank) * BM;      // rows of my half that are real
      const bool live = row_in_half < my_rows;
      const long long row = static_cast<long long>(t.row0) + rank * BM + row_in_half;
      epilogue_rows<EPI>(taddr, g, &tmC, ew, row, t.row0 + static_cast<int>(rank) * BM + quarter * 32, t.n_idx, live,
                         quarter * 32 < my_rows);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));
    }
    epilogue_drain(ew);
  }

  tc_fence_before();
  cluster_sync_all();      // neither CTA leaves while the other may still signal it or use its TMEM
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}


// =======================================================================================
// W8A16 on one CTA: FP8 weight tiles are converted to bf16 inside the kernel.  The 8 converter
// warps read the FP8 bytes straight from global memory into registers, four k-blocks ahead,
// scale them, and write the bf16 tile, swizzled as TMA would, into one of a ring of slots for
// the MMA warp; the bytes never pass through shared memory as FP8 (shared-memory bandwidth is
// what limits these kernels) and TMA carries A only.
//   TM = 128: one MMA per k-block, two accumulators in tensor memory (the epilogue of a tile
//             overlaps the next tile's main loop).  Not dispatched: with few rows per expert the
//             weights stream from HBM, register loads then expose its latency, and the TMA-staged
//             grouped_gemm_kernel<EPI, true> measured 1.25x faster (2.56 against 3.20 ms for the
//             gate/up GEMM of 256 DeepSeek-V3 experts at 32 rows each).
//   TM = 256: the converted tile feeds two MMAs, one per 128-row half of A, into the two halves
//             of tensor memory, so the conversion is paid once per 256 rows.  Both accumulators
//             are in use, so a tile's epilogue is not overlapped (the converters and the TMA
//             ring do run ahead into it); a tile with at most 128 live rows skips the second MMA.
// =======================================================================================
template <int TM>
struct CfgW8 {
  static constexpr int SUBS = TM / BM;                               // MMAs per k-block
  static constexpr int A_STAGE = SUBS * A_BYTES;                     // 16 / 32 KiB
  static constexpr int STAGES = TM == 128 ? 4 : 3;
  static constexpr int SLOTS = TM == 128 ? 4 : 3;                    // converted B tiles, 32 KiB each
  static constexpr int NACC = TM == 128 ? 2 : 1;                     // accumulator sets
  static constexpr int RING_BYTES = STAGES * A_STAGE + SLOTS * B_BYTES;
  static constexpr int BARS = 2 * STAGES + 2 * NACC + 2 * SLOTS;
  static constexpr size_t CTRL_BYTES = 8 * BARS + 16 + 4 * (3 * kMaxExperts + 3);
  static constexpr size_t SMEM_BYTES = 1024 + RING_BYTES + CTRL_BYTES + 1024 + 4 * 2 * EPI_PIECE_BYTES;
};
constexpr int W8_THREADS = GEMM_THREADS + CONVERT_THREADS;
constexpr int W8_UNITS = 256 * (BK / 16) / CONVERT_THREADS;         // 16-byte FP8 units per thread per k-block

// where the converter's load (or convert) cursor stands: k-block `kb` of tile `tile`
struct B8Cursor {
  int tile, kb;
  const uint8_t* src;     // this thread's first unit of the current k-block
  const float* srow;      // scales of the tile's first 128 B rows
};

template <int TM>
__device__ __forceinline__ Tile2 locate_w8(int tile, const int* s_pad, const int* s_cnt, const int* s_pp,
                                           const GemmArgs& g) {
  if (TM == 256) return locate_tile2(tile, s_pad, s_cnt, s_pp, g.n_groups, g.n_tiles, g.n_per_group);
  const Tile t = locate_tile(tile, s_pad, s_cnt, g.n_groups, g.n_tiles, g.n_per_group, g.bn, g.group_m);
  Tile2 r;
  r.row0 = t.row0;
  r.rows_left = t.valid_rows;
  r.b_row = t.b_row;
  r.n_idx = t.n_idx;
  return r;
}

// 16 bytes of weights through the read-only path.  Plain: with `.L1::no_allocate.L2::256B` on the
// load the 256-row kernel was 15-25 % slower (21.8 against 17.2 ms for the gate/up GEMM of 256
// DeepSeek-V3 experts at 1024 rows each).
__device__ __forceinline__ uint4 ld_weights16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

template <int EPI, int TM>
__global__ void __launch_bounds__(W8_THREADS, 1)
grouped_gemm_w8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmC,
                       const uint8_t* __restrict__ b8, const GemmArgs g) {
  using C = CfgW8<TM>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::RING_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint64_t* tempty = tfull + C::NACC;
  uint64_t* bready = tempty + C::NACC;
  uint64_t* bfree = bready + C::SLOTS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_pad = reinterpret_cast<int*>(tmem_slot + 4);
  int* s_cnt = s_pad + kMaxExperts + 1;
  int* s_pp = s_cnt + kMaxExperts + 1;
  uint8_t* epi_stage = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem + C::RING_BYTES + C::CTRL_BYTES) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
    for (int a = 0; a < C::NACC; ++a) { mbar_init(smem_u32(&tfull[a]), 1); mbar_init(smem_u32(&tempty[a]), 4); }
    for (int j = 0; j < C::SLOTS; ++j) { mbar_init(smem_u32(&bready[j]), CONVERT_THREADS / 32); mbar_init(smem_u32(&bfree[j]), 1); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i <= g.n_groups; i += blockDim.x) s_pad[i] = g.pad_offsets[i];
  for (int i = threadIdx.x; i < g.n_groups; i += blockDim.x) s_cnt[i] = g.counts[i];
  __syncthreads();
  if (TM == 256 && threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < g.n_groups; ++e) {
      s_pp[e] = acc;
      acc += ((s_pad[e + 1] - s_pad[e]) / BM + 1) / 2;
    }
    s_pp[g.n_groups] = acc;
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles =
      TM == 256 ? s_pp[g.n_groups] * g.n_tiles : ((s_pad[g.n_groups] - s_pad[0]) / BM) * g.n_tiles;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bslot_base = smem_base + C::STAGES * C::A_STAGE;

  if (warp == 0) {
    // ---------------- TMA producer: TM rows of A per k-block, one box ----------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const Tile2 t = locate_w8<TM>(tile, s_pad, s_cnt, s_pp, g);
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, abort_flag, g.status, 21)) break;
          const uint32_t fb = smem_u32(&full[s]);
          mbar_expect_tx(fb, C::A_STAGE);
          tma_load_2d(smem_base + s * C::A_STAGE, &tmA, kb * BK, t.row0, fb);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
        // a 256-row tile with at most 128 live rows needs its first half only
        const int n_sub = (TM == 256 && locate_w8<TM>(tile, s_pad, s_cnt, s_pp, g).rows_left > BM) ? 2 : 1;
        const uint32_t acc = C::NACC == 2 ? (tcount & 1u) : 0u;
        const uint32_t acc_ph = C::NACC == 2 ? ((tcount >> 1) & 1u) : (tcount & 1u);
        if (!mbar_wait(smem_u32(&tempty[acc]), acc_ph ^ 1u, abort_flag, g.status, 22)) break;
        tc_fence_after();
        bool ok = true;
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1u;
          const uint32_t j = it % C::SLOTS, jph = (it / C::SLOTS) & 1u;
          if (!mbar_wait(smem_u32(&full[s]), ph, abort_flag, g.status, 23)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&bready[j]), jph, abort_flag, g.status, 25)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * C::A_STAGE;
          const uint64_t db = make_smem_desc(bslot_base + j * B_BYTES);
          for (int sub = 0; sub < n_sub; ++sub) {
            const uint64_t da = make_smem_desc(sa + sub * A_BYTES);
            const uint32_t d_tmem = tmem_base + (acc + sub) * ACC_COLS;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              tc_mma_bf16(d_tmem, da + 2 * k, db + 2 * k, g.idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(smem_u32(&empty[s]));
          tc_commit(smem_u32(&bfree[j]));
        }
        if (!ok) break;
        tc_commit(smem_u32(&tfull[acc]));
      }
    }
  } else if (warp >= 6) {
    // ---------------- FP8 -> bf16 converter: global -> registers -> swizzled shared ----------------
    const int ct = threadIdx.x - GEMM_THREADS;             // 0..255; unit i of this thread is row ct/4 + 64 i
    const int r0 = ct >> 2, c = ct & 3;
    const long long row_bytes = static_cast<long long>(g.k_blocks) * BK;     // FP8: one byte per element
    const int my_tiles = blockIdx.x < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t n_it = static_cast<uint32_t>(my_tiles) * g.k_blocks;

    auto seek = [&](B8Cursor& cur) {                        // point the cursor at k-block 0 of cur.tile
      const Tile2 t = locate_w8<TM>(cur.tile, s_pad, s_cnt, s_pp, g);
      cur.kb = 0;
      cur.src = b8 + (static_cast<long long>(t.b_row) + r0) * row_bytes + c * 16;
      cur.srow = g.scales + static_cast<long long>(t.b_row >> 7) * g.scale_cols;
    };
    auto step = [&](B8Cursor& cur) {
      if (++cur.kb == g.k_blocks) {
        cur.tile += gridDim.x;
        if (cur.tile < total_tiles) seek(cur);
      } else {
        cur.src += BK;
      }
    };
    auto fetch = [&](B8Cursor& cur, uint4 (&q)[W8_UNITS]) {
      if (cur.tile >= total_tiles) return;
#pragma unroll
      for (int i = 0; i < W8_UNITS; ++i) q[i] = ld_weights16(cur.src + static_cast<long long>(64 * i) * row_bytes);
      step(cur);
    };
    // converts the fetched k-block `it` into its slot; false when a wait gave up
    auto emit = [&](B8Cursor& cur, const uint4 (&q)[W8_UNITS], uint32_t it) -> bool {
      const uint32_t j = it % C::SLOTS, jph = (it / C::SLOTS) & 1u;
      const float s0 = __ldg(cur.srow + (cur.kb >> 1));
      const float s1 = __ldg(cur.srow + g.scale_cols + (cur.kb >> 1));
      int good = 1;
      if (lane == 0) good = mbar_wait(smem_u32(&bfree[j]), jph ^ 1u, abort_flag, g.status, 27);
      good = __shfl_sync(0xFFFFFFFFu, good, 0);
      if (!good) return false;
      uint8_t* dst = smem + C::STAGES * C::A_STAGE + j * B_BYTES;
#pragma unroll
      for (int i = 0; i < W8_UNITS; ++i) {
        const int r = r0 + 64 * i;
        uint4 lo, hi;
        convert16(q[i], i < W8_UNITS / 2 ? s0 : s1, lo, hi);
        uint8_t* drow = dst + r * 128;
        *reinterpret_cast<uint4*>(drow + (((2 * c) ^ (r & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(drow + (((2 * c + 1) ^ (r & 7)) << 4)) = hi;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bready[j]));
      step(cur);
      return true;
    };

    if (n_it > 0) {
      B8Cursor ld{static_cast<int>(blockIdx.x), 0, nullptr, nullptr}, cv;
      seek(ld);
      cv = ld;
      // four k-blocks of FP8 bytes in flight in registers: the converters are the busiest warps, so
      // the distance has to cover memory latency in units of their own work, not of the MMAs'
      uint4 qa[W8_UNITS], qb[W8_UNITS], qc[W8_UNITS], qd[W8_UNITS];
      fetch(ld, qa);
      fetch(ld, qb);
      fetch(ld, qc);
      fetch(ld, qd);
      for (uint32_t it = 0; it < n_it && !*abort_flag; it += 4) {
        if (!emit(cv, qa, it)) break;
        fetch(ld, qa);
        if (it + 1 >= n_it || !emit(cv, qb, it + 1)) break;
        fetch(ld, qb);
        if (it + 2 >= n_it || !emit(cv, qc, it + 2)) break;
        fetch(ld, qc);
        if (it + 3 >= n_it || !emit(cv, qd, it + 3)) break;
        fetch(ld, qd);
      }
    }
  } else {
    // ---------------- epilogue: the tile's 128-row halves, one after the other ----------------
    const int quarter = warp & 3;
    EpiWarp ew{epi_stage + quarter * 2 * EPI_PIECE_BYTES, 0u, lane, 2};
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
      const Tile2 t = locate_w8<TM>(tile, s_pad, s_cnt, s_pp, g);
      const uint32_t acc = C::NACC == 2 ? (tcount & 1u) : 0u;
      const uint32_t acc_ph = C::NACC == 2 ? ((tcount >> 1) & 1u) : (tcount & 1u);
      if (!mbar_wait(smem_u32(&tfull[acc]), acc_ph, abort_flag, g.status, 24)) break;
      tc_fence_after();
#pragma unroll 1
      for (int sub = 0; sub < C::SUBS; ++sub) {
        const int first = sub * BM + quarter * 32;                 // first row of this warp inside the tile
        if (first >= t.rows_left) break;                           // nothing of this warp's to store
        const uint32_t taddr = tmem_base + (acc + sub) * ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
        const bool live = first + lane < t.rows_left;
        epilogue_rows<EPI>(taddr, g, &tmC, ew, static_cast<long long>(t.row0) + first + lane, t.row0 + first, t.n_idx,
                           live, true);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty[acc]));
    }
    epilogue_drain(ew);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// =======================================================================================
// W8A16 through an L2-resident ring ("convert once, share through L2").
//
// The kernels above convert a weight tile again for every row tile that uses it (8 to 16 times per
// weight at large batch), or read a bf16 copy that a separate pass wrote to HBM.  Here every FP8
// weight is read from HBM and converted ONCE per group of row tiles: the eight converter warps of all
// CTAs together turn one "granule" of weights (a few MB: one or more 256-row panels of B, whole K)
// into bf16 in a small ring in global memory, sized to stay in the 126 MB L2; the CTAs whose tiles use
// that panel fetch their B tiles from the ring by TMA exactly as the bf16 kernel fetches them from a
// weight buffer.  A ring slot is written again only after every tile that reads it has finished, so
// the bf16 copy lives in L2 between its one write and its ~16 reads and, at best, never reaches HBM.
//
//   granule g      PG consecutive N tiles of one (expert, group of <= 16 row tiles), in tile order
//   ready[g]       += 1 by every CTA when its share of granule g is in the ring (release);
//                  a producer warp waits for ready[g] == gridDim.x before its first B load of a tile
//   done[g]        += 1 by a CTA's MMA thread when the last operand block of one of its tiles of
//                  granule g has landed in shared memory; the converters wait for
//                  done[g - slots] == tiles of that granule before they overwrite its slot
// All CTAs convert a part of every granule, so all of them must be resident: the kernel is launched
// cooperatively with at most one CTA per SM.  Every wait is bounded (status MG_DEV_WAIT_TIMEOUT).
// Results are bit-identical to de-quantising first: same bf16(float(q) * scale), same MMA order.
// =======================================================================================
struct RingArgs {
  const uint8_t* b8;     // FP8 weights, [n_groups * n_per_group][K] row-major
  uint8_t* ring;         // bf16 ring, [slots * pg * 256][K] row-major
  int32_t* ready;        // [granules]
  int32_t* done;         // [granules]
  int slots;             // granules the ring holds
  int pg;                // N tiles (256 weight rows each) per granule; divides n_tiles
  int keep_in_l2;        // ring stores and loads carry the L2 evict_last policy
};
constexpr int RING_MAX_SLOTS = 64;
constexpr int RING_GROUP_M = 16;
constexpr size_t SMEM_RING_CTRL_BYTES = 8 * NUM_BARS + 32 + 4 * (3 * kMaxExperts + 3) + 4 * RING_MAX_SLOTS;
constexpr size_t SMEM_RING_BYTES = 1024 + Cfg<false>::RING_BYTES + SMEM_RING_CTRL_BYTES + 1024 + 4 * 2 * EPI_PIECE_BYTES;
static_assert(SMEM_RING_BYTES <= 232448, "shared memory of the ring kernel exceeds the 227 KiB a CTA may have");
constexpr int RING_THREADS = GEMM_THREADS + CONVERT_THREADS;

__device__ __forceinline__ int ld_acquire_gpu(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int32_t* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded poll of a global counter; false when the wait ran out or another role gave up
__device__ __forceinline__ bool wait_counter(const int32_t* p, int target, volatile int* abort_flag, int32_t* status,
                                             int where) {
  if (ld_acquire_gpu(p) >= target) return true;
  const unsigned long long t0 = global_timer();
  uint32_t spins = 0;
  while (true) {
    if (ld_acquire_gpu(p) >= target) return true;
    __nanosleep(64);
    if ((++spins & 15u) == 0u) {
      if (*abort_flag) return false;
      if (timed_out(t0, WAIT_LIMIT_NS)) {
        *abort_flag = 1;
        if (atomicCAS(status, MG_DEV_OK, MG_DEV_WAIT_TIMEOUT) == MG_DEV_OK) status[1] = where;
        return false;
      }
    }
  }
}

struct RingTile {
  int row0, valid_rows, b_row, n_idx;
  int granule;      // index of the tile's granule in conversion order
  int ring_row;     // first row of the tile's B panel inside the ring
};

// s_gb[e] = granules of the experts before e.  Tile order as locate_tile: expert-major, groups of 16 row
// tiles, N-major inside a group, row tiles fastest.
__device__ __forceinline__ RingTile locate_ring(int tile, const int* s_pad, const int* s_cnt, const int* s_gb,
                                                const GemmArgs& g, const RingArgs& r) {
  const int base0 = s_pad[0];
  int lo = 0, hi = g.n_groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (((s_pad[mid] - base0) / BM) * g.n_tiles <= tile) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int local = tile - ((s_pad[e] - base0) / BM) * g.n_tiles;
  const int m_e = (s_pad[e + 1] - s_pad[e]) / BM;
  const int per_group = RING_GROUP_M * g.n_tiles;
  const int grp = local / per_group;
  const int rem = local - grp * per_group;
  const int gm = min(RING_GROUP_M, m_e - grp * RING_GROUP_M);
  const int n = rem / gm;
  const int m = grp * RING_GROUP_M + (rem - n * gm);
  RingTile t;
  t.row0 = s_pad[e] + m * BM;
  t.valid_rows = min(BM, s_cnt[e] - m * BM);
  t.b_row = e * g.n_per_group + n * BN_MAX;
  t.n_idx = n;
  const int per_exp = g.n_tiles / r.pg;
  t.granule = s_gb[e] + grp * per_exp + n / r.pg;
  t.ring_row = ((t.granule % r.slots) * r.pg + n % r.pg) * BN_MAX;
  return t;
}

template <int EPI>
__global__ void __launch_bounds__(RING_THREADS, 1)
grouped_gemm_ring_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC, const GemmArgs g, const RingArgs r) {
  constexpr int STAGE_BYTES = Cfg<false>::STAGE_BYTES;
  constexpr int NS = STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg<false>::RING_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* conv_ok = reinterpret_cast<volatile int*>(tmem_slot + 2);
  int* s_pad = reinterpret_cast<int*>(tmem_slot + 8);
  int* s_cnt = s_pad + kMaxExperts + 1;
  int* s_gb = s_cnt + kMaxExperts + 1;
  int* s_uses = s_gb + kMaxExperts + 1;                  // tiles of the granule that last used each slot
  uint8_t* epi_stage = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem + Cfg<false>::RING_BYTES + SMEM_RING_CTRL_BYTES) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull[a]), 1); mbar_init(smem_u32(&tempty[a]), 4); }
    *abort_flag = 0;
    conv_ok[0] = 1;
    conv_ok[1] = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i <= g.n_groups; i += blockDim.x) s_pad[i] = g.pad_offsets[i];
  for (int i = threadIdx.x; i < g.n_groups; i += blockDim.x) s_cnt[i] = g.counts[i];
  __syncthreads();
  const int per_exp = g.n_tiles / r.pg;                  // granules per (expert, group of row tiles)
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < g.n_groups; ++e) {
      s_gb[e] = acc;
      const int m_e = (s_pad[e + 1] - s_pad[e]) / BM;
      acc += ((m_e + RING_GROUP_M - 1) / RING_GROUP_M) * per_exp;
    }
    s_gb[g.n_groups] = acc;
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = ((s_pad[g.n_groups] - s_pad[0]) / BM) * g.n_tiles;
  const uint32_t smem_base = smem_u32(smem);
  const int n_ctas = static_cast<int>(gridDim.x);

  if (warp == 0) {
    // ---------------- TMA producer: A from the rows, B from the ring ----------------
    if (lane == 0) {
      uint32_t it = 0;
      int have = -1;                                    // granule already known to be in the ring
      const uint64_t keep = policy_evict_last();
      const uint32_t tx_bytes = A_BYTES + B_BYTES;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const RingTile t = locate_ring(tile, s_pad, s_cnt, s_gb, g, r);
        if (t.granule != have) {
          if (!wait_counter(r.ready + t.granule, n_ctas, abort_flag, g.status, 41)) break;
          // the bf16 bytes were written with ordinary stores by other SMs: order them before the TMA reads
          asm volatile("fence.proxy.async.global;" ::: "memory");
          have = t.granule;
        }
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % NS, ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, abort_flag, g.status, 42)) break;
          const uint32_t fb = smem_u32(&full[s]);
          mbar_expect_tx(fb, tx_bytes);
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          tma_load_2d(sa, &tmA, kb * BK, t.row0, fb);
          if (r.keep_in_l2) tma_load_2d_hint(sa + A_BYTES, &tmB, kb * BK, t.ring_row, fb, keep);
          else tma_load_2d(sa + A_BYTES, &tmB, kb * BK, t.ring_row, fb);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
        const RingTile t = locate_ring(tile, s_pad, s_cnt, s_gb, g, r);
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&tempty[acc]), acc_ph ^ 1u, abort_flag, g.status, 43)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        bool ok = true;
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t s = it % NS, ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&full[s]), ph, abort_flag, g.status, 44)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc_mma_bf16(d_tmem, da + 2 * k, db + 2 * k, g.idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(smem_u32(&empty[s]));
        }
        if (!ok) break;
        // every B block of this tile has left the ring (its loads completed on the barriers above)
        red_release_gpu_add(r.done + t.granule, 1);
        tc_commit(smem_u32(&tfull[acc]));
      }
    }
  } else if (warp >= 6) {
    // ---------------- converters: FP8 panel -> bf16 ring slot, this CTA's share of every granule ----------
    // Two groups of four warps take alternate granules, so that one group's hand-off latencies (the poll
    // for a free slot, the drain of its stores, the barriers) overlap the other group's conversion.  The
    // FP8 bytes of a group's next granule are fetched into registers before it waits for the current
    // slot, which keeps the HBM latency of the weights off the hand-off path.
    constexpr int GT = CONVERT_THREADS / 2;              // threads per group
    const int ct = (threadIdx.x - GEMM_THREADS) & (GT - 1);
    const int grp_id = (threadIdx.x - GEMM_THREADS) / GT;
    const int units_per_row = g.k_blocks * (BK / 16);    // 16-byte FP8 units per weight row
    const int units = r.pg * BN_MAX * units_per_row;      // per granule; the host keeps it below 2^31
    const long long row_bytes = static_cast<long long>(g.k_blocks) * BK;
    const int stride = n_ctas * GT;
    const int u_first = static_cast<int>(blockIdx.x) * GT + ct;
    constexpr int PF = 8;                                // units of a granule a thread keeps in registers
    volatile int* my_ok = conv_ok + grp_id;
    const uint64_t keep = policy_evict_last();

    struct Cursor { int e, grp, nb, m_e; };
    auto settle = [&](Cursor& c) {                       // skip experts without rows; false at the end
      while (c.e < g.n_groups) {
        c.m_e = (s_pad[c.e + 1] - s_pad[c.e]) / BM;
        if (c.grp * RING_GROUP_M < c.m_e) return true;
        ++c.e; c.grp = 0; c.nb = 0;
      }
      return false;
    };
    auto advance = [&](Cursor& c) {
      if (++c.nb == per_exp) { c.nb = 0; ++c.grp; }
      return settle(c);
    };
    auto fetch = [&](const Cursor& c, uint4 (&q)[PF], float (&sc)[PF]) {
      const int b_row0 = c.e * g.n_per_group + c.nb * r.pg * BN_MAX;
      const uint8_t* src = r.b8 + static_cast<long long>(b_row0) * row_bytes;
#pragma unroll
      for (int i = 0; i < PF; ++i) {
        const int u = u_first + i * stride;
        if (u < units) {
          const int row = u / units_per_row;
          const int cu = u - row * units_per_row;
          q[i] = __ldcs(reinterpret_cast<const uint4*>(src + static_cast<long long>(u) * 16));
          sc[i] = __ldg(g.scales + static_cast<long long>((b_row0 + row) >> 7) * g.scale_cols + (cu >> 3));
        }
      }
    };

    Cursor cur{0, 0, 0, 0};
    bool more = settle(cur);
    if (more && grp_id == 1) more = advance(cur);        // group 1 starts at granule 1
    uint4 qn[PF];
    float sn[PF];
    if (more) fetch(cur, qn, sn);
    for (int gi = grp_id; more; gi += 2) {
      uint4 q[PF];
      float sc[PF];
#pragma unroll
      for (int i = 0; i < PF; ++i) { q[i] = qn[i]; sc[i] = sn[i]; }
      const Cursor me = cur;
      more = advance(cur);
      if (more) more = advance(cur);
      if (more) fetch(cur, qn, sn);
      const int slot = gi % r.slots;
      if (ct == 0) {
        // one thread decides for its group (the others meet it at the barrier below, so the decision
        // must be uniform): another role gave up, or the tiles that read this slot's previous granule
        // have not all fetched their last block within the limit
        if (*abort_flag) *my_ok = 0;
        else if (gi >= r.slots && !wait_counter(r.done + (gi - r.slots), s_uses[slot], abort_flag, g.status, 45))
          *my_ok = 0;
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp_id), "n"(GT) : "memory");
      if (!*my_ok) break;
      const int gm = min(RING_GROUP_M, me.m_e - me.grp * RING_GROUP_M);
      if (ct == 0) s_uses[slot] = r.pg * gm;
      uint8_t* dst = r.ring + static_cast<long long>(slot) * r.pg * BN_MAX * row_bytes * 2;
#pragma unroll
      for (int i = 0; i < PF; ++i) {
        const int u = u_first + i * stride;
        if (u < units) {
          uint4 lo, hi;
          convert16(q[i], sc[i], lo, hi);
          uint4* o = reinterpret_cast<uint4*>(dst + static_cast<long long>(u) * 32);
          if (r.keep_in_l2) { st_global_hint16(o, lo, keep); st_global_hint16(o + 1, hi, keep); }
          else { o[0] = lo; o[1] = hi; }
        }
      }
      // a grid smaller than the one PF was sized for leaves units beyond the prefetched ones
      if (u_first + PF * stride < units) {
        const int b_row0 = me.e * g.n_per_group + me.nb * r.pg * BN_MAX;
        const uint8_t* src = r.b8 + static_cast<long long>(b_row0) * row_bytes;
        for (int u = u_first + PF * stride; u < units; u += stride) {
          const int row = u / units_per_row;
          const int cu = u - row * units_per_row;
          const float s1 = __ldg(g.scales + static_cast<long long>((b_row0 + row) >> 7) * g.scale_cols + (cu >> 3));
          const uint4 q1 = __ldcs(reinterpret_cast<const uint4*>(src + static_cast<long long>(u) * 16));
          uint4 lo, hi;
          convert16(q1, s1, lo, hi);
          uint4* o = reinterpret_cast<uint4*>(dst + static_cast<long long>(u) * 32);
          if (r.keep_in_l2) { st_global_hint16(o, lo, keep); st_global_hint16(o + 1, hi, keep); }
          else { o[0] = lo; o[1] = hi; }
        }
      }
      // ordinary stores -> ordered before the TMA (async proxy) reads of other SMs; the barrier orders the
      // group's stores before thread 0's release, which publishes them at GPU scope
      asm volatile("fence.proxy.async.global;" ::: "memory");
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp_id), "n"(GT) : "memory");
      if (ct == 0) red_release_gpu_add(r.ready + gi, 1);
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    EpiWarp ew{epi_stage + quarter * 2 * EPI_PIECE_BYTES, 0u, lane, 2};
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tcount) {
      const RingTile t = locate_ring(tile, s_pad, s_cnt, s_gb, g, r);
      const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
      if (!mbar_wait(smem_u32(&tfull[acc]), acc_ph, abort_flag, g.status, 46)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool live = row_in_tile < t.valid_rows;
      const long long row = static_cast<long long>(t.row0) + row_in_tile;
      epilogue_rows<EPI>(taddr, g, &tmC, ew, row, t.row0 + quarter * 32, t.n_idx, live, quarter * 32 < t.valid_rows);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty[acc]));
    }
    epilogue_drain(ew);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}


// Self-test of the bounded wait: one thread waits on a barrier that nothing will ever complete,
// with a short limit; the wait must give up, record MG_DEV_WAIT_TIMEOUT and let the kernel end.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 99, limit_ns);
  }
}

int launch_wait_probe(const Handle* h, int limit_ms, cudaStream_t st) {
  wait_probe_kernel<<<1, 32, 0, st>>>(static_cast<unsigned long long>(limit_ms) * 1000000ull, h->d_status);
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 operands land 128B-swizzled (what the UMMA descriptor expects); FP8 bytes land as plain
// rows of 64 bytes for the converter warps
// `out_piece`: the 32 x 32 bf16 pieces the epilogue stores (rows of 64 bytes, SWIZZLE_64B in shared memory)
// A layer calls the same few (pointer, shape) combinations on every forward, so the encoded maps
// are kept in the handle: a forward at decode sizes is short enough for ~60 driver calls to show.
static int encode_2d(const Handle* h, CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                     uint32_t box_rows, bool fp8 = false, bool out_piece = false) {
  const uint32_t kind = (fp8 ? 1u : 0u) | (out_piece ? 2u : 0u);
  TensorMapCache& c = h->tmaps;
  for (int i = 0; i < c.used; ++i) {
    const TensorMapCache::Entry& e = c.e[i];
    if (e.base == base && e.rows == rows && e.cols == cols && e.box_rows == box_rows && e.kind == kind) {
      *map = e.map;
      return MG_OK;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  MG_REQUIRE(fn != nullptr, MG_ERR_DRIVER, "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (fp8 ? 1 : 2)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(out_piece ? 32 : BK), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  out_piece ? CU_TENSOR_MAP_SWIZZLE_64B
                            : fp8 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MG_REQUIRE(r == CUDA_SUCCESS, MG_ERR_DRIVER, "cuTensorMapEncodeTiled failed (%d) rows=%llu cols=%llu box=%u",
             static_cast<int>(r), static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols),
             box_rows);
  TensorMapCache::Entry& e = c.e[c.next];
  e.base = base; e.rows = rows; e.cols = cols; e.box_rows = box_rows; e.kind = kind; e.map = *map;
  c.next = (c.next + 1) % TensorMapCache::kEntries;
  if (c.used < TensorMapCache::kEntries) ++c.used;
  return MG_OK;
}

// the opt-in to more than 48 KiB of dynamic shared memory is a per-device attribute of the kernel:
// set once per (kernel, device)
template <typename K>
static int allow_smem(K kernel, size_t bytes, int device, bool (&done)[64]) {
  if (device >= 0 && device < 64 && done[device]) return MG_OK;
  MG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
  if (device >= 0 && device < 64) done[device] = true;
  return MG_OK;
}

template <int EPI, bool F8B>
static int launch_epi(const Handle* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                      const GemmArgs& args, int grid, cudaStream_t st) {
  constexpr size_t smem = gemm_smem_bytes<F8B>();
  static bool done[64];
  int rc = allow_smem(grouped_gemm_kernel<EPI, F8B>, smem, h->device, done);
  if (rc != MG_OK) return rc;
  grouped_gemm_kernel<EPI, F8B><<<grid, Cfg<F8B>::THREADS, smem, st>>>(ta, tb, tc, args);
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

template <int EPI, bool F8B>
static int launch_pair(const Handle* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                       const GemmArgs& args, int grid, cudaStream_t st) {
  constexpr size_t smem = gemm2_smem_bytes<F8B>();
  static bool done[64];
  int rc = allow_smem(grouped_gemm2_kernel<EPI, F8B>, smem, h->device, done);
  if (rc != MG_OK) return rc;
  grouped_gemm2_kernel<EPI, F8B><<<grid, Cfg2<F8B>::THREADS, smem, st>>>(ta, tb, tc, args);
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

RingPlan ring_plan(int n_per_group, int K, int64_t a_rows, int n_groups, size_t budget_bytes) {
  RingPlan r;
  const int n_tiles = n_per_group / BN_MAX;
  const size_t panel = static_cast<size_t>(BN_MAX) * K * 2;
  r.pg = 1;
  for (int d = 1; d <= n_tiles; ++d)
    if (n_tiles % d == 0 && d * panel <= (static_cast<size_t>(9) << 19)) r.pg = d;       // granules of up to 4.5 MiB
  r.granule_bytes = r.pg * panel;
  long long slots = static_cast<long long>(budget_bytes / r.granule_bytes);
  r.slots = static_cast<int>(slots < 2 ? 2 : slots > RING_MAX_SLOTS ? RING_MAX_SLOTS : slots);
  r.ring_bytes = r.slots * r.granule_bytes;
  r.max_granules = ((a_rows / BM + RING_GROUP_M - 1) / RING_GROUP_M + n_groups) * (n_tiles / r.pg);
  return r;
}

template <int EPI>
static int launch_ring(const Handle* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                       const GemmArgs& args, const RingArgs& ring, int grid, cudaStream_t st) {
  static bool done[64];
  int rc = allow_smem(grouped_gemm_ring_kernel<EPI>, SMEM_RING_BYTES, h->device, done);
  if (rc != MG_OK) return rc;
  // every CTA converts a share of every granule and waits for the others': all must be resident at once
  void* params[] = {const_cast<CUtensorMap*>(&ta), const_cast<CUtensorMap*>(&tb), const_cast<CUtensorMap*>(&tc),
                    const_cast<GemmArgs*>(&args), const_cast<RingArgs*>(&ring)};
  MG_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(grouped_gemm_ring_kernel<EPI>), dim3(grid),
                                      dim3(RING_THREADS), params, SMEM_RING_BYTES, st));
  return MG_OK;
}

template <int EPI, int TM>
static int launch_w8(const Handle* h, const CUtensorMap& ta, const CUtensorMap& tc, const void* b8,
                     const GemmArgs& args, int grid, cudaStream_t st) {
  constexpr size_t smem = CfgW8<TM>::SMEM_BYTES;
  static_assert(smem <= 232448, "shared memory of the W8A16 kernel exceeds the 227 KiB a CTA may have");
  static bool done[64];
  int rc = allow_smem(grouped_gemm_w8_kernel<EPI, TM>, smem, h->device, done);
  if (rc != MG_OK) return rc;
  grouped_gemm_w8_kernel<EPI, TM><<<grid, W8_THREADS, smem, st>>>(ta, tc, static_cast<const uint8_t*>(b8), args);
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

// W8A16 through the L2-resident ring: p.ring / p.ring_counters are the caller's scratch (ring_plan)
static int launch_ring_gemm(const Handle* h, const GemmProblem& p, cudaStream_t st) {
  MG_REQUIRE(p.b_fp8 && p.scales != nullptr && p.pad_offsets != nullptr, MG_ERR_CONFIG, "ring GEMM needs grouped FP8 weights");
  MG_REQUIRE(p.K % 128 == 0 && p.n_per_group % BN_MAX == 0, MG_ERR_SHAPE, "ring GEMM: K %% 128 and N %% 256 required");
  MG_REQUIRE(p.epilogue == EPI_SWIGLU_BF16 || p.epilogue == EPI_PLAIN_BF16, MG_ERR_CONFIG, "ring GEMM: bf16 epilogues only");
  const RingPlan rp = ring_plan(p.n_per_group, p.K, p.a_rows, p.n_groups, p.ring_bytes);
  MG_REQUIRE(rp.ring_bytes <= p.ring_bytes && 2 * rp.max_granules <= p.ring_counter_ints, MG_ERR_WORKSPACE,
             "ring scratch too small: %zu bytes / %lld counters given, %zu / %lld needed", p.ring_bytes,
             static_cast<long long>(p.ring_counter_ints), rp.ring_bytes, static_cast<long long>(2 * rp.max_granules));
  MG_REQUIRE(static_cast<long long>(rp.pg) * BN_MAX * (p.K / 16) < (1ll << 31), MG_ERR_LIMIT, "granule too large");
  CUtensorMap ta, tb, tc;
  int rc = encode_2d(h, &ta, p.a, static_cast<uint64_t>(p.a_rows), static_cast<uint64_t>(p.K), BM);
  if (rc != MG_OK) return rc;
  rc = encode_2d(h, &tb, p.ring, static_cast<uint64_t>(rp.slots) * rp.pg * BN_MAX, static_cast<uint64_t>(p.K), BN_MAX);
  if (rc != MG_OK) return rc;
  MG_REQUIRE(p.ldo % 8 == 0, MG_ERR_SHAPE, "output row length %lld must be a multiple of 8", static_cast<long long>(p.ldo));
  rc = encode_2d(h, &tc, p.out, static_cast<uint64_t>(p.a_rows), static_cast<uint64_t>(p.ldo), 32, false, true);
  if (rc != MG_OK) return rc;
  GemmArgs a;
  a.pad_offsets = p.pad_offsets;
  a.counts = p.counts;
  a.n_groups = p.n_groups;
  a.dense_rows = 0;
  a.n_tiles = p.n_per_group / BN_MAX;
  a.bn = BN_MAX;
  a.n_per_group = p.n_per_group;
  a.k_blocks = p.K / BK;
  a.group_m = RING_GROUP_M;
  a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN_MAX >> 3) << 17) |
            (static_cast<uint32_t>(BM >> 4) << 24);
  a.scales = p.scales;
  a.scale_cols = p.K / 128;
  a.out = p.out;
  a.ldo = p.ldo;
  a.status = h->d_status;
  RingArgs r;
  r.b8 = static_cast<const uint8_t*>(p.b);
  r.ring = static_cast<uint8_t*>(p.ring);
  r.ready = p.ring_counters;
  r.done = p.ring_counters + rp.max_granules;
  r.slots = rp.slots;
  r.pg = rp.pg;
  r.keep_in_l2 = h->opt_ring_persist ? 1 : 0;
  MG_CUDA(cudaMemsetAsync(p.ring_counters, 0, sizeof(int32_t) * 2 * rp.max_granules, st));
  int grid = h->sm_count;
  const long long max_tiles = (p.a_rows / BM) * a.n_tiles;
  if (max_tiles < grid) grid = static_cast<int>(max_tiles);
  if (grid < 1) return MG_OK;
  switch (p.epilogue) {
    case EPI_SWIGLU_BF16: return launch_ring<EPI_SWIGLU_BF16>(h, ta, tb, tc, a, r, grid, st);
    default: return launch_ring<EPI_PLAIN_BF16>(h, ta, tb, tc, a, r, grid, st);
  }
}

int launch_grouped_gemm(const Handle* h, const GemmProblem& p, cudaStream_t st) {
  const bool dense = p.pad_offsets == nullptr;
  if (p.a_rows <= 0 || (dense && p.dense_rows <= 0)) return MG_OK;
  MG_REQUIRE(p.K % BK == 0, MG_ERR_SHAPE, "GEMM K=%d must be a multiple of %d", p.K, BK);
  MG_REQUIRE(p.n_groups >= 1 && p.n_groups <= kMaxExperts, MG_ERR_SHAPE, "n_groups=%d out of range", p.n_groups);
  int bn;
  const bool f32_out = p.epilogue == EPI_PLAIN_F32 || p.epilogue == EPI_ROUND_BF16_F32;
  if (f32_out) {
    bn = static_cast<int>(round_up(p.n_per_group, 16));
    MG_REQUIRE(bn <= BN_MAX && p.n_groups == 1 && p.n_per_group % 4 == 0, MG_ERR_SHAPE,
               "fp32-output GEMM needs one group of <=256 columns (multiple of 4), got %d", p.n_per_group);
  } else {
    bn = BN_MAX;
    MG_REQUIRE(p.n_per_group % BN_MAX == 0, MG_ERR_SHAPE, "GEMM N per expert (%d) must be a multiple of %d",
               p.n_per_group, BN_MAX);
  }
  // SM pairs (2-CTA tiles of 256 x 256) for the bf16 expert GEMMs when switched on
  const bool pair = h->opt_pair_gemm && !f32_out;
  // FP8 weights converted in the kernel (one CTA per SM): 256-row tiles once experts average 120
  // live rows (a_rows also counts up to 127 rows of padding per expert); below that most tall tiles
  // would be half empty, the layer is bound by streaming the weights from HBM, and the 128-row
  // kernel, whose FP8 bytes arrive by TMA, streams them faster than register loads do
  const bool m256 = p.b_fp8 && !pair && !f32_out && !dense && h->opt_fp8_m256 &&
                    p.a_rows >= static_cast<int64_t>(p.n_groups) * (h->opt_fp8_m256 == 2 ? 0 : 120 + 127);
  if (p.ring != nullptr) return launch_ring_gemm(h, p, st);
  CUtensorMap ta, tb;
  int rc = encode_2d(h, &ta, p.a, static_cast<uint64_t>(p.a_rows), static_cast<uint64_t>(p.K), m256 ? 2 * BM : BM);
  if (rc != MG_OK) return rc;
  rc = encode_2d(h, &tb, p.b, static_cast<uint64_t>(p.n_groups) * p.n_per_group, static_cast<uint64_t>(p.K),
                 pair ? 128 : bn, p.b_fp8);
  if (rc != MG_OK) return rc;
  CUtensorMap tc = ta;   // unused by the fp32 epilogue
  if (!f32_out) {
    // output tensor [a_rows, ldo] bf16, written in 32 x 32 pieces
    MG_REQUIRE(p.ldo % 8 == 0, MG_ERR_SHAPE, "output row length %lld must be a multiple of 8", static_cast<long long>(p.ldo));
    rc = encode_2d(h, &tc, p.out, static_cast<uint64_t>(p.a_rows), static_cast<uint64_t>(p.ldo), 32, false, true);
    if (rc != MG_OK) return rc;
  }
  if (p.b_fp8) {
    MG_REQUIRE(!f32_out && p.scales != nullptr && p.K % 128 == 0 && p.K <= 128 * 128, MG_ERR_SHAPE,
               "FP8 weights need scales, K a multiple of 128 up to 16384 and a bf16 epilogue");
  }

  GemmArgs a;
  a.pad_offsets = p.pad_offsets;
  a.counts = p.counts;
  a.n_groups = p.n_groups;
  a.dense_rows = static_cast<int>(p.dense_rows);
  a.n_tiles = f32_out ? 1 : p.n_per_group / bn;
  a.bn = bn;
  a.n_per_group = p.n_per_group;
  a.k_blocks = p.K / BK;
  a.group_m = 16;
  // kind::f16: D fp32 (bit 4), A bf16 (bit 7), B bf16 (bit 10), both K-major, N>>3 at 17, M>>4 at 24
  a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) |
            (static_cast<uint32_t>(BM >> 4) << 24);
  a.scales = p.scales;
  a.scale_cols = p.K / 128;
  a.out = p.out;
  a.ldo = p.ldo;
  a.status = h->d_status;

  int grid = h->sm_count;
  if (dense) {
    long long tiles = (p.dense_rows + BM - 1) / BM * a.n_tiles;
    if (tiles < grid) grid = static_cast<int>(tiles);
  } else {
    long long max_tiles = (p.a_rows / BM) * a.n_tiles;
    if (max_tiles < grid) grid = static_cast<int>(max_tiles);
  }
  if (grid < 1) return MG_OK;
  if (m256) {
    long long tall_tiles = ((p.a_rows / BM + p.n_groups) / 2 + 1) * static_cast<long long>(a.n_tiles);
    int ctas = tall_tiles < h->sm_count ? static_cast<int>(tall_tiles) : h->sm_count;
    switch (p.epilogue) {
      case EPI_SWIGLU_BF16: return launch_w8<EPI_SWIGLU_BF16, 256>(h, ta, tc, p.b, a, ctas, st);
      case EPI_PLAIN_BF16: return launch_w8<EPI_PLAIN_BF16, 256>(h, ta, tc, p.b, a, ctas, st);
    }
  }
  if (pair) {
    // UMMA M = 256 across the two CTAs; one cluster per SM pair
    a.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) |
              (static_cast<uint32_t>(256 >> 4) << 24);
    int pairs = h->sm_count / 2;
    long long max_pair_tiles = dense ? ((p.dense_rows + 2 * BM - 1) / (2 * BM)) * a.n_tiles
                                     : ((p.a_rows / BM + p.n_groups) / 2 + 1) * static_cast<long long>(a.n_tiles);
    if (max_pair_tiles < pairs) pairs = static_cast<int>(max_pair_tiles);
    if (pairs < 1) pairs = 1;
    if (p.b_fp8) {
      switch (p.epilogue) {
        case EPI_SWIGLU_BF16: return launch_pair<EPI_SWIGLU_BF16, true>(h, ta, tb, tc, a, 2 * pairs, st);
        case EPI_PLAIN_BF16: return launch_pair<EPI_PLAIN_BF16, true>(h, ta, tb, tc, a, 2 * pairs, st);
      }
    }
    switch (p.epilogue) {
      case EPI_SWIGLU_BF16: return launch_pair<EPI_SWIGLU_BF16, false>(h, ta, tb, tc, a, 2 * pairs, st);
      case EPI_PLAIN_BF16: return launch_pair<EPI_PLAIN_BF16, false>(h, ta, tb, tc, a, 2 * pairs, st);
    }
  }
  if (p.b_fp8) {
    switch (p.epilogue) {
      case EPI_SWIGLU_BF16: return launch_epi<EPI_SWIGLU_BF16, true>(h, ta, tb, tc, a, grid, st);
      case EPI_PLAIN_BF16: return launch_epi<EPI_PLAIN_BF16, true>(h, ta, tb, tc, a, grid, st);
    }
  } else {
    switch (p.epilogue) {
      case EPI_SWIGLU_BF16: return launch_epi<EPI_SWIGLU_BF16, false>(h, ta, tb, tc, a, grid, st);
      case EPI_PLAIN_BF16: return launch_epi<EPI_PLAIN_BF16, false>(h, ta, tb, tc, a, grid, st);
      case EPI_PLAIN_F32: return launch_epi<EPI_PLAIN_F32, false>(h, ta, tb, tc, a, grid, st);
      case EPI_ROUND_BF16_F32: return launch_epi<EPI_ROUND_BF16_F32, false>(h, ta, tb, tc, a, grid, st);
    }
  }
  set_error("bad epilogue");
  return MG_ERR_CONFIG;
}

}  // namespace mg
