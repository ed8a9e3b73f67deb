// Packed per-expert weight layout and FP8 (e4m3, 128x128 block scale) de-quantisation.
//
// Packed buffer of one layer on one rank (E_l = experts owned, I = intermediate, H = hidden):
//   W13 [E_l][2I][H]  gate and up rows interleaved in 128-row blocks: rows [256b, 256b+128)
//                     are gate rows [128b, 128b+128), rows [256b+128, 256b+256) the matching
//                     up rows.  A 256-row N tile of the first GEMM therefore holds the gate
//                     and up columns of the same 128 outputs, and every 128x128 FP8 scale
//                     block stays whole.
//   W2  [E_l][H][I]   down_proj as stored by nn.Linear.
//   S13 [E_l][2I/128][H/128], S2 [E_l][H/128][I/128]  fp32 scales (FP8 layers only), in the
//                     same block order as the rows they scale.
//   SH13 [2I_s][H], SH2 [H][I_s]   shared expert, always bf16, same interleave.
// nn.Linear weights are [out, in] row-major = "N x K, K-major", which is the B operand
// layout of the GEMM, so packing is a copy.
#include <cuda_fp8.h>

#include "common.cuh"

namespace mg {

PackedLayout packed_layout(const Handle* h) {
  const mg_layer_desc& d = h->d;
  PackedLayout L;
  const size_t E = h->e_local, I = d.inter, H = d.hidden, Is = d.inter_shared;
  L.w_elem = d.weight_format == MG_WEIGHT_FP8_BLOCK128 ? 1 : 2;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) / 256 * 256; return o; };
  L.w13 = take(E * 2 * I * H * L.w_elem);
  L.w2 = take(E * H * I * L.w_elem);
  if (d.weight_format == MG_WEIGHT_FP8_BLOCK128) {
    L.s13 = take(E * (2 * I / 128) * (H / 128) * 4);
    L.s2 = take(E * (H / 128) * (I / 128) * 4);
  } else {
    L.s13 = L.s2 = off;
  }
  L.sh13 = take(2 * Is * H * 2);
  L.sh2 = take(H * Is * 2);
  L.total = off;
  return L;
}

// copy `rows` rows of `vec_per_row` uint4 each; destination row = map(r)
__global__ void __launch_bounds__(256) interleave_rows_kernel(const uint4* __restrict__ gate,
                                                              const uint4* __restrict__ up, int rows_each,
                                                              int vec_per_row, uint4* __restrict__ dst) {
  // one block per source row pair (gate row r and up row r)
  const int r = blockIdx.x;
  const int64_t g_dst = (static_cast<int64_t>(r / 128) * 256 + (r % 128)) * vec_per_row;
  const int64_t u_dst = g_dst + static_cast<int64_t>(128) * vec_per_row;
  for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
    dst[g_dst + v] = gate[static_cast<int64_t>(r) * vec_per_row + v];
    dst[u_dst + v] = up[static_cast<int64_t>(r) * vec_per_row + v];
  }
}

__global__ void __launch_bounds__(256) copy_vec_kernel(const uint4* __restrict__ src, int64_t n,
                                                       uint4* __restrict__ dst) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

// scales of gate/up ([I/128][H/128] each) -> interleaved [2I/128][H/128]
__global__ void interleave_scales_kernel(const float* __restrict__ gs, const float* __restrict__ us,
                                         int brows, int bcols, float* __restrict__ dst) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < brows * bcols) {
    int r = i / bcols, c = i % bcols;
    dst[(2 * r) * bcols + c] = gs[i];
    dst[(2 * r + 1) * bcols + c] = us[i];
  }
}

int launch_pack_expert(const Handle* h, int local_expert, const void* g, const void* u, const void* dn,
                       const float* gs, const float* us, const float* ds, void* packed, cudaStream_t st) {
  const mg_layer_desc& d = h->d;
  const PackedLayout L = packed_layout(h);
  uint8_t* base = static_cast<uint8_t*>(packed);
  const size_t H = d.hidden;
  if (local_expert < 0) {
    const size_t Is = d.inter_shared;
    MG_REQUIRE(Is > 0, MG_ERR_CONFIG, "layer has no shared expert");
    const int vpr = static_cast<int>(H * 2 / 16);
    interleave_rows_kernel<<<static_cast<unsigned>(Is), 256, 0, st>>>(
        static_cast<const uint4*>(g), static_cast<const uint4*>(u), static_cast<int>(Is), vpr,
        reinterpret_cast<uint4*>(base + L.sh13));
    MG_CUDA(cudaGetLastError());
    copy_vec_kernel<<<1024, 256, 0, st>>>(static_cast<const uint4*>(dn), static_cast<int64_t>(H * Is * 2 / 16),
                                          reinterpret_cast<uint4*>(base + L.sh2));
    MG_CUDA(cudaGetLastError());
    return MG_OK;
  }
  MG_REQUIRE(local_expert < h->e_local, MG_ERR_SHAPE, "local_expert %d out of range [0,%d)", local_expert,
             h->e_local);
  const size_t I = d.inter, w = L.w_elem;
  const int vpr = static_cast<int>(H * w / 16);
  interleave_rows_kernel<<<static_cast<unsigned>(I), 256, 0, st>>>(
      static_cast<const uint4*>(g), static_cast<const uint4*>(u), static_cast<int>(I), vpr,
      reinterpret_cast<uint4*>(base + L.w13 + static_cast<size_t>(local_expert) * 2 * I * H * w));
  MG_CUDA(cudaGetLastError());
  copy_vec_kernel<<<1024, 256, 0, st>>>(static_cast<const uint4*>(dn), static_cast<int64_t>(H * I * w / 16),
                                        reinterpret_cast<uint4*>(base + L.w2 + static_cast<size_t>(local_expert) * H * I * w));
  MG_CUDA(cudaGetLastError());
  if (d.weight_format == MG_WEIGHT_FP8_BLOCK128) {
    MG_REQUIRE(gs && us && ds, MG_ERR_NULL, "FP8 layer needs the three scale tensors");
    const int br = static_cast<int>(I / 128), bc = static_cast<int>(H / 128);
    float* s13 = reinterpret_cast<float*>(base + L.s13) + static_cast<size_t>(local_expert) * 2 * br * bc;
    interleave_scales_kernel<<<(br * bc + 255) / 256, 256, 0, st>>>(gs, us, br, bc, s13);
    MG_CUDA(cudaGetLastError());
    float* s2 = reinterpret_cast<float*>(base + L.s2) + static_cast<size_t>(local_expert) * bc * br;
    MG_CUDA(cudaMemcpyAsync(s2, ds, sizeof(float) * bc * br, cudaMemcpyDeviceToDevice, st));
  }
  return MG_OK;
}

// ---------------------------------------------------------------------------------------
// FP8 e4m3 -> bf16 with 128x128 block scales: bf16(float(q) * s)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void dequant16(const uint4& q, float s, uint4* out2) {
  const __nv_fp8x2_storage_t* p = reinterpret_cast<const __nv_fp8x2_storage_t*>(&q);
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p[i], __NV_E4M3);
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
    __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(f.x, s), __fmul_rn(f.y, s));
    o[i] = *reinterpret_cast<uint32_t*>(&b);
  }
  out2[0] = make_uint4(o[0], o[1], o[2], o[3]);
  out2[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// matrices stacked along rows: n_mat matrices of [rows, cols]; scales [n_mat][ceil(rows/128)][ceil(cols/128)]
__global__ void __launch_bounds__(256) dequant_kernel(const uint4* __restrict__ q, const float* __restrict__ scale,
                                                      int64_t total_rows, int rows_per_mat, int cols,
                                                      uint4* __restrict__ out) {
  const int vpr = cols / 16;
  const int brows = (rows_per_mat + 127) / 128, bcols = (cols + 127) / 128;
  const int64_t n = total_rows * vpr;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vpr;
    const int v = static_cast<int>(i - r * vpr);
    const int64_t mat = r / rows_per_mat;
    const int rr = static_cast<int>(r - mat * rows_per_mat);
    const float s = __ldg(scale + (mat * brows + rr / 128) * bcols + (v * 16) / 128);
    uint4 o[2];
    dequant16(__ldg(q + i), s, o);
    out[2 * i] = o[0];
    out[2 * i + 1] = o[1];
  }
}

int launch_dequant(const void* q, const float* s, int64_t rows, int64_t cols, void* out, cudaStream_t st) {
  MG_REQUIRE(cols % 16 == 0, MG_ERR_SHAPE, "dequant: cols=%lld must be a multiple of 16", static_cast<long long>(cols));
  if (rows == 0) return MG_OK;
  int64_t n = rows * (cols / 16);
  int grid = static_cast<int>(n / 256 + 1 < 148 * 16 ? n / 256 + 1 : 148 * 16);
  dequant_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(q), s, rows, static_cast<int>(rows),
                                       static_cast<int>(cols), static_cast<uint4*>(out));
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

// The packed matrices are stacks of [rows, cols] blocks whose rows and cols are multiples of 128, so
// the scales of the stack are one contiguous [total_rows/128][cols/128] array.  One warp converts 512
// consecutive bytes of a row per step (32 lanes x 16 bytes, four scale blocks), four steps in flight
// per lane: pure streaming at 3 bytes of HBM traffic per element, no per-element index arithmetic.
constexpr int kDeqUnroll = 4;
__global__ void __launch_bounds__(256) dequant_rows_kernel(const uint4* __restrict__ q, const float* __restrict__ scale,
                                                           int64_t total_rows, int cols, uint4* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int segs = cols >> 9;                              // 512-byte segments per row
  const int bcols = cols >> 7;
  const int64_t n_units = total_rows * segs;
  const int64_t warp0 = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t u0 = warp0 * kDeqUnroll; u0 < n_units; u0 += n_warps * kDeqUnroll) {
    uint4 v[kDeqUnroll];
    float sc[kDeqUnroll];
    int64_t at[kDeqUnroll];
#pragma unroll
    for (int j = 0; j < kDeqUnroll; ++j) {
      const int64_t u = u0 + j;
      at[j] = -1;
      if (u < n_units) {
        const int64_t row = u / segs;
        const int seg = static_cast<int>(u - row * segs);
        at[j] = (row * cols + (seg << 9)) / 16 + lane;     // 16-byte vector index of this lane's FP8 bytes
        v[j] = __ldcs(q + at[j]);
        sc[j] = __ldg(scale + (row >> 7) * bcols + (seg << 2) + (lane >> 3));
      }
    }
#pragma unroll
    for (int j = 0; j < kDeqUnroll; ++j) {
      if (at[j] >= 0) {
        uint4 o[2];
        dequant16(v[j], sc[j], o);
        out[2 * at[j]] = o[0];
        out[2 * at[j] + 1] = o[1];
      }
    }
  }
}

// which = 0: W13 of experts [e_lo, e_lo+e_n) -> bf16_out (same element layout as the packed
// W13); which = 1: W2 likewise into the W2 part of bf16_out
int launch_dequant_packed(const Handle* h, const void* packed, void* bf16_out, int which, int e_lo, int e_n,
                          cudaStream_t st) {
  const mg_layer_desc& d = h->d;
  const PackedLayout L = packed_layout(h);
  const uint8_t* base = static_cast<const uint8_t*>(packed);
  const int64_t E = h->e_local, I = d.inter, H = d.hidden;
  __nv_bfloat16* o13 = static_cast<__nv_bfloat16*>(bf16_out);
  __nv_bfloat16* o2 = o13 + E * 2 * I * H;
  if (e_n <= 0) return MG_OK;
  const int grid = h->sm_count * 8;
  const int64_t rows = which == 0 ? 2 * I : H, cols = which == 0 ? H : I;
  const int64_t off = e_lo * rows;
  const uint8_t* src = base + (which == 0 ? L.w13 : L.w2) + off * cols;
  const float* sc = reinterpret_cast<const float*>(base + (which == 0 ? L.s13 : L.s2)) + off / 128 * (cols / 128);
  __nv_bfloat16* dst = (which == 0 ? o13 : o2) + off * cols;
  if (cols % 512 == 0 && rows % 128 == 0) {
    dequant_rows_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), sc, e_n * rows,
                                              static_cast<int>(cols), reinterpret_cast<uint4*>(dst));
  } else {
    dequant_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), sc, e_n * rows,
                                         static_cast<int>(rows), static_cast<int>(cols), reinterpret_cast<uint4*>(dst));
  }
  MG_CUDA(cudaGetLastError());
  return MG_OK;
}

}  // namespace mg
