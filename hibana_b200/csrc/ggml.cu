// GGML block formats served in place: Q8_0, IQ2_XXS and IQ2_XS weight matrices stay in their checkpoint bytes on
// the device and are decoded inside the kernels that read them.
//
//   ggml_gemv_kernel     decode-sized products y[m][n] = sum_k x[m][k] W[n][k] for up to 8 activation rows: one
//                        warp per weight row, lanes striding over the row's blocks, every weight byte read once and
//                        expanded in registers (a decode step is bound by the weight stream: 2.06 to 8.5 bits per
//                        weight instead of 16). With `pairs` it is the grouped form a mixture-of-experts layer needs:
//                        work item p multiplies activation row pair_row[p] with expert pair_expert[p]'s matrix.
//   ggml_dequant_kernel  bf16 expansion of a matrix (or of a row range) for prefill-sized products, which then run
//                        on the tcgen05 GEMM.
//
// IQ2 formats index an E8-lattice codebook (256 x 8 or 512 x 8 magnitudes) that is part of the file format; the
// table comes with the checkpoint and is passed in as a device pointer, staged in shared memory per CTA.
// Block layouts (little endian): Q8_0 = fp16 d, 32 x int8; IQ2_XXS = fp16 d, 8 x {4 index bytes, u32: 4 x 7 sign
// bits + 4-bit scale}; IQ2_XS = fp16 d, 32 x u16 {9-bit index, 7 sign bits}, 8 scale bytes (two 4-bit scales).
// The eighth sign of every group of eight makes the number of negative signs even.
// Reference: hibana/kernels/csrc/iq2_moe.cu:72-338, hibana/kernels/csrc/ggml_codec.cuh, hibana/kernels/ggml_bf16.py.
#include "hb_api.h"
#include "hb_common.cuh"

#include <cuda_fp16.h>

namespace hb {
namespace {

constexpr int T_Q8_0 = 8, T_IQ2_XXS = 16, T_IQ2_XS = 17;
constexpr int GEMV_MAX_ROWS = 8;

__device__ __forceinline__ float half_at(const uint8_t* p) {
  const uint16_t raw = static_cast<uint16_t>(p[0]) | (static_cast<uint16_t>(p[1]) << 8);
  return __half2float(__ushort_as_half(raw));
}
__device__ __forceinline__ uint32_t u32_at(const uint8_t* p) {   // blocks are only 2-byte aligned
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
  return static_cast<uint32_t>(q[0]) | (static_cast<uint32_t>(q[1]) << 16);
}
// 7 stored sign bits -> 8 sign bits (even parity).
__device__ __forceinline__ uint32_t signs8(uint32_t s7) { return s7 | ((__popc(s7) & 1u) << 7); }

// Decodes 8 consecutive weights: group `g8` (0 .. K / 8) of a row.
template <int TYPE>
__device__ __forceinline__ void decode8(const uint8_t* row, int g8, const uint8_t* grid, float (&w)[8]) {
  if constexpr (TYPE == T_Q8_0) {
    const uint8_t* blk = row + (g8 >> 2) * 34;
    const float d = half_at(blk);
    const int8_t* q = reinterpret_cast<const int8_t*>(blk + 2 + (g8 & 3) * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = d * static_cast<float>(q[i]);
  } else if constexpr (TYPE == T_IQ2_XXS) {
    const uint8_t* blk = row + (g8 >> 5) * 66;
    const int sub = (g8 >> 2) & 7, j = g8 & 3;              // 32-weight sub-block, group of 8 inside it
    const uint8_t* qs = blk + 2 + sub * 8;
    const uint32_t aux = u32_at(qs + 4);
    const float db = half_at(blk) * (0.5f + static_cast<float>(aux >> 28)) * 0.25f;
    const uint8_t* gr = grid + static_cast<int>(qs[j]) * 8;
    const uint32_t sg = signs8((aux >> (7 * j)) & 127u);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = db * static_cast<float>(gr[i]) * (((sg >> i) & 1u) ? -1.f : 1.f);
  } else {
    const uint8_t* blk = row + (g8 >> 5) * 74;
    const int sub = (g8 >> 2) & 7, j = g8 & 3;
    const uint8_t* q = blk + 2 + (sub * 4 + j) * 2;
    const uint32_t v = static_cast<uint32_t>(q[0]) | (static_cast<uint32_t>(q[1]) << 8);
    const uint32_t sc = blk[66 + sub];
    const float db = half_at(blk) * (0.5f + static_cast<float>((j < 2) ? (sc & 15u) : (sc >> 4))) * 0.25f;
    const uint8_t* gr = grid + static_cast<int>(v & 511u) * 8;
    const uint32_t sg = signs8(v >> 9);
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = db * static_cast<float>(gr[i]) * (((sg >> i) & 1u) ? -1.f : 1.f);
  }
}

template <int TYPE>
__device__ __forceinline__ int grid_bytes() { return TYPE == T_IQ2_XXS ? 256 * 8 : TYPE == T_IQ2_XS ? 512 * 8 : 0; }

// grid (ceil(n / 4), items): 4 warps per CTA, one weight row per warp. items = 1 (plain) or the number of pairs.
template <int TYPE, int M>
__global__ void __launch_bounds__(128)
ggml_gemv_kernel(const uint8_t* __restrict__ w, long long row_bytes, long long expert_bytes, int n, int k,
                 const __nv_bfloat16* __restrict__ x, long long ldx, const uint8_t* __restrict__ grid_table,
                 const int* __restrict__ pair_expert, const int* __restrict__ pair_row, int relu2,
                 __nv_bfloat16* __restrict__ y, long long ldy) {
  extern __shared__ uint8_t grid_s[];
  constexpr int GB = TYPE == T_IQ2_XXS ? 2048 : TYPE == T_IQ2_XS ? 4096 : 0;
  for (int i = threadIdx.x * 4; i < GB; i += blockDim.x * 4)
    *reinterpret_cast<uint32_t*>(grid_s + i) = *reinterpret_cast<const uint32_t*>(grid_table + i);
  if (GB) __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + warp;
  if (row >= n) return;
  const int item = blockIdx.y;
  const uint8_t* wbase = w;
  const __nv_bfloat16* xb = x;
  __nv_bfloat16* yb = y;
  if (pair_expert != nullptr) {            // grouped: one activation row against its expert's matrix
    const int e = pair_expert[item];
    if (e < 0) return;
    wbase = w + static_cast<long long>(e) * expert_bytes;
    xb = x + static_cast<long long>(pair_row[item]) * ldx;
    yb = y + static_cast<long long>(item) * ldy;
  }
  const uint8_t* wr = wbase + static_cast<long long>(row) * row_bytes;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int g8 = lane; g8 < (k >> 3); g8 += 32) {
    float wv[8];
    decode8<TYPE>(wr, g8, grid_s, wv);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 xa = *reinterpret_cast<const uint4*>(xb + static_cast<long long>(m) * ldx + g8 * 8);
      const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[m] += wv[2 * i] * bf16_lo(xw[i]) + wv[2 * i + 1] * bf16_hi(xw[i]);
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float v = warp_sum(acc[m]);
    if (relu2) v = v > 0.f ? v * v : 0.f;
    if (lane == 0) yb[static_cast<long long>(m) * ldy + row] = __float2bfloat16(v);
  }
}

// One thread per 8 weights: rows [row0, row0 + rows) of the matrix -> bf16 [rows, k].
template <int TYPE>
__global__ void ggml_dequant_kernel(const uint8_t* __restrict__ w, long long row_bytes, int row0, int rows, int k,
                                    const uint8_t* __restrict__ grid_table, __nv_bfloat16* __restrict__ out) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = k >> 3;
  if (idx >= static_cast<long long>(rows) * per_row) return;
  const int r = static_cast<int>(idx / per_row), g8 = static_cast<int>(idx % per_row);
  float wv[8];
  decode8<TYPE>(w + static_cast<long long>(row0 + r) * row_bytes, g8, grid_table, wv);
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = pack_bf16(wv[2 * i], wv[2 * i + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<long long>(r) * k + g8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

template <int TYPE>
int launch_gemv(const uint8_t* w, long long row_bytes, long long expert_bytes, int n, int k, const __nv_bfloat16* x,
                long long ldx, int m, const uint8_t* grid, const int* pe, const int* pr, int items, int relu2,
                __nv_bfloat16* y, long long ldy, cudaStream_t st) {
  const dim3 g((n + 3) / 4, items);
  const int smem = TYPE == T_IQ2_XXS ? 2048 : TYPE == T_IQ2_XS ? 4096 : 0;
#define HB_GEMV(MM)                                                                                              \
  ggml_gemv_kernel<TYPE, MM><<<g, 128, smem, st>>>(w, row_bytes, expert_bytes, n, k, x, ldx, grid, pe, pr, relu2, y, ldy)
  switch (m) {
    case 1: HB_GEMV(1); break;
    case 2: HB_GEMV(2); break;
    case 4: HB_GEMV(4); break;
    default: HB_GEMV(8); break;
  }
#undef HB_GEMV
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

// y [m, n] = x [m, k] @ W^T for m in {1, 2, 4, 8} activation rows (the caller pads x and y to one of those).
// type: 8 Q8_0, 16 IQ2_XXS, 17 IQ2_XS. grid: the format's lattice table on the device (null for Q8_0).
int hb_ggml_gemv(int type, const void* w, long long row_bytes, int n, int k, const void* x, long long ldx, int m,
                 const void* grid, int relu2, void* y, long long ldy, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k % 256 != 0 && !(type == T_Q8_0 && k % 32 == 0)) return 1;
  if ((m != 1 && m != 2 && m != 4 && m != 8) || ldx % 8 != 0) return 1;
  if (type != T_Q8_0 && grid == nullptr) return 1;
  auto st = static_cast<cudaStream_t>(stream);
  auto W = static_cast<const uint8_t*>(w);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const uint8_t*>(grid);
  auto Y = static_cast<__nv_bfloat16*>(y);
  if (type == T_Q8_0) return launch_gemv<T_Q8_0>(W, row_bytes, 0, n, k, X, ldx, m, G, nullptr, nullptr, 1, relu2, Y, ldy, st);
  if (type == T_IQ2_XXS) return launch_gemv<T_IQ2_XXS>(W, row_bytes, 0, n, k, X, ldx, m, G, nullptr, nullptr, 1, relu2, Y, ldy, st);
  if (type == T_IQ2_XS) return launch_gemv<T_IQ2_XS>(W, row_bytes, 0, n, k, X, ldx, m, G, nullptr, nullptr, 1, relu2, Y, ldy, st);
  return 1;
}

// Grouped form: y [pairs, n], row p = x[pair_row[p]] @ W[pair_expert[p]]^T (pair_expert < 0: skipped).
int hb_ggml_gemv_pairs(int type, const void* w, long long row_bytes, long long expert_bytes, int n, int k,
                       const void* x, long long ldx, const void* grid, const void* pair_expert, const void* pair_row,
                       int pairs, int relu2, void* y, long long ldy, void* stream) {
  if (pairs <= 0 || n <= 0) return 0;
  if ((k % 256 != 0 && !(type == T_Q8_0 && k % 32 == 0)) || ldx % 8 != 0 || pairs > 65535) return 1;
  if (type != T_Q8_0 && grid == nullptr) return 1;
  auto st = static_cast<cudaStream_t>(stream);
  auto W = static_cast<const uint8_t*>(w);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const uint8_t*>(grid);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto PE = static_cast<const int*>(pair_expert);
  auto PR = static_cast<const int*>(pair_row);
  if (type == T_Q8_0) return launch_gemv<T_Q8_0>(W, row_bytes, expert_bytes, n, k, X, ldx, 1, G, PE, PR, pairs, relu2, Y, ldy, st);
  if (type == T_IQ2_XXS) return launch_gemv<T_IQ2_XXS>(W, row_bytes, expert_bytes, n, k, X, ldx, 1, G, PE, PR, pairs, relu2, Y, ldy, st);
  if (type == T_IQ2_XS) return launch_gemv<T_IQ2_XS>(W, row_bytes, expert_bytes, n, k, X, ldx, 1, G, PE, PR, pairs, relu2, Y, ldy, st);
  return 1;
}

int hb_ggml_dequant(int type, const void* w, long long row_bytes, int row0, int rows, int k, const void* grid,
                    void* out, void* stream) {
  if (rows <= 0) return 0;
  if (k % 8 != 0 || (type != T_Q8_0 && grid == nullptr)) return 1;
  const long long n = static_cast<long long>(rows) * (k >> 3);
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  auto st = static_cast<cudaStream_t>(stream);
  auto W = static_cast<const uint8_t*>(w);
  auto G = static_cast<const uint8_t*>(grid);
  auto O = static_cast<__nv_bfloat16*>(out);
  if (type == T_Q8_0) ggml_dequant_kernel<T_Q8_0><<<blocks, 256, 0, st>>>(W, row_bytes, row0, rows, k, G, O);
  else if (type == T_IQ2_XXS) ggml_dequant_kernel<T_IQ2_XXS><<<blocks, 256, 0, st>>>(W, row_bytes, row0, rows, k, G, O);
  else if (type == T_IQ2_XS) ggml_dequant_kernel<T_IQ2_XS><<<blocks, 256, 0, st>>>(W, row_bytes, row0, rows, k, G, O);
  else return 1;
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
