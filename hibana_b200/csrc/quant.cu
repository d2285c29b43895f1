// Activation quantisers for sm_100a.
//
// NVFP4: e2m1 values packed two per byte, one ue4m3 scale per 16 elements written straight into the
// 128x4-swizzled block layout that tcgen05.cp moves into TMEM, and a per-tensor fp32 scale supplied by the
// caller (x ~= q * sf * global_scale). Variants fuse the producer op so the bf16 activation is read once:
//   plain, RMSNorm -> quant, residual-add + RMSNorm -> quant, SiLU(gate) * up -> quant.
// FP8: static per-tensor e4m3, dynamic per-row e4m3.
//
// Covers what the reference does in hibana/kernels/nvfp4_quant.py:46-156, hibana/kernels/fp8_quant.py:19-88
// and hibana/kernels/cute/residual_norm.py:62-160.
#include "hb_common.cuh"
#include "hb_api.h"
#include "rownorm.cuh"

namespace hb {
namespace {

// One thread per 16-element group over the padded scale extent (padding scales are written as zero).
// mode 0: y = x; mode 1: y = silu(x[:, :K]) * x[:, K:2K] (x has 2K columns, gate first);
// mode 2: gate/up interleaved pairwise (x[:, 2j], x[:, 2j+1]).
__global__ void quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int m, int k, int ka,
                                   const float* __restrict__ gscale, uint8_t* __restrict__ q,
                                   uint8_t* __restrict__ sf, int mode, const int* __restrict__ src_rows,
                                   const int* __restrict__ total_rows) {
  grid_dep_wait();     // launched as a programmatic dependent: the producer of x must have completed
  grid_dep_launch();   // a GEMM launched as a programmatic dependent may start prefetching its weights
  const int groups_pad = ka * 4;
  const int rows_pad = ((m + 127) >> 7) << 7;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(rows_pad) * groups_pad) return;
  const int row = static_cast<int>(idx / groups_pad);
  const int g = static_cast<int>(idx % groups_pad);
  if (total_rows != nullptr && row >= *total_rows) return;   // beyond the planned segments: never read
  // Row-indirect mode (MoE): output row `row` of the sorted buffer takes input row src_rows[row] (-1 = padding).
  const int in_row = src_rows != nullptr ? (row < m ? src_rows[row] : -1) : row;
  if (row >= m || in_row < 0 || g * 16 >= k) {
    sf[row_sf_off(row, g, ka)] = 0;
    return;
  }
  const float inv_gs = 1.f / *gscale;
  float v[16];
  if (mode == 0) {
    load16(x + in_row * ldx + g * 16, v);
  } else if (mode == 1) {
    float u[16];
    load16(x + in_row * ldx + g * 16, v);
    load16(x + in_row * ldx + k + g * 16, u);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float s = v[i] / (1.f + __expf(-v[i]));
      v[i] = __bfloat162float(__float2bfloat16(s * u[i]));
    }
  } else {
    float a[16], b[16];
    load16(x + in_row * ldx + g * 32, a);
    load16(x + in_row * ldx + g * 32 + 16, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float g0 = a[2 * i], u0 = a[2 * i + 1], g1 = b[2 * i], u1 = b[2 * i + 1];
      v[i] = __bfloat162float(__float2bfloat16(g0 / (1.f + __expf(-g0)) * u0));
      v[8 + i] = __bfloat162float(__float2bfloat16(g1 / (1.f + __expf(-g1)) * u1));
    }
  }
  uint2 packed;
  const uint32_t sfb = quant16(v, inv_gs, &packed);
  *reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * (k / 2) + g * 8) = packed;
  sf[row_sf_off(row, g, ka)] = static_cast<uint8_t>(sfb);
}

// MoE sorted buffers at decode sizes: one thread per ((token, expert) pair, group of 16). The pair's row in the
// sorted buffer is pos[pair] (-1: routed elsewhere); its input row is the pair's token (topk > 0: x holds the
// tokens) or the sorted row itself (topk == 0: x is already sorted, e.g. the experts' hidden activations). Padding
// rows of the 128-row expert segments are not touched: the grouped GEMM computes token columns it never stores
// from them, so their codes and scales may hold anything.
__global__ void quant_nvfp4_pairs_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                         const int* __restrict__ pos, int pairs, int topk, int k, int ka,
                                         const float* __restrict__ gscale, uint8_t* __restrict__ q,
                                         uint8_t* __restrict__ sf) {
  grid_dep_wait();
  grid_dep_launch();
  const int groups_pad = ka * 4;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(pairs) * groups_pad) return;
  const int pair = static_cast<int>(idx / groups_pad), g = static_cast<int>(idx % groups_pad);
  const int row = pos[pair];
  if (row < 0) return;
  if (g * 16 >= k) {       // scale groups that pad the last K tile read as zero
    sf[row_sf_off(row, g, ka)] = 0;
    return;
  }
  const long long in_row = topk > 0 ? pair / topk : row;
  float v[16];
  load16(x + in_row * ldx + g * 16, v);
  uint2 packed;
  const uint32_t sfb = quant16(v, 1.f / *gscale, &packed);
  *reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * (k / 2) + g * 8) = packed;
  sf[row_sf_off(row, g, ka)] = static_cast<uint8_t>(sfb);
}

// (residual add +) RMSNorm -> NVFP4 (and / or bf16). One CTA per row on the register-resident row core.
// Writes the updated residual (bf16) when `residual` is given. gemma != 0 uses weight (1 + w).
template <int T, int MAXC>
__global__ void __launch_bounds__(T)
norm_quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                        const __nv_bfloat16* __restrict__ w, float eps, int gemma, int m, int k, int ka,
                        const float* __restrict__ gscale, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                        __nv_bfloat16* __restrict__ normed) {
  grid_dep_wait();     // launched as a programmatic dependent: the producer of x must have completed
  grid_dep_launch();   // a GEMM launched as a programmatic dependent may start prefetching its weights
  __shared__ float red[40];
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  if (row >= m) {   // padding rows of the last 128-row scale block: zero scales, nothing else
    for (int g = tid; g < ka * 4; g += T) sf[row_sf_off(row, g, ka)] = 0;
    return;
  }
  const int nchunk = k >> 3;
  float v[MAXC][8];
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * k);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + static_cast<size_t>(row) * k) : nullptr;
  uint4 xa[MAXC], ra[MAXC];
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = tid + i * T;
    if (c < nchunk) {
      xa[i] = xr[c];
      if (rr) ra[i] = rr[c];
    }
  }
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = tid + i * T;
    if (c < nchunk) {
      unpack8(xa[i], v[i]);
      if (rr) {
        float r[8];
        unpack8(ra[i], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16(v[i][e] + r[e]));
        rr[c] = pack8(v[i]);
      }
    }
  }
  RowOut out;
  out.n = 1;
  out.q[0] = q; out.sf[0] = sf; out.bf[0] = normed;
  row_finish<T, MAXC>(v, k, w, eps, gemma, red, out, row, ka, gscale);
}

// Zeroes the scale bytes of the padding rows [m, round_up(m, 128)) (used after the per-row kernel).
__global__ void sf_pad_rows_kernel(uint8_t* sf, int m, int ka) {
  const int rows_pad = ((m + 127) >> 7) << 7;
  const int groups_pad = ka * 4;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long n = static_cast<long long>(rows_pad - m) * groups_pad;
  if (idx >= n) return;
  sf[row_sf_off(m + static_cast<int>(idx / groups_pad), static_cast<int>(idx % groups_pad), ka)] = 0;
}

// Static per-tensor FP8 (e4m3): q = sat(x / scale). 8 elements per thread.
__global__ void quant_fp8_static_kernel(const __nv_bfloat16* __restrict__ x, long long n,
                                        const float* __restrict__ scale, uint8_t* __restrict__ q) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  const float inv = 1.f / *scale;
  if (i + 8 <= n) {
    const uint4 a = *reinterpret_cast<const uint4*>(x + i);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
    uint32_t o[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j >> 1] |= float_to_e4m3(bf16_lo(w[j]) * inv) << (16 * (j & 1));
      o[j >> 1] |= float_to_e4m3(bf16_hi(w[j]) * inv) << (16 * (j & 1) + 8);
    }
    *reinterpret_cast<uint2*>(q + i) = make_uint2(o[0], o[1]);
  } else {
    for (long long j = i; j < n; ++j) q[j] = static_cast<uint8_t>(float_to_e4m3(__bfloat162float(x[j]) * inv));
  }
}

// Dynamic per-row FP8: scale[row] = amax / 448, q = x / scale. One warp per row.
__global__ void quant_fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, int m, int k, uint8_t* __restrict__ q,
                                      float* __restrict__ scales) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= m) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * k;
  float amax = 0.f;
  for (int i = lane; i < k; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(xr[i])));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  for (int i = lane; i < k; i += 32)
    q[static_cast<size_t>(row) * k + i] = static_cast<uint8_t>(float_to_e4m3(__bfloat162float(xr[i]) * inv));
  if (lane == 0) scales[row] = scale;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

// src_rows / total_rows (both may be null): row-indirect mode for MoE sorted buffers; m is then the row capacity.
int hb_quant_nvfp4_rows(const void* x, long long ldx, int m, int k, int ka, const void* gscale, void* q, void* sf,
                        int mode, const void* src_rows, const void* total_rows, void* stream) {
  if (k % 16 != 0 || ka * 64 < k) return 1;
  const int rows_pad = ((m + 127) / 128) * 128;
  const long long n = static_cast<long long>(rows_pad) * ka * 4;
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  launch_dep(quant_nvfp4_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), ldx, m, k, ka, static_cast<const float*>(gscale),
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), mode, static_cast<const int*>(src_rows),
      static_cast<const int*>(total_rows));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_quant_nvfp4_pairs(const void* x, long long ldx, const void* pos, int pairs, int topk, int k, int ka,
                         const void* gscale, void* q, void* sf, void* stream) {
  if (pairs <= 0) return 0;
  if (k % 16 != 0 || ka * 64 < k) return 1;
  const long long n = static_cast<long long>(pairs) * ka * 4;
  launch_dep(quant_nvfp4_pairs_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), ldx,
             static_cast<const int*>(pos), pairs, topk, k, ka, static_cast<const float*>(gscale),
             static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_quant_nvfp4(const void* x, long long ldx, int m, int k, int ka, const void* gscale, void* q, void* sf,
                   int mode, void* stream) {
  if (k % 16 != 0 || ka * 64 < k) return 1;
  const int rows_pad = ((m + 127) / 128) * 128;
  const long long n = static_cast<long long>(rows_pad) * ka * 4;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
  launch_dep(quant_nvfp4_kernel, dim3(blocks), dim3(threads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const __nv_bfloat16*>(x), ldx, m, k, ka, static_cast<const float*>(gscale),
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), mode, nullptr, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_norm_quant_nvfp4(const void* x, void* residual, const void* w, float eps, int gemma, int m, int k, int ka,
                        const void* gscale, void* q, void* sf, void* normed, void* stream) {
  if (k % 16 != 0 || (q != nullptr && ka * 64 < k) || k > 8192) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  constexpr int T = 256;
  const int rows_pad = q != nullptr ? ((m + 127) / 128) * 128 : m;
  const int nchunk = k / 8;
#define HB_NQ(MAXC)                                                                                              \
  launch_dep(norm_quant_nvfp4_kernel<T, MAXC>, dim3(rows_pad), dim3(T), 0, st,                                   \
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(residual),                               \
      static_cast<const __nv_bfloat16*>(w), eps, gemma, m, k, ka, static_cast<const float*>(gscale),             \
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), static_cast<__nv_bfloat16*>(normed))
  if (nchunk <= T) HB_NQ(1);
  else if (nchunk <= 2 * T) HB_NQ(2);
  else if (nchunk <= 3 * T) HB_NQ(3);
  else HB_NQ(4);
#undef HB_NQ
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_quant_fp8_static(const void* x, long long n, const void* scale, void* q, void* stream) {
  const long long threads = (n + 7) / 8;
  quant_fp8_static_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), n, static_cast<const float*>(scale), static_cast<uint8_t*>(q));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_quant_fp8_rows(const void* x, int m, int k, void* q, void* scales, void* stream) {
  quant_fp8_rows_kernel<<<(m + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), m, k, static_cast<uint8_t*>(q), static_cast<float*>(scales));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
