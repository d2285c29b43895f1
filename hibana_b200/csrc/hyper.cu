// Hyper-connections (hc residual streams of width H per token, mixed into one block input and re-injected after the
// block), the three memory-bound steps around the two small GEMMs of a site:
//   grouped_norm   normed[t, s, :] = hyper[t, s, :] * rsqrt(mean_s(hyper^2) + eps) * (1 + w[s, :])    per stream s
//   gate_mean      mixed[t, :]     = (1 / hc) * sum_s sigmoid(gate_logits[t, s, :]) * normed[t, s, :]
//   inject_combine hyper'[t, s, :] = hyper[t, s, :] + block_out[t, :] * 2 * sigmoid(inject_logits[t, s])
// One CTA per token; every thread keeps 8-element chunks in registers, so each tensor is read once.
// Reference: hibana/model/flashnext/hyper.py:1-121 (math), hibana/kernels/flashnext_fused.py:25-250 (its Triton
// kernels for the same steps).
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

__device__ __forceinline__ void unpack(const uint4& a, float (&f)[8]) {
  f[0] = bf16_lo(a.x); f[1] = bf16_hi(a.x); f[2] = bf16_lo(a.y); f[3] = bf16_hi(a.y);
  f[4] = bf16_lo(a.z); f[5] = bf16_hi(a.z); f[6] = bf16_lo(a.w); f[7] = bf16_hi(a.w);
}
__device__ __forceinline__ uint4 pack(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// grid (tokens, hc): one CTA normalises one stream of one token. H <= 8 * 256 * MAXC.
template <int MAXC>
__global__ void __launch_bounds__(256) hc_norm_kernel(const __nv_bfloat16* __restrict__ hyper,
                                                      const __nv_bfloat16* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ normed, int hc, int h, float eps) {
  __shared__ float red[33];
  const long long base = (static_cast<long long>(blockIdx.x) * hc + blockIdx.y) * h;
  const int nchunk = h >> 3;
  float v[MAXC][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nchunk) {
      unpack(reinterpret_cast<const uint4*>(hyper + base)[c], v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) red[32] = rsqrtf(t / h + eps);
  }
  __syncthreads();
  const float rstd = red[32];
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nchunk) {
      float ww[8], y[8];
      unpack(reinterpret_cast<const uint4*>(w + static_cast<long long>(blockIdx.y) * h)[c], ww);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = v[i][e] * rstd * (1.f + ww[e]);
      reinterpret_cast<uint4*>(normed + base)[c] = pack(y);
    }
  }
}

__global__ void __launch_bounds__(256) hc_gate_mean_kernel(const __nv_bfloat16* __restrict__ gate,
                                                           const __nv_bfloat16* __restrict__ normed,
                                                           __nv_bfloat16* __restrict__ mixed, int hc, int h) {
  const long long base = static_cast<long long>(blockIdx.x) * hc * h;
  const float inv = 1.f / hc;
  for (int c = threadIdx.x; c < (h >> 3); c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < hc; ++s) {
      float g[8], n[8];
      unpack(reinterpret_cast<const uint4*>(gate + base + static_cast<long long>(s) * h)[c], g);
      unpack(reinterpret_cast<const uint4*>(normed + base + static_cast<long long>(s) * h)[c], n);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += sigmoidf(g[e]) * n[e];
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv;
    reinterpret_cast<uint4*>(mixed + static_cast<long long>(blockIdx.x) * h)[c] = pack(acc);
  }
}

__global__ void __launch_bounds__(256) hc_inject_kernel(const __nv_bfloat16* __restrict__ hyper,
                                                        const __nv_bfloat16* __restrict__ block_out,
                                                        const float* __restrict__ inject_logits, long long ld_logits,
                                                        __nv_bfloat16* __restrict__ out, int hc, int h) {
  const long long base = static_cast<long long>(blockIdx.x) * hc * h;
  for (int c = threadIdx.x; c < (h >> 3); c += blockDim.x) {
    float b[8];
    unpack(reinterpret_cast<const uint4*>(block_out + static_cast<long long>(blockIdx.x) * h)[c], b);
    for (int s = 0; s < hc; ++s) {
      const float inj = 2.f * sigmoidf(inject_logits[static_cast<long long>(blockIdx.x) * ld_logits + s]);
      float x[8];
      unpack(reinterpret_cast<const uint4*>(hyper + base + static_cast<long long>(s) * h)[c], x);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] += b[e] * inj;
      reinterpret_cast<uint4*>(out + base + static_cast<long long>(s) * h)[c] = pack(x);
    }
  }
}

// low[t][j] = silu(bf16(x[t][j])) for the first `rank` columns of the fp32 rows x (pitch ldx): the activation
// between the two low-rank gate projections, applied to the bf16-rounded value as a bf16 GEMM output would carry it.
__global__ void hc_low_kernel(const float* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ low, int rows,
                              int rank) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * rank) return;
  const int r = i / rank, j = i - r * rank;
  const float v = __bfloat162float(__float2bfloat16(x[r * ldx + j]));
  low[i] = __float2bfloat16(v / (1.f + __expf(-v)));
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

int hb_hc_norm(const void* hyper, const void* w, void* normed, int tokens, int hc, int h, float eps, void* stream) {
  if (tokens <= 0) return 0;
  if (h % 8 != 0 || h > 8 * 256 * 4) return 1;
  const dim3 grid(tokens, hc);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto a = static_cast<const __nv_bfloat16*>(hyper);
  auto b = static_cast<const __nv_bfloat16*>(w);
  auto o = static_cast<__nv_bfloat16*>(normed);
  const int nchunk = h >> 3;
  if (nchunk <= 256) hc_norm_kernel<1><<<grid, 256, 0, st>>>(a, b, o, hc, h, eps);
  else if (nchunk <= 512) hc_norm_kernel<2><<<grid, 256, 0, st>>>(a, b, o, hc, h, eps);
  else hc_norm_kernel<4><<<grid, 256, 0, st>>>(a, b, o, hc, h, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_hc_gate_mean(const void* gate, const void* normed, void* mixed, int tokens, int hc, int h, void* stream) {
  if (tokens <= 0) return 0;
  if (h % 8 != 0) return 1;
  hc_gate_mean_kernel<<<tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(normed),
      static_cast<__nv_bfloat16*>(mixed), hc, h);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_hc_inject(const void* hyper, const void* block_out, const void* inject_logits, long long ld_logits, void* out,
                 int tokens, int hc, int h, void* stream) {
  if (tokens <= 0) return 0;
  if (h % 8 != 0) return 1;
  hc_inject_kernel<<<tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(hyper), static_cast<const __nv_bfloat16*>(block_out),
      static_cast<const float*>(inject_logits), ld_logits, static_cast<__nv_bfloat16*>(out), hc, h);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_hc_low(const void* x, long long ldx, void* low, int rows, int rank, void* stream) {
  if (rows <= 0) return 0;
  hc_low_kernel<<<(rows * rank + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(x), ldx, static_cast<__nv_bfloat16*>(low), rows, rank);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
