// Register-resident row core shared by the norm + quantise kernels (local, fused all-reduce, reduce-scatter +
// all-gather): one CTA per row, every thread owns chunks of 8 consecutive elements (one 16-byte load each), so all
// loads of a row are in flight at once and the row never goes through shared memory. Two neighbouring lanes hold
// one 16-element NVFP4 group; its amax is a single shuffle.
#pragma once
#include "hb_common.cuh"

namespace hb {

constexpr int ROW_MAX_DST = 8;

struct RowOut {
  int n;                          // destinations (1 = local, world = push to every rank)
  uint8_t* q[ROW_MAX_DST];        // packed e2m1 base of [rows, h / 2] (null = no NVFP4 output)
  uint8_t* sf[ROW_MAX_DST];       // swizzled scale blocks
  __nv_bfloat16* bf[ROW_MAX_DST]; // bf16 base of [rows, h] (null = no bf16 output)
};

__device__ __forceinline__ size_t row_sf_off(int row, int g, int ka) {
  const int rb = row >> 7, ri = row & 127;
  return (static_cast<size_t>(rb) * ka + (g >> 2)) * 512 + (ri & 31) * 16 + (ri >> 5) * 4 + (g & 3);
}

// Quantises 16 floats to NVFP4: writes 8 packed bytes and returns the ue4m3 scale byte (x ~= q * sf * global scale).
__device__ __forceinline__ uint32_t quant16(const float (&x)[16], float inv_gs, uint2* packed) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const uint32_t sfb = float_to_e4m3(amax * (1.f / 6.f) * inv_gs);
  const float sf = e4m3_to_float(sfb);
  const float inv = sf > 0.f ? 1.f / (sf * (1.f / inv_gs)) : 0.f;
  uint32_t w[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i >> 2] |= e2m1x2(x[2 * i] * inv, x[2 * i + 1] * inv) << (8 * (i & 3));
  *packed = make_uint2(w[0], w[1]);
  return sfb;
}

// 16 consecutive bf16 values (32-byte aligned address, global or shared) as floats.
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&x)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0];
  const uint4 b = reinterpret_cast<const uint4*>(p)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[2 * i] = bf16_lo(w[i]);
    x[2 * i + 1] = bf16_hi(w[i]);
  }
}

__device__ __forceinline__ void unpack8(const uint4& a, float (&f)[8]) {
  f[0] = bf16_lo(a.x); f[1] = bf16_hi(a.x); f[2] = bf16_lo(a.y); f[3] = bf16_hi(a.y);
  f[4] = bf16_lo(a.z); f[5] = bf16_hi(a.z); f[6] = bf16_lo(a.w); f[7] = bf16_hi(a.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

// v[i] holds chunk (tid + i * T) of the row (values already rounded to bf16 precision). Computes the RMS over the
// row, applies the weight, and writes bf16 and / or NVFP4 to every destination at row `out_row`.
// `red` is shared scratch of >= 33 floats. weight == null skips the normalisation (plain quantise / copy).
template <int T, int MAXC>
__device__ __forceinline__ void row_finish(float (&v)[MAXC][8], int h, const __nv_bfloat16* __restrict__ weight,
                                           float eps, int gemma, float* red, const RowOut& out, long long out_row,
                                           int ka, const float* __restrict__ gscale) {
  const int tid = threadIdx.x;
  const int nchunk = h >> 3;
  float rstd = 1.f;
  if (weight != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXC; ++i)
      if (tid + i * T < nchunk) {
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
      }
    ss = warp_sum(ss);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid < 32) {
      float t = tid < T / 32 ? red[tid] : 0.f;
      t = warp_sum(t);
      if (tid == 0) red[32] = rsqrtf(t / h + eps);
    }
    __syncthreads();
    rstd = red[32];
  }
  const bool want_q = out.q[0] != nullptr;
  const float inv_gs = want_q ? 1.f / *gscale : 0.f;
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = tid + i * T;
    const bool live = c < nchunk;
    float y[8];
    if (live) {
      if (weight != nullptr) {
        float w[8];
        unpack8(reinterpret_cast<const uint4*>(weight)[c], w);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          y[e] = __bfloat162float(__float2bfloat16(v[i][e] * rstd * (gemma ? 1.f + w[e] : w[e])));
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = v[i][e];
      }
      if (out.bf[0] != nullptr) {
        const uint4 pk = pack8(y);
        for (int d = 0; d < out.n; ++d) reinterpret_cast<uint4*>(out.bf[d] + out_row * h)[c] = pk;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = 0.f;
    }
    if (want_q) {
      // chunks c and c ^ 1 form one 16-element group; T is even, so they sit in neighbouring lanes
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(y[e]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      if (live) {
        const uint32_t sfb = float_to_e4m3(amax * (1.f / 6.f) * inv_gs);
        const float sfv = e4m3_to_float(sfb);
        const float inv = sfv > 0.f ? 1.f / (sfv * (1.f / inv_gs)) : 0.f;
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) w |= e2m1x2(y[2 * e] * inv, y[2 * e + 1] * inv) << (8 * e);
        const size_t so = row_sf_off(static_cast<int>(out_row), c >> 1, ka);
        for (int d = 0; d < out.n; ++d) {
          reinterpret_cast<uint32_t*>(out.q[d] + out_row * (h >> 1))[c] = w;
          if ((c & 1) == 0) out.sf[d][so] = static_cast<uint8_t>(sfb);
        }
      }
    }
  }
  if (want_q) {
    // padding groups of the last 256-element K tile get zero scales
    const int groups = h >> 4, groups_pad = ka * 4;
    for (int g = groups + tid; g < groups_pad; g += T)
      for (int d = 0; d < out.n; ++d) out.sf[d][row_sf_off(static_cast<int>(out_row), g, ka)] = 0;
  }
}

}  // namespace hb
