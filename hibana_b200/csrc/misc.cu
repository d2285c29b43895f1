// Memory-bound pointwise / row kernels for sm_100a: RMSNorm family, RoPE + q/k norm + KV-pool write,
// SiLU-mul, ReLU^2, sigmoid gates, embedding gather, residual add.
//
// Reference counterparts: hibana/model/norm.py:14-71, hibana/model/nemotron/norm.py:23-84,
// hibana/kernels/qk_norm_rope.py:16, hibana/model/rope.py:12, hibana/kernels/nemotron_fused.py:20,
// hibana/cache/kv_pool.py:120-132, hibana/kernels/flashnext_fused.py:624-660, hibana/kernels/mamba2.py:797.
#include "hb_api.h"
#include "hb_common.cuh"
#include "rownorm.cuh"

namespace hb {
namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}

// y = rmsnorm(x (+ residual)) * w; when residual != null it is updated in place with x + residual.
// One CTA per row; 8 bf16 per thread per step; row cached in registers for H <= 8 * 8 * blockDim.
template <int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int h, long long ldx,
               long long ldy, float eps, int gemma) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = h >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + static_cast<long long>(row) * h) : nullptr;
  float v[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      const uint4 a = xr[idx];
      v[i][0] = bf16_lo(a.x); v[i][1] = bf16_hi(a.x); v[i][2] = bf16_lo(a.y); v[i][3] = bf16_hi(a.y);
      v[i][4] = bf16_lo(a.z); v[i][5] = bf16_hi(a.z); v[i][6] = bf16_lo(a.w); v[i][7] = bf16_hi(a.w);
      if (rr) {
        const uint4 b = rr[idx];
        const float r[8] = {bf16_lo(b.x), bf16_hi(b.x), bf16_lo(b.y), bf16_hi(b.y),
                            bf16_lo(b.z), bf16_hi(b.z), bf16_lo(b.w), bf16_hi(b.w)};
#pragma unroll
        for (int t = 0; t < 8; ++t) v[i][t] = __bfloat162float(__float2bfloat16(v[i][t] + r[t]));
        rr[idx] = make_uint4(pack_bf16(v[i][0], v[i][1]), pack_bf16(v[i][2], v[i][3]), pack_bf16(v[i][4], v[i][5]),
                             pack_bf16(v[i][6], v[i][7]));
      }
#pragma unroll
      for (int t = 0; t < 8; ++t) ss += v[i][t] * v[i][t];
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / h + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      const uint4 b = wr[idx];
      float ww[8] = {bf16_lo(b.x), bf16_hi(b.x), bf16_lo(b.y), bf16_hi(b.y),
                     bf16_lo(b.z), bf16_hi(b.z), bf16_lo(b.w), bf16_hi(b.w)};
      float o[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) o[t] = v[i][t] * rstd * (gemma ? 1.f + ww[t] : ww[t]);
      yr[idx] = make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
    }
  }
}

// Gated grouped RMSNorm (Mamba-2 / GDN output): y = rmsnorm_g(x * silu(z)) * w with groups of `gs` channels,
// or norm-before-gate when norm_first != 0: y = rmsnorm_g(x) * w * silu(z). One warp per (row, group).
__global__ void gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ z,
                                     const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int rows,
                                     int h, int gs, long long ldx, long long ldz, float eps, int norm_first,
                                     int sigmoid_gate, int gemma, uint8_t* __restrict__ q_out,
                                     uint8_t* __restrict__ q_sf, const float* __restrict__ q_gscale, int q_ka) {
  const int groups = h / gs;
  const long long wid0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  // Fast path: the group fits in registers as 16-byte chunks (up to 4 per lane = 1024 features): one read of x and
  // z, one exp per element, 16-byte stores.
  if (gs % 8 == 0 && gs <= 1024 && ldx % 8 == 0 && (z == nullptr || ldz % 8 == 0) && h % 8 == 0) {
    if (wid0 >= static_cast<long long>(rows) * groups) return;
    const int lane_ = threadIdx.x & 31;
    const int row_ = static_cast<int>(wid0 / groups), g_ = static_cast<int>(wid0 % groups);
    const uint4* xr4 = reinterpret_cast<const uint4*>(x + row_ * ldx + g_ * gs);
    const uint4* zr4 = z ? reinterpret_cast<const uint4*>(z + row_ * ldz + g_ * gs) : nullptr;
    const uint4* wr4 = reinterpret_cast<const uint4*>(w + g_ * gs);
    const int nchunk = gs >> 3;
    float v[4][8], gt[4][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int ci = lane_ + c * 32;
      if (ci < nchunk) {
        const uint4 xa = xr4[ci];
        const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w};
        uint32_t zw[4] = {0, 0, 0, 0};
        if (zr4) {
          const uint4 za = zr4[ci];
          zw[0] = za.x; zw[1] = za.y; zw[2] = za.z; zw[3] = za.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xv = (e & 1) ? bf16_hi(xw[e >> 1]) : bf16_lo(xw[e >> 1]);
          float gate = 1.f;
          if (zr4) {
            const float zz = (e & 1) ? bf16_hi(zw[e >> 1]) : bf16_lo(zw[e >> 1]);
            gate = sigmoid_gate ? 1.f / (1.f + __expf(-zz)) : zz / (1.f + __expf(-zz));
          }
          gt[c][e] = gate;
          v[c][e] = norm_first ? xv : xv * gate;
          ss += v[c][e] * v[c][e];
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(ss) / gs + eps);
    uint4* yr4 = reinterpret_cast<uint4*>(y + static_cast<long long>(row_) * h + g_ * gs);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int ci = lane_ + c * 32;
      const unsigned act = __ballot_sync(0xffffffffu, ci < nchunk);     // lanes that share the shuffle below
      if (ci < nchunk) {
        const uint4 wa = wr4[ci];
        const uint32_t ww4[4] = {wa.x, wa.y, wa.z, wa.w};
        uint32_t o4[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float o2[2];
#pragma unroll
          for (int d = 0; d < 2; ++d) {
            const float ww = d ? bf16_hi(ww4[e >> 1]) : bf16_lo(ww4[e >> 1]);
            const float wv = gemma ? 1.f + ww : ww;
            o2[d] = norm_first ? v[c][e + d] * rstd * wv * gt[c][e + d] : v[c][e + d] * rstd * wv;
          }
          const __nv_bfloat162 pk = __floats2bfloat162_rn(o2[0], o2[1]);
          o4[e >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
        }
        if (q_out == nullptr) {
          yr4[ci] = make_uint4(o4[0], o4[1], o4[2], o4[3]);
          continue;
        }
        // NVFP4 output for the projection that follows: chunks ci and ci ^ 1 (neighbouring lanes) are one
        // 16-element scale group; values are the bf16-rounded outputs, as a separate quantiser would see them
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          f[2 * e] = bf16_lo(o4[e]);
          f[2 * e + 1] = bf16_hi(o4[e]);
        }
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
        amax = fmaxf(amax, __shfl_xor_sync(act, amax, 1));
        const float inv_gs = 1.f / *q_gscale;
        const uint32_t sfb = float_to_e4m3(amax * (1.f / 6.f) * inv_gs);
        const float sfv = e4m3_to_float(sfb);
        const float inv = sfv > 0.f ? 1.f / (sfv * (1.f / inv_gs)) : 0.f;
        uint32_t wq = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) wq |= e2m1x2(f[2 * e] * inv, f[2 * e + 1] * inv) << (8 * e);
        const int col8 = (g_ * gs >> 3) + ci;                  // 8-element chunk index inside the row
        reinterpret_cast<uint32_t*>(q_out + static_cast<size_t>(row_) * (h >> 1))[col8] = wq;
        if ((ci & 1) == 0) q_sf[row_sf_off(row_, col8 >> 1, q_ka)] = static_cast<uint8_t>(sfb);
      }
    }
    return;
  }
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(rows) * groups) return;
  const int row = static_cast<int>(wid / groups), g = static_cast<int>(wid % groups);
  const __nv_bfloat16* xr = x + row * ldx + g * gs;
  const __nv_bfloat16* zr = z ? z + row * ldz + g * gs : nullptr;
  float ss = 0.f;
  for (int i = lane; i < gs; i += 32) {
    float v = __bfloat162float(xr[i]);
    if (zr && !norm_first) {
      const float zz = __bfloat162float(zr[i]);
      v *= sigmoid_gate ? 1.f / (1.f + __expf(-zz)) : zz / (1.f + __expf(-zz));
    }
    ss += v * v;
  }
  const float rstd = rsqrtf(warp_sum(ss) / gs + eps);
  for (int i = lane; i < gs; i += 32) {
    float v = __bfloat162float(xr[i]);
    float gate = 1.f;
    if (zr) {
      const float zz = __bfloat162float(zr[i]);
      gate = sigmoid_gate ? 1.f / (1.f + __expf(-zz)) : zz / (1.f + __expf(-zz));
    }
    const float ww = __bfloat162float(w[g * gs + i]);
    const float wv = gemma ? 1.f + ww : ww;
    const float o = norm_first ? v * rstd * wv * gate : v * gate * rstd * wv;
    y[static_cast<long long>(row) * h + g * gs + i] = __float2bfloat16(o);
  }
}

// Per token: optional per-head RMSNorm of q and k, NeoX rotary on the first `rot` dims of q and k, q written to
// q_out [T, Hq, D], k and v rows written into the paged pools at slot[t] (bf16 or e4m3 with scale 1/kv_scale).
// qkv row layout: [Hq * D | Hkv * D | Hkv * D]. One CTA per token, one warp per head (looping).
__global__ void rope_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_qkv,
                                     const int* __restrict__ positions, const int* __restrict__ slots,
                                     const float* __restrict__ inv_freq, const __nv_bfloat16* __restrict__ q_norm_w,
                                     const __nv_bfloat16* __restrict__ k_norm_w, float eps, int gemma_norm,
                                     __nv_bfloat16* __restrict__ q_out, void* __restrict__ k_pool,
                                     void* __restrict__ v_pool, long long pool_stride, long long head_stride, int hq, int hkv,
                                     int d, int rot,
                                     int kv_fp8, float kv_inv_scale, int q_gate, uint8_t* __restrict__ k_sf,
                                     uint8_t* __restrict__ v_sf, long long sf_pool_stride, long long sf_head_stride,
                                     const float2* __restrict__ table) {
  grid_dep_wait();     // may run as a programmatic dependent of the QKV projection
  grid_dep_launch();
  const int t = blockIdx.x;
  const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int nw = gridDim.y * (blockDim.x >> 5);
  const float pos = static_cast<float>(positions[t]);
  int slot = slots ? slots[t] : -1;
  if (slot >= 0 && !index_ok(slot, kBoundKvSlots, kKerRopeKvWrite)) slot = -1;   // reported; nothing is written
  const int half = rot >> 1;
  // With q_gate the q block holds [q | gate] per head (2 * D per head); the gate half is left untouched.
  const int q_head_stride = q_gate ? 2 * d : d;
  const __nv_bfloat16* row = qkv + t * ld_qkv;
  for (int hd = warp; hd < hq + 2 * hkv; hd += nw) {
    const bool is_q = hd < hq, is_k = !is_q && hd < hq + hkv;
    const __nv_bfloat16* src = is_q ? row + hd * q_head_stride
                                    : row + hq * q_head_stride + (hd - hq) * d;
    float rstd = 1.f;
    const __nv_bfloat16* nw_ptr = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    if (nw_ptr != nullptr) {
      float ss = 0.f;
      for (int i = lane; i < d; i += 32) {
        const float v = __bfloat162float(src[i]);
        ss += v * v;
      }
      rstd = rsqrtf(warp_sum(ss) / d + eps);
    }
    __nv_bfloat16* dst_bf = nullptr;
    uint8_t* dst_f8 = nullptr;
    uint8_t* dst_f4 = nullptr;      // kv_fp8 == 2: packed e2m1 row (d / 2 bytes) + its d / 16 ue4m3 block scales
    uint8_t* dst_sf = nullptr;
    if (is_q) {
      dst_bf = q_out + (static_cast<long long>(t) * hq + hd) * d;
    } else {
      if (slot < 0) continue;
      const int kh = is_k ? hd - hq : hd - hq - hkv;
      void* pool = is_k ? k_pool : v_pool;
      const long long off = static_cast<long long>(slot) * pool_stride + static_cast<long long>(kh) * head_stride;
      if (kv_fp8 == 2) {
        dst_f4 = static_cast<uint8_t*>(pool) + off;       // strides of the packed pool are in bytes
        dst_sf = (is_k ? k_sf : v_sf) + static_cast<long long>(slot) * sf_pool_stride +
                 static_cast<long long>(kh) * sf_head_stride;
      } else if (kv_fp8) {
        dst_f8 = static_cast<uint8_t*>(pool) + off;
      } else {
        dst_bf = static_cast<__nv_bfloat16*>(pool) + off;
      }
    }
    for (int i = lane; i < d; i += 32) {
      float v = __bfloat162float(src[i]);
      if (nw_ptr != nullptr) {
        const float ww = __bfloat162float(nw_ptr[i]);
        v = __bfloat162float(__float2bfloat16(v * rstd * (gemma_norm ? 1.f + ww : ww)));
      }
      float o = v;
      if ((is_q || is_k) && i < rot) {
        const int j = i < half ? i : i - half;
        const int pi = i < half ? i + half : i - half;
        float pv = __bfloat162float(src[pi]);
        if (nw_ptr != nullptr) {
          const float ww = __bfloat162float(nw_ptr[pi]);
          pv = __bfloat162float(__float2bfloat16(pv * rstd * (gemma_norm ? 1.f + ww : ww)));
        }
        float sn, cs;
        if (table != nullptr) {     // (cos, sin) of this token's angles, computed once per forward for all layers
          const float2 csn = table[static_cast<long long>(t) * half + j];
          cs = csn.x;
          sn = csn.y;
        } else {
          sincosf(pos * inv_freq[j], &sn, &cs);
        }
        o = i < half ? v * cs - pv * sn : v * cs + pv * sn;
      }
      if (dst_f4) {
        // NVFP4 row: 16 consecutive elements (16 consecutive lanes) share a ue4m3 scale; x ~= code * scale / kv_inv_scale.
        // d is a multiple of 32 here, so every lane of the warp takes part in the shuffles.
        const float ob = __bfloat162float(__float2bfloat16(o));
        float amax = fabsf(ob);
#pragma unroll
        for (int sh = 1; sh < 16; sh <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sh));
        const uint32_t sfb = float_to_e4m3(amax * (1.f / 6.f) * kv_inv_scale);
        const float sf = e4m3_to_float(sfb);
        const float inv = sf > 0.f ? 1.f / (sf * (1.f / kv_inv_scale)) : 0.f;
        const float other = __shfl_xor_sync(0xffffffffu, ob, 1);
        if ((lane & 1) == 0) dst_f4[i >> 1] = static_cast<uint8_t>(e2m1x2(ob * inv, other * inv));
        if ((lane & 15) == 0) dst_sf[i >> 4] = static_cast<uint8_t>(sfb);
      } else if (dst_f8) dst_f8[i] = static_cast<uint8_t>(float_to_e4m3(o * kv_inv_scale));
      else dst_bf[i] = __float2bfloat16(o);
    }
  }
}

// out[t, j] = act(x[t, j]) * x[t, I + j] (mode 0: silu split), pairs interleaved (mode 1), relu^2 (mode 2, no mul),
// x * sigmoid(gate) with separate gate pointer (mode 3).
__global__ void act_mul_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                               __nv_bfloat16* __restrict__ out, long long rows, int inter, long long ldx, int mode) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * inter) return;
  const long long r = idx / inter;
  const int j = static_cast<int>(idx % inter);
  float o;
  if (mode == 0) {
    const float g = __bfloat162float(x[r * ldx + j]), u = __bfloat162float(x[r * ldx + inter + j]);
    o = g / (1.f + __expf(-g)) * u;
  } else if (mode == 1) {
    const float g = __bfloat162float(x[r * ldx + 2 * j]), u = __bfloat162float(x[r * ldx + 2 * j + 1]);
    o = g / (1.f + __expf(-g)) * u;
  } else if (mode == 2) {
    const float g = fmaxf(__bfloat162float(x[r * ldx + j]), 0.f);
    o = g * g;
  } else {
    const float v = __bfloat162float(x[r * ldx + j]), g = __bfloat162float(gate[r * ldx + j]);
    o = v / (1.f + __expf(-g));
  }
  out[r * inter + j] = __float2bfloat16(o);
}

// beta = sigmoid(b), g = -exp(a_log) * softplus(a + dt_bias) from the bf16 b | a projection [T, 2 * heads].
__global__ void gdn_gates_kernel(const __nv_bfloat16* __restrict__ ba, long long ld, const float* __restrict__ a_log,
                                 const float* __restrict__ dt_bias, int rows, int heads, float* __restrict__ beta,
                                 float* __restrict__ g) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * heads) return;
  const int r = i / heads, hd = i - r * heads;
  const float b = __bfloat162float(ba[r * ld + hd]);
  const float a = __bfloat162float(ba[r * ld + heads + hd]) + dt_bias[hd];
  beta[i] = 1.f / (1.f + __expf(-b));
  const float sp = a > 20.f ? a : log1pf(__expf(a));
  g[i] = -__expf(a_log[hd]) * sp;
}

__global__ void embedding_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int h, long long vocab) {
  const int t = blockIdx.x;
  long long id = ids[t];
  if (id < 0 || id >= vocab || !index_ok(id, kBoundVocab, kKerEmbedding)) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + id * h);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * h);
  for (int i = threadIdx.x; i < (h >> 3); i += blockDim.x) dst[i] = src[i];
}

__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, long long n) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
  if (i + 1 < n) {
    const uint32_t x = *reinterpret_cast<const uint32_t*>(a + i), y = *reinterpret_cast<const uint32_t*>(b + i);
    *reinterpret_cast<uint32_t*>(out + i) = pack_bf16(bf16_lo(x) + bf16_lo(y), bf16_hi(x) + bf16_hi(y));
  } else if (i < n) {
    out[i] = __float2bfloat16(__bfloat162float(a[i]) + __bfloat162float(b[i]));
  }
}

}  // namespace
}  // namespace hb

using namespace hb;
#define ST(s) static_cast<cudaStream_t>(s)
#define BF(p) static_cast<const __nv_bfloat16*>(p)
#define BFM(p) static_cast<__nv_bfloat16*>(p)
#define OK() (cudaGetLastError() == cudaSuccess ? 0 : 2)

extern "C" {

int hb_rmsnorm(const void* x, void* residual, const void* w, void* y, int rows, int h, long long ldx, long long ldy,
               float eps, int gemma, void* stream) {
  if (h % 8 != 0 || rows <= 0) return 1;
  const int nvec = h / 8;
  if (nvec <= 256) rmsnorm_kernel<1><<<rows, 256, 0, ST(stream)>>>(BF(x), BFM(residual), BF(w), BFM(y), h, ldx, ldy, eps, gemma);
  else if (nvec <= 512) rmsnorm_kernel<2><<<rows, 256, 0, ST(stream)>>>(BF(x), BFM(residual), BF(w), BFM(y), h, ldx, ldy, eps, gemma);
  else if (nvec <= 1024) rmsnorm_kernel<4><<<rows, 256, 0, ST(stream)>>>(BF(x), BFM(residual), BF(w), BFM(y), h, ldx, ldy, eps, gemma);
  else if (nvec <= 2048) rmsnorm_kernel<8><<<rows, 256, 0, ST(stream)>>>(BF(x), BFM(residual), BF(w), BFM(y), h, ldx, ldy, eps, gemma);
  else return 1;
  return OK();
}

int hb_gated_rmsnorm(const void* x, const void* z, const void* w, void* y, int rows, int h, int gs, long long ldx,
                     long long ldz, float eps, int norm_first, int sigmoid_gate, int gemma, void* stream) {
  if (h % gs != 0) return 1;
  const long long warps = static_cast<long long>(rows) * (h / gs);
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  gated_rmsnorm_kernel<<<blocks, 256, 0, ST(stream)>>>(BF(x), BF(z), BF(w), BFM(y), rows, h, gs, ldx, ldz, eps,
                                                       norm_first, sigmoid_gate, gemma, nullptr, nullptr, nullptr, 0);
  return OK();
}

int hb_gdn_gates(const void* ba, long long ld, const void* a_log, const void* dt_bias, int rows, int heads,
                 void* beta, void* g, void* stream) {
  if (rows <= 0) return 0;
  gdn_gates_kernel<<<(rows * heads + 255) / 256, 256, 0, ST(stream)>>>(
      BF(ba), ld, static_cast<const float*>(a_log), static_cast<const float*>(dt_bias), rows, heads,
      static_cast<float*>(beta), static_cast<float*>(g));
  return OK();
}

// Same norm, written as NVFP4 rows (packed codes [rows, h / 2] + swizzled block scales) for the projection that
// follows. Needs the register-resident path: group size a multiple of 16 and at most 1024, 16-byte aligned rows.
int hb_gated_rmsnorm_quant(const void* x, const void* z, const void* w, int rows, int h, int gs, long long ldx,
                           long long ldz, float eps, int norm_first, int sigmoid_gate, int gemma, void* q, void* sf,
                           const void* gscale, int ka, void* stream) {
  if (h % gs != 0 || gs % 16 != 0 || gs > 1024 || ldx % 8 != 0 || (z != nullptr && ldz % 8 != 0) || ka * 64 != h)
    return 1;   // (h a multiple of 64: no scale groups pad the last K tile)
  const long long warps = static_cast<long long>(rows) * (h / gs);
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  gated_rmsnorm_kernel<<<blocks, 256, 0, ST(stream)>>>(BF(x), BF(z), BF(w), nullptr, rows, h, gs, ldx, ldz, eps,
                                                       norm_first, sigmoid_gate, gemma, static_cast<uint8_t*>(q),
                                                       static_cast<uint8_t*>(sf), static_cast<const float*>(gscale), ka);
  return OK();
}

// Prefill-sized RoPE + KV write for the plain case (bf16 pools, full rotary, no q / k norm, angles from the table):
// a lane owns 8 consecutive features of a head (one 16-byte load, its rotation partners in a second one, the 8
// angles in four), a half-warp owns a head of up to 128 features, so the per-element cost is a few instructions
// instead of the generic kernel's scalar loop (which is instruction-bound: 55 us for 58 MB at 2048 tokens).
__global__ void __launch_bounds__(256) rope_kv_write_vec_kernel(
    const __nv_bfloat16* __restrict__ qkv, long long ld_qkv, const int* __restrict__ slots,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
    long long pool_stride, long long head_stride, int tokens, int hq, int hkv, int d, int q_gate,
    const float2* __restrict__ table) {
  grid_dep_wait();
  grid_dep_launch();
  const int lanes_per_head = d >> 3;                       // 8, 16 or 32
  const int heads_per_warp = 32 / lanes_per_head;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes_per_head, l = lane % lanes_per_head;
  const int heads = hq + 2 * hkv;
  const int groups = (heads + heads_per_warp - 1) / heads_per_warp;     // warp-sized units of work per token
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= static_cast<long long>(tokens) * groups) return;
  const int t = static_cast<int>(unit / groups);
  const int hd = static_cast<int>(unit % groups) * heads_per_warp + sub;
  if (hd >= heads) return;
  const bool is_q = hd < hq, is_k = !is_q && hd < hq + hkv;
  const int q_head_stride = q_gate ? 2 * d : d;
  const __nv_bfloat16* src = qkv + t * ld_qkv + (is_q ? hd * q_head_stride : hq * q_head_stride + (hd - hq) * d);
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (static_cast<long long>(t) * hq + hd) * d;
  } else {
    int slot = slots ? slots[t] : -1;
    if (slot >= 0 && !index_ok(slot, kBoundKvSlots, kKerRopeKvWrite)) slot = -1;
    if (slot < 0) return;
    const int kh = is_k ? hd - hq : hd - hq - hkv;
    dst = (is_k ? k_pool : v_pool) + static_cast<long long>(slot) * pool_stride + static_cast<long long>(kh) * head_stride;
  }
  const uint4 own = *reinterpret_cast<const uint4*>(src + 8 * l);
  if (!is_q && !is_k) {                                    // values: a copy
    *reinterpret_cast<uint4*>(dst + 8 * l) = own;
    return;
  }
  const int half = d >> 1, half_lanes = lanes_per_head >> 1;
  const bool low = l < half_lanes;
  const uint4 other = *reinterpret_cast<const uint4*>(src + 8 * (low ? l + half_lanes : l - half_lanes));
  const float4* tb = reinterpret_cast<const float4*>(table + static_cast<long long>(t) * half + 8 * (low ? l : l - half_lanes));
  const uint32_t ow[4] = {own.x, own.y, own.z, own.w}, pw[4] = {other.x, other.y, other.z, other.w};
  uint32_t out[4];
#pragma unroll
  for (int e2 = 0; e2 < 4; ++e2) {
    const float4 cs2 = tb[e2];                             // (cos, sin) of features 2 e2 and 2 e2 + 1
    const float v0 = bf16_lo(ow[e2]), v1 = bf16_hi(ow[e2]), p0 = bf16_lo(pw[e2]), p1 = bf16_hi(pw[e2]);
    const float o0 = low ? v0 * cs2.x - p0 * cs2.y : v0 * cs2.x + p0 * cs2.y;
    const float o1 = low ? v1 * cs2.z - p1 * cs2.w : v1 * cs2.z + p1 * cs2.w;
    out[e2] = pack_bf16(o0, o1);
  }
  *reinterpret_cast<uint4*>(dst + 8 * l) = make_uint4(out[0], out[1], out[2], out[3]);
}

// Scale pools of an NVFP4 KV cache for the NEXT hb_rope_kv_write call of this thread (kv_fp8 = 2): ue4m3 scale rows
// [slots, kv heads, d / 16] of K and V with their strides in bytes. Consumed by that call.
struct KvSf {
  uint8_t* k = nullptr;
  uint8_t* v = nullptr;
  long long pool_stride = 0, head_stride = 0;
};
static thread_local KvSf g_kv_sf;
// (cos, sin) table [tokens, rot / 2] for the NEXT hb_rope_kv_write call of this thread (null = compute in the kernel).
static thread_local const float2* g_rope_table = nullptr;
void hb_rope_use_table(const void* table) { g_rope_table = static_cast<const float2*>(table); }

__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int tokens,
                                  int half, float2* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(tokens) * half) return;
  const int t = static_cast<int>(i / half), j = static_cast<int>(i % half);
  float sn, cs;
  sincosf(static_cast<float>(positions[t]) * inv_freq[j], &sn, &cs);      // the same call the kernel makes without a table
  out[i] = make_float2(cs, sn);
}

// out[t][j] = (cos, sin)(positions[t] * inv_freq[j]), j < half: one table per forward serves every layer's RoPE.
int hb_rope_table(const void* positions, const void* inv_freq, int tokens, int half, void* out, void* stream) {
  if (tokens <= 0 || half <= 0) return 0;
  const long long n = static_cast<long long>(tokens) * half;
  rope_table_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ST(stream)>>>(
      static_cast<const int*>(positions), static_cast<const float*>(inv_freq), tokens, half, static_cast<float2*>(out));
  return OK();
}

void hb_kv_fp4_scales(void* k_sf, void* v_sf, long long pool_stride, long long head_stride) {
  g_kv_sf.k = static_cast<uint8_t*>(k_sf); g_kv_sf.v = static_cast<uint8_t*>(v_sf);
  g_kv_sf.pool_stride = pool_stride; g_kv_sf.head_stride = head_stride;
}

int hb_rope_kv_write(const void* qkv, long long ld_qkv, const void* positions, const void* slots,
                     const void* inv_freq, const void* q_norm_w, const void* k_norm_w, float eps, int gemma_norm,
                     void* q_out, void* k_pool, void* v_pool, long long pool_stride, long long head_stride, int tokens,
                     int hq, int hkv,
                     int d, int rot, int kv_fp8, float kv_inv_scale, int q_gate, void* stream) {
  if (tokens <= 0) return 0;
  if (rot > d || (rot & 1)) return 1;
  if (kv_fp8 == 2 && (d % 32 != 0 || g_kv_sf.k == nullptr || g_kv_sf.v == nullptr)) return 1;
  if (g_rope_table != nullptr && q_norm_w == nullptr && k_norm_w == nullptr && kv_fp8 == 0 && rot == d &&
      (d == 64 || d == 128 || d == 256) && ld_qkv % 8 == 0 && k_pool != nullptr && v_pool != nullptr &&
      pool_stride % 8 == 0 && head_stride % 8 == 0) {
    const int per_warp = 32 / (d >> 3);
    const long long units = static_cast<long long>(tokens) * ((hq + 2 * hkv + per_warp - 1) / per_warp);
    const float2* table = g_rope_table;
    g_rope_table = nullptr;
    g_kv_sf = KvSf{};
    launch_dep(rope_kv_write_vec_kernel, dim3(static_cast<unsigned>((units + 7) / 8)), dim3(256), 0, ST(stream),
               BF(qkv), ld_qkv, static_cast<const int*>(slots), BFM(q_out), static_cast<__nv_bfloat16*>(k_pool),
               static_cast<__nv_bfloat16*>(v_pool), pool_stride, head_stride, tokens, hq, hkv, d, q_gate, table);
    return OK();
  }
  // One warp per head: a warp that walks several heads in turn is a chain of load latencies (measured 62 us for
  // 2048 tokens of the 27B geometry, 58 MB of traffic), so the heads of a token are spread over CTAs at every size.
  const int heads = hq + 2 * hkv;
  const int ysplit = (heads + 7) / 8;
  launch_dep(rope_kv_write_kernel, dim3(tokens, ysplit), dim3(256), 0, ST(stream),
      BF(qkv), ld_qkv, static_cast<const int*>(positions), static_cast<const int*>(slots),
      static_cast<const float*>(inv_freq), BF(q_norm_w), BF(k_norm_w), eps, gemma_norm, BFM(q_out), k_pool, v_pool,
      pool_stride, head_stride, hq, hkv, d, rot, kv_fp8, kv_inv_scale, q_gate, g_kv_sf.k, g_kv_sf.v,
      g_kv_sf.pool_stride, g_kv_sf.head_stride, g_rope_table);
  g_kv_sf = KvSf{};
  g_rope_table = nullptr;
  return OK();
}

int hb_act_mul(const void* x, const void* gate, void* out, long long rows, int inter, long long ldx, int mode,
               void* stream) {
  const long long n = rows * inter;
  if (n <= 0) return 0;
  act_mul_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ST(stream)>>>(BF(x), BF(gate), BFM(out), rows,
                                                                                inter, ldx, mode);
  return OK();
}

int hb_embedding(const void* ids, const void* table, void* out, int tokens, int h, long long vocab, void* stream) {
  if (tokens <= 0) return 0;
  if (h % 8 != 0) return 1;
  embedding_kernel<<<tokens, 128, 0, ST(stream)>>>(static_cast<const long long*>(ids), BF(table), BFM(out), h, vocab);
  return OK();
}

int hb_add(const void* a, const void* b, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  const long long threads = (n + 1) / 2;
  add_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, ST(stream)>>>(BF(a), BF(b), BFM(out), n);
  return OK();
}

}  // extern "C"
