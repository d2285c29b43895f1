// Recurrent-layer kernels for sm_100a: depthwise causal conv1d, Mamba-2 selective state scan, gated delta rule.
//
// One code path serves chunked prefill (many tokens per sequence, state carried in from / out to a pool slot),
// decode (one token) and speculative verify (k + 1 tokens written to a scratch slot, then the accepted prefix is
// replayed from the untouched committed state with the same kernel, so verify and commit are bitwise equal).
// Sequences are ragged: rows [q_indptr[b], q_indptr[b+1]) belong to sequence b (null = one row each); state lives
// in `*_pool[slot]` with separate read and write slots.
//
//   conv1d : y[t, c] = act(bias[c] + sum_j w[c, j] * x[t - (W-1) + j, c]); window state = last W-1 raw rows.
//   mamba2 : S = exp(dt A) S + dt x B^T ; y = S C + D x   (per head, state [P, N] fp32, dt = softplus(dt + bias))
//   gdn    : S = exp(g) S ; u = S k ; v' = beta (v - u) ; S += v' k^T ; o = S q   (per value head, state [V, K])
//
// Reference counterparts: hibana/kernels/mamba2.py:226-470 and :854-1139 (Triton conv / SSU / SSD chunk scan),
// hibana/kernels/fla/* and hibana/kernels/csrc/gdn_verify.cu:172-330 (gated delta rule prefill / verify / commit).
#include <cuda_fp16.h>

#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// One thread per (sequence, channel): walks the sequence's tokens keeping the W-1 previous raw inputs.
template <int W>
__global__ void conv1d_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, long long ldy,
                              __nv_bfloat16* __restrict__ state, long long state_stride,
                              const int* __restrict__ q_indptr, const int* __restrict__ slot_in,
                              const int* __restrict__ slot_out, const int* __restrict__ has_init, int channels,
                              int act_silu) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  if (!index_ok(slot_in[b], kBoundStateSlots, kKerConvState) ||
      (slot_out != nullptr && !index_ok(slot_out[b], kBoundStateSlots, kKerConvState)))
    return;   // reported; the sequence is skipped
  const int r0 = q_indptr ? q_indptr[b] : b;
  const int r1 = q_indptr ? q_indptr[b + 1] : b + 1;
  float win[W - 1];
  const bool init = has_init == nullptr || has_init[b] != 0;
  const __nv_bfloat16* sin = state + static_cast<long long>(slot_in[b]) * state_stride + static_cast<long long>(c) * (W - 1);
#pragma unroll
  for (int j = 0; j < W - 1; ++j) win[j] = init ? __bfloat162float(sin[j]) : 0.f;
  float wt[W];
#pragma unroll
  for (int j = 0; j < W; ++j) wt[j] = __bfloat162float(w[static_cast<long long>(c) * W + j]);
  const float bs = bias ? __bfloat162float(bias[c]) : 0.f;
  for (int t = r0; t < r1; ++t) {
    const float xv = __bfloat162float(x[t * ldx + c]);
    float acc = bs + wt[W - 1] * xv;
#pragma unroll
    for (int j = 0; j < W - 1; ++j) acc += wt[j] * win[j];
#pragma unroll
    for (int j = 0; j < W - 2; ++j) win[j] = win[j + 1];
    win[W - 2] = xv;
    y[t * ldy + c] = __float2bfloat16(act_silu ? silu_f(acc) : acc);
  }
  if (slot_out != nullptr) {
    __nv_bfloat16* so = state + static_cast<long long>(slot_out[b]) * state_stride + static_cast<long long>(c) * (W - 1);
#pragma unroll
    for (int j = 0; j < W - 1; ++j) so[j] = __float2bfloat16(win[j]);
  }
}

// Prefill form: one thread per (sequence, channel, tile of CONV_TT tokens), so a long chunk is not walked serially.
// The window of a tile's first token comes from the rows before it (or the stored state at the sequence start);
// the new state is written by conv1d_state_kernel afterwards.
constexpr int CONV_TT = 32;
template <int W>
__global__ void conv1d_tiled_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                    const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                                    __nv_bfloat16* __restrict__ y, long long ldy, __nv_bfloat16* __restrict__ state,
                                    long long state_stride, const int* __restrict__ q_indptr,
                                    const int* __restrict__ slot_in, const int* __restrict__ slot_out,
                                    const int* __restrict__ has_init, int channels, int act_silu) {
  const int b = blockIdx.z;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  if (!index_ok(slot_in[b], kBoundStateSlots, kKerConvState) ||
      (slot_out != nullptr && !index_ok(slot_out[b], kBoundStateSlots, kKerConvState)))
    return;   // reported; the sequence is skipped
  const int r0 = q_indptr ? q_indptr[b] : b;
  const int r1 = q_indptr ? q_indptr[b + 1] : b + 1;
  const int t0 = r0 + blockIdx.y * CONV_TT;
  if (t0 >= r1) return;
  const int t1 = min(t0 + CONV_TT, r1);
  const bool init = has_init == nullptr || has_init[b] != 0;
  const __nv_bfloat16* sin = state + static_cast<long long>(slot_in[b]) * state_stride + static_cast<long long>(c) * (W - 1);
  float win[W - 1];
#pragma unroll
  for (int j = 0; j < W - 1; ++j) {
    const int t = t0 - (W - 1) + j;        // row of the j-th window entry; rows before r0 live in the state
    if (t >= r0) win[j] = __bfloat162float(x[t * ldx + c]);
    else win[j] = init ? __bfloat162float(sin[j + (t0 - r0)]) : 0.f;   // state holds rows r0-(W-1) .. r0-1
  }
  float wt[W];
#pragma unroll
  for (int j = 0; j < W; ++j) wt[j] = __bfloat162float(w[static_cast<long long>(c) * W + j]);
  const float bs = bias ? __bfloat162float(bias[c]) : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float xv = __bfloat162float(x[t * ldx + c]);
    float acc = bs + wt[W - 1] * xv;
#pragma unroll
    for (int j = 0; j < W - 1; ++j) acc += wt[j] * win[j];
#pragma unroll
    for (int j = 0; j < W - 2; ++j) win[j] = win[j + 1];
    win[W - 2] = xv;
    y[t * ldy + c] = __float2bfloat16(act_silu ? silu_f(acc) : acc);
  }
}

// New window of every sequence after a tiled pass: the last W - 1 raw inputs (rows before the sequence start come
// from the old state). One thread per (sequence, channel) reads everything it needs before it writes, so the input
// and output slots may be the same.
template <int W>
__global__ void conv1d_state_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                    __nv_bfloat16* __restrict__ state, long long state_stride,
                                    const int* __restrict__ q_indptr, const int* __restrict__ slot_in,
                                    const int* __restrict__ slot_out, const int* __restrict__ has_init,
                                    int channels) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  if (!index_ok(slot_in[b], kBoundStateSlots, kKerConvState) ||
      (slot_out != nullptr && !index_ok(slot_out[b], kBoundStateSlots, kKerConvState)))
    return;   // reported; the sequence is skipped
  const int r0 = q_indptr ? q_indptr[b] : b;
  const int r1 = q_indptr ? q_indptr[b + 1] : b + 1;
  const bool init = has_init == nullptr || has_init[b] != 0;
  const __nv_bfloat16* sin = state + static_cast<long long>(slot_in[b]) * state_stride + static_cast<long long>(c) * (W - 1);
  __nv_bfloat16 win[W - 1];
#pragma unroll
  for (int j = 0; j < W - 1; ++j) {
    const int t = r1 - (W - 1) + j;
    if (t >= r0) win[j] = x[t * ldx + c];
    else win[j] = init ? sin[j + (r1 - r0)] : __float2bfloat16(0.f);
  }
  __nv_bfloat16* so = state + static_cast<long long>(slot_out[b]) * state_stride + static_cast<long long>(c) * (W - 1);
#pragma unroll
  for (int j = 0; j < W - 1; ++j) so[j] = win[j];
}

struct MambaParams {
  const __nv_bfloat16* x;    // [T, heads * P]   (row pitch ldx)
  const __nv_bfloat16* bmat; // [T, groups * N]  (row pitch ldb)
  const __nv_bfloat16* cmat; // [T, groups * N]
  const __nv_bfloat16* dt;   // [T, heads]       (row pitch lddt)
  long long ldx, ldb, lddt;
  const float* a_log;        // [heads]  A = -exp(a_log)
  const float* dt_bias;      // [heads]
  const float* dskip;        // [heads]
  __nv_bfloat16* y;          // [T, heads * P]
  long long ldy;
  float* state;              // [slots, heads, P, N] (fp32; __half or int8 with the quantised formats)
  float* state_scale;        // int8 format: [slots, heads, P] row scales (stride = state_stride / N)
  unsigned sr_seed;          // fp16 format: 0 = round to nearest, else seed of the stochastic rounding
  long long state_stride;
  const int* q_indptr;
  const int* slot_in;
  const int* slot_out;
  const int* has_init;
  int heads, groups;
};

// One CTA per (sequence, head). Thread layout: P rows x (THREADS / P) column groups; each thread keeps
// N / (THREADS / P) state columns of one row in registers for the whole sequence. The columns of a thread are
// groups of four interleaved with the other threads of its row (group j of column group cg is columns
// 4 * (j * CG + cg) ...), so that the CG threads of a row move 16 * CG contiguous bytes per instruction and every
// sector a warp touches is used whole: a decode step is nothing but this state traffic.
// State formats: 0 fp32; 1 fp16 (optionally stochastically rounded on store, so that rounding errors do not
// accumulate as a bias over thousands of steps); 2 int8 with one fp32 scale per state row (absmax / 127).
// The recurrence itself always runs in fp32 registers; only the pool representation changes.
__device__ __forceinline__ unsigned mix32(unsigned x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

template <int P, int N, int THREADS, int FMT>
__global__ void __launch_bounds__(THREADS) mamba2_scan_kernel(const MambaParams p) {
  constexpr int CG = THREADS / P;          // column groups
  constexpr int NC = N / CG;               // state columns per thread
  static_assert(THREADS % P == 0 && N % CG == 0 && CG <= 32 && (CG & (CG - 1)) == 0 && NC % 4 == 0, "bad Mamba tiling");
  auto col = [&](int i, int cg_) { return ((i >> 2) * CG + cg_) * 4 + (i & 3); };   // state column of register i
  __shared__ float bs[N], cs[N];
  const int b = blockIdx.y, h = blockIdx.x;
  if (!index_ok(p.slot_in[b], kBoundStateSlots, kKerMambaScan) ||
      (p.slot_out != nullptr && !index_ok(p.slot_out[b], kBoundStateSlots, kKerMambaScan)))
    return;   // reported; uniform over the CTA, before any barrier
  const int g = h / (p.heads / p.groups);
  const int row = threadIdx.x / CG, cg = threadIdx.x % CG;
  const int r0 = p.q_indptr ? p.q_indptr[b] : b;
  const int r1 = p.q_indptr ? p.q_indptr[b + 1] : b + 1;
  float s[NC];
  const bool init = p.has_init == nullptr || p.has_init[b] != 0;
  {
    const long long off = static_cast<long long>(p.slot_in[b]) * p.state_stride +
                          (static_cast<long long>(h) * P + row) * N;
    if constexpr (FMT == 0) {
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) {
        const float4 v = init ? *reinterpret_cast<const float4*>(p.state + off + col(4 * j, cg)) : make_float4(0, 0, 0, 0);
        s[4 * j] = v.x; s[4 * j + 1] = v.y; s[4 * j + 2] = v.z; s[4 * j + 3] = v.w;
      }
    } else if constexpr (FMT == 1) {
      const __half* sin = reinterpret_cast<const __half*>(p.state) + off;
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) {
        const uint2 raw = init ? *reinterpret_cast<const uint2*>(sin + col(4 * j, cg)) : make_uint2(0, 0);
        const __half2 lo = *reinterpret_cast<const __half2*>(&raw.x), hi = *reinterpret_cast<const __half2*>(&raw.y);
        s[4 * j] = __low2float(lo); s[4 * j + 1] = __high2float(lo);
        s[4 * j + 2] = __low2float(hi); s[4 * j + 3] = __high2float(hi);
      }
    } else {
      const int8_t* sin = reinterpret_cast<const int8_t*>(p.state) + off;
      const float sc = p.state_scale[static_cast<long long>(p.slot_in[b]) * (p.state_stride / N) +
                                     static_cast<long long>(h) * P + row];
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) {
        const char4 raw = init ? *reinterpret_cast<const char4*>(sin + col(4 * j, cg)) : make_char4(0, 0, 0, 0);
        s[4 * j] = raw.x * sc; s[4 * j + 1] = raw.y * sc; s[4 * j + 2] = raw.z * sc; s[4 * j + 3] = raw.w * sc;
      }
    }
  }
  const float a = -__expf(p.a_log[h]);
  const float dtb = p.dt_bias ? p.dt_bias[h] : 0.f;
  const float dsk = p.dskip ? p.dskip[h] : 0.f;
  for (int t = r0; t < r1; ++t) {
    __syncthreads();
    for (int i = threadIdx.x; i < N; i += THREADS) {
      bs[i] = __bfloat162float(p.bmat[t * p.ldb + g * N + i]);
      cs[i] = __bfloat162float(p.cmat[t * p.ldb + g * N + i]);
    }
    __syncthreads();
    const float dt = softplus_f(__bfloat162float(p.dt[t * p.lddt + h]) + dtb);
    const float decay = __expf(dt * a);
    const float xv = __bfloat162float(p.x[t * p.ldx + h * P + row]);
    const float dx = dt * xv;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      s[i] = s[i] * decay + dx * bs[col(i, cg)];
      acc += s[i] * cs[col(i, cg)];
    }
#pragma unroll
    for (int o = CG / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (cg == 0) p.y[t * p.ldy + h * P + row] = __float2bfloat16(acc + dsk * xv);
  }
  if (p.slot_out != nullptr) {
    const long long off = static_cast<long long>(p.slot_out[b]) * p.state_stride +
                          (static_cast<long long>(h) * P + row) * N;
    if constexpr (FMT == 0) {
#pragma unroll
      for (int j = 0; j < NC / 4; ++j)
        *reinterpret_cast<float4*>(p.state + off + col(4 * j, cg)) =
            make_float4(s[4 * j], s[4 * j + 1], s[4 * j + 2], s[4 * j + 3]);
    } else if constexpr (FMT == 1) {
      __half* so = reinterpret_cast<__half*>(p.state) + off;
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) {
        __half r4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = 4 * j + e;
          if (p.sr_seed == 0) {
            r4[e] = __float2half_rn(s[i]);
          } else {
            // stochastic rounding: up with probability (x - lo) / (hi - lo)
            const __half lo = __float2half_rd(s[i]), hi = __float2half_ru(s[i]);
            const float fl = __half2float(lo), fh = __half2float(hi);
            const unsigned r = mix32(p.sr_seed ^ mix32(static_cast<unsigned>(off + col(i, cg)) * 2654435761u + r1));
            const float u = (r >> 8) * (1.f / 16777216.f);
            r4[e] = (fh > fl && (s[i] - fl) > u * (fh - fl)) ? hi : lo;
          }
        }
        *reinterpret_cast<uint2*>(so + col(4 * j, cg)) = *reinterpret_cast<const uint2*>(r4);
      }
    } else {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < NC; ++i) amax = fmaxf(amax, fabsf(s[i]));
#pragma unroll
      for (int o = CG / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float sc = amax > 0.f ? amax / 127.f : 1.f;
      const float inv = 1.f / sc;
      int8_t* so = reinterpret_cast<int8_t*>(p.state) + off;
#pragma unroll
      for (int j = 0; j < NC / 4; ++j) {
        char4 r4;
        r4.x = static_cast<signed char>(__float2int_rn(fminf(fmaxf(s[4 * j] * inv, -127.f), 127.f)));
        r4.y = static_cast<signed char>(__float2int_rn(fminf(fmaxf(s[4 * j + 1] * inv, -127.f), 127.f)));
        r4.z = static_cast<signed char>(__float2int_rn(fminf(fmaxf(s[4 * j + 2] * inv, -127.f), 127.f)));
        r4.w = static_cast<signed char>(__float2int_rn(fminf(fmaxf(s[4 * j + 3] * inv, -127.f), 127.f)));
        *reinterpret_cast<char4*>(so + col(4 * j, cg)) = r4;
      }
      if (cg == 0)
        p.state_scale[static_cast<long long>(p.slot_out[b]) * (p.state_stride / N) + static_cast<long long>(h) * P + row] = sc;
    }
  }
}

struct GdnParams {
  const __nv_bfloat16* q;     // [T, k_heads * K]  (pitch ldq), already l2-normalised when requested by the caller
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;     // [T, v_heads * V]  (pitch ldv)
  const float* g;             // [T, v_heads] log decay (<= 0)
  const float* beta;          // [T, v_heads]
  long long ldq, ldv;
  __nv_bfloat16* o;           // [T, v_heads * V]
  long long ldo;
  float* state;               // [slots, v_heads, V, K]
  long long state_stride;
  const int* q_indptr;
  const int* slot_in;
  const int* slot_out;
  const int* has_init;
  int k_heads, v_heads;
  float scale;                // applied to q
  int l2norm;                 // normalise q and k rows in the kernel
};

// One CTA per (sequence, value head), V threads: thread v holds state row S[v, 0..K) in registers.
template <int V, int K>
__global__ void __launch_bounds__(V) gdn_scan_kernel(const GdnParams p) {
  // The head's [V, K] fp32 state travels through shared memory (rows padded by four floats): global traffic is
  // then whole rows per warp instruction in both directions, and thread v picks up / drops its own row from the
  // padded tile without bank conflicts. Reading rows straight from global, 512 bytes apart per lane, used half of
  // every sector and made a decode step take twice its state traffic.
  extern __shared__ __align__(16) float gdn_tile[];
  constexpr int TS = K + 4;
  __shared__ float qs[K], ks[K];
  __shared__ float red[2][V / 32];
  const int b = blockIdx.y, hv = blockIdx.x;
  if (!index_ok(p.slot_in[b], kBoundStateSlots, kKerGdnScan) ||
      (p.slot_out != nullptr && !index_ok(p.slot_out[b], kBoundStateSlots, kKerGdnScan)))
    return;   // reported; uniform over the CTA, before any barrier
  const int hk = hv / (p.v_heads / p.k_heads);
  const int v = threadIdx.x;
  const int r0 = p.q_indptr ? p.q_indptr[b] : b;
  const int r1 = p.q_indptr ? p.q_indptr[b + 1] : b + 1;
  float s[K];
  const bool init = p.has_init == nullptr || p.has_init[b] != 0;
  if (init) {
    const float* sin = p.state + static_cast<long long>(p.slot_in[b]) * p.state_stride +
                       static_cast<long long>(hv) * V * K;
    for (int idx = v; idx < V * K / 4; idx += V) {
      const int row = idx / (K / 4), c4 = idx % (K / 4);
      const unsigned dst = smem_u32(gdn_tile + row * TS + c4 * 4);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(sin + static_cast<long long>(idx) * 4)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < K; i += 4) {
    const float4 t = init ? *reinterpret_cast<const float4*>(gdn_tile + v * TS + i) : make_float4(0, 0, 0, 0);
    s[i] = t.x; s[i + 1] = t.y; s[i + 2] = t.z; s[i + 3] = t.w;
  }
  for (int t = r0; t < r1; ++t) {
    __syncthreads();
    float qv = 0.f, kv = 0.f;
    if (v < K) {
      qv = __bfloat162float(p.q[t * p.ldq + hk * K + v]);
      kv = __bfloat162float(p.k[t * p.ldq + hk * K + v]);
    }
    if (p.l2norm) {
      float q2 = warp_sum(qv * qv), k2 = warp_sum(kv * kv);
      if ((v & 31) == 0) {
        red[0][v >> 5] = q2;
        red[1][v >> 5] = k2;
      }
      __syncthreads();
      q2 = 0.f;
      k2 = 0.f;
#pragma unroll
      for (int w = 0; w < V / 32; ++w) {
        q2 += red[0][w];
        k2 += red[1][w];
      }
      qv *= rsqrtf(q2 + 1e-6f);
      kv *= rsqrtf(k2 + 1e-6f);
    }
    if (v < K) {
      qs[v] = qv * p.scale;
      ks[v] = kv;
    }
    __syncthreads();
    const float decay = __expf(p.g[static_cast<long long>(t) * p.v_heads + hv]);
    const float bt = p.beta[static_cast<long long>(t) * p.v_heads + hv];
    const float vv = __bfloat162float(p.v[t * p.ldv + hv * V + v]);
    float u = 0.f;
#pragma unroll
    for (int i = 0; i < K; ++i) {
      s[i] *= decay;
      u += s[i] * ks[i];
    }
    const float dv = bt * (vv - u);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < K; ++i) {
      s[i] += dv * ks[i];
      o += s[i] * qs[i];
    }
    p.o[t * p.ldo + hv * V + v] = __float2bfloat16(o);
  }
  if (p.slot_out != nullptr) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < K; i += 4)
      *reinterpret_cast<float4*>(gdn_tile + v * TS + i) = make_float4(s[i], s[i + 1], s[i + 2], s[i + 3]);
    __syncthreads();
    float* so = p.state + static_cast<long long>(p.slot_out[b]) * p.state_stride + static_cast<long long>(hv) * V * K;
    for (int idx = v; idx < V * K / 4; idx += V) {
      const int row = idx / (K / 4), c4 = idx % (K / 4);
      *reinterpret_cast<float4*>(so + static_cast<long long>(idx) * 4) =
          *reinterpret_cast<const float4*>(gdn_tile + row * TS + c4 * 4);
    }
  }
}

}  // namespace
}  // namespace hb

using namespace hb;
#define ST(s) static_cast<cudaStream_t>(s)
#define BF(p) static_cast<const __nv_bfloat16*>(p)
#define BFM(p) static_cast<__nv_bfloat16*>(p)
#define IP(p) static_cast<const int*>(p)
#define FP(p) static_cast<const float*>(p)

template <int FMT>
static int launch_mamba(const MambaParams& p, dim3 grid, int head_dim, int d_state, cudaStream_t st) {
  if (head_dim == 32 && d_state == 64) mamba2_scan_kernel<32, 64, 128, FMT><<<grid, 128, 0, st>>>(p);
  else if (head_dim == 64 && d_state == 128) mamba2_scan_kernel<64, 128, 256, FMT><<<grid, 256, 0, st>>>(p);
  else if (head_dim == 64 && d_state == 64) mamba2_scan_kernel<64, 64, 256, FMT><<<grid, 256, 0, st>>>(p);
  else if (head_dim == 32 && d_state == 16) mamba2_scan_kernel<32, 16, 128, FMT><<<grid, 128, 0, st>>>(p);
  else return 1;
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

extern "C" {

int hb_conv1d(const void* x, long long ldx, const void* w, const void* bias, void* y, long long ldy, void* state,
              long long state_stride, const void* q_indptr, const void* slot_in, const void* slot_out,
              const void* has_init, int batch, int channels, int width, int act_silu, int max_rows, void* stream) {
  if (batch <= 0) return 0;
  if (width != 4) return 1;
  if (max_rows > CONV_TT) {   // prefill: parallel over tiles of tokens, then the new windows
    const dim3 tg((channels + 127) / 128, (max_rows + CONV_TT - 1) / CONV_TT, batch);
    conv1d_tiled_kernel<4><<<tg, 128, 0, ST(stream)>>>(BF(x), ldx, BF(w), BF(bias), BFM(y), ldy, BFM(state),
                                                       state_stride, IP(q_indptr), IP(slot_in), IP(slot_out),
                                                       IP(has_init), channels, act_silu);
    if (slot_out != nullptr)
      conv1d_state_kernel<4><<<dim3((channels + 127) / 128, batch), 128, 0, ST(stream)>>>(
          BF(x), ldx, BFM(state), state_stride, IP(q_indptr), IP(slot_in), IP(slot_out), IP(has_init), channels);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  const dim3 grid((channels + 127) / 128, batch);
  conv1d_kernel<4><<<grid, 128, 0, ST(stream)>>>(BF(x), ldx, BF(w), BF(bias), BFM(y), ldy, BFM(state), state_stride,
                                                 IP(q_indptr), IP(slot_in), IP(slot_out), IP(has_init), channels,
                                                 act_silu);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// state_fmt: 0 fp32, 1 fp16 (sr_seed != 0: stochastic rounding on store), 2 int8 + state_scale [slots, heads, P].
int hb_mamba2_scan_fmt(const void* x, const void* bmat, const void* cmat, const void* dt, long long ldx,
                       long long ldb, long long lddt, const void* a_log, const void* dt_bias, const void* dskip,
                       void* y, long long ldy, void* state, long long state_stride, const void* q_indptr,
                       const void* slot_in, const void* slot_out, const void* has_init, int batch, int heads,
                       int groups, int head_dim, int d_state, int state_fmt, void* state_scale, unsigned sr_seed,
                       void* stream) {
  if (batch <= 0) return 0;
  if (state_fmt < 0 || state_fmt > 2 || (state_fmt == 2 && state_scale == nullptr)) return 1;
  MambaParams p;
  p.x = BF(x); p.bmat = BF(bmat); p.cmat = BF(cmat); p.dt = BF(dt);
  p.ldx = ldx; p.ldb = ldb; p.lddt = lddt;
  p.a_log = FP(a_log); p.dt_bias = FP(dt_bias); p.dskip = FP(dskip);
  p.y = BFM(y); p.ldy = ldy;
  p.state = static_cast<float*>(state); p.state_stride = state_stride;
  p.state_scale = static_cast<float*>(state_scale); p.sr_seed = sr_seed;
  p.q_indptr = IP(q_indptr); p.slot_in = IP(slot_in); p.slot_out = IP(slot_out); p.has_init = IP(has_init);
  p.heads = heads; p.groups = groups;
  const dim3 grid(heads, batch);
  if (state_fmt == 0) return launch_mamba<0>(p, grid, head_dim, d_state, ST(stream));
  if (state_fmt == 1) return launch_mamba<1>(p, grid, head_dim, d_state, ST(stream));
  return launch_mamba<2>(p, grid, head_dim, d_state, ST(stream));
}

int hb_mamba2_scan(const void* x, const void* bmat, const void* cmat, const void* dt, long long ldx, long long ldb,
                   long long lddt, const void* a_log, const void* dt_bias, const void* dskip, void* y, long long ldy,
                   void* state, long long state_stride, const void* q_indptr, const void* slot_in,
                   const void* slot_out, const void* has_init, int batch, int heads, int groups, int head_dim,
                   int d_state, void* stream) {
  return hb_mamba2_scan_fmt(x, bmat, cmat, dt, ldx, ldb, lddt, a_log, dt_bias, dskip, y, ldy, state, state_stride,
                            q_indptr, slot_in, slot_out, has_init, batch, heads, groups, head_dim, d_state, 0, nullptr,
                            0, stream);
}

int hb_gdn_scan(const void* q, const void* k, const void* v, const void* g, const void* beta, long long ldq,
                long long ldv, void* o, long long ldo, void* state, long long state_stride, const void* q_indptr,
                const void* slot_in, const void* slot_out, const void* has_init, int batch, int k_heads,
                int v_heads, int kdim, int vdim, float scale, int l2norm, void* stream) {
  if (batch <= 0) return 0;
  GdnParams p;
  p.q = BF(q); p.k = BF(k); p.v = BF(v); p.g = FP(g); p.beta = FP(beta);
  p.ldq = ldq; p.ldv = ldv; p.o = BFM(o); p.ldo = ldo;
  p.state = static_cast<float*>(state); p.state_stride = state_stride;
  p.q_indptr = IP(q_indptr); p.slot_in = IP(slot_in); p.slot_out = IP(slot_out); p.has_init = IP(has_init);
  p.k_heads = k_heads; p.v_heads = v_heads; p.scale = scale; p.l2norm = l2norm;
  const dim3 grid(v_heads, batch);
  if (kdim == 128 && vdim == 128) {
    constexpr int SMEM = 128 * (128 + 4) * 4;     // above the 48 KB default: opt in once
    static bool armed = false;
    if (!armed) {
      if (cudaFuncSetAttribute(gdn_scan_kernel<128, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) !=
          cudaSuccess)
        return 3;
      armed = true;
    }
    gdn_scan_kernel<128, 128><<<grid, 128, SMEM, ST(stream)>>>(p);
  } else if (kdim == 64 && vdim == 64) {
    gdn_scan_kernel<64, 64><<<grid, 64, 64 * 68 * 4, ST(stream)>>>(p);
  } else if (kdim == 32 && vdim == 32) {
    gdn_scan_kernel<32, 32><<<grid, 32, 32 * 36 * 4, ST(stream)>>>(p);
  } else {
    return 1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
