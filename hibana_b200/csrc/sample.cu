// Sampling and speculative verify-and-accept kernels for sm_100a.
//
//  * argmax over bf16 / fp32 logits rows (greedy), optional grammar bitmask.
//  * temperature / top-k / top-p sampling, one CTA per row, counter-based RNG keyed by (seed, offset) so a
//    request's draws do not depend on batch composition.
//  * exact greedy acceptance of a drafted block (longest matching prefix + the target's own token), with stop
//    ids and a token budget, producing device-resident counts.
//  * rank / logit gap of a drafted token in its verify row (relaxed acceptance).
//
// Reference counterparts: hibana/engine/sampler.py:87-123, hibana/engine/accept.py:18-56,
// hibana/kernels/relaxed_rank.py:13, hibana/kernels/sampled_verify.py:17, hibana/engine/accept_graphs.py.
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

__device__ __forceinline__ bool mask_ok(const int* mask, int i) {
  return mask == nullptr || ((mask[i >> 5] >> (i & 31)) & 1);
}

// Lowest index wins ties (same as torch.argmax on CPU for exact ties).
template <typename T>
__global__ void __launch_bounds__(256)
argmax_kernel(const T* __restrict__ logits, long long ld, int vocab, const int* __restrict__ bitmask, int mask_words,
              long long* __restrict__ out, float* __restrict__ out_val) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int row = blockIdx.x;
  const T* lr = logits + row * ld;
  const int* mask = bitmask ? bitmask + static_cast<long long>(row) * mask_words : nullptr;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    if (!mask_ok(mask, i)) continue;
    const float v = ldf<T>(lr, i);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
        best = sv[w];
        bi = si[w];
      }
    out[row] = bi == 0x7fffffff ? 0 : bi;
    if (out_val) out_val[row] = best;
  }
}

// Two-stage argmax for wide vocabularies: `nch` CTAs per row each scan a slice, then one warp per row combines.
template <typename T>
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const T* __restrict__ logits, long long ld, int vocab, const int* __restrict__ bitmask,
                      int mask_words, int nch, float* __restrict__ pv, int* __restrict__ pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int row = blockIdx.x, ch = blockIdx.y;
  const T* lr = logits + row * ld;
  const int* mask = bitmask ? bitmask + static_cast<long long>(row) * mask_words : nullptr;
  const int per = (vocab + nch - 1) / nch;
  const int lo = ch * per, hi = min(vocab, lo + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    if (!mask_ok(mask, i)) continue;
    const float v = ldf<T>(lr, i);
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
        best = sv[w];
        bi = si[w];
      }
    pv[row * nch + ch] = best;
    pi[row * nch + ch] = bi;
  }
}

// One warp per row. Rows whose temperature is > 0 are left to the sampling kernel.
__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int nch, int rows,
                                    const float* __restrict__ temperature, long long* __restrict__ out,
                                    float* __restrict__ out_val) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  if (temperature != nullptr && temperature[row] > 0.f) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < nch; c += 32) {
    const float v = pv[row * nch + c];
    const int i = pi[row * nch + c];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (lane == 0) {
    out[row] = bi == 0x7fffffff ? 0 : bi;
    if (out_val) out_val[row] = best;
  }
}

// splitmix64-based counter RNG -> uniform in [0, 1).
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long offset) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (offset + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

// ---- full-vocabulary sampling (top-k off or above SAMPLE_K): softmax over every allowed token, nucleus by an exact
// threshold search, inverse-CDF draw in index order. Same law as engine/rejection.py `distribution`.
__device__ __forceinline__ unsigned order_key(float v) {   // order-preserving map float -> uint32
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ float block_sum256(float v, float* red) {   // 256 threads, deterministic
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w];
  return t;
}

__device__ __forceinline__ int block_sum256i(int v, int* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  int t = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w];
  return t;
}

// The sampling law of one row as engine/rejection.py `distribution` defines it: softmax(logits / temp) over the
// allowed tokens, cut to the first `k_lim` tokens in (value desc, index asc) order (0 = no cut), then to the
// smallest prefix of that order whose mass reaches p_lim. Draws one token by inverse CDF in index order from the
// law with token `exclude` removed (-1: nothing removed; the residual of a point-mass draft in speculative
// sampling) and reports the probability of token `probe` under the law. 256 threads, whole CTA.
template <typename T>
__device__ void law_row(const T* __restrict__ lr, int vocab, const int* __restrict__ mask, float temp, int k_lim,
                        float p_lim, float u01, int exclude, int probe, long long* out, float* out_prob,
                        float* out_probe) {
  __shared__ float red[8];
  __shared__ int redi[8];
  __shared__ float csum[256];
  __shared__ int ceq[256];
  __shared__ int s_pick_thread;
  __shared__ float s_base;
  __shared__ int s_eq_base;
  const int tid = threadIdx.x;
  const float inv_t = 1.f / temp;
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += 256)
    if (mask_ok(mask, i)) mx = fmaxf(mx, ldf<T>(lr, i));
  mx = warp_max(mx);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  // ---- top-k cut: tk_key = value of the k-th token, need_k = how many of the tokens equal to it are inside
  unsigned tk_key = 0;     // finite values have keys above 0x007fffff: 0 keeps everything
  int need_k = 0x7fffffff;
  const bool cut_k = k_lim > 0 && k_lim < vocab;
  if (cut_k) {
    unsigned lo = 0, hi = order_key(mx);
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo + 1) >> 1);
      int cnt = 0;
      for (int i = tid; i < vocab; i += 256)
        if (mask_ok(mask, i)) {
          const float v = ldf<T>(lr, i);
          cnt += v > -INFINITY && order_key(v) >= mid;
        }
      cnt = block_sum256i(cnt, redi);
      if (cnt >= k_lim) lo = mid;
      else hi = mid - 1;
    }
    tk_key = lo;
    int above = 0;
    for (int i = tid; i < vocab; i += 256)
      if (mask_ok(mask, i)) {
        const float v = ldf<T>(lr, i);
        above += v > -INFINITY && order_key(v) > tk_key;
      }
    need_k = k_lim - block_sum256i(above, redi);
  }
  // mass above a key and number of tokens equal to it
  float m_above = 0.f;
  int n_eq = 0;
  for (int i = tid; i < vocab; i += 256)
    if (mask_ok(mask, i)) {
      const float v = ldf<T>(lr, i);
      if (v > -INFINITY) {
        const unsigned k = order_key(v);
        if (k > tk_key) m_above += __expf((v - mx) * inv_t);
        else n_eq += k == tk_key;
      }
    }
  m_above = block_sum256(m_above, red);
  n_eq = block_sum256i(n_eq, redi);
  unsigned t_key = tk_key;
  int need_eq = min(need_k, n_eq);
  float w_t = cut_k ? __expf((key_value(tk_key) - mx) * inv_t) : 0.f;
  float kept = m_above + (cut_k ? need_eq * w_t : 0.f);
  // ---- nucleus inside the cut: the smallest prefix, in the same order, whose mass reaches p_lim * kept
  if (p_lim < 1.f) {
    const float want = p_lim * kept;
    unsigned lo = tk_key, hi = order_key(mx);      // mass(key >= lo) = kept >= want
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo + 1) >> 1);     // mid > tk_key: every token at or above it is inside the cut
      float mass = 0.f;
      for (int i = tid; i < vocab; i += 256)
        if (mask_ok(mask, i)) {
          const float v = ldf<T>(lr, i);
          if (v > -INFINITY && order_key(v) >= mid) mass += __expf((v - mx) * inv_t);
        }
      mass = block_sum256(mass, red);
      if (mass >= want) lo = mid;
      else hi = mid - 1;
    }
    if (lo != tk_key || !cut_k) {
      t_key = lo;
      float above = 0.f;
      int eq = 0;
      for (int i = tid; i < vocab; i += 256)
        if (mask_ok(mask, i)) {
          const float v = ldf<T>(lr, i);
          if (v > -INFINITY) {
            const unsigned k = order_key(v);
            if (k > t_key) above += __expf((v - mx) * inv_t);
            else eq += k == t_key;
          }
        }
      m_above = block_sum256(above, red);
      n_eq = block_sum256i(eq, redi);
      w_t = __expf((key_value(t_key) - mx) * inv_t);
      need_eq = n_eq;
    }
    int need = w_t > 0.f ? static_cast<int>(ceilf((want - m_above) / w_t)) : 1;
    need_eq = max(1, min(need, need_eq));
    kept = m_above + need_eq * w_t;
  }
  // ---- membership and weight of the probed / excluded token (its rank among equals decides at the threshold)
  float w_probe = 0.f, w_ex = 0.f;
  for (int pass = 0; pass < 2; ++pass) {
    const int tok = pass == 0 ? probe : exclude;
    if (tok < 0 || tok >= vocab || !mask_ok(mask, tok)) continue;
    if (pass == 1 && exclude == probe) {
      w_ex = w_probe;
      continue;
    }
    const float v = ldf<T>(lr, tok);
    float w = 0.f;
    if (v > -INFINITY) {
      const unsigned k = order_key(v);
      if (k > t_key) w = __expf((v - mx) * inv_t);
      else if (k == t_key) {
        int before = 0;
        for (int i = tid; i < tok; i += 256)
          if (mask_ok(mask, i)) {
            const float o = ldf<T>(lr, i);
            before += o > -INFINITY && order_key(o) == t_key;
          }
        before = block_sum256i(before, redi);
        if (before < need_eq) w = w_t;
      }
    }
    if (pass == 0) w_probe = w;
    else w_ex = w;
  }
  if (out_probe != nullptr && tid == 0) *out_probe = w_probe / kept;
  if (!(kept - w_ex > kept * 1e-6f)) {      // nothing left beside the excluded token: the law itself is drawn from
    exclude = -1;
    w_ex = 0.f;
  }
  const float kept_draw = kept - w_ex;
  // ---- draw: contiguous chunk per thread, chunk sums scanned by thread 0, the owning thread walks its chunk
  const int per = (vocab + 255) / 256;
  const int lo_i = tid * per, hi_i = min(vocab, lo_i + per);
  float mine = 0.f;
  int my_eq = 0;
  for (int i = lo_i; i < hi_i; ++i)
    if (mask_ok(mask, i)) {
      const float v = ldf<T>(lr, i);
      if (v > -INFINITY) {
        const unsigned k = order_key(v);
        if (k > t_key) mine += __expf((v - mx) * inv_t);
        else if (k == t_key) ++my_eq;
      }
    }
  csum[tid] = mine;
  ceq[tid] = my_eq;
  __syncthreads();
  const float u = u01 * kept_draw;
  const int ex_thread = exclude >= 0 ? exclude / per : -1;
  if (tid == 0) {
    float acc = 0.f;
    int eq_seen = 0, pick = -1, last = 0;
    float base = 0.f;
    int eq_base = 0;
    for (int t = 0; t < 256; ++t) {
      const int take = max(0, min(ceq[t], need_eq - eq_seen));
      float w = csum[t] + take * w_t;
      if (t == ex_thread) w = fmaxf(w - w_ex, 0.f);
      if (w > 0.f) last = t;
      if (pick < 0 && u < acc + w) {
        pick = t;
        base = acc;
        eq_base = eq_seen;
      }
      acc += w;
      eq_seen += ceq[t];
    }
    if (pick < 0) {   // rounding: u landed past the last kept token
      pick = last;
      base = -1.f;
    }
    s_pick_thread = pick;
    s_base = base;
    s_eq_base = eq_base;
  }
  __syncthreads();
  if (tid == s_pick_thread) {
    float acc = s_base;
    int eq_seen = s_eq_base, chosen = -1, last_kept = -1;
    float w_chosen = 0.f, w_last = 0.f;
    for (int i = lo_i; i < hi_i; ++i) {
      if (!mask_ok(mask, i)) continue;
      const float v = ldf<T>(lr, i);
      if (!(v > -INFINITY)) continue;
      const unsigned k = order_key(v);
      float w = 0.f;
      if (k > t_key) w = __expf((v - mx) * inv_t);
      else if (k == t_key) {
        if (eq_seen < need_eq) w = w_t;
        ++eq_seen;
      }
      if (i == exclude) w = 0.f;
      if (w <= 0.f) continue;
      last_kept = i;
      w_last = w;
      if (s_base >= 0.f && u < acc + w) {
        chosen = i;
        w_chosen = w;
        break;
      }
      acc += w;
    }
    if (chosen < 0) {
      chosen = last_kept < 0 ? 0 : last_kept;
      w_chosen = w_last;
    }
    *out = chosen;
    if (out_prob) *out_prob = w_chosen / kept_draw;
  }
  __syncthreads();
}

template <typename T>
__device__ void sample_full_row(const T* __restrict__ lr, int vocab, const int* __restrict__ mask, float temp,
                                int k_lim, float p_lim, float u01, long long* out, float* out_prob) {
  law_row<T>(lr, vocab, mask, temp, k_lim, p_lim, u01, -1, -1, out, out_prob, nullptr);
}

constexpr int SAMPLE_K = 64;  // candidates kept per row for 1 <= top-k <= 64 (top-p is applied inside them)

// One CTA per row. Keeps the SAMPLE_K largest logits by repeated threshold passes (vocab is read a few times from
// L2), then softmax / top-p / inverse-CDF draw on the candidates. temperature <= 0 means greedy.
template <typename T>
__global__ void __launch_bounds__(256)
sample_kernel(const T* __restrict__ logits, long long ld, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ offsets,
              const int* __restrict__ bitmask, int mask_words, long long* __restrict__ out,
              float* __restrict__ out_prob, int skip_greedy) {
  __shared__ float cv[SAMPLE_K];
  __shared__ int ci[SAMPLE_K];
  __shared__ float wv[8];
  __shared__ int wi[8];
  __shared__ float s_prev_v;
  __shared__ int s_prev_i;
  const int row = blockIdx.x;
  const T* lr = logits + row * ld;
  const int* mask = bitmask ? bitmask + static_cast<long long>(row) * mask_words : nullptr;
  const float temp = temperature ? temperature[row] : 0.f;
  if (skip_greedy && temp <= 0.f) return;   // the two-stage argmax owns greedy rows
  int k = top_k ? top_k[row] : 0;
  if (temp > 0.f && (k <= 0 || k > SAMPLE_K)) {
    // top-k off (the API default) or wider than the candidate list: the law is the softmax over the whole
    // vocabulary (then top-p), not over the SAMPLE_K largest logits
    sample_full_row<T>(lr, vocab, mask, temp, k > SAMPLE_K ? k : 0, top_p ? top_p[row] : 1.f,
                       uniform01(seeds ? seeds[row] : 0ull, offsets ? offsets[row] : 0ull), out + row,
                       out_prob ? out_prob + row : nullptr);
    return;
  }
  if (temp <= 0.f) k = 1;
  if (threadIdx.x == 0) {
    s_prev_v = INFINITY;
    s_prev_i = -1;
  }
  __syncthreads();
  // Selection by successive maxima in (value desc, index asc) order: exact and deterministic.
  for (int c = 0; c < k; ++c) {
    const float pv = s_prev_v;
    const int pi = s_prev_i;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      if (!mask_ok(mask, i)) continue;
      const float v = ldf<T>(lr, i);
      const bool after_prev = v < pv || (v == pv && i > pi);
      if (after_prev && (v > best || (v == best && i < bi))) {
        best = v;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if ((threadIdx.x & 31) == 0) {
      wv[threadIdx.x >> 5] = best;
      wi[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < 8; ++w)
        if (wv[w] > best || (wv[w] == best && wi[w] < bi)) {
          best = wv[w];
          bi = wi[w];
        }
      cv[c] = best;
      ci[c] = bi == 0x7fffffff ? 0 : bi;
      s_prev_v = best;
      s_prev_i = bi;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    if (k == 1) {
      out[row] = ci[0];
      if (out_prob) out_prob[row] = 1.f;
      return;
    }
    const float inv_t = 1.f / temp;
    const float m = cv[0];
    float sum = 0.f;
    for (int c = 0; c < k; ++c) {
      cv[c] = (cv[c] == -INFINITY) ? 0.f : __expf((cv[c] - m) * inv_t);
      sum += cv[c];
    }
    const float p_lim = top_p ? top_p[row] : 1.f;
    int keep = k;
    if (p_lim < 1.f) {
      float acc = 0.f;
      for (int c = 0; c < k; ++c) {
        acc += cv[c] / sum;
        if (acc >= p_lim) {
          keep = c + 1;
          break;
        }
      }
    }
    float ksum = 0.f;
    for (int c = 0; c < keep; ++c) ksum += cv[c];
    const float u = uniform01(seeds ? seeds[row] : 0ull, offsets ? offsets[row] : 0ull) * ksum;
    float acc = 0.f;
    int pick = keep - 1;
    for (int c = 0; c < keep; ++c) {
      acc += cv[c];
      if (u < acc) {
        pick = c;
        break;
      }
    }
    out[row] = ci[pick];
    if (out_prob) out_prob[row] = cv[pick] / ksum;
  }
}

// Walk of a block drafter's candidate lattice, one warp per request, lane = candidate (width <= 32). Step j scores
// candidate w as scores[b][j][previous choice][w]; the greedy walk takes the best (lowest index on ties), the
// sampled walk draws from softmax(row / T) by inverse CDF with the caller's uniform. Writes the chosen tokens and
// candidate indices, the probability of every candidate at every step (the draft law on its support, what
// speculative sampling divides by) and the unit-temperature probability of the chosen one (acceptance estimate).
__global__ void lattice_walk_kernel(const long long* __restrict__ cand, const float* __restrict__ scores,
                                    const float* __restrict__ temperature, const float* __restrict__ uniforms,
                                    int batch, int k, int width, long long* __restrict__ tokens,
                                    int* __restrict__ chosen, float* __restrict__ probs, float* __restrict__ estimate) {
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (b >= batch) return;
  const float temp = temperature ? temperature[b] : 0.f;
  const bool sampled = temp > 0.f && uniforms != nullptr;
  int prev = 0;
  for (int j = 0; j < k; ++j) {
    const long long base = (static_cast<long long>(b) * k + j) * width;
    const float x = lane < width ? scores[(base + prev) * width + lane] : -INFINITY;
    const float mx = warp_max(x);
    const float e1 = lane < width ? __expf(x - mx) : 0.f;              // unit temperature: the estimate
    const float z1 = warp_sum(e1);
    float p = e1 / z1;
    int pick;
    if (sampled) {
      const float et = lane < width ? __expf((x - mx) / temp) : 0.f;
      p = et / warp_sum(et);
      float cdf = p;                                                   // inclusive scan over the lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, cdf, o);
        if (lane >= o) cdf += up;
      }
      const unsigned below = __ballot_sync(0xffffffffu, lane < width && cdf < uniforms[static_cast<long long>(b) * k + j]);
      pick = min(__popc(below), width - 1);
    } else {
      const unsigned best = __ballot_sync(0xffffffffu, lane < width && x == mx);
      pick = __ffs(best) - 1;
    }
    if (probs != nullptr && lane < width) probs[base + lane] = p;
    const float p1 = __shfl_sync(0xffffffffu, e1 / z1, pick);
    if (lane == 0) {
      tokens[static_cast<long long>(b) * k + j] = cand[base + pick];
      chosen[static_cast<long long>(b) * k + j] = pick;
      if (estimate != nullptr) estimate[static_cast<long long>(b) * k + j] = p1;
    }
    prev = pick;
  }
}

// Speculative rejection sampling against point-mass drafts, one CTA per verified row. Request b owns logits rows
// [b * (k + 1), (b + 1) * (k + 1)); row j < k sees draft d = drafts[b][j]: with p the row's law (law_row) the draft
// stands when u * 1 < p[d] (or, for a relaxed request, u < e^soft * p[d]); otherwise the row's token is a draw from
// max(p - onehot(d), 0) renormalised. Row k draws the bonus token from p. The kernel writes, per row, the token the
// target "says" there: d where the draft stands, the draw where it does not; the exact-prefix accept kernel below
// then yields the emitted tokens, so sampled and greedy rounds share one accept path (greedy requests, temp <= 0,
// fall out of the same rule: their law is the one-hot argmax). Uniforms are counter draws at (seed, 2 * (draws + j)
// + 1) for the test and + 2 for the draw.
template <typename T>
__global__ void __launch_bounds__(256)
spec_targets_kernel(const T* __restrict__ logits, long long ld, int vocab, int k, const long long* __restrict__ drafts,
                    const float* __restrict__ temperature, const int* __restrict__ top_k,
                    const float* __restrict__ top_p, const unsigned long long* __restrict__ seeds,
                    const unsigned long long* __restrict__ draws, const float* __restrict__ soft,
                    const int* __restrict__ bitmask, int mask_words, const long long* __restrict__ greedy_pick,
                    long long* __restrict__ target, float* __restrict__ p_draft) {
  __shared__ long long s_tok;
  __shared__ float s_probe;
  const int row = blockIdx.x, b = row / (k + 1), j = row - b * (k + 1);
  const T* lr = logits + row * ld;
  const int* mask = bitmask ? bitmask + static_cast<long long>(row) * mask_words : nullptr;
  float temp = temperature ? temperature[b] : 0.f;
  int k_lim = top_k ? top_k[b] : 0;
  float p_lim = top_p ? top_p[b] : 1.f;
  if (temp <= 0.f && greedy_pick != nullptr) {      // the caller already has this row's argmax
    if (threadIdx.x == 0) {
      target[row] = greedy_pick[row];
      if (p_draft) p_draft[row] = j < k && greedy_pick[row] == drafts[static_cast<long long>(b) * k + j] ? 1.f : 0.f;
    }
    return;
  }
  if (temp <= 0.f) {
    temp = 1.f;
    k_lim = 1;
    p_lim = 1.f;
  }
  const unsigned long long seed = seeds ? seeds[b] : 0ull, base = draws ? draws[b] : 0ull;
  const int d = j < k ? static_cast<int>(drafts[static_cast<long long>(b) * k + j]) : -1;
  law_row<T>(lr, vocab, mask, temp, k_lim, p_lim, uniform01(seed, 2 * (base + j) + 2), d, d, &s_tok, nullptr,
             &s_probe);
  if (threadIdx.x == 0) {
    long long tok = s_tok;
    if (j < k) {
      const float u = uniform01(seed, 2 * (base + j) + 1), pd = s_probe;
      const float sf = soft ? soft[b] : 0.f;
      if (u < pd || (sf > 0.f && u < __expf(sf) * pd)) tok = d;
      if (p_draft) p_draft[row] = pd;
    } else if (p_draft) {
      p_draft[row] = 1.f;
    }
    target[row] = tok;
  }
}

// Exact greedy acceptance. Row layout: request b owns rows [b*(k+1), (b+1)*(k+1)); row j holds the target's
// argmax after consuming [pending, draft_1..draft_j]. Accept drafts while draft[j] == target[j-1]; emit the
// accepted drafts plus the target token of the first mismatch (or the bonus token). Emission stops at a stop id
// (inclusive) or when `budget[b]` tokens are out. Writes emitted[b, 0..count) and count[b].
__global__ void accept_greedy_kernel(const long long* __restrict__ target, const long long* __restrict__ drafts,
                                     const long long* __restrict__ stop_ids, int n_stop,
                                     const int* __restrict__ budget, const int* __restrict__ depth, int k_max, int batch,
                                     long long* __restrict__ emitted, int* __restrict__ count,
                                     int* __restrict__ accepted) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int k = depth ? min(depth[b], k_max) : k_max;
  const long long* t = target + static_cast<long long>(b) * (k_max + 1);
  const long long* d = drafts + static_cast<long long>(b) * k_max;
  long long* e = emitted + static_cast<long long>(b) * (k_max + 1);
  const int lim = budget ? budget[b] : k + 1;
  int n = 0, acc = 0;
  bool stopped = false;
  for (int j = 0; j <= k && n < lim && !stopped; ++j) {
    const long long tok = t[j];
    e[n++] = tok;
    for (int s = 0; s < n_stop; ++s)
      if (stop_ids[static_cast<long long>(b) * n_stop + s] == tok) stopped = true;
    if (j < k && d[j] == tok) ++acc;
    else break;
  }
  count[b] = n;
  if (accepted) accepted[b] = acc;
}

// Rank (number of strictly larger logits) and gap to the row maximum of token ids[row].
template <typename T>
__global__ void __launch_bounds__(256)
rank_gap_kernel(const T* __restrict__ logits, long long ld, int vocab, const long long* __restrict__ ids,
                int* __restrict__ rank, float* __restrict__ gap) {
  __shared__ float smax[8];
  __shared__ int scnt[8];
  const int row = blockIdx.x;
  const T* lr = logits + row * ld;
  const float mine = ldf<T>(lr, ids[row]);
  float mx = -INFINITY;
  int cnt = 0;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = ldf<T>(lr, i);
    mx = fmaxf(mx, v);
    cnt += v > mine;
  }
  mx = warp_max(mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) {
    smax[threadIdx.x >> 5] = mx;
    scnt[threadIdx.x >> 5] = cnt;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) {
      mx = fmaxf(mx, smax[w]);
      cnt += scnt[w];
    }
    rank[row] = cnt;
    gap[row] = mx - mine;
  }
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

int hb_argmax(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* bitmask, int mask_words,
              void* out, void* out_val, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_f32)
    argmax_kernel<float><<<rows, 256, 0, st>>>(static_cast<const float*>(logits), ld, vocab,
                                               static_cast<const int*>(bitmask), mask_words,
                                               static_cast<long long*>(out), static_cast<float*>(out_val));
  else
    argmax_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, vocab,
                                                       static_cast<const int*>(bitmask), mask_words,
                                                       static_cast<long long*>(out), static_cast<float*>(out_val));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_sample(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* temperature,
              const void* top_k, const void* top_p, const void* seeds, const void* offsets, const void* bitmask,
              int mask_words, void* out, void* out_prob, int skip_greedy, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define HB_SAMPLE_ARGS                                                                                     \
  ld, vocab, static_cast<const float*>(temperature), static_cast<const int*>(top_k),                       \
      static_cast<const float*>(top_p), static_cast<const unsigned long long*>(seeds),                     \
      static_cast<const unsigned long long*>(offsets), static_cast<const int*>(bitmask), mask_words,       \
      static_cast<long long*>(out), static_cast<float*>(out_prob), skip_greedy
  if (is_f32) sample_kernel<float><<<rows, 256, 0, st>>>(static_cast<const float*>(logits), HB_SAMPLE_ARGS);
  else sample_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), HB_SAMPLE_ARGS);
#undef HB_SAMPLE_ARGS
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_lattice_walk(const void* cand, const void* scores, const void* temperature, const void* uniforms, int batch,
                    int k, int width, void* tokens, void* chosen, void* probs, void* estimate, void* stream) {
  if (batch <= 0 || k <= 0) return 0;
  if (width < 1 || width > 32) return 1;
  lattice_walk_kernel<<<(batch + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(cand), static_cast<const float*>(scores), static_cast<const float*>(temperature),
      static_cast<const float*>(uniforms), batch, k, width, static_cast<long long*>(tokens),
      static_cast<int*>(chosen), static_cast<float*>(probs), static_cast<float*>(estimate));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_spec_targets(const void* logits, long long ld, int batch, int k, int vocab, int is_f32, const void* drafts,
                    const void* temperature, const void* top_k, const void* top_p, const void* seeds,
                    const void* draws, const void* soft, const void* bitmask, int mask_words,
                    const void* greedy_pick, void* target, void* p_draft, void* stream) {
  if (batch <= 0) return 0;
  if (k < 0 || vocab <= 0) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rows = batch * (k + 1);
#define HB_SPEC_ARGS                                                                                          \
  ld, vocab, k, static_cast<const long long*>(drafts), static_cast<const float*>(temperature),                \
      static_cast<const int*>(top_k), static_cast<const float*>(top_p),                                       \
      static_cast<const unsigned long long*>(seeds), static_cast<const unsigned long long*>(draws),           \
      static_cast<const float*>(soft), static_cast<const int*>(bitmask), mask_words,                          \
      static_cast<const long long*>(greedy_pick), static_cast<long long*>(target), static_cast<float*>(p_draft)
  if (is_f32) spec_targets_kernel<float><<<rows, 256, 0, st>>>(static_cast<const float*>(logits), HB_SPEC_ARGS);
  else
    spec_targets_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), HB_SPEC_ARGS);
#undef HB_SPEC_ARGS
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_accept_greedy(const void* target, const void* drafts, const void* stop_ids, int n_stop, const void* budget,
                     const void* depth, int k_max, int batch, void* emitted, void* count, void* accepted,
                     void* stream) {
  if (batch <= 0) return 0;
  accept_greedy_kernel<<<(batch + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(target), static_cast<const long long*>(drafts),
      static_cast<const long long*>(stop_ids), n_stop, static_cast<const int*>(budget),
      static_cast<const int*>(depth), k_max, batch, static_cast<long long*>(emitted), static_cast<int*>(count),
      static_cast<int*>(accepted));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_rank_gap(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* ids, void* rank,
                void* gap, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_f32)
    rank_gap_kernel<float><<<rows, 256, 0, st>>>(static_cast<const float*>(logits), ld, vocab,
                                                 static_cast<const long long*>(ids), static_cast<int*>(rank),
                                                 static_cast<float*>(gap));
  else
    rank_gap_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, vocab,
                                                         static_cast<const long long*>(ids),
                                                         static_cast<int*>(rank), static_cast<float*>(gap));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Two-stage greedy argmax. scratch_v / scratch_i hold rows * nch partials. With `temperature` given, rows whose
// temperature is > 0 are skipped (their token comes from hb_sample with skip_greedy).
int hb_argmax2(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* bitmask, int mask_words,
               int nch, void* scratch_v, void* scratch_i, const void* temperature, void* out, void* out_val,
               void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(rows, nch);
  if (is_f32)
    argmax_partial_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(logits), ld, vocab,
                                                       static_cast<const int*>(bitmask), mask_words, nch,
                                                       static_cast<float*>(scratch_v), static_cast<int*>(scratch_i));
  else
    argmax_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, vocab, static_cast<const int*>(bitmask), mask_words, nch,
        static_cast<float*>(scratch_v), static_cast<int*>(scratch_i));
  argmax_final_kernel<<<(rows + 3) / 4, 128, 0, st>>>(static_cast<const float*>(scratch_v),
                                                      static_cast<const int*>(scratch_i), nch, rows,
                                                      static_cast<const float*>(temperature),
                                                      static_cast<long long*>(out), static_cast<float*>(out_val));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
