// Mixture-of-experts routing, planning, row gather and combine for sm_100a.
//
//   route   : per token, softmax (or sigmoid + selection bias) over E router logits, top-k, renormalise, scale.
//   plan    : counts per expert, 128-row-aligned segment starts, and a deterministic position of every
//             (token, k) pair inside its expert's segment (pairs keep token order, so sums are reproducible).
//   gather  : bf16 rows of the sorted activation buffer (padding rows zero) for bf16 experts; NVFP4 experts
//             quantise through the row-indirect mode of the activation quantiser instead.
//   combine : out[t] = sum_k w[t, k] * y[pos[t, k]] (+ shared expert output) in selection order.
//
// The grouped GEMMs between plan and combine are the grouped mode of csrc/gemm.cu. Reference counterparts:
// hibana/kernels/flashnext_fused.py:279-620 (route_topk, moe_combine*), hibana/model/nemotron/moe.py:76-306,
// hibana/kernels/csrc/w3_gemm.cu:711-1289 (prep / combine), hibana/kernels/csrc/nemotron_moe.cu:496-618.
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int MAX_TOPK = 32;

// One warp per token; E <= 32 * PER. Selection order is (value desc, index asc): every candidate is one 64-bit key
// (order-preserving bits of the value above the complemented index), a lane keeps the best of its PER keys, and
// each of the top-k rounds is two warp-wide `redux.max` instructions plus a rescan by the one lane that owned the
// winner, instead of a shuffle tree over (value, index) pairs.
__device__ __forceinline__ unsigned route_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Decode-sized routing: one CTA per token, one thread per expert. The k-th largest key is found by a 32-step bit
// search on block-wide counts (`__syncthreads_count`), ties at the threshold go to the lower expert index, and the
// at most 32 selected experts rank themselves against each other, so the ids come out in the same order as the
// round-by-round extraction of `moe_route_kernel` (descending score, lower index first) in ~2 us instead of one
// dependent round per selected expert in a single warp.
__global__ void __launch_bounds__(1024) moe_route_block_kernel(
    const float* __restrict__ logits, long long ld, const float* __restrict__ sel_bias, int experts, int topk,
    int sigmoid, int renorm, float scale, int* __restrict__ ids, float* __restrict__ weights) {
  __shared__ float s_red[32];
  __shared__ int s_warp_tie[32], s_warp_sel[32];
  __shared__ unsigned s_key[MAX_TOPK];
  __shared__ int s_id[MAX_TOPK];
  __shared__ float s_sc[MAX_TOPK], s_sorted[MAX_TOPK];
  const int t = blockIdx.x, e = threadIdx.x, lane = e & 31, warp = e >> 5, nwarps = blockDim.x >> 5;
  const bool live = e < experts;
  const float x = live ? logits[t * ld + e] : -INFINITY;
  float score;
  unsigned key;
  if (sigmoid) {
    score = live ? 1.f / (1.f + __expf(-x)) : 0.f;
    key = live ? route_key(score + (sel_bias ? sel_bias[e] : 0.f)) : 0u;
  } else {
    float m = warp_max(x);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = lane < nwarps ? s_red[lane] : -INFINITY;
    m = warp_max(m);
    __syncthreads();
    const float ex = live ? __expf(x - m) : 0.f;
    float sum = warp_sum(ex);
    if (lane == 0) s_red[warp] = sum;
    __syncthreads();
    sum = lane < nwarps ? s_red[lane] : 0.f;
    sum = warp_sum(sum);
    score = ex * (1.f / sum);
    key = live ? route_key(score) : 0u;
  }
  unsigned thr = 0u;                       // the largest value with at least topk keys at or above it
  for (int b = 31; b >= 0; --b) {
    const unsigned cand = thr | (1u << b);
    if (__syncthreads_count(key >= cand) >= topk) thr = cand;
  }
  const int above = __syncthreads_count(key > thr);
  const bool tie = key == thr && thr != 0u;
  // exclusive prefix counts over the expert index: of the ties (who gets the remaining places) and, below, of the
  // selected (their slot in the shared list)
  const unsigned tie_mask = __ballot_sync(0xffffffffu, tie);
  if (lane == 0) s_warp_tie[warp] = __popc(tie_mask);
  __syncthreads();
  int tie_rank = __popc(tie_mask & ((1u << lane) - 1u));
  for (int w = 0; w < warp; ++w) tie_rank += s_warp_tie[w];
  const bool sel = key > thr || (tie && tie_rank < topk - above);
  const unsigned sel_mask = __ballot_sync(0xffffffffu, sel);
  if (lane == 0) s_warp_sel[warp] = __popc(sel_mask);
  __syncthreads();
  int slot = __popc(sel_mask & ((1u << lane) - 1u));
  for (int w = 0; w < warp; ++w) slot += s_warp_sel[w];
  if (sel && slot < MAX_TOPK) {
    s_key[slot] = key;
    s_id[slot] = e;
    s_sc[slot] = score;
  }
  __syncthreads();
  if (e < topk) {                           // thread j places list entry j: its rank among the selected
    const unsigned kj = s_key[e];
    const int ij = s_id[e];
    int rank = 0;
    for (int i = 0; i < topk; ++i) rank += (s_key[i] > kj || (s_key[i] == kj && s_id[i] < ij)) ? 1 : 0;
    s_sorted[rank] = s_sc[e];
    ids[static_cast<long long>(t) * topk + rank] = ij;
  }
  __syncthreads();
  if (e < topk) {
    float wsum = 0.f;
    for (int i = 0; i < topk; ++i) wsum += s_sorted[i];       // in rank order, like the round-by-round kernel
    const float w = (renorm ? s_sorted[e] / fmaxf(wsum, 1e-20f) : s_sorted[e]) * scale;
    weights[static_cast<long long>(t) * topk + e] = w;
  }
}

template <int PER>
__global__ void moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ sel_bias,
                                 int tokens, int experts, int topk, int sigmoid, int renorm, float scale,
                                 int* __restrict__ ids, float* __restrict__ weights) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  float score[PER];
  unsigned key[PER];     // selection key of entry i (expert lane + 32 i); 0 = taken or absent
  const float* lr = logits + t * ld;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + i * 32;
    score[i] = e < experts ? lr[e] : -INFINITY;
    mx = fmaxf(mx, score[i]);
  }
  if (sigmoid) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      if (e < experts) {
        score[i] = 1.f / (1.f + __expf(-score[i]));
        key[i] = route_key(score[i] + (sel_bias ? sel_bias[e] : 0.f));
      } else {
        score[i] = 0.f;
        key[i] = 0u;
      }
    }
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      score[i] = e < experts ? __expf(score[i] - mx) : 0.f;
      sum += score[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      score[i] *= inv;
      key[i] = e < experts ? route_key(score[i]) : 0u;
    }
  }
  // lane-local best: highest key, lowest slot on ties (slots of a lane ascend with the expert index)
  // (every index below is a compile-time constant after unrolling: the arrays must stay in registers)
  unsigned bk = 0u;
  int bs = 0;
#define HB_ROUTE_RESCAN()                              \
  bk = 0u;                                             \
  bs = 0;                                              \
  _Pragma("unroll") for (int i = PER - 1; i >= 0; --i) { \
    const bool better = key[i] >= bk && key[i] != 0u;  \
    bk = better ? key[i] : bk;                         \
    bs = better ? i : bs;                              \
  }
  HB_ROUTE_RESCAN()
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < topk; ++k) {
    const unsigned top = __reduce_max_sync(0xffffffffu, bk);
    // among the lanes that hold the top key, the lowest expert index: expert = lane + 32 * slot
    const unsigned cand = (bk == top && top != 0u) ? 0xffffffffu - static_cast<unsigned>(lane + bs * 32) : 0u;
    const unsigned win = __reduce_max_sync(0xffffffffu, cand);
    const int bi = top != 0u ? static_cast<int>(0xffffffffu - win) : 0;
    float sc = 0.f;
    if (top != 0u && (bi & 31) == lane) {
      const int slot = bi >> 5;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        sc = i == slot ? score[i] : sc;
        key[i] = i == slot ? 0u : key[i];
      }
      HB_ROUTE_RESCAN()
    }
    sc = __shfl_sync(0xffffffffu, sc, bi & 31);
    wsum += sc;
    if (lane == k) {
      my_w = sc;
      my_id = bi;
    }
  }
  if (lane < topk) {
    const float w = (renorm ? my_w / fmaxf(wsum, 1e-20f) : my_w) * scale;
    ids[static_cast<long long>(t) * topk + lane] = my_id;
    weights[static_cast<long long>(t) * topk + lane] = w;
  }
#undef HB_ROUTE_RESCAN
}

// Budgeted expert sharing for small batches (decode, verify): a step whose rows pick their experts independently
// streams almost rows x top-k distinct experts' weights; here the call as a whole reads at most `budget` distinct
// experts. Every row keeps its best `keep` choices; the rest of the budget goes to the experts with the largest
// summed routing weight over the call (ties: the lower id); a row then uses those of its top-k that made the set, in
// rank order, with its weights renormalised over them (times `scale`), and fills the slots it lost with its best
// expert at weight 0 so that shapes stay fixed. ids / weights are the router's output [rows, k], updated in place.
// One CTA of 1024 threads; experts <= 1024, rows * k <= 16384. Sums are integers (2^-24 units): order-independent.
__global__ void __launch_bounds__(1024)
moe_share_kernel(int* __restrict__ ids, float* __restrict__ weights, int rows, int k, int experts, int keep, int budget,
                 float scale) {
  __shared__ unsigned score[1024];
  __shared__ unsigned char in_set[1024];
  __shared__ int s_core;
  const int tid = threadIdx.x;
  if (tid < 1024) {
    score[tid] = 0u;
    in_set[tid] = 0;
  }
  if (tid == 0) s_core = 0;
  __syncthreads();
  for (int i = tid; i < rows * k; i += blockDim.x) {
    const int r = i / k, j = i - r * k;
    const int e = ids[i];
    if (e < 0 || e >= experts) continue;
    float sum = 0.f;
    for (int q = 0; q < k; ++q) sum += weights[r * k + q];
    const float w = sum > 0.f ? weights[i] / sum : 0.f;
    atomicAdd(&score[e], static_cast<unsigned>(w * 16777216.f));
    if (j < keep) in_set[e] = 1;
  }
  __syncthreads();
  if (tid < experts && in_set[tid]) atomicAdd(&s_core, 1);
  __syncthreads();
  const int need = budget - s_core;
  bool add = false;
  if (tid < experts && !in_set[tid] && score[tid] > 0u && need > 0) {
    const unsigned mine = score[tid];
    int ahead = 0;
    for (int e = 0; e < experts; ++e)
      ahead += !in_set[e] && (score[e] > mine || (score[e] == mine && e < tid));
    add = ahead < need;
  }
  __syncthreads();      // every rank was counted against the guaranteed set alone
  if (add) in_set[tid] = 2;
  __syncthreads();
  for (int r = tid; r < rows; r += blockDim.x) {
    int* ri = ids + static_cast<long long>(r) * k;
    float* rw = weights + static_cast<long long>(r) * k;
    const int first = ri[0];
    float sum = 0.f;
    int used = 0;
    for (int j = 0; j < k; ++j) {
      const int e = ri[j];
      const float w = rw[j];
      if (e >= 0 && e < experts && in_set[e]) {
        ri[used] = e;
        rw[used] = w;
        sum += w;
        ++used;
      }
    }
    const float inv = sum > 0.f ? scale / sum : 0.f;
    for (int j = 0; j < used; ++j) rw[j] *= inv;
    for (int j = used; j < k; ++j) {
      ri[j] = first;
      rw[j] = 0.f;
    }
  }
}

// Exclusive prefix sum over the 1024 threads of the CTA (thread i contributes v); `total` receives the sum.
__device__ __forceinline__ int block_excl_scan_1024(int v, int* wtot, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  __syncthreads();
  if (lane == 31) wtot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const int w = wtot[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += up;
    }
    wtot[lane] = winc - w;
    if (lane == 31 && total != nullptr) *total = winc;
  }
  __syncthreads();
  return wtot[warp] + inc - v;
}

// Single CTA. e_lo / e_n restrict planning to the experts [e_lo, e_lo + e_n) this rank owns (expert parallelism):
// pairs routed elsewhere get pos = -1 and are skipped by the combine.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int pairs, int topk, int experts, int e_lo, int e_n, int id_base,
                int* __restrict__ cnt, int* __restrict__ start, int* __restrict__ pos, int* __restrict__ src_row,
                int rows_cap, int* __restrict__ total_rows, int tile_bn, int* __restrict__ tiles,
                int* __restrict__ n_tiles, int tile_cap) {
  extern __shared__ int sm[];   // [experts] counts, [experts] starts, [experts] running, [warps][experts]
  int* c = sm;
  int* s = sm + experts;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) c[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i] - id_base;   // `experts` counts the experts held here; ids are global
    if (e >= e_lo && e < e_lo + e_n) atomicAdd(&c[e], 1);
  }
  __syncthreads();
  __shared__ int wtot[32];
  __shared__ int s_total;
  const bool par = experts <= static_cast<int>(blockDim.x) && blockDim.x == 1024;   // one expert per thread
  if (par) {
    const int mine = static_cast<int>(threadIdx.x) < experts ? ((c[threadIdx.x] + 127) >> 7) << 7 : 0;
    const int off = block_excl_scan_1024(mine, wtot, &s_total);
    if (static_cast<int>(threadIdx.x) < experts) s[threadIdx.x] = off;
    __syncthreads();
    if (threadIdx.x == 0) *total_rows = s_total;
  } else if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < experts; ++e) {
      s[e] = acc;
      acc += ((c[e] + 127) >> 7) << 7;
    }
    *total_rows = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    cnt[e] = c[e];
    start[e] = s[e];
  }
  // Work list of the grouped GEMMs: one entry (expert * 4096 + chunk) per tile of `tile_bn` rows that has rows.
  if (tiles != nullptr) {
    int* tb = s + experts;   // scratch (reused as the running counts below)
    if (par) {
      const int mine = static_cast<int>(threadIdx.x) < experts ? (c[threadIdx.x] + tile_bn - 1) / tile_bn : 0;
      const int off = block_excl_scan_1024(mine, wtot, &s_total);
      if (static_cast<int>(threadIdx.x) < experts) tb[threadIdx.x] = off;
      __syncthreads();
      if (threadIdx.x == 0) *n_tiles = s_total < tile_cap ? s_total : tile_cap;
    } else if (threadIdx.x == 0) {
      int acc = 0;
      for (int e = 0; e < experts; ++e) {
        tb[e] = acc;
        acc += (c[e] + tile_bn - 1) / tile_bn;
      }
      *n_tiles = acc < tile_cap ? acc : tile_cap;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
      const int nt = (c[e] + tile_bn - 1) / tile_bn;
      for (int k = 0; k < nt; ++k)
        if (tb[e] + k < tile_cap) tiles[tb[e] + k] = e * 4096 + k;
    }
    __syncthreads();
  }
  for (int r = threadIdx.x; r < rows_cap; r += blockDim.x) src_row[r] = -1;
  __syncthreads();
  // Deterministic positions (pairs of an expert keep their order): chunks of blockDim.x pairs; inside a chunk a
  // warp ranks its 32 pairs by expert with match_any, per-warp counts are prefix-summed over the warps, and a
  // running count per expert carries from chunk to chunk.
  int* run = s + experts;                 // [experts] rows handed out so far
  int* wc = run + experts;                // [warps][experts] pairs of this chunk per warp and expert
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) run[e] = 0;
  for (int base = 0; base < pairs; base += blockDim.x) {
    for (int k = threadIdx.x; k < warps * experts; k += blockDim.x) wc[k] = 0;
    __syncthreads();
    const int i = base + threadIdx.x;
    int e = i < pairs ? ids[i] - id_base : -1;
    if (e < e_lo || e >= e_lo + e_n) e = -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) wc[warp * experts + e] = __popc(same);
    __syncthreads();
    for (int x = threadIdx.x; x < experts; x += blockDim.x) {   // exclusive prefix over warps, in place
      int acc = run[x];
      for (int w = 0; w < warps; ++w) {
        const int v = wc[w * experts + x];
        wc[w * experts + x] = acc;
        acc += v;
      }
      run[x] = acc;
    }
    __syncthreads();
    if (i < pairs) {
      if (e >= 0) {
        const int r = s[e] + wc[warp * experts + e] + rank;
        if (r < rows_cap) {
          pos[i] = r;
          src_row[r] = i / topk;
        } else {
          pos[i] = -1;
        }
      } else {
        pos[i] = -1;
      }
    }
    __syncthreads();
  }
}

// Work list from per-expert row counts alone (for plans made elsewhere, e.g. the expert-parallel one): one entry
// expert * 4096 + chunk per tile of `tile_bn` rows that has rows. Single CTA.
__global__ void moe_tiles_kernel(const int* __restrict__ cnt, int experts, int tile_bn, int* __restrict__ tiles,
                                 int* __restrict__ n_tiles, int tile_cap) {
  extern __shared__ int base[];
  __shared__ int wtot[32];
  __shared__ int s_total;
  if (experts <= 1024 && blockDim.x == 1024) {      // one expert per thread: parallel prefix
    const int mine = static_cast<int>(threadIdx.x) < experts ? (cnt[threadIdx.x] + tile_bn - 1) / tile_bn : 0;
    const int off = block_excl_scan_1024(mine, wtot, &s_total);
    if (static_cast<int>(threadIdx.x) < experts) base[threadIdx.x] = off;
    __syncthreads();
    if (threadIdx.x == 0) *n_tiles = s_total < tile_cap ? s_total : tile_cap;
  } else if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < experts; ++e) {
      base[e] = acc;
      acc += (cnt[e] + tile_bn - 1) / tile_bn;
    }
    *n_tiles = acc < tile_cap ? acc : tile_cap;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int nt = (cnt[e] + tile_bn - 1) / tile_bn;
    for (int k = 0; k < nt; ++k)
      if (base[e] + k < tile_cap) tiles[base[e] + k] = e * 4096 + k;
  }
}

__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ src_row,
                                  const int* __restrict__ total_rows, __nv_bfloat16* __restrict__ out, int h) {
  const int r = blockIdx.x;
  if (r >= *total_rows) return;
  const int src = src_row[r];
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(r) * h);
  if (src < 0) {
    for (int i = threadIdx.x; i < (h >> 3); i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* s = reinterpret_cast<const uint4*>(x + src * ldx);
    for (int i = threadIdx.x; i < (h >> 3); i += blockDim.x) dst[i] = s[i];
  }
}

// out[t, :] = sum_k w[t, k] * y[pos[t, k], :] (+ shared[t, :] * shared_scale). One CTA per token.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long long ldy, const int* __restrict__ pos,
                                   const float* __restrict__ weights, const __nv_bfloat16* __restrict__ shared,
                                   long long ld_shared, __nv_bfloat16* __restrict__ out, long long ldo, int topk,
                                   int h) {
  const int t = blockIdx.x;
  __shared__ int ps[MAX_TOPK];
  __shared__ float ws[MAX_TOPK];
  if (threadIdx.x < topk) {
    ps[threadIdx.x] = pos[static_cast<long long>(t) * topk + threadIdx.x];
    ws[threadIdx.x] = weights[static_cast<long long>(t) * topk + threadIdx.x];
  }
  __syncthreads();
  for (int i = threadIdx.x * 2; i < h; i += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int k = 0; k < topk; ++k) {
      if (ps[k] < 0) continue;
      const uint32_t v = *reinterpret_cast<const uint32_t*>(y + ps[k] * ldy + i);
      a0 += ws[k] * bf16_lo(v);
      a1 += ws[k] * bf16_hi(v);
    }
    if (shared != nullptr) {
      const uint32_t v = *reinterpret_cast<const uint32_t*>(shared + t * ld_shared + i);
      a0 += bf16_lo(v);
      a1 += bf16_hi(v);
    }
    *reinterpret_cast<uint32_t*>(out + t * ldo + i) = pack_bf16(a0, a1);
  }
}

}  // namespace
}  // namespace hb

using namespace hb;
#define ST(s) static_cast<cudaStream_t>(s)

extern "C" {

int hb_moe_route(const void* logits, long long ld, const void* sel_bias, int tokens, int experts, int topk,
                 int sigmoid, int renorm, float scale, void* ids, void* weights, void* stream) {
  if (tokens <= 0) return 0;
  if (experts > 1024 || topk > MAX_TOPK || topk > experts) return 1;
  if (tokens <= 256 && experts > 128) {      // decode / verify sizes: latency matters, one CTA per token
    const int threads = (experts + 31) / 32 * 32;
    moe_route_block_kernel<<<tokens, threads, 0, ST(stream)>>>(
        static_cast<const float*>(logits), ld, static_cast<const float*>(sel_bias), experts, topk, sigmoid, renorm,
        scale, static_cast<int*>(ids), static_cast<float*>(weights));
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
#define HB_ROUTE(PER)                                                                                        \
  moe_route_kernel<PER><<<(tokens + 3) / 4, 128, 0, ST(stream)>>>(                                           \
      static_cast<const float*>(logits), ld, static_cast<const float*>(sel_bias), tokens, experts, topk, sigmoid, \
      renorm, scale, static_cast<int*>(ids), static_cast<float*>(weights))
  if (experts <= 128) HB_ROUTE(4);
  else if (experts <= 512) HB_ROUTE(16);
  else HB_ROUTE(32);
#undef HB_ROUTE
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_moe_share(void* ids, void* weights, int rows, int k, int experts, int keep, int budget, float scale,
                 void* stream) {
  if (rows <= 0) return 0;
  if (experts > 1024 || k > MAX_TOPK || keep < 0 || keep > k || rows * k > 16384) return 1;
  moe_share_kernel<<<1, 1024, 0, ST(stream)>>>(static_cast<int*>(ids), static_cast<float*>(weights), rows, k, experts,
                                               keep, budget, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_moe_plan(const void* ids, int tokens, int topk, int experts, int e_lo, int e_n, int id_base, void* cnt, void* start,
                void* pos, void* src_row, int rows_cap, void* total_rows, int tile_bn, void* tiles, void* n_tiles,
                int tile_cap, void* stream) {
  if (tokens <= 0) return 0;
  if (tiles != nullptr && (tile_bn < 16 || n_tiles == nullptr || tile_cap <= 0)) return 1;
  const size_t smem = static_cast<size_t>(3 + 1024 / 32) * experts * sizeof(int);
  static size_t attr = 0;
  if (smem > 48 * 1024 && smem > attr) {
    if (cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return 3;
    attr = smem;
  }
  moe_plan_kernel<<<1, 1024, smem, ST(stream)>>>(
      static_cast<const int*>(ids), tokens * topk, topk, experts, e_lo, e_n, id_base, static_cast<int*>(cnt),
      static_cast<int*>(start), static_cast<int*>(pos), static_cast<int*>(src_row), rows_cap,
      static_cast<int*>(total_rows), tile_bn, static_cast<int*>(tiles), static_cast<int*>(n_tiles), tile_cap);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_moe_tiles(const void* cnt, int experts, int tile_bn, void* tiles, void* n_tiles, int tile_cap, void* stream) {
  if (experts <= 0 || tile_bn < 16 || tile_cap <= 0) return 1;
  moe_tiles_kernel<<<1, 1024, experts * sizeof(int), ST(stream)>>>(static_cast<const int*>(cnt), experts, tile_bn,
                                                                  static_cast<int*>(tiles),
                                                                  static_cast<int*>(n_tiles), tile_cap);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_moe_gather(const void* x, long long ldx, const void* src_row, const void* total_rows, void* out, int rows_cap,
                  int h, void* stream) {
  if (rows_cap <= 0) return 0;
  moe_gather_kernel<<<rows_cap, 128, 0, ST(stream)>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                      static_cast<const int*>(src_row),
                                                      static_cast<const int*>(total_rows),
                                                      static_cast<__nv_bfloat16*>(out), h);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_moe_combine(const void* y, long long ldy, const void* pos, const void* weights, const void* shared,
                   long long ld_shared, void* out, long long ldo, int tokens, int topk, int h, void* stream) {
  if (tokens <= 0) return 0;
  if (topk > MAX_TOPK || (h & 1)) return 1;
  moe_combine_kernel<<<tokens, 256, 0, ST(stream)>>>(static_cast<const __nv_bfloat16*>(y), ldy,
                                                     static_cast<const int*>(pos), static_cast<const float*>(weights),
                                                     static_cast<const __nv_bfloat16*>(shared), ld_shared,
                                                     static_cast<__nv_bfloat16*>(out), ldo, topk, h);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
