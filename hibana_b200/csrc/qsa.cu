// Sparse attention with a learned indexer ("QSA"): every `ratio` consecutive tokens of a sequence form a group with
// one compressed index key; a query scores the groups that are complete at its position, keeps the best
// budget / ratio of them and attends only to their tokens plus the tail of its own incomplete group.
//
//   compress  ckey[group] = RoPE_at(group's first position)( GemmaRMSNorm( mean of the group's raw index keys ) ),
//             stored in the row of the group's FIRST token of an index pool parallel to the KV pool
//   score     s[row, g] = sum over index heads of relu(q[row, h, :] . ckey[g]) / sqrt(D) for g < (pos + 1) / ratio,
//             -inf beyond
//   expand    chosen group ids (top-k, done with torch.topk on the device) -> KV slot list per query row:
//             the groups' tokens, then the tail tokens; the paged attention kernels then run over that list
// One warp per group (compress) or per (row, group) score; D = 128 (four elements per lane).
// Reference: hibana/model/flashnext/reference.py:29-64 (the rule), hibana/kernels/qsa/csrc/{compression,query_prep,
// score_exact,topk_pages}.cu.
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int QD = 128;

// grid: total groups (prefix-summed over sequences via grp_indptr); block: 32 threads (one warp per group).
__global__ void qsa_compress_kernel(const __nv_bfloat16* __restrict__ raw_k, __nv_bfloat16* __restrict__ ckey,
                                    const int* __restrict__ kv_indices, long long ld_idx,
                                    const int* __restrict__ seq_rows, const int* __restrict__ grp_indptr,
                                    const int* __restrict__ grp_first, int batch, int ratio,
                                    const __nv_bfloat16* __restrict__ norm_w, float eps,
                                    const float* __restrict__ inv_freq, int rot) {
  const int gi = blockIdx.x;
  if (gi >= grp_indptr[batch]) return;      // the grid may cover a host-side bound of the number of groups
  int b = 0;
  while (b + 1 < batch && grp_indptr[b + 1] <= gi) ++b;
  const int g = grp_first[b] + (gi - grp_indptr[b]);     // group number inside the sequence
  const int lane = threadIdx.x;
  const int* idx = kv_indices + static_cast<long long>(seq_rows ? seq_rows[b] : b) * ld_idx;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < ratio; ++j) {
    const uint2 raw = *reinterpret_cast<const uint2*>(raw_k + static_cast<long long>(idx[g * ratio + j]) * QD + lane * 4);
    v[0] += bf16_lo(raw.x); v[1] += bf16_hi(raw.x); v[2] += bf16_lo(raw.y); v[3] += bf16_hi(raw.y);
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    v[e] *= 1.f / ratio;
    ss += v[e] * v[e];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / QD + eps);
  const uint2 wr = *reinterpret_cast<const uint2*>(norm_w + lane * 4);
  const float w[4] = {bf16_lo(wr.x), bf16_hi(wr.x), bf16_lo(wr.y), bf16_hi(wr.y)};
#pragma unroll
  for (int e = 0; e < 4; ++e) v[e] = __bfloat162float(__float2bfloat16(v[e] * rstd * (1.f + w[e])));
  // NeoX rotary over the first `rot` dims at the group's first position: element d pairs with d + rot / 2
  const float pos = static_cast<float>(g * ratio);
  const int half = rot >> 1;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int d = lane * 4 + e;
    float other = __shfl_sync(0xffffffffu, v[e], (d < half ? d + half : d - half) >> 2);
    // the partner sits in another lane at the same e (half is a multiple of 4)
    if (d < rot) {
      const int fi = d < half ? d : d - half;
      float s, c;
      __sincosf(pos * inv_freq[fi], &s, &c);
      v[e] = d < half ? v[e] * c - other * s : v[e] * c + other * s;
    }
  }
  const long long dst = static_cast<long long>(idx[g * ratio]) * QD + lane * 4;
  *reinterpret_cast<uint2*>(ckey + dst) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
}

// grid (rows, ceil(max_groups / 8)); 8 warps per CTA, one group per warp.
__global__ void __launch_bounds__(256)
qsa_score_kernel(const __nv_bfloat16* __restrict__ q, int heads, const __nv_bfloat16* __restrict__ ckey,
                 const int* __restrict__ kv_indices, long long ld_idx, const int* __restrict__ row_seq,
                 const int* __restrict__ row_pos, int ratio, int max_groups, float* __restrict__ scores) {
  const int row = blockIdx.x;
  const int g = blockIdx.y * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (g >= max_groups) return;
  const int visible = (row_pos[row] + 1) / ratio;
  float out = -INFINITY;
  if (g < visible) {
    const int* idx = kv_indices + static_cast<long long>(row_seq[row]) * ld_idx;
    const uint2 kr = *reinterpret_cast<const uint2*>(ckey + static_cast<long long>(idx[g * ratio]) * QD + lane * 4);
    const float k[4] = {bf16_lo(kr.x), bf16_hi(kr.x), bf16_lo(kr.y), bf16_hi(kr.y)};
    float acc = 0.f;
    for (int h = 0; h < heads; ++h) {
      const uint2 qr = *reinterpret_cast<const uint2*>(q + (static_cast<long long>(row) * heads + h) * QD + lane * 4);
      float d = bf16_lo(qr.x) * k[0] + bf16_hi(qr.x) * k[1] + bf16_lo(qr.y) * k[2] + bf16_hi(qr.y) * k[3];
      d = warp_sum(d);
      acc += fmaxf(d, 0.f);
    }
    out = acc * rsqrtf(static_cast<float>(QD));
  }
  if (lane == 0) scores[static_cast<long long>(row) * max_groups + g] = out;
}

// One CTA per query row: writes the KV slots of the chosen groups (ascending group order is not required by the
// attention kernels), then the tail tokens; sel_len = tokens written.
__global__ void __launch_bounds__(128)
qsa_expand_kernel(const long long* __restrict__ chosen, const float* __restrict__ chosen_scores, int width,
                  const int* __restrict__ kv_indices, long long ld_idx, const int* __restrict__ row_seq,
                  const int* __restrict__ row_pos, int ratio, int* __restrict__ sel, long long ld_sel,
                  int* __restrict__ sel_len) {
  __shared__ int count;
  const int row = blockIdx.x;
  const int* idx = kv_indices + static_cast<long long>(row_seq[row]) * ld_idx;
  if (threadIdx.x == 0) count = 0;
  __syncthreads();
  // valid choices form a prefix of the top-k output (scores of invisible groups are -inf and sort last)
  int nvalid = 0;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    if (chosen_scores[static_cast<long long>(row) * width + i] > -INFINITY) atomicAdd(&count, 1);
  __syncthreads();
  nvalid = count;
  for (int i = threadIdx.x; i < nvalid * ratio; i += blockDim.x) {
    const int g = static_cast<int>(chosen[static_cast<long long>(row) * width + i / ratio]);
    sel[static_cast<long long>(row) * ld_sel + i] = idx[g * ratio + i % ratio];
  }
  const int pos = row_pos[row];
  const int tail0 = (pos + 1) / ratio * ratio;
  for (int p = tail0 + threadIdx.x; p <= pos; p += blockDim.x)
    sel[static_cast<long long>(row) * ld_sel + nvalid * ratio + (p - tail0)] = idx[p];
  if (threadIdx.x == 0) sel_len[row] = nvalid * ratio + (pos - tail0 + 1);
}

}  // namespace
}  // namespace hb

using namespace hb;
#define ST(s) static_cast<cudaStream_t>(s)

extern "C" {

// Index keys have 128 dims. grp_indptr [batch + 1]: prefix sum of groups to compress per sequence; grp_first [batch]:
// number of the first of them inside its sequence.
int hb_qsa_compress(const void* raw_k, void* ckey, const void* kv_indices, long long ld_idx, const void* seq_rows,
                    const void* grp_indptr, const void* grp_first, int batch, int total_groups, int ratio,
                    const void* norm_w, float eps, const void* inv_freq, int rot, void* stream) {
  if (total_groups <= 0) return 0;
  if (rot % 8 != 0 || rot > QD) return 1;
  qsa_compress_kernel<<<total_groups, 32, 0, ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(raw_k), static_cast<__nv_bfloat16*>(ckey), static_cast<const int*>(kv_indices),
      ld_idx, static_cast<const int*>(seq_rows), static_cast<const int*>(grp_indptr),
      static_cast<const int*>(grp_first), batch, ratio, static_cast<const __nv_bfloat16*>(norm_w), eps,
      static_cast<const float*>(inv_freq), rot);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_qsa_score(const void* q, int rows, int heads, const void* ckey, const void* kv_indices, long long ld_idx,
                 const void* row_seq, const void* row_pos, int ratio, int max_groups, void* scores, void* stream) {
  if (rows <= 0 || max_groups <= 0) return 0;
  qsa_score_kernel<<<dim3(rows, (max_groups + 7) / 8), 256, 0, ST(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), heads, static_cast<const __nv_bfloat16*>(ckey),
      static_cast<const int*>(kv_indices), ld_idx, static_cast<const int*>(row_seq), static_cast<const int*>(row_pos),
      ratio, max_groups, static_cast<float*>(scores));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_qsa_expand(const void* chosen, const void* chosen_scores, int rows, int width, const void* kv_indices,
                  long long ld_idx, const void* row_seq, const void* row_pos, int ratio, void* sel, long long ld_sel,
                  void* sel_len, void* stream) {
  if (rows <= 0) return 0;
  qsa_expand_kernel<<<rows, 128, 0, ST(stream)>>>(
      static_cast<const long long*>(chosen), static_cast<const float*>(chosen_scores), width,
      static_cast<const int*>(kv_indices), ld_idx, static_cast<const int*>(row_seq), static_cast<const int*>(row_pos),
      ratio, static_cast<int*>(sel), ld_sel, static_cast<int*>(sel_len));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
