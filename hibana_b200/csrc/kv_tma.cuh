// Tensor maps over a token-granular KV pool, for bulk tensor copies of runs of consecutive slots.
//
// A pool is logically [slots, kv_heads, D] bf16 with arbitrary slot and head strides. Two physical layouts occur:
//   slot-major  (head stride = D, slot stride = kv_heads * D): one token's heads are adjacent;
//   head-major  (slot stride = D, head stride = slots * D):     one head's tokens are adjacent, so a run of slots
//               of one head is one contiguous stream (full DRAM page locality when a kernel walks one head).
// Either is described to the TMA unit as a 2-D matrix with row pitch = slot stride; a box is `box_rows` slots x
// 64 elements (128 bytes, the 128-byte-swizzle limit). Head h, column block c, first slot s of a run:
//   x = h * xh + c * 64,   y = h * yh + s.
#pragma once
#include "gemm.cuh"

namespace hb {

struct KvTma {
  CUtensorMap k = {};     // copies: valid for as long as this struct lives (the launch that follows)
  CUtensorMap v = {};
  int xh = 0, yh = 0;
  int ok = 0;
};

inline KvTma make_kv_tma(const void* k_pool, const void* v_pool, long long slot_stride, long long head_stride,
                         long long pool_slots, int hkv, int d, int box_rows) {
  KvTma t;
  if (pool_slots < box_rows || slot_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(k_pool) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(v_pool) & 15) != 0 || d % 64 != 0)
    return t;
  uint64_t rows, cols;
  if (head_stride == d && slot_stride >= static_cast<long long>(hkv) * d) {
    rows = static_cast<uint64_t>(pool_slots);
    cols = static_cast<uint64_t>(hkv) * d;
    t.xh = d;
    t.yh = 0;
  } else if (slot_stride >= d && head_stride % slot_stride == 0 && head_stride / slot_stride >= pool_slots) {
    rows = static_cast<uint64_t>(hkv) * (head_stride / slot_stride);
    cols = static_cast<uint64_t>(d);
    t.xh = 0;
    t.yh = static_cast<int>(head_stride / slot_stride);
  } else {
    return t;
  }
  TmapKey kk{k_pool, rows, cols, static_cast<uint64_t>(slot_stride) * 2, static_cast<uint32_t>(box_rows), 64u, 0};
  TmapKey kv = kk;
  kv.ptr = v_pool;
  t.ok = get_tmap_2d(kk, &t.k) && get_tmap_2d(kv, &t.v);
  return t;
}

}  // namespace hb
