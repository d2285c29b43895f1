// Gather / scatter of token rows between the paged KV pool of ALL layers and one linear payload buffer, in one
// launch per direction: the data mover of the SSD tier (pool -> pinned host staging -> file, and back).
//
// Pool storage is [layers][2 (k, v)][kv_heads][slots][D] (head-major, csrc/kv_tma.cuh); the payload of token i is
// [layers][2][kv_heads][D] contiguous, tokens one after another, so a block of 256 tokens is one contiguous
// object on disk. The payload pointer may be pinned host memory (unified addressing): the kernel then moves the
// rows over PCIe itself, and no intermediate device buffer or per-row copy call exists.
// Reference counterpart: hibana/kernels/csrc/kv_copy.cu (gather/scatter between pools and host-mapped payload
// buffers, all pools in one launch), hibana/cache/ssd.py:176-246.
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

// grid (tokens, layers * 2); a CTA moves the kv_heads rows of one (token, layer, k|v): kv_heads * row_bytes bytes.
__global__ void kv_copy_kernel(uint8_t* __restrict__ pool, uint8_t* __restrict__ payload,
                               const int* __restrict__ slots, long long plane_bytes, long long head_bytes,
                               int row_bytes, int kv_heads, long long token_bytes, int to_pool) {
  const int slot = slots[blockIdx.x];
  if (slot < 0 || !index_ok(slot, kBoundKvSlots, kKerKvCopy)) return;
  uint8_t* pl = payload + static_cast<long long>(blockIdx.x) * token_bytes +
                static_cast<long long>(blockIdx.y) * kv_heads * row_bytes;
  uint8_t* pp = pool + static_cast<long long>(blockIdx.y) * plane_bytes + static_cast<long long>(slot) * row_bytes;
  const int chunks = row_bytes >> 4;
  for (int i = threadIdx.x; i < kv_heads * chunks; i += blockDim.x) {
    const int hd = i / chunks, c = i % chunks;
    uint4* a = reinterpret_cast<uint4*>(pp + hd * head_bytes) + c;
    uint4* b = reinterpret_cast<uint4*>(pl + hd * row_bytes) + c;
    if (to_pool) *a = *b;
    else *b = *a;
  }
}

}  // namespace
}  // namespace hb

extern "C" {

// pool: base of [layers][2][kv_heads][slots_dim][D] with element size `esize`; payload: `tokens` rows of
// layers * 2 * kv_heads * D elements; slots: int32 [tokens] on the device (-1 = skip). to_pool = 1 scatters.
int hb_kv_copy(void* pool, void* payload, const void* slots, int tokens, int layers, int kv_heads,
               long long slots_dim, int d, int esize, int to_pool, void* stream) {
  if (tokens <= 0) return 0;
  const int row_bytes = d * esize;
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(pool) & 15) || (reinterpret_cast<uintptr_t>(payload) & 15))
    return 1;
  const long long head_bytes = slots_dim * row_bytes;
  const long long plane_bytes = head_bytes * kv_heads;
  const long long token_bytes = static_cast<long long>(layers) * 2 * kv_heads * row_bytes;
  hb::kv_copy_kernel<<<dim3(tokens, layers * 2), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(pool), static_cast<uint8_t*>(payload), static_cast<const int*>(slots), plane_bytes,
      head_bytes, row_bytes, kv_heads, token_bytes, to_pool);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
