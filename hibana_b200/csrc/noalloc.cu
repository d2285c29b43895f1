// Allocation-free greedy argmax: see hb_noalloc.h for who needs it and the rules of use.
#include "hb_noalloc.h"

#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

// The scratch lives in the library image: partial maxima first, their indices after them.
static __device__ __align__(256) unsigned char g_noalloc_scratch[HB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};   // device address of the array, per device, filled on first use

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

__device__ __forceinline__ void keep_better(float& best, int& bi, float v, int i) {
  if (v > best || (v == best && i < bi)) {
    best = v;
    bi = i;
  }
}

// Stage 1: HB_NOALLOC_CHUNKS CTAs per row, each reduces one slice of the vocabulary into one partial.
template <typename T>
__global__ void __launch_bounds__(256)
noalloc_partial_kernel(const T* __restrict__ logits, long long ld, int vocab, float* __restrict__ pv,
                       int* __restrict__ pi) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const int row = blockIdx.x, ch = blockIdx.y;
  const T* lr = logits + row * ld;
  const int per = (vocab + HB_NOALLOC_CHUNKS - 1) / HB_NOALLOC_CHUNKS;
  const int lo = ch * per, hi = min(vocab, lo + per);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) keep_better(best, bi, load_logit<T>(lr, i), i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    keep_better(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) keep_better(best, bi, sv[w], si[w]);
    pv[row * HB_NOALLOC_CHUNKS + ch] = best;      // every partial that stage 2 reads is written here first
    pi[row * HB_NOALLOC_CHUNKS + ch] = bi;
  }
}

// Stage 2: one warp per row combines the partials.
__global__ void noalloc_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int rows,
                                     long long* __restrict__ out) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < HB_NOALLOC_CHUNKS; c += 32)
    keep_better(best, bi, pv[row * HB_NOALLOC_CHUNKS + c], pi[row * HB_NOALLOC_CHUNKS + c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    keep_better(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
}

void explain(char* buf, int len, const char* msg) {
  if (buf != nullptr && len > 0) snprintf(buf, static_cast<size_t>(len), "%s", msg);
}

}  // namespace

extern "C" int hb_argmax_noalloc(const void* logits, long long ld, int rows, int vocab, int is_f32, void* out,
                                 void* stream, char* errbuf, int errbuf_len) {
  if (logits == nullptr || out == nullptr || vocab <= 0 || rows < 0 || ld < vocab) {
    explain(errbuf, errbuf_len, "hb_argmax_noalloc: bad argument (null pointer, vocab <= 0, rows < 0 or ld < vocab)");
    return HB_NOALLOC_BAD_ARGUMENT;
  }
  if (rows > HB_NOALLOC_MAX_ROWS) {
    if (errbuf != nullptr && errbuf_len > 0)
      snprintf(errbuf, static_cast<size_t>(errbuf_len),
               "hb_argmax_noalloc: %d rows exceed the built-in scratch (at most %d rows per call)", rows,
               HB_NOALLOC_MAX_ROWS);
    return HB_NOALLOC_TOO_MANY_ROWS;
  }
  if (rows == 0) return HB_NOALLOC_OK;
  // Set-up, once per device, with that device current: in host code the array's name is only a stand-in, the
  // kernels need its device address.
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    explain(errbuf, errbuf_len, "hb_argmax_noalloc: no current CUDA device");
    return HB_NOALLOC_SETUP_FAILED;
  }
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      explain(errbuf, errbuf_len, "hb_argmax_noalloc: cudaGetSymbolAddress failed for the scratch array");
      return HB_NOALLOC_SETUP_FAILED;
    }
    g_scratch_addr[dev] = p;
  }
  float* pv = static_cast<float*>(g_scratch_addr[dev]);
  int* pi = reinterpret_cast<int*>(static_cast<unsigned char*>(g_scratch_addr[dev]) +
                                   HB_NOALLOC_MAX_ROWS * HB_NOALLOC_CHUNKS * 4);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(rows, HB_NOALLOC_CHUNKS);
  if (is_f32)
    noalloc_partial_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(logits), ld, vocab, pv, pi);
  else
    noalloc_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, vocab,
                                                               pv, pi);
  noalloc_final_kernel<<<(rows + 3) / 4, 128, 0, st>>>(pv, pi, rows, static_cast<long long*>(out));
  if (cudaGetLastError() != cudaSuccess) {
    explain(errbuf, errbuf_len, "hb_argmax_noalloc: kernel launch failed");
    return HB_NOALLOC_LAUNCH_FAILED;
  }
  return HB_NOALLOC_OK;
}
