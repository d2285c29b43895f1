// Expert-parallel all-to-all over NVLink peer memory, fused with the work on either side of it.
//
// Every rank routes its own tokens; the experts are split into contiguous ranges, one per rank. One mixture-of-
// experts call on every rank is the kernel sequence
//
//   ep_count     my (token, expert) pairs per expert -> row `rank` of the count matrix on EVERY rank + a flag
//   ep_plan      waits for all rows of the count matrix; from it every rank derives, without further traffic,
//                the layout of every owner's receive buffer (expert segments padded to 128 rows, sources in
//                rank order inside a segment): the owner side gets segment starts / counts for the grouped
//                GEMMs, the sender side the destination (rank, row) of each of its pairs
//   ep_dispatch  one CTA per token: quantises the row to NVFP4 once (or keeps bf16) and stores it straight into
//                the receive buffers of the owners of its top-k experts, with a note saying where the result has
//                to go; the last CTA raises this rank's "rows" flag on every rank
//   grouped fc1  (csrc/gemm.cu) weights stream in first; the activation loads wait for the "rows" flags
//   grouped fc2  (csrc/gemm.cu, epilogue 5) stores every output row into the return buffer of its source rank;
//                the last CTA raises the "returned" flag on every rank
//   ep_combine   one CTA per token: waits for the "returned" flags, then sums its top-k rows with the routing
//                weights in selection order (deterministic) and adds the shared expert; the last CTA completes
//                the call's sequence number
//
// All flags carry the call's sequence number, every wait is bounded, and a timeout leaves a status code for the
// host. Buffers are single: a rank can only start call n + 1 after its combine of call n, which needed every
// rank's fc2 of call n, so nothing of call n is still being read when call n + 1 writes.
// The reference has no multi-GPU expert parallelism (its w3 MoE takes an expert range e_lo / e_n for two ranks
// with replicated activations: hibana/kernels/csrc/w3_gemm.cu:640-1300, hibana/model/flashnext/moe.py:68-192).
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int EP_MAX_WORLD = 8;
constexpr int EP_MAX_TOPK = 32;

struct EpCtrl {                 // first bytes of every rank's expert-parallel heap
  int flag_cnt[EP_MAX_WORLD];   // [src] count-matrix row of rank src has landed (sequence number)
  int flag_rows[EP_MAX_WORLD];  // [src] dispatched rows of rank src have landed
  int flag_ret[EP_MAX_WORLD];   // [src] rank src has returned all results it owed anyone
  int seq;                      // calls completed on this rank
  int done_dispatch, done_fc2, done_combine;
  int pad[4];
};
static_assert(sizeof(EpCtrl) == 128, "layout is part of the host interface");

struct EpPeers {
  uint8_t* base[EP_MAX_WORLD];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Threads 0..world-1 wait until flags[thread] has reached seq. Returns (to every thread) whether all did.
__device__ __forceinline__ bool wait_flags(const int* flags, int world, int seq, unsigned long long limit_ns,
                                           int* status, int* ok_smem) {
  if (threadIdx.x == 0) *ok_smem = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const unsigned long long t0 = globaltimer_ns();
    bool ok = false;
    for (unsigned long long it = 0, cap = spin_cap(limit_ns); it < cap; ++it) {
      if (ld_acquire_sys(flags + threadIdx.x) - seq >= 0) {
        ok = true;
        break;
      }
      if ((it & 63u) == 63u &&
          (globaltimer_ns() - t0 > limit_ns || *reinterpret_cast<volatile int*>(status) != 0))
        break;
    }
    if (!ok) {
      *ok_smem = 0;
      set_status(status, kTimeoutPeer);
    }
  }
  __syncthreads();
  return *ok_smem != 0;
}

// ------------------------------------------------------------------------------------------------ count
__global__ void __launch_bounds__(1024)
ep_count_kernel(const int* __restrict__ ids, int pairs, int experts, EpPeers peers, int world, int rank,
                long long cnt_mat_off) {
  extern __shared__ int c[];
  EpCtrl* mine = reinterpret_cast<EpCtrl*>(peers.base[rank]);
  const int seq = ld_relaxed_sys(&mine->seq) + 1;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) c[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < experts) atomicAdd(&c[e], 1);
  }
  __syncthreads();
  for (int r = 0; r < world; ++r) {
    int* row = reinterpret_cast<int*>(peers.base[r] + cnt_mat_off) + static_cast<size_t>(rank) * experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) row[e] = c[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(&reinterpret_cast<EpCtrl*>(peers.base[threadIdx.x])->flag_cnt[rank], seq);
}

// ------------------------------------------------------------------------------------------------ plan
// Shared memory: mat [world][E], total [E], start [E], fill [E].
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int* __restrict__ ids, int pairs, int experts, int e_per, EpPeers peers, int world, int rank,
               long long cnt_mat_off, int rows_cap, int* __restrict__ grp_cnt, int* __restrict__ grp_start,
               int* __restrict__ total_rows, int* __restrict__ dst_rank, int* __restrict__ dst_row,
               unsigned long long limit_ns, int* status) {
  extern __shared__ int sm[];
  __shared__ int ok_s;
  int* mat = sm;
  int* total = mat + world * experts;
  int* start = total + experts;
  int* fill = start + experts;
  EpCtrl* mine = reinterpret_cast<EpCtrl*>(peers.base[rank]);
  const int seq = ld_relaxed_sys(&mine->seq) + 1;
  const bool ok = wait_flags(mine->flag_cnt, world, seq, limit_ns, status, &ok_s);
  const int* gmat = reinterpret_cast<const int*>(peers.base[rank] + cnt_mat_off);
  for (int i = threadIdx.x; i < world * experts; i += blockDim.x) mat[i] = ok ? ld_relaxed_sys(gmat + i) : 0;
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int t = 0, before = 0;
    for (int s = 0; s < world; ++s) {
      if (s == rank) before = t;
      t += mat[s * experts + e];
    }
    total[e] = t;
    fill[e] = before;   // my first row inside the expert's segment: sources sit in rank order
  }
  __syncthreads();
  // segment starts of every owner (thread r walks rank r's experts): 128-row aligned prefix
  if (threadIdx.x < world) {
    int acc = 0;
    for (int e = threadIdx.x * e_per; e < (threadIdx.x + 1) * e_per && e < experts; ++e) {
      start[e] = acc;
      acc += ((total[e] + 127) >> 7) << 7;
    }
    if (static_cast<int>(threadIdx.x) == rank) *total_rows = min(acc, rows_cap);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < e_per; e += blockDim.x) {
    const int ge = rank * e_per + e;
    // a segment that does not fit is left out (nothing is written past the buffer) and the call is marked failed:
    // the host reads the status word with the step's result and raises
    const bool in = ge < experts && start[ge] + total[ge] <= rows_cap;
    if (!in && ge < experts && total[ge] > 0) set_status(status, kOverflow);
    grp_cnt[e] = in ? total[ge] : 0;
    grp_start[e] = in ? start[ge] : 0;
  }
  for (int e = threadIdx.x; e < experts; e += blockDim.x) fill[e] += start[e];
  __syncthreads();
  // Rows inside a segment are handed out in arrival order of the atomics; a row's result does not depend on
  // where it sits, and the combine sums in selection order, so the output stays deterministic.
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0 || e >= experts) {
      dst_rank[i] = -1;
      dst_row[i] = -1;
      continue;
    }
    const int row = atomicAdd(&fill[e], 1);
    const bool in = row < rows_cap && start[e] + total[e] <= rows_cap;
    if (!in) set_status(status, kOverflow);
    dst_rank[i] = in ? e / e_per : -1;
    dst_row[i] = in ? row : -1;
  }
}

// ------------------------------------------------------------------------------------------------ dispatch
struct DispatchParams {
  const __nv_bfloat16* x;
  long long ldx;
  int tokens, topk, h, ka;
  const int* dst_rank;
  const int* dst_row;
  const float* gscale;       // null = bf16 rows
  EpPeers peers;
  int world, rank;
  long long q_off, sf_off, bf_off, row_ret_off;
};

template <int T>
__global__ void __launch_bounds__(T) ep_dispatch_kernel(const DispatchParams p) {
  __shared__ int dr[EP_MAX_TOPK], dw[EP_MAX_TOPK];
  EpCtrl* mine = reinterpret_cast<EpCtrl*>(p.peers.base[p.rank]);
  const int seq = ld_relaxed_sys(&mine->seq) + 1;
  const int t = blockIdx.x;
  if (t < p.tokens) {
    if (threadIdx.x < p.topk) {
      dr[threadIdx.x] = p.dst_rank[static_cast<long long>(t) * p.topk + threadIdx.x];
      dw[threadIdx.x] = p.dst_row[static_cast<long long>(t) * p.topk + threadIdx.x];
    }
    __syncthreads();
    const int nchunk = p.h >> 3;   // 8 elements = one 16-byte load
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(t) * p.ldx);
    const float inv_gs = p.gscale != nullptr ? 1.f / *p.gscale : 0.f;
    for (int c0 = 0; c0 < nchunk; c0 += T) {
      const int c = c0 + threadIdx.x;
      const bool live = c < nchunk;
      const uint4 raw = live ? src[c] : make_uint4(0, 0, 0, 0);
      if (p.gscale == nullptr) {
        if (live)
          for (int k = 0; k < p.topk; ++k)
            if (dr[k] >= 0)
              reinterpret_cast<uint4*>(p.peers.base[dr[k]] + p.bf_off + static_cast<long long>(dw[k]) * p.h * 2)[c] = raw;
        continue;
      }
      float y[8] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y),
                    bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w)};
      // chunks c and c ^ 1 form one 16-element group (T is even: neighbouring lanes)
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(y[e]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      const uint32_t sfb = float_to_e4m3(amax * (1.f / 6.f) * inv_gs);
      const float sfv = e4m3_to_float(sfb);
      const float inv = sfv > 0.f ? 1.f / (sfv * (1.f / inv_gs)) : 0.f;
      uint32_t w = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) w |= float_to_e2m1(y[e] * inv) << (4 * e);
      if (live) {
        const int g = c >> 1;
        for (int k = 0; k < p.topk; ++k) {
          if (dr[k] < 0) continue;
          uint8_t* base = p.peers.base[dr[k]];
          const int row = dw[k];
          reinterpret_cast<uint32_t*>(base + p.q_off + static_cast<long long>(row) * (p.h >> 1))[c] = w;
          if ((c & 1) == 0) {
            const int rb = row >> 7, ri = row & 127;
            base[p.sf_off + (static_cast<size_t>(rb) * p.ka + (g >> 2)) * 512 + (ri & 31) * 16 + (ri >> 5) * 4 +
                 (g & 3)] = static_cast<uint8_t>(sfb);
          }
        }
      }
    }
    if (p.gscale != nullptr) {
      // scale groups that pad the last 256-element K tile read as zero
      const int groups = p.h >> 4, groups_pad = p.ka * 4;
      for (int g = groups + threadIdx.x; g < groups_pad; g += T)
        for (int k = 0; k < p.topk; ++k)
          if (dr[k] >= 0) {
            const int row = dw[k], rb = row >> 7, ri = row & 127;
            p.peers.base[dr[k]][p.sf_off + (static_cast<size_t>(rb) * p.ka + (g >> 2)) * 512 + (ri & 31) * 16 +
                                (ri >> 5) * 4 + (g & 3)] = 0;
          }
    }
    if (threadIdx.x < p.topk && dr[threadIdx.x] >= 0)
      reinterpret_cast<int*>(p.peers.base[dr[threadIdx.x]] + p.row_ret_off)[dw[threadIdx.x]] =
          (p.rank << 24) | (t * p.topk + static_cast<int>(threadIdx.x));
  }
  // the last CTA tells every rank that this rank's rows are in place
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&mine->done_dispatch, 1) == static_cast<int>(gridDim.x) - 1) {
      mine->done_dispatch = 0;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        st_release_sys(&reinterpret_cast<EpCtrl*>(p.peers.base[r])->flag_rows[p.rank], seq);
    }
  }
}

// ------------------------------------------------------------------------------------------------ combine
struct CombineParams {
  const float* weights;
  const int* dst_rank;       // pairs that were dropped (-1) contribute nothing
  const __nv_bfloat16* shared;
  long long ld_shared;
  __nv_bfloat16* out;
  long long ldo;
  int tokens, topk, h;
  EpPeers peers;
  int world, rank;
  long long ret_off;
  unsigned long long limit_ns;
  int* status;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(const CombineParams p) {
  __shared__ float ws[EP_MAX_TOPK];
  __shared__ int live[EP_MAX_TOPK];
  __shared__ int ok_s;
  EpCtrl* mine = reinterpret_cast<EpCtrl*>(p.peers.base[p.rank]);
  const int seq = ld_relaxed_sys(&mine->seq) + 1;
  const int t = blockIdx.x;
  const bool ok = wait_flags(mine->flag_ret, p.world, seq, p.limit_ns, p.status, &ok_s);
  if (t < p.tokens) {
    if (threadIdx.x < p.topk) {
      ws[threadIdx.x] = p.weights[static_cast<long long>(t) * p.topk + threadIdx.x];
      live[threadIdx.x] = ok && p.dst_rank[static_cast<long long>(t) * p.topk + threadIdx.x] >= 0;
    }
    __syncthreads();
    const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(p.peers.base[p.rank] + p.ret_off) +
                               static_cast<long long>(t) * p.topk * p.h;
    for (int i = threadIdx.x * 2; i < p.h; i += blockDim.x * 2) {
      float a0 = 0.f, a1 = 0.f;
      for (int k = 0; k < p.topk; ++k) {
        if (!live[k]) continue;
        uint32_t v;   // written by another GPU during this kernel's lifetime: not through the read-only path
        asm volatile("ld.relaxed.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(ret + static_cast<long long>(k) * p.h + i) : "memory");
        a0 += ws[k] * bf16_lo(v);
        a1 += ws[k] * bf16_hi(v);
      }
      if (p.shared != nullptr) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(p.shared + t * p.ld_shared + i);
        a0 += bf16_lo(v);
        a1 += bf16_hi(v);
      }
      *reinterpret_cast<uint32_t*>(p.out + t * p.ldo + i) = pack_bf16(a0, a1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&mine->done_combine, 1) == static_cast<int>(gridDim.x) - 1) {
      mine->done_combine = 0;
      mine->seq = seq;   // the call is complete on this rank
    }
  }
}

}  // namespace
}  // namespace hb

using namespace hb;
#define ST(s) static_cast<cudaStream_t>(s)

static EpPeers make_peers(const void* const* bases, int world) {
  EpPeers p;
  for (int i = 0; i < EP_MAX_WORLD; ++i) p.base[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(bases[i])) : nullptr;
  return p;
}

extern "C" {

int hb_ep_ctrl_bytes(void) { return static_cast<int>(sizeof(EpCtrl)); }
// Byte offsets of {flag_rows, flag_ret, seq, done_fc2} inside the control block.
void hb_ep_ctrl_layout(long long* out4) {
  out4[0] = offsetof(EpCtrl, flag_rows);
  out4[1] = offsetof(EpCtrl, flag_ret);
  out4[2] = offsetof(EpCtrl, seq);
  out4[3] = offsetof(EpCtrl, done_fc2);
}

int hb_ep_count(const void* ids, int pairs, int experts, const void* const* bases, int world, int rank,
                long long cnt_mat_off, void* stream) {
  if (world < 1 || world > EP_MAX_WORLD || experts < 1) return 1;
  ep_count_kernel<<<1, 1024, experts * sizeof(int), ST(stream)>>>(static_cast<const int*>(ids), pairs, experts,
                                                                 make_peers(bases, world), world, rank, cnt_mat_off);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_ep_plan(const void* ids, int pairs, int experts, const void* const* bases, int world, int rank,
               long long cnt_mat_off, int rows_cap, void* grp_cnt, void* grp_start, void* total_rows, void* dst_rank,
               void* dst_row, long long limit_ns, void* status, void* stream) {
  if (world < 1 || world > EP_MAX_WORLD || experts % world != 0) return 1;
  const size_t smem = (static_cast<size_t>(world) + 3) * experts * sizeof(int);
  if (smem > 48 * 1024) {
    static bool attr = false;
    if (!attr) {
      if (cudaFuncSetAttribute(ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
        return 3;
      attr = true;
    }
    if (smem > 160 * 1024) return 1;
  }
  ep_plan_kernel<<<1, 1024, smem, ST(stream)>>>(
      static_cast<const int*>(ids), pairs, experts, experts / world, make_peers(bases, world), world, rank,
      cnt_mat_off, rows_cap, static_cast<int*>(grp_cnt), static_cast<int*>(grp_start), static_cast<int*>(total_rows),
      static_cast<int*>(dst_rank), static_cast<int*>(dst_row), static_cast<unsigned long long>(limit_ns),
      static_cast<int*>(status));
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// gscale null: rows travel as bf16 into the buffer at bf_off; else as NVFP4 (q_off, sf_off with `ka` K atoms).
int hb_ep_dispatch(const void* x, long long ldx, int tokens, int topk, int h, int ka, const void* dst_rank,
                   const void* dst_row, const void* gscale, const void* const* bases, int world, int rank,
                   long long q_off, long long sf_off, long long bf_off, long long row_ret_off, void* stream) {
  if (topk > EP_MAX_TOPK || (h & 15) || world > EP_MAX_WORLD) return 1;
  DispatchParams p;
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx; p.tokens = tokens; p.topk = topk; p.h = h; p.ka = ka;
  p.dst_rank = static_cast<const int*>(dst_rank); p.dst_row = static_cast<const int*>(dst_row);
  p.gscale = static_cast<const float*>(gscale); p.peers = make_peers(bases, world); p.world = world; p.rank = rank;
  p.q_off = q_off; p.sf_off = sf_off; p.bf_off = bf_off; p.row_ret_off = row_ret_off;
  ep_dispatch_kernel<256><<<tokens > 0 ? tokens : 1, 256, 0, ST(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_ep_combine(const void* weights, const void* dst_rank, const void* shared, long long ld_shared, void* out,
                  long long ldo, int tokens, int topk, int h, const void* const* bases, int world, int rank,
                  long long ret_off, long long limit_ns, void* status, void* stream) {
  if (topk > EP_MAX_TOPK || (h & 1) || world > EP_MAX_WORLD) return 1;
  CombineParams p;
  p.weights = static_cast<const float*>(weights); p.dst_rank = static_cast<const int*>(dst_rank);
  p.shared = static_cast<const __nv_bfloat16*>(shared); p.ld_shared = ld_shared;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo; p.tokens = tokens; p.topk = topk; p.h = h;
  p.peers = make_peers(bases, world); p.world = world; p.rank = rank; p.ret_off = ret_off;
  p.limit_ns = static_cast<unsigned long long>(limit_ns); p.status = static_cast<int*>(status);
  ep_combine_kernel<<<tokens > 0 ? tokens : 1, 256, 0, ST(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
