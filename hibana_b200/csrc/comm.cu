// NVLink peer-memory communicator for one NVSwitch box: symmetric heap + fused collective kernels.
//
// Every rank cudaMallocs one heap and maps every peer's heap through CUDA IPC, so kernels reach peer memory with
// plain loads and stores over NVLink. The heap starts with a control block (per-slot arrival flags, per-slot
// sequence numbers, completion counters) followed by NSLOT data slots. Collectives are sequence-numbered per slot
// entirely on the device, so a captured CUDA graph replays them without host involvement.
//
//   hb_ar_norm : one-shot all-reduce of a [rows, H] bf16 partial that already sits in this rank's slot (the
//                producing GEMM writes there), fused with residual add, RMSNorm and optionally NVFP4 quantisation
//                of the next GEMM's input. Every rank sums the world's partials in rank order, so all ranks get
//                bitwise identical results (what lets tensor-parallel ranks sample without exchanging tokens).
//   hb_barrier : flag barrier over the same slots.
//
// Every wait on a peer is bounded (nanosecond limit passed per launch): on expiry the kernel records
// kTimeoutPeer in the status word, skips the dependent math and returns; the context stays usable.
// Replaces the reference's two-rank host-proxied RDMA one-shot (hibana/kernels/csrc/rdma_oneshot.cu:66-295) and the
// separate residual+norm kernel that follows it (hibana/kernels/cute/residual_norm.py).
#include "hb_api.h"
#include "hb_common.cuh"
#include <cstddef>

namespace hb {
namespace {

constexpr int MAX_WORLD = 8;
constexpr int NSLOT = 8;
constexpr int CTRL_BYTES = 4096;

// Control block at the start of every rank's heap.
struct Ctrl {
  int flags[NSLOT][MAX_WORLD];   // flags[slot][src] = sequence number src has published for this slot
  int seq[NSLOT];                // sequence number of the last completed collective on this slot
  int done[NSLOT];               // CTAs of the running collective that have finished
  // sequence-parallel prefill chain (GEMM -> reduce-scatter -> norm -> all-gather -> GEMM)
  int sp_cnt[MAX_WORLD];         // sp_cnt[src]: tiles of the running scatter that rank src has delivered (monotonic)
  int sp_flag[MAX_WORLD];        // sp_flag[src]: gather sequence number rank src has pushed its rows for
  int sp_seq_scatter;            // scatters completed on this rank
  int sp_seq_gather;             // gathers this rank has pushed
  int sp_done;                   // CTAs of the running reduce kernel that have finished
  int pad[13];
};
static_assert(sizeof(Ctrl) <= CTRL_BYTES, "control block too large");

struct Peers {
  uint8_t* base[MAX_WORLD];
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

// Publishes `seq` to every peer's flags[slot][rank] (threads 0..world-1 of the calling CTA).
__device__ __forceinline__ void signal_peers(const Peers& peers, int world, int rank, int slot, int seq) {
  if (threadIdx.x < world) {
    Ctrl* c = reinterpret_cast<Ctrl*>(peers.base[threadIdx.x]);
    st_release_sys(&c->flags[slot][rank], seq);
  }
}
// Waits until every rank has published `seq` on this rank's flags[slot]. Returns false on timeout.
__device__ __forceinline__ bool wait_peers(Ctrl* mine, int world, int slot, int seq, unsigned long long limit_ns,
                                           int* status, int* ok_smem) {
  if (threadIdx.x == 0) *ok_smem = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const unsigned long long t0 = globaltimer_ns();
    bool ok = false;
    for (unsigned it = 0; it < HB_SPIN_LIMIT; ++it) {
      if (ld_relaxed_sys(&mine->flags[slot][threadIdx.x]) - seq >= 0) {
        ok = true;
        break;
      }
      if ((it & 63u) == 63u && globaltimer_ns() - t0 > limit_ns) break;
    }
    __threadfence_system();   // acquire: order the peer data reads after the flag observation
    if (!ok) {
      *ok_smem = 0;
      set_status(status, kTimeoutPeer);
    }
  }
  __syncthreads();
  return *ok_smem != 0;
}

struct ArNormParams {
  Peers peers;
  int world, rank, slot;
  long long data_offset;        // byte offset of the partial inside every rank's heap (same on all ranks)
  int rows, h;
  __nv_bfloat16* residual;      // [rows, h] updated in place (may be null: no residual)
  const __nv_bfloat16* weight;  // RMSNorm weight (null: no norm, output = reduced sum (+ residual))
  float eps;
  int gemma;
  __nv_bfloat16* out;           // normed (or summed) output bf16 (may be null when only the quantised form is used)
  uint8_t* q;                   // optional NVFP4 output
  uint8_t* sf;
  const float* gscale;
  int ka;
  unsigned long long limit_ns;
  int* status;
};

__device__ __forceinline__ size_t sf_off(int row, int g, int ka) {
  const int rb = row >> 7, ri = row & 127;
  return (static_cast<size_t>(rb) * ka + (g >> 2)) * 512 + (ri & 31) * 16 + (ri >> 5) * 4 + (g & 3);
}

// One CTA per row. Thread t owns 16-element groups t, t + T, ...
template <int T>
__global__ void __launch_bounds__(T) ar_norm_kernel(const ArNormParams p) {
  extern __shared__ float row_s[];   // h floats
  __shared__ float red[32];
  __shared__ int ok_s;
  Ctrl* mine = reinterpret_cast<Ctrl*>(p.peers.base[p.rank]);
  const int seq = ld_relaxed_sys(&mine->seq[p.slot]) + 1;
  const int row = blockIdx.x;
  if (blockIdx.x == 0) signal_peers(p.peers, p.world, p.rank, p.slot, seq);
  const bool ok = wait_peers(mine, p.world, p.slot, seq, p.limit_ns, p.status, &ok_s);
  const int groups = p.h / 16;
  const int rows_pad = p.q ? ((p.rows + 127) / 128) * 128 : p.rows;
  if (ok && row < p.rows) {
    float ss = 0.f;
    for (int g = threadIdx.x; g < groups; g += T) {
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.f;
      for (int r = 0; r < p.world; ++r) {   // fixed rank order: bitwise identical on every rank
        const uint4* src = reinterpret_cast<const uint4*>(p.peers.base[r] + p.data_offset +
                                                          (static_cast<size_t>(row) * p.h + g * 16) * 2);
        const uint4 a = src[0], b = src[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[2 * i] += bf16_lo(w[i]);
          acc[2 * i + 1] += bf16_hi(w[i]);
        }
      }
      if (p.residual != nullptr) {
        uint4* rp = reinterpret_cast<uint4*>(p.residual + static_cast<size_t>(row) * p.h + g * 16);
        const uint4 a = rp[0], b = rp[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          // the reduced sum is rounded to bf16 first, like an unfused all-reduce followed by add
          const float s0 = __bfloat162float(__float2bfloat16(acc[2 * i])) + bf16_lo(w[i]);
          const float s1 = __bfloat162float(__float2bfloat16(acc[2 * i + 1])) + bf16_hi(w[i]);
          o[i] = pack_bf16(s0, s1);
          acc[2 * i] = bf16_lo(o[i]);
          acc[2 * i + 1] = bf16_hi(o[i]);
        }
        rp[0] = make_uint4(o[0], o[1], o[2], o[3]);
        rp[1] = make_uint4(o[4], o[5], o[6], o[7]);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = __bfloat162float(__float2bfloat16(acc[i]));
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        row_s[g * 16 + i] = acc[i];
        ss += acc[i] * acc[i];
      }
    }
    float rstd = 1.f;
    if (p.weight != nullptr) {
      ss = warp_sum(ss);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < T / 32 ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) red[0] = rsqrtf(t / p.h + p.eps);
      }
      __syncthreads();
      rstd = red[0];
    } else {
      __syncthreads();
    }
    const float inv_gs = p.q ? 1.f / *p.gscale : 0.f;
    const int groups_pad = p.q ? p.ka * 4 : groups;
    for (int g = threadIdx.x; g < groups_pad; g += T) {
      if (g >= groups) {
        p.sf[sf_off(row, g, p.ka)] = 0;
        continue;
      }
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float x = row_s[g * 16 + i];
        if (p.weight != nullptr) {
          const float w = __bfloat162float(p.weight[g * 16 + i]);
          x = x * rstd * (p.gemma ? 1.f + w : w);
        }
        v[i] = __bfloat162float(__float2bfloat16(x));
      }
      if (p.out != nullptr) {
        uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(row) * p.h + g * 16);
        dst[0] = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        dst[1] = make_uint4(pack_bf16(v[8], v[9]), pack_bf16(v[10], v[11]), pack_bf16(v[12], v[13]),
                            pack_bf16(v[14], v[15]));
      }
      if (p.q != nullptr) {
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
        const uint32_t sfb = float_to_e4m3(amax * (1.f / 6.f) * inv_gs);
        const float sfv = e4m3_to_float(sfb);
        const float inv = sfv > 0.f ? 1.f / (sfv * (1.f / inv_gs)) : 0.f;
        uint32_t w[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i >> 3] |= float_to_e2m1(v[i] * inv) << (4 * (i & 7));
        *reinterpret_cast<uint2*>(p.q + static_cast<size_t>(row) * (p.h / 2) + g * 8) = make_uint2(w[0], w[1]);
        p.sf[sf_off(row, g, p.ka)] = static_cast<uint8_t>(sfb);
      }
    }
  } else if (ok && p.q != nullptr && row < rows_pad) {
    for (int g = threadIdx.x; g < p.ka * 4; g += T) p.sf[sf_off(row, g, p.ka)] = 0;   // scale padding rows
  }
  // The last CTA to finish completes the collective on this slot.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(&mine->done[p.slot], 1);
    if (prev == static_cast<int>(gridDim.x) - 1) {
      mine->done[p.slot] = 0;
      __threadfence();
      mine->seq[p.slot] = seq;
    }
  }
}

struct RsNormAgParams {
  Peers peers;
  int world, rank, rows_per_rank, h;
  long long stage_offset;       // [world][rows_per_rank][h] bf16 partials delivered by the GEMM epilogues
  int expected;                 // tile arrivals per source and scatter
  __nv_bfloat16* residual;      // [rows_per_rank, h] this rank's rows of the residual stream (updated in place)
  const __nv_bfloat16* weight;
  float eps;
  int gemma;
  long long gather_q_offset;    // NVFP4: packed rows [world * rows_per_rank, h / 2] in every heap (-1 = off)
  long long gather_sf_offset;   //        swizzled scale blocks
  long long gather_bf_offset;   // bf16 rows [world * rows_per_rank, h] in every heap (-1 = off)
  const float* gscale;
  int ka;
  unsigned long long limit_ns;
  int* status;
};

// One CTA per owned row: waits for every source's tiles, sums the partials in rank order, adds the residual,
// normalises, quantises and pushes the row into every rank's gather buffer; the last CTA publishes the flag.
template <int T>
__global__ void __launch_bounds__(T) rs_norm_ag_kernel(const RsNormAgParams p) {
  extern __shared__ float row_s[];
  __shared__ float red[32];
  __shared__ int ok_s;
  Ctrl* mine = reinterpret_cast<Ctrl*>(p.peers.base[p.rank]);
  const int sseq = ld_relaxed_sys(&mine->sp_seq_scatter) + 1;
  const int gseq = ld_relaxed_sys(&mine->sp_seq_gather) + 1;
  const int row = blockIdx.x;                       // local (owned) row
  const int grow = p.rank * p.rows_per_rank + row;  // global row
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const long long want = static_cast<long long>(sseq) * p.expected;
    const unsigned long long t0 = globaltimer_ns();
    bool ok = false;
    for (unsigned it = 0; it < HB_SPIN_LIMIT; ++it) {
      if (ld_relaxed_sys(&mine->sp_cnt[threadIdx.x]) >= want) {
        ok = true;
        break;
      }
      if ((it & 63u) == 63u && globaltimer_ns() - t0 > p.limit_ns) break;
    }
    __threadfence_system();
    if (!ok) {
      ok_s = 0;
      set_status(p.status, kTimeoutPeer);
    }
  }
  __syncthreads();
  const bool ok = ok_s != 0;
  const int groups = p.h / 16;
  if (ok) {
    float ss = 0.f;
    const uint8_t* stage = p.peers.base[p.rank] + p.stage_offset;
    for (int g = threadIdx.x; g < groups; g += T) {
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.f;
      for (int r = 0; r < p.world; ++r) {
        const uint4* src = reinterpret_cast<const uint4*>(
            stage + ((static_cast<size_t>(r) * p.rows_per_rank + row) * p.h + g * 16) * 2);
        const uint4 a = src[0], b = src[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          acc[2 * i] += bf16_lo(w[i]);
          acc[2 * i + 1] += bf16_hi(w[i]);
        }
      }
      uint4* rp = reinterpret_cast<uint4*>(p.residual + static_cast<size_t>(row) * p.h + g * 16);
      const uint4 a = rp[0], b = rp[1];
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float s0 = __bfloat162float(__float2bfloat16(acc[2 * i])) + bf16_lo(w[i]);
        const float s1 = __bfloat162float(__float2bfloat16(acc[2 * i + 1])) + bf16_hi(w[i]);
        o[i] = pack_bf16(s0, s1);
        acc[2 * i] = bf16_lo(o[i]);
        acc[2 * i + 1] = bf16_hi(o[i]);
      }
      rp[0] = make_uint4(o[0], o[1], o[2], o[3]);
      rp[1] = make_uint4(o[4], o[5], o[6], o[7]);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        row_s[g * 16 + i] = acc[i];
        ss += acc[i] * acc[i];
      }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < T / 32 ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) red[0] = rsqrtf(t / p.h + p.eps);
    }
    __syncthreads();
    const float rstd = red[0];
    const float inv_gs = p.gather_q_offset >= 0 ? 1.f / *p.gscale : 0.f;
    const int groups_pad = p.gather_q_offset >= 0 ? p.ka * 4 : groups;
    for (int g = threadIdx.x; g < groups_pad; g += T) {
      if (g >= groups) {
        for (int r = 0; r < p.world; ++r) (p.peers.base[r] + p.gather_sf_offset)[sf_off(grow, g, p.ka)] = 0;
        continue;
      }
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float w = __bfloat162float(p.weight[g * 16 + i]);
        v[i] = __bfloat162float(__float2bfloat16(row_s[g * 16 + i] * rstd * (p.gemma ? 1.f + w : w)));
      }
      if (p.gather_bf_offset >= 0) {
        const uint4 lo = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
        const uint4 hi = make_uint4(pack_bf16(v[8], v[9]), pack_bf16(v[10], v[11]), pack_bf16(v[12], v[13]), pack_bf16(v[14], v[15]));
        for (int r = 0; r < p.world; ++r) {
          uint4* dst = reinterpret_cast<uint4*>(p.peers.base[r] + p.gather_bf_offset +
                                                (static_cast<size_t>(grow) * p.h + g * 16) * 2);
          dst[0] = lo;
          dst[1] = hi;
        }
      }
      if (p.gather_q_offset >= 0) {
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
        const uint32_t sfb = float_to_e4m3(amax * (1.f / 6.f) * inv_gs);
        const float sfv = e4m3_to_float(sfb);
        const float inv = sfv > 0.f ? 1.f / (sfv * (1.f / inv_gs)) : 0.f;
        uint32_t w[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i >> 3] |= float_to_e2m1(v[i] * inv) << (4 * (i & 7));
        const uint2 packed = make_uint2(w[0], w[1]);
        const size_t so = sf_off(grow, g, p.ka);
        for (int r = 0; r < p.world; ++r) {
          *reinterpret_cast<uint2*>(p.peers.base[r] + p.gather_q_offset + static_cast<size_t>(grow) * (p.h / 2) + g * 8) = packed;
          (p.peers.base[r] + p.gather_sf_offset)[so] = static_cast<uint8_t>(sfb);
        }
      }
    }
  }
  // The last CTA publishes this rank's rows to every peer and completes both sequence numbers.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&mine->sp_done, 1);
    ok_s = prev == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (ok_s) {
    if (threadIdx.x < p.world) {
      Ctrl* c = reinterpret_cast<Ctrl*>(p.peers.base[threadIdx.x]);
      st_release_sys(&c->sp_flag[p.rank], gseq);
    }
    if (threadIdx.x == 0) {
      mine->sp_done = 0;
      mine->sp_seq_scatter = sseq;
      mine->sp_seq_gather = gseq;
    }
  }
}

struct BarrierParams {
  Peers peers;
  int world, rank, slot;
  unsigned long long limit_ns;
  int* status;
};

__global__ void barrier_kernel(const BarrierParams p) {
  __shared__ int ok_s;
  Ctrl* mine = reinterpret_cast<Ctrl*>(p.peers.base[p.rank]);
  const int seq = ld_relaxed_sys(&mine->seq[p.slot]) + 1;
  __threadfence_system();
  signal_peers(p.peers, p.world, p.rank, p.slot, seq);
  wait_peers(mine, p.world, p.slot, seq, p.limit_ns, p.status, &ok_s);
  if (threadIdx.x == 0) mine->seq[p.slot] = seq;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

int hb_comm_ctrl_bytes(void) { return CTRL_BYTES; }
int hb_comm_nslot(void) { return NSLOT; }

// Allocates a zeroed heap with cudaMalloc and returns its device pointer through *out.
int hb_comm_alloc(long long bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  *out = p;
  return 0;
}
int hb_comm_free(void* p) { return static_cast<int>(cudaFree(p)); }
// 64-byte IPC handle of a heap allocated by hb_comm_alloc.
int hb_comm_ipc_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
int hb_comm_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return static_cast<int>(e);
  *out = p;
  return 0;
}
int hb_comm_ipc_close(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

// peer_bases: host array of `world` heap base pointers as seen from this process (own heap at index rank).
int hb_ar_norm(const void* const* peer_bases, int world, int rank, int slot, long long data_offset, int rows, int h,
               void* residual, const void* weight, float eps, int gemma, void* out, void* q, void* sf,
               const void* gscale, int ka, long long limit_ns, void* status, void* stream) {
  if (world < 1 || world > MAX_WORLD || slot < 0 || slot >= NSLOT || h % 16 != 0 || rows <= 0) return 1;
  if (static_cast<size_t>(h) * sizeof(float) > 96 * 1024) return 1;
  ArNormParams p;
  for (int i = 0; i < MAX_WORLD; ++i)
    p.peers.base[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(peer_bases[i])) : nullptr;
  p.world = world; p.rank = rank; p.slot = slot; p.data_offset = data_offset; p.rows = rows; p.h = h;
  p.residual = static_cast<__nv_bfloat16*>(residual);
  p.weight = static_cast<const __nv_bfloat16*>(weight);
  p.eps = eps; p.gemma = gemma;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q = static_cast<uint8_t*>(q); p.sf = static_cast<uint8_t*>(sf);
  p.gscale = static_cast<const float*>(gscale); p.ka = ka;
  p.limit_ns = static_cast<unsigned long long>(limit_ns);
  p.status = static_cast<int*>(status);
  constexpr int T = 256;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(ar_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    attr = true;
  }
  // The caller keeps persistent output buffers whose padding scale rows were zeroed once, so only real rows run.
  ar_norm_kernel<T><<<rows, T, h * sizeof(float), static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_barrier(const void* const* peer_bases, int world, int rank, int slot, long long limit_ns, void* status,
               void* stream) {
  if (world < 1 || world > MAX_WORLD || slot < 0 || slot >= NSLOT) return 1;
  BarrierParams p;
  for (int i = 0; i < MAX_WORLD; ++i)
    p.peers.base[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(peer_bases[i])) : nullptr;
  p.world = world; p.rank = rank; p.slot = slot;
  p.limit_ns = static_cast<unsigned long long>(limit_ns);
  p.status = static_cast<int*>(status);
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Offsets inside the control block: {sp_cnt, sp_flag, sp_seq_gather} in bytes.
int hb_comm_sp_layout(long long* out3) {
  out3[0] = offsetof(Ctrl, sp_cnt);
  out3[1] = offsetof(Ctrl, sp_flag);
  out3[2] = offsetof(Ctrl, sp_seq_gather);
  return 0;
}

int hb_rs_norm_ag(const void* const* peer_bases, int world, int rank, int rows_per_rank, int h, long long stage_offset,
                  int expected, void* residual, const void* weight, float eps, int gemma, long long gather_q_offset,
                  long long gather_sf_offset, long long gather_bf_offset, const void* gscale, int ka,
                  long long limit_ns, void* status, void* stream) {
  if (world < 1 || world > MAX_WORLD || h % 16 != 0 || rows_per_rank <= 0) return 1;
  if (static_cast<size_t>(h) * sizeof(float) > 96 * 1024) return 1;
  RsNormAgParams p;
  for (int i = 0; i < MAX_WORLD; ++i)
    p.peers.base[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(peer_bases[i])) : nullptr;
  p.world = world; p.rank = rank; p.rows_per_rank = rows_per_rank; p.h = h; p.stage_offset = stage_offset;
  p.expected = expected; p.residual = static_cast<__nv_bfloat16*>(residual);
  p.weight = static_cast<const __nv_bfloat16*>(weight); p.eps = eps; p.gemma = gemma;
  p.gather_q_offset = gather_q_offset; p.gather_sf_offset = gather_sf_offset; p.gather_bf_offset = gather_bf_offset;
  p.gscale = static_cast<const float*>(gscale); p.ka = ka;
  p.limit_ns = static_cast<unsigned long long>(limit_ns); p.status = static_cast<int*>(status);
  constexpr int T = 256;
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(rs_norm_ag_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    attr = true;
  }
  rs_norm_ag_kernel<T><<<rows_per_rank, T, h * sizeof(float), static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
