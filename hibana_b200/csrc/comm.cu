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
#include "rownorm.cuh"
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
  int sp_target;                 // tile arrivals every source owes after the scatters completed so far
  int pick_seq;                  // vocab-parallel (value, index) exchanges completed on this rank
  int pad[11];
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
    for (unsigned long long it = 0, cap = spin_cap(limit_ns); it < cap; ++it) {
      if (ld_acquire_sys(&mine->flags[slot][threadIdx.x]) - seq >= 0) {
        ok = true;
        break;
      }
      // once any wait of this job has timed out, later waits give up at their first check instead of each
      // spending the full limit (thousands of CTAs x the limit would look like a hang)
      if ((it & 63u) == 63u && (globaltimer_ns() - t0 > limit_ns || *reinterpret_cast<volatile int*>(status) != 0)) break;
    }
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

// One CTA per row on the register-resident row core: all peers' chunks of the row are loaded at once.
template <int T, int MAXC>
__global__ void __launch_bounds__(T) ar_norm_kernel(const ArNormParams p) {
  __shared__ float red[40];
  __shared__ int ok_s;
  Ctrl* mine = reinterpret_cast<Ctrl*>(p.peers.base[p.rank]);
  const int seq = ld_relaxed_sys(&mine->seq[p.slot]) + 1;
  const int row = blockIdx.x;
  if (blockIdx.x == 0) signal_peers(p.peers, p.world, p.rank, p.slot, seq);
  const bool ok = wait_peers(mine, p.world, p.slot, seq, p.limit_ns, p.status, &ok_s);
  const int nchunk = p.h >> 3;
  if (ok) {
    float v[MAXC][8];
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = threadIdx.x + i * T;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
      if (c < nchunk) {
        uint4 part[MAX_WORLD];
#pragma unroll
        for (int r = 0; r < MAX_WORLD; ++r)
          if (r < p.world)
            part[r] = reinterpret_cast<const uint4*>(p.peers.base[r] + p.data_offset +
                                                     static_cast<size_t>(row) * p.h * 2)[c];
#pragma unroll
        for (int r = 0; r < MAX_WORLD; ++r)     // fixed rank order: bitwise identical on every rank
          if (r < p.world) {
            float f[8];
            unpack8(part[r], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[i][e] += f[e];
          }
        // the reduced sum is rounded to bf16 first, like an unfused all-reduce followed by an add
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16(v[i][e]));
        if (p.residual != nullptr) {
          uint4* rp = reinterpret_cast<uint4*>(p.residual + static_cast<size_t>(row) * p.h) + c;
          float f[8];
          unpack8(*rp, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16(v[i][e] + f[e]));
          *rp = pack8(v[i]);
        }
      }
    }
    RowOut out;
    out.n = 1;
    out.q[0] = p.q; out.sf[0] = p.sf; out.bf[0] = p.out;
    row_finish<T, MAXC>(v, p.h, p.weight, p.eps, p.gemma, red, out, row, p.ka, p.gscale);
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

// Low-latency variant for small messages: every rank pushes its partial into all peers as 8-byte words
// {two bf16 values, sequence number}; the receiver spins on the words themselves, so a collective costs one
// one-way NVLink hop and needs neither flags nor fences. The LL area of a slot is ll[src][row][h / 2] words and
// lives at `ll_offset` in every heap; stale words carry an older sequence number and are never mistaken for data.
struct ArNormLlParams {
  ArNormParams base;
  long long ll_offset;
  int ll_rows;                  // row capacity of the LL area (stride between sources)
};

template <int T, int MAXC>
__global__ void __launch_bounds__(T) ar_norm_ll_kernel(const ArNormLlParams pp) {
  const ArNormParams& p = pp.base;
  __shared__ float red[40];
  __shared__ int bad_s;
  Ctrl* mine = reinterpret_cast<Ctrl*>(p.peers.base[p.rank]);
  const int seq = ld_relaxed_sys(&mine->seq[p.slot]) + 1;
  const int row = blockIdx.x;
  const int nchunk = p.h >> 3;
  if (threadIdx.x == 0) bad_s = 0;
  // ---- push my chunks to every other rank
  uint4 own[MAXC];
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = threadIdx.x + i * T;
    if (c < nchunk) {
      own[i] = reinterpret_cast<const uint4*>(p.peers.base[p.rank] + p.data_offset + static_cast<size_t>(row) * p.h * 2)[c];
      const size_t word = (static_cast<size_t>(p.rank) * pp.ll_rows + row) * (p.h >> 1) + static_cast<size_t>(c) * 4;
      for (int d = 0; d < p.world; ++d) {
        if (d == p.rank) continue;
        uint2* dst = reinterpret_cast<uint2*>(p.peers.base[d] + pp.ll_offset) + word;
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(own[i].x), "r"(seq) : "memory");
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst + 1), "r"(own[i].y), "r"(seq) : "memory");
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst + 2), "r"(own[i].z), "r"(seq) : "memory");
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst + 3), "r"(own[i].w), "r"(seq) : "memory");
      }
    }
  }
  __syncthreads();
  // ---- collect every source's chunks (spin on the data words), sum in rank order
  float v[MAXC][8];
  const unsigned long long t0 = globaltimer_ns();
#pragma unroll
  for (int i = 0; i < MAXC; ++i) {
    const int c = threadIdx.x + i * T;
#pragma unroll
    for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
    if (c < nchunk) {
      for (int r = 0; r < p.world; ++r) {
        uint4 part = own[i];
        if (r != p.rank) {
          const uint2* src = reinterpret_cast<const uint2*>(p.peers.base[p.rank] + pp.ll_offset) +
                             (static_cast<size_t>(r) * pp.ll_rows + row) * (p.h >> 1) + static_cast<size_t>(c) * 4;
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint32_t data = 0, flag = 0;
            bool got = false;
            for (unsigned long long it = 0, cap = spin_cap(p.limit_ns); it < cap; ++it) {
              asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(data), "=r"(flag) : "l"(src + k) : "memory");
              if (static_cast<int>(flag) == seq) {
                got = true;
                break;
              }
              if ((it & 255u) == 255u && (bad_s || globaltimer_ns() - t0 > p.limit_ns ||
                                          *reinterpret_cast<volatile int*>(p.status) != 0))
                break;
            }
            if (!got) {
              bad_s = 1;
              set_status(p.status, kTimeoutLowLatency);
            }
            w[k] = data;
          }
          part = make_uint4(w[0], w[1], w[2], w[3]);
        }
        float f[8];
        unpack8(part, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += f[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16(v[i][e]));
      if (p.residual != nullptr) {
        uint4* rp = reinterpret_cast<uint4*>(p.residual + static_cast<size_t>(row) * p.h) + c;
        float f[8];
        unpack8(*rp, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16(v[i][e] + f[e]));
        *rp = pack8(v[i]);
      }
    }
  }
  RowOut out;
  out.n = 1;
  out.q[0] = p.q; out.sf[0] = p.sf; out.bf[0] = p.out;
  row_finish<T, MAXC>(v, p.h, p.weight, p.eps, p.gemma, red, out, row, p.ka, p.gscale);
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
template <int T, int MAXC>
__global__ void __launch_bounds__(T) rs_norm_ag_kernel(const RsNormAgParams p) {
  __shared__ float red[40];
  __shared__ int ok_s;
  Ctrl* mine = reinterpret_cast<Ctrl*>(p.peers.base[p.rank]);
  const int sseq = ld_relaxed_sys(&mine->sp_seq_scatter) + 1;
  const int gseq = ld_relaxed_sys(&mine->sp_seq_gather) + 1;
  const int row = blockIdx.x;                       // local (owned) row
  const int grow = p.rank * p.rows_per_rank + row;  // global row
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    // cumulative, so calls with different row counts can follow one another
    const int want = ld_relaxed_sys(&mine->sp_target) + p.expected;
    const unsigned long long t0 = globaltimer_ns();
    bool ok = false;
    for (unsigned long long it = 0, cap = spin_cap(p.limit_ns); it < cap; ++it) {
      if (ld_relaxed_sys(&mine->sp_cnt[threadIdx.x]) - want >= 0) {
        ok = true;
        break;
      }
      if ((it & 63u) == 63u && (globaltimer_ns() - t0 > p.limit_ns || *reinterpret_cast<volatile int*>(p.status) != 0)) break;
    }
    __threadfence_system();
    if (!ok) {
      ok_s = 0;
      set_status(p.status, kTimeoutCounter);
    }
  }
  __syncthreads();
  const int nchunk = p.h >> 3;
  if (ok_s) {
    float v[MAXC][8];
    const uint8_t* stage = p.peers.base[p.rank] + p.stage_offset;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = threadIdx.x + i * T;
#pragma unroll
      for (int e = 0; e < 8; ++e) v[i][e] = 0.f;
      if (c < nchunk) {
        uint4 part[MAX_WORLD];
#pragma unroll
        for (int r = 0; r < MAX_WORLD; ++r)
          if (r < p.world)
            part[r] = reinterpret_cast<const uint4*>(stage + (static_cast<size_t>(r) * p.rows_per_rank + row) * p.h * 2)[c];
        uint4* rp = reinterpret_cast<uint4*>(p.residual + static_cast<size_t>(row) * p.h) + c;
        const uint4 rv = *rp;
#pragma unroll
        for (int r = 0; r < MAX_WORLD; ++r)
          if (r < p.world) {
            float f[8];
            unpack8(part[r], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[i][e] += f[e];
          }
        float f[8];
        unpack8(rv, f);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          v[i][e] = __bfloat162float(__float2bfloat16(__bfloat162float(__float2bfloat16(v[i][e])) + f[e]));
        *rp = pack8(v[i]);
      }
    }
    RowOut out;
    out.n = p.world;
    for (int r = 0; r < ROW_MAX_DST; ++r) {
      const bool on = r < p.world;
      out.q[r] = on && p.gather_q_offset >= 0 ? p.peers.base[r] + p.gather_q_offset : nullptr;
      out.sf[r] = on && p.gather_q_offset >= 0 ? p.peers.base[r] + p.gather_sf_offset : nullptr;
      out.bf[r] = on && p.gather_bf_offset >= 0
                      ? reinterpret_cast<__nv_bfloat16*>(p.peers.base[r] + p.gather_bf_offset) : nullptr;
    }
    row_finish<T, MAXC>(v, p.h, p.weight, p.eps, p.gemma, red, out, grow, p.ka, p.gscale);
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
      mine->sp_target += p.expected;
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

// Vocab-parallel greedy pick: every rank holds, per row, the best (logit, global token id) of its vocabulary shard.
// Each rank pushes its pairs into every peer's landing area as two 8-byte words {payload, sequence number} (the
// low-latency protocol: the receiver spins on the words themselves), then takes the best of the world's pairs in
// (value desc, id asc) order, which is the same choice on every rank. 16 bytes per row and rank cross NVLink
// instead of the rows x vocabulary fp32 logits of an all-gather.
struct PickParams {
  Peers peers;
  int world, rank, rows, rows_cap;
  long long area_offset;          // landing area [world][rows_cap] x 16 bytes in every heap
  const float* val;               // [rows] best local logit
  const long long* idx;           // [rows] its id inside the shard
  long long idx_offset;           // first global id of this rank's shard
  long long* out;                 // [rows] global id of the world's best
  unsigned long long limit_ns;
  int* status;
};

__global__ void __launch_bounds__(256) pick_exchange_kernel(const PickParams p) {
  Ctrl* mine = reinterpret_cast<Ctrl*>(p.peers.base[p.rank]);
  const int seq = ld_relaxed_sys(&mine->pick_seq) + 1;
  const unsigned long long t0 = globaltimer_ns();
  for (int row = threadIdx.x; row < p.rows; row += blockDim.x) {
    float best = p.val[row];
    long long bi = p.idx[row] + p.idx_offset;
    const size_t slot = static_cast<size_t>(p.rank) * p.rows_cap + row;
    for (int d = 0; d < p.world; ++d) {
      if (d == p.rank) continue;
      uint2* dst = reinterpret_cast<uint2*>(p.peers.base[d] + p.area_offset) + slot * 2;
      asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(best)), "r"(seq) : "memory");
      asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst + 1), "r"(static_cast<unsigned>(bi)), "r"(seq) : "memory");
    }
    for (int r = 0; r < p.world; ++r) {
      if (r == p.rank) continue;
      const uint2* src = reinterpret_cast<const uint2*>(p.peers.base[p.rank] + p.area_offset) +
                         (static_cast<size_t>(r) * p.rows_cap + row) * 2;
      unsigned w[2] = {0, 0};
      bool ok = true;
      for (int k = 0; k < 2 && ok; ++k) {
        ok = false;
        for (unsigned long long it = 0, cap = spin_cap(p.limit_ns); it < cap; ++it) {
          unsigned data, flag;
          asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(data), "=r"(flag) : "l"(src + k) : "memory");
          if (static_cast<int>(flag) == seq) {
            w[k] = data;
            ok = true;
            break;
          }
          if ((it & 255u) == 255u &&
              (globaltimer_ns() - t0 > p.limit_ns || *reinterpret_cast<volatile int*>(p.status) != 0))
            break;
        }
      }
      if (!ok) {
        set_status(p.status, kTimeoutLowLatency);
        continue;
      }
      const float v = __uint_as_float(w[0]);
      const long long i = static_cast<long long>(w[1]);
      if (v > best || (v == best && i < bi)) {
        best = v;
        bi = i;
      }
    }
    p.out[row] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) mine->pick_seq = seq;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

// Vocab-parallel greedy pick (see pick_exchange_kernel). rows <= rows_cap; area_offset + world * rows_cap * 16 bytes
// must lie inside every heap and must not be a slot another collective writes.
int hb_pick_exchange(const void* const* peer_bases, int world, int rank, int rows, int rows_cap, long long area_offset,
                     const void* val, const void* idx, long long idx_offset, void* out, long long limit_ns,
                     void* status, void* stream) {
  if (world < 1 || world > MAX_WORLD || rows <= 0 || rows > rows_cap) return 1;
  PickParams p;
  for (int i = 0; i < MAX_WORLD; ++i)
    p.peers.base[i] = i < world ? static_cast<uint8_t*>(const_cast<void*>(peer_bases[i])) : nullptr;
  p.world = world; p.rank = rank; p.rows = rows; p.rows_cap = rows_cap; p.area_offset = area_offset;
  p.val = static_cast<const float*>(val); p.idx = static_cast<const long long*>(idx); p.idx_offset = idx_offset;
  p.out = static_cast<long long*>(out); p.limit_ns = static_cast<unsigned long long>(limit_ns);
  p.status = static_cast<int*>(status);
  pick_exchange_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

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
               const void* gscale, int ka, long long limit_ns, void* status, long long ll_offset, int ll_rows,
               void* stream) {
  if (world < 1 || world > MAX_WORLD || slot < 0 || slot >= NSLOT || h % 16 != 0 || rows <= 0) return 1;
  if (h > 8192) return 1;
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
  // The caller keeps persistent output buffers whose padding scale rows were zeroed once, so only real rows run.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nchunk = h / 8;
  if (ll_offset >= 0 && rows <= ll_rows && world > 1) {
    ArNormLlParams pp;
    pp.base = p;
    pp.ll_offset = ll_offset;
    pp.ll_rows = ll_rows;
    if (nchunk <= T) ar_norm_ll_kernel<T, 1><<<rows, T, 0, st>>>(pp);
    else if (nchunk <= 2 * T) ar_norm_ll_kernel<T, 2><<<rows, T, 0, st>>>(pp);
    else if (nchunk <= 3 * T) ar_norm_ll_kernel<T, 3><<<rows, T, 0, st>>>(pp);
    else ar_norm_ll_kernel<T, 4><<<rows, T, 0, st>>>(pp);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  if (nchunk <= T) ar_norm_kernel<T, 1><<<rows, T, 0, st>>>(p);
  else if (nchunk <= 2 * T) ar_norm_kernel<T, 2><<<rows, T, 0, st>>>(p);
  else if (nchunk <= 3 * T) ar_norm_kernel<T, 3><<<rows, T, 0, st>>>(p);
  else ar_norm_kernel<T, 4><<<rows, T, 0, st>>>(p);
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
  if (h > 8192) return 1;
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nchunk = h / 8;
  if (nchunk <= T) rs_norm_ag_kernel<T, 1><<<rows_per_rank, T, 0, st>>>(p);
  else if (nchunk <= 2 * T) rs_norm_ag_kernel<T, 2><<<rows_per_rank, T, 0, st>>>(p);
  else if (nchunk <= 3 * T) rs_norm_ag_kernel<T, 3><<<rows_per_rank, T, 0, st>>>(p);
  else rs_norm_ag_kernel<T, 4><<<rows_per_rank, T, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
