// Decode / verify attention on tcgen05 for head dim 128 and up to 16 query rows per (sequence, kv head).
//
// The tile math runs transposed so that the KEYS take the 128-row side of the MMA and the handful of query rows its
// (cheap) N side:   S^T[key, row] = K Q^T        (A = K tile, K-major;  B = Q, 16 rows, K-major; N = 16)
//                   O^T[d, row]  += V^T P^T      (A = V tile read MN-major; B = P^T, 16 rows x 128 keys, K-major)
// Both accumulators live in TMEM (16 columns each). A softmax thread owns one KEY (one TMEM lane): it loads its 16
// scores, exponentiates against a per-row reference maximum shared by all threads, adds to its private row sums
// (reduced over threads once, at the end) and stores 16 bf16 probabilities into the swizzled P^T tile. The
// reference maximum is only raised when some score exceeds it by more than 2^8 (one block-wide vote per tile;
// the full cross-thread maximum and the TMEM rescale of O^T run only then), so the steady state has no
// cross-thread reduction at all. K / V tiles of 128 keys travel as bulk tensor copies (32-row boxes of a run of
// consecutive slots) or cp.async gathers into a 3-stage ring. The kernel is persistent: one CTA per SM walks its
// share of the (sequence, kv head, split) items, and loads, MMAs and softmax of consecutive items overlap (the
// ring, the S^T double buffer and a ring of Q tiles are indexed by running counters), so the only pipeline fill is
// the first one. KV splits and their merge are as in attn_decode.cu (same partial format).
// Replaces the FlashInfer decode wrapper of the reference (hibana/engine/graphs.py:55) and its multi-row verify kernel
// (hibana/kernels/csrc/verify_attn.cu:469).
#include "kv_tma.cuh"
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int TD = 128;          // head dim
constexpr int TKT = 128;         // keys per tile
constexpr int TSTAGES = 3;
constexpr int TQ = 16;           // query rows (padded)
constexpr int TPRODUCERS = 96;   // warps 4, 5, 6
constexpr int TTHREADS = 256;
constexpr float TGAP = 8.f;

constexpr int T_KV_TILE = TKT * TD * 2;                 // 32 KiB, one of K or V
constexpr int T_STAGE = 2 * T_KV_TILE;
constexpr int T_Q_BYTES = TQ * TD * 2;                  // 4 KiB: two 64-column blocks of 16 rows
constexpr int T_P_BYTES = TQ * TKT * 2;                 // 4 KiB: two 64-key blocks of 16 rows
constexpr int TQBUF = 4;          // query tiles in flight (items overlap: loads run up to three tiles ahead)
constexpr int T_BAR_OFF = TSTAGES * T_STAGE + TQBUF * T_Q_BYTES + 2 * T_P_BYTES;   // P^T is double-buffered
constexpr int T_SMEM = T_BAR_OFF + 512 + 1024;

struct TcParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  long long pool_stride, head_stride;
  int tma_xh, tma_yh, use_tma;
  const int* kv_indices;
  long long ld_idx;
  const int* seq_rows;
  const int* ctx_len;
  const int* q_indptr;
  __nv_bfloat16* out;
  float* part_o;
  float* part_lse;
  int hq, hkv, splits, batch, total_items;
  float scale_log2;
  int causal;
  int* status;
  unsigned long long* prof;   // optional role counters (see hb_attn_decode_tc_profile)
};

__device__ __forceinline__ void cp16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void st_zero16(uint32_t saddr) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(saddr), "r"(0) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Reduces 16 per-lane values over the warp with 16 shuffles: each step trades half of the values still held with
// the lane 16, 8, 4, 2 apart, so that a lane ends up with the full reduction of ONE value; a last step folds the
// two lanes that hold the same one. The value index a lane ends up with is `bfly_index(lane)`.
template <bool MAX>
__device__ __forceinline__ float bfly_reduce16(const float (&v)[16], int lane) {
  auto op = [](float a, float b) { return MAX ? fmaxf(a, b) : a + b; };
  float a8[8], a4[4], a2[2];
  const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4, h2 = lane & 2;
#pragma unroll
  for (int i = 0; i < 8; ++i) {   // upper half-warp keeps values 8..15
    const float keep = h16 ? v[i + 8] : v[i], give = h16 ? v[i] : v[i + 8];
    a8[i] = op(keep, __shfl_xor_sync(0xffffffffu, give, 16));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float keep = h8 ? a8[i + 4] : a8[i], give = h8 ? a8[i] : a8[i + 4];
    a4[i] = op(keep, __shfl_xor_sync(0xffffffffu, give, 8));
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float keep = h4 ? a4[i + 2] : a4[i], give = h4 ? a4[i] : a4[i + 2];
    a2[i] = op(keep, __shfl_xor_sync(0xffffffffu, give, 4));
  }
  const float keep = h2 ? a2[1] : a2[0], give = h2 ? a2[0] : a2[1];
  float r = op(keep, __shfl_xor_sync(0xffffffffu, give, 2));
  r = op(r, __shfl_xor_sync(0xffffffffu, r, 1));
  return r;
}
// The value index whose reduction `bfly_reduce16` leaves in `lane`.
__device__ __forceinline__ int bfly_index(int lane) {
  return ((lane & 16) ? 8 : 0) + ((lane & 8) ? 4 : 0) + ((lane & 4) ? 2 : 0) + ((lane & 2) ? 1 : 0);
}
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort, int* status, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort, status, code));
}

// One unit of work: the keys [k0, k1) of one (sequence, kv head, split). Every role walks the same list (the CTA's
// contiguous share [item_lo, item_hi) of all items) and derives the same tile counts from ctx_len.
__device__ __forceinline__ int item_lo(int total, int cta) {
  return static_cast<int>(static_cast<long long>(total) * cta / static_cast<long long>(gridDim.x));
}
struct Item {
  int b, kvh, split, row0, R, nq, ctx, k0, k1, ntiles;
};
__device__ __forceinline__ Item load_item(const TcParams& p, int item) {
  Item w;
  // kv head slowest: with a head-major pool consecutive items read neighbouring memory (the splits of a sequence,
  // then the next sequence of the same head), so the handful of items of one CTA stays within a few pages
  w.split = item % p.splits;
  w.b = (item / p.splits) % p.batch;
  w.kvh = item / (p.splits * p.batch);
  w.row0 = p.q_indptr ? ldg_keep(p.q_indptr + w.b) : w.b;
  w.R = p.q_indptr ? ldg_keep(p.q_indptr + w.b + 1) - w.row0 : 1;
  w.nq = w.R * (p.hq / p.hkv);
  w.ctx = ldg_keep(p.ctx_len + w.b);
  const int per = (((w.ctx + p.splits - 1) / p.splits + TKT - 1) / TKT) * TKT;
  w.k0 = w.split * per;
  w.k1 = min(w.ctx, w.k0 + per);
  w.ntiles = w.k1 > w.k0 ? (w.k1 - w.k0 + TKT - 1) / TKT : 0;
  return w;
}
// Walks the tiles of this CTA's items in order, skipping items without keys. `q` counts the non-empty items
// (it selects the Q buffer), `g` the tiles (it selects ring stages and barrier phases).
struct TileIter {
  Item w;
  int item, end, t, q, g;
  bool valid;
  __device__ __forceinline__ void seek(const TcParams& p) {   // settles on a non-empty item at or after `item`
    while (item < end) {
      w = load_item(p, item);
      if (w.ntiles > 0) {
        valid = true;
        return;
      }
      ++item;
    }
    valid = false;
  }
  __device__ __forceinline__ void begin(const TcParams& p) {
    item = item_lo(p.total_items, blockIdx.x);
    end = item_lo(p.total_items, blockIdx.x + 1);
    t = 0; q = 0; g = 0;
    seek(p);
  }
  __device__ __forceinline__ void next(const TcParams& p) {
    ++g;
    if (++t >= w.ntiles) {
      t = 0;
      ++q;
      ++item;
      seek(p);
    }
  }
};

__global__ void __launch_bounds__(TTHREADS, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv,
                      const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv_s = smem;                                   // TSTAGES K tiles, then TSTAGES V tiles
  uint8_t* q_s = smem + TSTAGES * T_STAGE;                // TQBUF query tiles
  uint8_t* p_s = q_s + TQBUF * T_Q_BYTES;
  uint64_t* full_k = reinterpret_cast<uint64_t*>(smem + T_BAR_OFF);   // K and V tiles travel in rings of their own:
  uint64_t* full_v = full_k + TSTAGES;                                 // a K tile is free again after its score
  uint64_t* empty_k = full_v + TSTAGES;                                // product, a V tile only after the softmax
  uint64_t* empty_v = empty_k + TSTAGES;                               // and the value product
  uint64_t* s_ready = empty_v + TSTAGES;   // [2]
  uint64_t* p_ready = s_ready + 2;       // [2]: the softmax may run a tile ahead of the issuer, so one barrier per parity
  uint64_t* pv_ready = p_ready + 2;      // [2]: tile g completes a phase of pv_ready[g & 1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_ready + 2);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(smem + T_BAR_OFF + 192);   // [4 warps][16] cross-warp scratch
  int* vote = reinterpret_cast<int*>(red + 64);                    // [2 tile parities][4 warps]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = p.hq / p.hkv;

  if (tid == 0) {
    for (int s = 0; s < TSTAGES; ++s) {
      mbar_init(&full_k[s], TPRODUCERS);
      mbar_init(&full_v[s], TPRODUCERS);
      mbar_init(&empty_k[s], 1);
      mbar_init(&empty_v[s], 1);
    }
    mbar_init(&s_ready[0], 1);
    mbar_init(&s_ready[1], 1);
    mbar_init(&p_ready[0], 128);
    mbar_init(&p_ready[1], 128);
    mbar_init(&pv_ready[0], 1);
    mbar_init(&pv_ready[1], 1);
    *abort = 0;
    fence_mbar_init();
    if (p.use_tma) {
      prefetch_tmap(&tmk);
      prefetch_tmap(&tmv);
    }
  }
  if (warp == 7) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t o_tmem = tmem_base + 2 * TQ;

  if (warp >= 4 && warp < 7) {
    // ------------------------------------------------------------------ producers
    const int ptid = tid - 128, pw = warp - 4;
    constexpr int CPR = TD / 8;
    constexpr int SB = (TKT / 32 + 2) / 3;   // 32-key sub-blocks per warp and tile
    auto fetch_slots = [&](const TileIter& it, int (&sl)[SB]) {
      const int* idx_row = it.valid ? p.kv_indices + static_cast<long long>(p.seq_rows ? ldg_keep(p.seq_rows + it.w.b) : it.w.b) * p.ld_idx
                                    : p.kv_indices;
#pragma unroll
      for (int i = 0; i < SB; ++i) {
        const int j = pw + 3 * i;
        const int key = it.w.k0 + it.t * TKT + j * 32 + lane;
        sl[i] = (j < TKT / 32 && it.valid && key < it.w.k1) ? ldg_keep(idx_row + key) : -1;
      }
    };
    // returns whether this warp used the gather path for any of its sub-blocks (warp-uniform)
    auto copy_tile = [&](int kvh, const int (&sl)[SB], const __nv_bfloat16* pool, const CUtensorMap* tm, uint8_t* tile,
                         uint64_t* bar) -> bool {
      bool gathered = false;
#pragma unroll
      for (int i = 0; i < SB; ++i) {
        const int j = pw + 3 * i;
        if (j >= TKT / 32) break;
        const int slot = sl[i];
        const int slot0 = __shfl_sync(0xffffffffu, slot, 0);
        const bool run = p.use_tma && __all_sync(0xffffffffu, slot >= 0 && slot == slot0 + lane);
        if (run) {
          if (lane == 0) {
            mbar_add_tx(bar, 32 * TD * 2);
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_2d(tile + h * (TKT * 128) + j * (32 * 128), tm, bar, kvh * p.tma_xh + h * 64,
                          kvh * p.tma_yh + slot0);
          }
        } else {
          gathered = true;
          const int part = lane % CPR;
          const uint32_t dst0 = smem_u32(tile) + (part >> 3) * (TKT * 128);
#pragma unroll
          for (int ii = 0; ii < 16; ++ii) {
            const int rr = ii * 2 + lane / CPR;
            const int s1 = __shfl_sync(0xffffffffu, slot, rr);
            const int r = j * 32 + rr;
            const uint32_t dst = dst0 + r * 128 + (((part & 7) ^ (r & 7)) << 4);
            if (s1 >= 0)
              cp16(dst, pool + static_cast<long long>(s1) * p.pool_stride + kvh * p.head_stride + part * 8);
            else st_zero16(dst);
          }
        }
      }
      return gathered;
    };
    const bool prof = p.prof != nullptr && ptid == 0;
    long long c_wait = 0;
    int n_tma = 0, n_gather = 0;
    // this thread's own row copies (and the Q rows with a first tile) must have landed and be visible to the
    // tensor-core proxy before it reports in; bulk copies report by transaction bytes on their own
    auto settle = [&]() {
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      fence_proxy_async_smem();
    };
    // K tile (and, with the first tile of an item, its Q rows) of tile `a`; false when the stage wait gave up
    auto put_k = [&](const TileIter& a, const int (&ids)[SB]) -> bool {
      const int s = a.g % TSTAGES;
      const long long c0 = prof ? clock64() : 0;
      if (a.g >= TSTAGES && !mbar_wait(&empty_k[s], ((a.g / TSTAGES) - 1) & 1, abort, p.status, kTimeoutEmpty))
        return false;
      if (prof) c_wait += clock64() - c0;
      const bool first = a.t == 0;
      if (first) {
        // Q rows of the item (zero padded to 16) in two 64-column blocks of 16 swizzled rows; they ride on the
        // barrier of the item's first K tile. Buffer q % TQBUF was last read TQBUF items ago; the stage wait above
        // proves every MMA up to the score product three tiles back, hence of all items before the previous two,
        // has completed.
        const uint32_t qb = smem_u32(q_s) + (a.q % TQBUF) * T_Q_BYTES;
        for (int c = ptid; c < TQ * CPR; c += TPRODUCERS) {
          const int r = c / CPR, part = c % CPR;
          const uint32_t dst = qb + (part >> 3) * (TQ * 128) + r * 128 + (((part & 7) ^ (r & 7)) << 4);
          if (r < a.w.nq) {
            const int rr = r / g, gg = r % g;
            cp16(dst, p.q + (static_cast<long long>(a.w.row0 + rr) * p.hq + a.w.kvh * g + gg) * TD + part * 8);
          } else {
            st_zero16(dst);
          }
        }
      }
      const bool gathered = copy_tile(a.w.kvh, ids, p.k_pool, &tmk, kv_s + s * T_KV_TILE, &full_k[s]);
      if (gathered || first) settle();
      mbar_arrive(&full_k[s]);
      return true;
    };
    // Order of issue: K(0), then K(t + 1) before V(t): the score product is what the softmax waits for, the value
    // tile is only needed after it. Slot ids are fetched two tiles ahead of their use.
    TileIter it, nx, nx2;
    it.begin(p);
    int sl[SB], sl_n[SB], sl_n2[SB];
    fetch_slots(it, sl);
    nx = it;
    if (it.valid) nx.next(p);
    fetch_slots(nx, sl_n);
    bool live = !it.valid || put_k(it, sl);
    while (live && it.valid) {
      nx2 = nx;
      if (nx.valid) nx2.next(p);
      fetch_slots(nx2, sl_n2);
      if (nx.valid && !put_k(nx, sl_n)) break;
      const int s = it.g % TSTAGES;
      const long long c0 = prof ? clock64() : 0;
      if (it.g >= TSTAGES && !mbar_wait(&empty_v[s], ((it.g / TSTAGES) - 1) & 1, abort, p.status, kTimeoutEmpty)) break;
      if (prof) c_wait += clock64() - c0;
      const bool gathered =
          copy_tile(it.w.kvh, sl, p.v_pool, &tmv, kv_s + (TSTAGES + s) * T_KV_TILE, &full_v[s]);
      if (prof) (gathered ? n_gather : n_tma) += 1;
      if (gathered) settle();
      mbar_arrive(&full_v[s]);
#pragma unroll
      for (int i = 0; i < SB; ++i) {
        sl[i] = sl_n[i];
        sl_n[i] = sl_n2[i];
      }
      it = nx;
      nx = nx2;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (prof) {
      atomicAdd(p.prof + 0, static_cast<unsigned long long>(c_wait));
      atomicAdd(p.prof + 1, static_cast<unsigned long long>(n_tma));
      atomicAdd(p.prof + 2, static_cast<unsigned long long>(n_gather));
    }
  } else if (warp == 7) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(TKT, TQ);            // M = keys, N = query rows
      constexpr uint32_t idesc_pv = make_idesc_bf16(TD, TQ, 1, 0);       // A = V read MN-major (M = head dim)
      const uint32_t p_a = smem_u32(p_s);
      const bool prof = p.prof != nullptr;
      long long c_idle = 0;
      auto issue_qk = [&](const TileIter& it) {
        const int s = it.g % TSTAGES;
        tc_fence_after();
        const uint32_t k_a = smem_u32(kv_s + s * T_KV_TILE);
        const uint32_t q_a = smem_u32(q_s) + (it.q % TQBUF) * T_Q_BYTES;
        const uint32_t s_t = tmem_base + (it.g & 1) * TQ;
#pragma unroll
        for (int ks = 0; ks < TD / 16; ++ks) {
          const uint32_t in_row = (ks & 3) * 32;
          mma_f16(s_t, make_desc_sw128(k_a + (ks >> 2) * (TKT * 128) + in_row),
                  make_desc_sw128(q_a + (ks >> 2) * (TQ * 128) + in_row), idesc_qk, ks > 0 ? 1u : 0u);
        }
        tc_commit(&s_ready[it.g & 1]);
        tc_commit(&empty_k[s]);
      };
      // Two streams of work, each taken as soon as its barrier allows: S^T of the tile `ahead` (its K tile has
      // landed, and its S buffer is free: at most two score tiles ahead of the PV products) and the PV product of
      // the tile `cur` (its P^T is written). Neither waits behind the other.
      TileIter cur, ahead;
      cur.begin(p);
      ahead = cur;
      uint32_t idle = 0;
      uint64_t t_idle = 0;
      long long c0 = 0;
      while (cur.valid) {
        bool progressed = false;
        if (ahead.valid && ahead.g < cur.g + 2 &&
            mbar_test_wait(&full_k[ahead.g % TSTAGES], (ahead.g / TSTAGES) & 1)) {
          issue_qk(ahead);
          ahead.next(p);
          progressed = true;
        }
        if (mbar_test_wait(&p_ready[cur.g & 1], (cur.g >> 1) & 1) &&
            mbar_test_wait(&full_v[cur.g % TSTAGES], (cur.g / TSTAGES) & 1)) {
          const int s = cur.g % TSTAGES;
          tc_fence_after();
          const uint32_t v_a = smem_u32(kv_s + (TSTAGES + s) * T_KV_TILE);
#pragma unroll
          for (int kk = 0; kk < TKT / 16; ++kk) {
            // A: 16 keys = two 8-row groups 1024 bytes apart; the two 64-wide head-dim blocks are TKT * 128 apart
            const uint64_t adesc = make_desc_sw128_mn(v_a + kk * 2048, TKT * 128, 1024);
            const uint64_t bdesc =
                make_desc_sw128(p_a + (cur.g & 1) * T_P_BYTES + (kk >> 2) * (TQ * 128) + (kk & 3) * 32);
            mma_f16(o_tmem, adesc, bdesc, idesc_pv, (cur.t > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty_v[s]);
          tc_commit(&pv_ready[cur.g & 1]);
          cur.next(p);
          progressed = true;
        }
        if (progressed) {
          if (prof && idle > 0) c_idle += clock64() - c0;
          idle = 0;
          continue;
        }
        if (idle == 0) {
          t_idle = globaltimer_ns();
          if (prof) c0 = clock64();
        }
        if ((++idle & 255u) == 0u) {   // bounded: another role gave up, or nothing moved for the wait limit
          if (*abort) break;
          if (globaltimer_ns() - t_idle > HB_WAIT_NS || idle > HB_SPIN_LIMIT) {
            *abort = 1;
            set_status(p.status, kTimeoutAccum);
            break;
          }
        }
      }
      if (prof) atomicAdd(p.prof + 3, static_cast<unsigned long long>(c_idle));
    }
  } else {
    // ------------------------------------------------------------------ softmax: thread = key lane
    const uint32_t tlane = static_cast<uint32_t>(warp * 32) << 16;
    // byte offset of this key's column inside a P^T row: 64-key block, 16-byte chunk (swizzled per row), element
    const uint32_t p_blk = smem_u32(p_s) + (tid >> 6) * (TQ * 128) + (tid & 7) * 2;
    const int p_chunk = (tid & 63) >> 3;
    bool ok = true;
    int gt = 0;   // tiles done by this CTA (all items)
    const bool prof = p.prof != nullptr && tid == 0;
    const long long c_begin = prof ? clock64() : 0;
    long long c_s = 0, c_pv = 0, c_epi = 0;
    int n_raise = 0;
    const int it_lo = item_lo(p.total_items, blockIdx.x), it_hi = item_lo(p.total_items, blockIdx.x + 1);
    Item w_next = load_item(p, min(it_lo, p.total_items - 1));
    for (int item = it_lo; item < it_hi; ++item) {
      const Item w = w_next;
      // the next item's descriptor (dependent global loads) is fetched behind this item's tiles
      w_next = load_item(p, min(item + 1, p.total_items - 1));
      float m_ref[TQ], l_part[TQ];
      int lim[TQ];
#pragma unroll
      for (int j = 0; j < TQ; ++j) {
        m_ref[j] = -INFINITY;
        l_part[j] = 0.f;
        lim[j] = j < w.nq ? (p.causal ? w.ctx - w.R + (j / g) + 1 : w.ctx) : 0;   // keys [0, lim) visible to row j
      }
      for (int t = 0; t < w.ntiles; ++t, ++gt) {
        // A wait that gave up does not leave the loop: the named barriers below are counted, so every softmax
        // warp runs the same sequence to the end (later waits return at once through the abort flag; the math is
        // garbage and nothing is written out).
        const long long c0 = prof ? clock64() : 0;
        if (ok && !warp_wait(&s_ready[gt & 1], (gt >> 1) & 1, abort, p.status, kTimeoutAccum)) ok = false;
        if (prof) c_s += clock64() - c0;
        tc_fence_after();
        uint32_t raw[TQ];
        tmem_ld_32x16(tmem_base + (gt & 1) * TQ + tlane, raw);
        tmem_ld_wait();
        tc_fence_before();
        const int kp = w.k0 + t * TKT + tid;
        float x[TQ];
        bool exceed = false;
#pragma unroll
        for (int j = 0; j < TQ; ++j) {
          x[j] = (kp < w.k1 && kp < lim[j]) ? __uint_as_float(raw[j]) * p.scale_log2 : -INFINITY;
          exceed |= x[j] > m_ref[j] + TGAP;
        }
        // one vote over the 128 softmax threads: does anybody need a higher reference? (double-buffered by tile
        // parity: a warp that runs ahead writes its next vote into the other half)
        int* vt = vote + (gt & 1) * 4;
        const bool w_any = __any_sync(0xffffffffu, exceed);
        if (lane == 0) vt[warp] = w_any;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool raise = (vt[0] | vt[1] | vt[2] | vt[3]) != 0;
        // P(g) goes to the buffer that the PV product of tile g - 2 read; a rescale touches O^T and needs the
        // product of tile g - 1 done as well.
        const long long c1 = prof ? clock64() : 0;
        if (ok && gt > 1 && !warp_wait(&pv_ready[gt & 1], ((gt >> 1) - 1) & 1, abort, p.status, kTimeoutAccum))
          ok = false;
        if (ok && raise && gt > 0 &&
            !warp_wait(&pv_ready[(gt - 1) & 1], ((gt - 1) >> 1) & 1, abort, p.status, kTimeoutAccum))
          ok = false;
        if (prof) {
          c_pv += clock64() - c1;
          n_raise += raise;
        }
        if (raise) {
          const float mine = bfly_reduce16<true>(x, lane);
          if ((lane & 1) == 0) red[warp * TQ + bfly_index(lane)] = mine;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          uint32_t o[TQ];
          if (t > 0) {
            tc_fence_after();
            tmem_ld_32x16(o_tmem + tlane, o);
            tmem_ld_wait();
          }
#pragma unroll
          for (int j = 0; j < TQ; ++j) {
            const float m_new =
                fmaxf(m_ref[j], fmaxf(fmaxf(red[j], red[TQ + j]), fmaxf(red[2 * TQ + j], red[3 * TQ + j])));
            const float alpha = m_new == -INFINITY ? 1.f : ex2(m_ref[j] - m_new);
            m_ref[j] = m_new;
            l_part[j] *= alpha;
            if (t > 0) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          }
          if (t > 0) {
            tmem_st_32x16(o_tmem + tlane, o);
            tmem_st_wait();
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");   // `red` may be rewritten by the next raise
        }
#pragma unroll
        for (int j = 0; j < TQ; ++j) {
          const float pj = m_ref[j] == -INFINITY ? 0.f : ex2(x[j] - m_ref[j]);
          l_part[j] += pj;
          const uint32_t dst = p_blk + (gt & 1) * T_P_BYTES + j * 128 + ((p_chunk ^ (j & 7)) << 4);
          asm volatile("st.shared.b16 [%0], %1;" ::"r"(dst), "h"(__bfloat16_as_ushort(__float2bfloat16(pj)))
                       : "memory");
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(&p_ready[gt & 1]);
      }
      // ---- item epilogue: row sums over the 128 threads, O^T / l, store
      const long long c2 = prof ? clock64() : 0;
      if (ok && w.ntiles > 0 &&
          !warp_wait(&pv_ready[(gt - 1) & 1], ((gt - 1) >> 1) & 1, abort, p.status, kTimeoutAccum))
        ok = false;
      {
        const float mine = bfly_reduce16<false>(l_part, lane);
        if ((lane & 1) == 0) red[warp * TQ + bfly_index(lane)] = mine;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      uint32_t o[TQ];
      if (w.ntiles > 0) {
        tc_fence_after();
        tmem_ld_32x16(o_tmem + tlane, o);
        tmem_ld_wait();
        tc_fence_before();
      } else {
#pragma unroll
        for (int j = 0; j < TQ; ++j) o[j] = 0;
      }
      float l_row[TQ];
#pragma unroll
      for (int j = 0; j < TQ; ++j) l_row[j] = red[j] + red[TQ + j] + red[2 * TQ + j] + red[3 * TQ + j];
      if (ok) {
        // thread = head-dim element `tid` of every query row
#pragma unroll
        for (int j = 0; j < TQ; ++j) {
          if (j >= w.nq) break;
          const float l = l_row[j];
          const float val = l > 0.f ? __uint_as_float(o[j]) / l : 0.f;
          const int rr = j / g, gg = j % g;
          const long long rh = static_cast<long long>(w.row0 + rr) * p.hq + w.kvh * g + gg;
          if (p.splits == 1) {
            p.out[rh * TD + tid] = __float2bfloat16(val);
          } else {
            p.part_o[(rh * p.splits + w.split) * TD + tid] = val;
            if (tid == 0) p.part_lse[rh * p.splits + w.split] = l > 0.f ? m_ref[j] + log2f(l) : -INFINITY;
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // `red` is free again
      if (prof) c_epi += clock64() - c2;
    }
    if (prof) {
      atomicAdd(p.prof + 5, static_cast<unsigned long long>(c_s));
      atomicAdd(p.prof + 6, static_cast<unsigned long long>(c_pv));
      atomicAdd(p.prof + 7, static_cast<unsigned long long>(c_epi));
      atomicAdd(p.prof + 8, static_cast<unsigned long long>(clock64() - c_begin));
      atomicAdd(p.prof + 9, static_cast<unsigned long long>(n_raise));
      atomicAdd(p.prof + 10, static_cast<unsigned long long>(gt));
      atomicAdd(p.prof + 11, 1ull);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 7) tmem_dealloc(tmem_base, 64);
}

}  // namespace
}  // namespace hb

using namespace hb;

static unsigned long long* g_tc_prof = nullptr;

extern "C" {

// Optional role counters, accumulated over launches into 12 u64 (device memory; null switches them off). Cycles are
// summed over CTAs: [0] producer waits for a free stage, [1] / [2] tiles of producer warp 0 copied by bulk tensor
// copies only / with gathered rows, [3] issuer waits for a full stage, [4] issuer waits for P, [5] softmax waits for
// S, [6] softmax waits for the previous PV product, [7] item epilogues, [8] softmax role in total, [9] raises of the
// reference maximum, [10] tiles, [11] CTAs.
void hb_attn_decode_tc_profile(void* buf) { g_tc_prof = static_cast<unsigned long long*>(buf); }

// Head dim 128, bf16 KV, rows_per_seq * (hq / hkv) <= 16. Same outputs as hb_attn_decode (hb_attn_merge follows when
// splits > 1).
int hb_attn_decode_tc(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                      long long head_stride, const void* kv_indices, long long ld_idx, const void* seq_rows,
                      const void* ctx_len, const void* q_indptr, void* out, void* part_o, void* part_lse, int batch,
                      int max_rows, int hq, int hkv, int d, int splits, float scale, int causal, long long pool_slots,
                      void* status, void* stream) {
  if (batch <= 0) return 0;
  if (d != TD || hq % hkv != 0 || max_rows * (hq / hkv) > TQ) return 1;
  TcParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pool = static_cast<const __nv_bfloat16*>(k_pool);
  p.v_pool = static_cast<const __nv_bfloat16*>(v_pool);
  p.pool_stride = pool_stride; p.head_stride = head_stride;
  p.kv_indices = static_cast<const int*>(kv_indices); p.ld_idx = ld_idx;
  p.seq_rows = static_cast<const int*>(seq_rows); p.ctx_len = static_cast<const int*>(ctx_len);
  p.q_indptr = static_cast<const int*>(q_indptr);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = static_cast<float*>(part_o); p.part_lse = static_cast<float*>(part_lse);
  p.hq = hq; p.hkv = hkv; p.splits = splits < 1 ? 1 : splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = static_cast<int*>(status);
  p.prof = g_tc_prof;
  if (p.splits > 1 && (part_o == nullptr || part_lse == nullptr)) return 1;
  static const CUtensorMap dummy = {};
  const CUtensorMap *tk = &dummy, *tv = &dummy;
  const KvTma t = make_kv_tma(k_pool, v_pool, pool_stride, head_stride, pool_slots, hkv, d, 32);
  p.use_tma = t.ok; p.tma_xh = t.xh; p.tma_yh = t.yh;
  if (t.ok) {
    tk = &t.k;
    tv = &t.v;
  }
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM) != cudaSuccess)
      return 3;
    attr = true;
  }
  p.batch = batch;
  p.total_items = batch * hkv * p.splits;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  attn_decode_tc_kernel<<<dim3(p.total_items < sms ? p.total_items : sms), TTHREADS, T_SMEM, static_cast<cudaStream_t>(stream)>>>(*tk, *tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
