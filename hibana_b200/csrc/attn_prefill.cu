// Paged GQA prefill attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA owns one (sequence, kv head, block of query tokens). The block's query rows are packed as
// (token, group member) pairs, 128 rows = floor(128 / g) tokens x g query heads of the kv head, so a K / V tile
// gathered once from the token-granular pool serves the whole GQA group. Per 128-key tile:
//
//   producers (3 warps)   gather K and V rows by slot id with 16-byte cp.async into 128-byte-swizzled tiles
//                         (the layout TMA would produce; rows of a paged pool are not a TMA box). K and V have
//                         separate 2-stage rings: a K stage is free as soon as its S MMA has run, so K runs one
//                         tile ahead of V;
//   issuer (1 lane)       S = Q K^T (kind::f16, both operands K-major) into one of two TMEM score buffers, two
//                         tiles ahead of the softmax; once the softmax warps have published P, O += P V (V as
//                         MN-major B operand) accumulates in TMEM;
//   softmax (4 warps)     thread r owns query row r = TMEM lane r: one tcgen05.ld of the whole score row, row max,
//                         exp2, bf16 P tile into swizzled shared memory. The running maximum that O and the row
//                         sum refer to is only raised (and O rescaled in TMEM) when the new maximum exceeds it by
//                         more than 2^8, so the rescale is rare and the tensor pipe overlaps the softmax.
//
// Causal masking follows the ragged-batch rule of the engine: row token j of a sequence with R new rows and
// context ctx sees keys [0, ctx - R + j]. All waits are bounded; a timeout raises the status word and every role
// leaves.
//
// Replaces the reference's FlashInfer ragged-prefill wrapper + prefix kernel + LSE merge
// (hibana/kernels/ops.py:131-161, hibana/model/attention.py:73-96, hibana/kernels/csrc/verify_attn.cu prefix_kernel).
#include "kv_tma.cuh"
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int PF_THREADS = 256;
constexpr int PF_ROWS = 128;      // packed query rows per CTA
constexpr int PF_STAGES = 2;
constexpr int PF_PRODUCERS = 96;  // warps 4, 5, 6

struct PfParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  long long pool_stride;      // elements between slots
  long long head_stride;      // elements between kv heads
  int tma_xh, tma_yh;         // tensor-map coordinates per kv head (kv_tma.cuh)
  const int* kv_indices;
  long long ld_idx;
  const int* seq_rows;
  const int* ctx_len;
  const int* q_indptr;
  __nv_bfloat16* out;
  int hq, hkv;
  int use_tma;                // pools are TMA-addressable: contiguous slot runs travel as bulk tensor copies
  float scale_log2;
  int causal;
  int* status;
  unsigned long long* prof;   // optional cycle counters (null = off)
};

template <int D>
struct PfCfg {
  static constexpr int KT = D > 128 ? 64 : 128;               // keys per tile (head dim 256: 64, to fit shared memory)
  static constexpr int HALVES = D / 64;                      // 64-element (128-byte) column blocks of a row
  static constexpr int Q_BYTES = PF_ROWS * D * 2;
  static constexpr int KV_TILE = KT * D * 2;              // one stage of K or of V
  static constexpr int P_BYTES = PF_ROWS * KT * 2;
  static constexpr int BAR_OFF = Q_BYTES + 2 * PF_STAGES * KV_TILE + P_BYTES;
  static constexpr int SMEM = BAR_OFF + 256 + 1024;
  static constexpr int TMEM_COLS = 512;                      // S0 [0, KT) S1 [KT, 2 KT) O [2 KT, 2 KT + D)
  static constexpr float RESCALE_GAP = 8.f;                  // log2 units
};

__device__ __forceinline__ void cp16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Cycle accounting of one representative thread per role (softmax thread 0, producer 0, the issuer), summed over
// CTAs into p.prof: where each role's time goes. Costs one predictable branch per site when off.
#define PF_T0() const long long _t0 = p.prof ? clock64() : 0
#define PF_ACC(slot, cond) do { if (p.prof && (cond)) atomicAdd(p.prof + (slot), (unsigned long long)(clock64() - _t0)); } while (0)

// Bounded wait with a warp-uniform verdict, for warps that go on to warp-wide tcgen05.ld / st.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort, int* status, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort, status, code));
}
__device__ __forceinline__ void st_zero16(uint32_t saddr) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(saddr), "r"(0) : "memory");
}

// Byte offset of 16-byte chunk `part` of row `r` in a tile of `rows` rows whose 128-byte column blocks are stored
// one after another, each with the 128-byte swizzle (chunk index xor row % 8).
__device__ __forceinline__ uint32_t sw_off(int r, int part, int rows) {
  return static_cast<uint32_t>((part >> 3) * rows * 128 + r * 128 + (((part & 7) ^ (r & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv, const PfParams p) {
  using C = PfCfg<D>;
  constexpr int KT = C::KT;
  constexpr int CPR = D / 8;   // 16-byte chunks per row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = smem + C::Q_BYTES;
  uint8_t* v_s = k_s + PF_STAGES * C::KV_TILE;
  uint8_t* p_s = v_s + PF_STAGES * C::KV_TILE;
  uint64_t* kfull = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  uint64_t* vfull = kfull + PF_STAGES;
  uint64_t* kempty = vfull + PF_STAGES;
  uint64_t* vempty = kempty + PF_STAGES;
  uint64_t* s_ready = vempty + PF_STAGES;   // [2], one per score buffer
  uint64_t* p_ready = s_ready + 2;
  uint64_t* pv_ready = p_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_ready + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = p.hq / p.hkv;
  const int tok_per_blk = PF_ROWS / g;
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int qb = gridDim.x - 1 - blockIdx.x;   // heaviest (latest) query blocks first
  const int row0 = p.q_indptr ? p.q_indptr[b] : b;
  const int R = p.q_indptr ? p.q_indptr[b + 1] - row0 : 1;
  const int tok0 = qb * tok_per_blk;
  if (tok0 >= R) return;   // uniform: before any barrier or TMEM allocation
  const int ntok = min(tok_per_blk, R - tok0);
  const int nrows = ntok * g;
  const int ctx = p.ctx_len[b];
  // keys [0, kmax) are visible to at least one row of the block
  const int kmax = p.causal ? min(ctx, ctx - R + tok0 + ntok) : ctx;
  const int ntiles = (kmax + KT - 1) / KT;

  if (tid == 0) {
    for (int s = 0; s < PF_STAGES; ++s) {
      mbar_init(&kfull[s], PF_PRODUCERS);
      mbar_init(&vfull[s], PF_PRODUCERS);
      mbar_init(&kempty[s], 1);
      mbar_init(&vempty[s], 1);
    }
    mbar_init(&s_ready[0], 1);
    mbar_init(&s_ready[1], 1);
    mbar_init(p_ready, PF_ROWS);
    mbar_init(pv_ready, 1);
    *abort = 0;
    fence_mbar_init();
    if (p.use_tma) {
      prefetch_tmap(&tmk);
      prefetch_tmap(&tmv);
    }
  }
  if (warp == 7) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t o_tmem = tmem_base + 2 * KT;

  if (warp >= 4 && warp < 7) {
    // ------------------------------------------------------------------ producers
    const int ptid = tid - 128;
    const int* idx_row = p.kv_indices + static_cast<long long>(p.seq_rows ? p.seq_rows[b] : b) * p.ld_idx;
    // Q rows (zero padded); they travel in the first cp.async group, i.e. with K tile 0.
    for (int c = ptid; c < PF_ROWS * CPR; c += PF_PRODUCERS) {
      const int r = c / CPR, part = c % CPR;
      const uint32_t dst = smem_u32(q_s) + sw_off(r, part, PF_ROWS);
      if (r < nrows) {
        const int tok = tok0 + r / g, gg = r % g;
        cp16(dst, p.q + (static_cast<long long>(row0 + tok) * p.hq + kvh * g + gg) * D + part * 8);
      } else {
        st_zero16(dst);
      }
    }
    // A tile is moved as four 32-key sub-blocks, one producer warp each (warp j % 3). Lane l fetches the slot id
    // of key l of the sub-block. Slots of a sequence are handed out in ascending runs, so most sub-blocks sit in
    // 32 consecutive pool rows: then one lane issues a bulk tensor copy per 128-byte column block (box = 32 rows
    // x 64 elements, 128-byte swizzle, row pitch = one pool slot) that completes on the tile's barrier by
    // transaction bytes. Otherwise (fragmented pool, tail of the context) the warp gathers the rows with 16-byte
    // cp.async: the LSU path keeps only ~16 KB in flight per SM, an order of magnitude less than the TMA unit.
    const int pw = warp - 4;
    constexpr int SB = (KT / 32 + 2) / 3;   // sub-blocks per warp and tile
    // Slot ids of this warp's sub-blocks of tile t (one per lane); -1 beyond the visible keys.
    auto fetch_slots = [&](int t, int (&sl)[SB]) {
#pragma unroll
      for (int i = 0; i < SB; ++i) {
        const int j = pw + 3 * i;
        const int key = t * KT + j * 32 + lane;
        sl[i] = (j < KT / 32 && t < ntiles && key < kmax) ? __ldg(idx_row + key) : -1;
      }
    };
    auto copy_tile = [&](int t, const int (&sl)[SB], const __nv_bfloat16* pool, const CUtensorMap* tm, uint8_t* ring,
                         uint64_t* bar) {
      uint8_t* tile = ring + (t % PF_STAGES) * C::KV_TILE;
#pragma unroll
      for (int i = 0; i < SB; ++i) {
        const int j = pw + 3 * i;
        if (j >= KT / 32) break;
        const int slot = sl[i];
        const int slot0 = __shfl_sync(0xffffffffu, slot, 0);
        const bool run = p.use_tma && __all_sync(0xffffffffu, slot >= 0 && slot == slot0 + lane);
        if (run) {
          if (lane == 0) {
            mbar_add_tx(bar, 32 * D * 2);   // bytes only: this lane's arrival comes with the other producers'
#pragma unroll
            for (int h = 0; h < C::HALVES; ++h)
              tma_load_2d(tile + h * (KT * 128) + j * (32 * 128), tm, bar, kvh * p.tma_xh + h * 64,
                          kvh * p.tma_yh + slot0);
          }
        } else {
          // lane -> (row = i * (32 / CPR) + lane / CPR, 16-byte column = lane % CPR)
          constexpr int RPI = 32 / CPR;
          const int part = lane % CPR;
          const uint32_t dst0 = smem_u32(tile) + (part >> 3) * (KT * 128);
#pragma unroll
          for (int ii = 0; ii < 32 / RPI; ++ii) {
            const int rr = ii * RPI + lane / CPR;
            const int s1 = __shfl_sync(0xffffffffu, slot, rr);
            const int r = j * 32 + rr;
            const uint32_t dst = dst0 + r * 128 + (((part & 7) ^ (r & 7)) << 4);
            if (s1 >= 0)
              cp16(dst, pool + static_cast<long long>(s1) * p.pool_stride + kvh * p.head_stride + part * 8);
            else st_zero16(dst);
          }
        }
      }
    };
    // cp.async groups in order: K0, [K1, V0], [K2, V1], ...  After iteration t commits V(t), "at most two groups
    // pending" means K(t) and V(t - 1) have landed: fence them for the tensor-core proxy and signal.
    bool live = ntiles > 0;
    int sl_v[SB], sl_k[SB], sl_pre[SB];   // slots of tile t (V copy), t + 1 (K copy), t + 2 (in flight)
    fetch_slots(0, sl_v);
    fetch_slots(1, sl_k);
    if (live) copy_tile(0, sl_v, p.k_pool, &tmk, k_s, &kfull[0]);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int t = 0; live && t < ntiles; ++t) {
      fetch_slots(t + 2, sl_pre);   // latency hides behind the stage waits below
      if (t + 1 < ntiles) {
        {
          PF_T0();
          if (t + 1 >= PF_STAGES && !mbar_wait(&kempty[(t + 1) % PF_STAGES], (((t + 1) / PF_STAGES) - 1) & 1, abort,
                                               p.status, kTimeoutEmpty)) {
            live = false;
            break;
          }
          PF_ACC(6, ptid == 0);
        }
        {
          PF_T0();
          copy_tile(t + 1, sl_k, p.k_pool, &tmk, k_s, &kfull[(t + 1) % PF_STAGES]);
          PF_ACC(8, ptid == 0);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      {
        PF_T0();
        if (t >= PF_STAGES &&
            !mbar_wait(&vempty[t % PF_STAGES], ((t / PF_STAGES) - 1) & 1, abort, p.status, kTimeoutEmpty)) {
          live = false;
          break;
        }
        PF_ACC(7, ptid == 0);
      }
      {
        PF_T0();
        copy_tile(t, sl_v, p.v_pool, &tmv, v_s, &vfull[t % PF_STAGES]);
        PF_ACC(8, ptid == 0);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      PF_T0();
      asm volatile("cp.async.wait_group 2;" ::: "memory");
      PF_ACC(9, ptid == 0);
      fence_proxy_async_smem();
      mbar_arrive(&kfull[t % PF_STAGES]);
      if (t >= 1) mbar_arrive(&vfull[(t - 1) % PF_STAGES]);
#pragma unroll
      for (int i = 0; i < SB; ++i) {
        sl_v[i] = sl_k[i];
        sl_k[i] = sl_pre[i];
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");   // nothing may land after the CTA has gone
    fence_proxy_async_smem();
    if (live) mbar_arrive(&vfull[(ntiles - 1) % PF_STAGES]);
  } else if (warp == 7) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(PF_ROWS, KT);
      constexpr uint32_t idesc_pv = make_idesc_bf16(PF_ROWS, D, 0, 1);
      const uint32_t q_a = smem_u32(q_s), p_a = smem_u32(p_s);
      // S(t) = Q K(t)^T into score buffer t % 2; releases the K stage and publishes the scores when done.
      auto issue_qk = [&](int t) -> bool {
        const int s = t % PF_STAGES;
        {
          PF_T0();
          if (!mbar_wait(&kfull[s], (t / PF_STAGES) & 1, abort, p.status, kTimeoutFull)) return false;
          PF_ACC(5, true);
        }
        tc_fence_after();
        const uint32_t k_a = smem_u32(k_s + s * C::KV_TILE);
        const uint32_t s_t = tmem_base + (t & 1) * KT;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t in_row = (ks & 3) * 32;   // 16 elements = 32 bytes inside the 128-byte swizzled row
          mma_f16(s_t, make_desc_sw128(q_a + (ks >> 2) * (PF_ROWS * 128) + in_row),
                  make_desc_sw128(k_a + (ks >> 2) * (KT * 128) + in_row), idesc_qk, ks > 0 ? 1u : 0u);
        }
        tc_commit(&kempty[s]);
        tc_commit(&s_ready[t & 1]);
        return true;
      };
      bool ok = ntiles > 0 && issue_qk(0);
      if (ok && ntiles > 1) ok = issue_qk(1);
      for (int t = 0; ok && t < ntiles; ++t) {
        const int s = t % PF_STAGES;
        {
          PF_T0();
          if (!mbar_wait(p_ready, t & 1, abort, p.status, kTimeoutAccum)) break;
          PF_ACC(3, true);
        }
        {
          PF_T0();
          if (!mbar_wait(&vfull[s], (t / PF_STAGES) & 1, abort, p.status, kTimeoutFull)) break;
          PF_ACC(4, true);
        }
        tc_fence_after();
        const uint32_t v_a = smem_u32(v_s + s * C::KV_TILE);
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
          const uint64_t adesc = make_desc_sw128(p_a + (kk >> 2) * (PF_ROWS * 128) + (kk & 3) * 32);
          // 16 keys = two 8-row groups 1024 bytes apart; the D / 64 column blocks are KT * 128 bytes apart
          const uint64_t bdesc = make_desc_sw128_mn(v_a + kk * 2048, KT * 128, 1024);
          mma_f16(o_tmem, adesc, bdesc, idesc_pv, (t > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&vempty[s]);
        tc_commit(pv_ready);
        // score buffer t % 2 was read completely before p_ready(t): refill it two tiles ahead
        if (t + 2 < ntiles) ok = issue_qk(t + 2);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output (warps 0-3)
    const int r = tid;                                   // packed query row = TMEM lane
    const uint32_t tlane = static_cast<uint32_t>(warp * 32) << 16;
    const bool row_ok = r < nrows;
    const int tok = tok0 + r / g;
    // last visible key position (inclusive)
    const int lim = row_ok ? (p.causal ? ctx - R + tok : ctx - 1) : -1;
    float m_ref = -INFINITY, l = 0.f;   // O and l are relative to 2^m_ref
    const uint32_t p_row = smem_u32(p_s) + r * 128;
    bool ok = true;
    const long long t_begin = p.prof ? clock64() : 0;
    for (int t = 0; t < ntiles; ++t) {
      {
        PF_T0();
        if (!warp_wait(&s_ready[t & 1], (t >> 1) & 1, abort, p.status, kTimeoutAccum)) {
          ok = false;
          break;
        }
        PF_ACC(0, tid == 0);
      }
      tc_fence_after();
      const int k0 = t * KT;
      const uint32_t s_t = tmem_base + (t & 1) * KT + tlane;
      // The two passes over the score row are rolled loops over 32-column chunks: fully unrolled, the softmax body
      // alone is several thousand instructions, and streaming that through the instruction cache every tile cost
      // more than the arithmetic. `rel` = last visible column of this tile for this row (>= 127: no masking).
      const int rel = lim - k0;
      const long long t_math = p.prof ? clock64() : 0;
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int c0 = 0; c0 < KT; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_t + c0, v);
        tmem_ld_wait();
        const int rc = rel - c0;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          mx4[j & 3] = fmaxf(mx4[j & 3], j <= rc ? __uint_as_float(v[j]) : -INFINITY);
      }
      const float m_tile = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      // P(t) overwrites the buffer O += P(t - 1) V(t - 1) reads, and a rescale touches O: both need that MMA done.
      {
        PF_T0();
        if (t > 0 && !warp_wait(pv_ready, (t - 1) & 1, abort, p.status, kTimeoutAccum)) {
          ok = false;
          break;
        }
        PF_ACC(1, tid == 0);
      }
      if (t == 0) {
        m_ref = m_tile;
      } else if (__any_sync(0xffffffffu, m_tile > m_ref + C::RESCALE_GAP)) {
        // Raise the reference (all lanes of the warp: tcgen05.ld / st are warp-wide) and rescale O and l.
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = m_new == -INFINITY ? 1.f : ex2(m_ref - m_new);
        m_ref = m_new;
        l *= alpha;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32(o_tmem + tlane + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st_32x32(o_tmem + tlane + c0, o);
        }
        tmem_st_wait();
      }
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int c0 = 0; c0 < KT; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_t + c0, v);
        tmem_ld_wait();
        const int rc = rel - c0;
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = j <= rc ? ex2(fmaf(__uint_as_float(v[j]), p.scale_log2, neg_m)) : 0.f;
          const float p1 = j + 1 <= rc ? ex2(fmaf(__uint_as_float(v[j + 1]), p.scale_log2, neg_m)) : 0.f;
          sum4[(j >> 1) & 3] += p0 + p1;
          w[j >> 1] = pack_bf16(p0, p1);
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int part = (c0 >> 3) + ch;   // 16-byte chunk (8 keys) of the row
          const uint32_t dst = p_row + (part >> 3) * (PF_ROWS * 128) + (((part & 7) ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[4 * ch]), "r"(w[4 * ch + 1]),
                       "r"(w[4 * ch + 2]), "r"(w[4 * ch + 3])
                       : "memory");
        }
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (p.prof && tid == 0) atomicAdd(p.prof + 13, (unsigned long long)(clock64() - t_math));
      {
        PF_T0();
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(p_ready);
        PF_ACC(14, tid == 0);
      }
    }
    if (p.prof && tid == 0) {
      atomicAdd(p.prof + 10, (unsigned long long)(clock64() - t_begin));
      atomicAdd(p.prof + 11, (unsigned long long)ntiles);
    }
    if (ok && ntiles > 0) ok = warp_wait(pv_ready, (ntiles - 1) & 1, abort, p.status, kTimeoutAccum);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (static_cast<long long>(row0 + tok) * p.hq + kvh * g + r % g) * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        if (ntiles > 0) {
          tmem_ld_32x32(o_tmem + tlane + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0;
        }
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8)
            *reinterpret_cast<uint4*>(dst + c0 + j) =
                make_uint4(pack_bf16(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv),
                           pack_bf16(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv),
                           pack_bf16(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv),
                           pack_bf16(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv));
        }
      }
      tc_fence_before();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 7) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D>
int launch_prefill(const PfParams& p, const CUtensorMap* tk, const CUtensorMap* tv, int qblocks, int batch,
                   cudaStream_t st) {
  using C = PfCfg<D>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) !=
        cudaSuccess)
      return 3;
    attr = true;
  }
  attn_prefill_kernel<D><<<dim3(qblocks, p.hkv, batch), PF_THREADS, C::SMEM, st>>>(*tk, *tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace
}  // namespace hb

using namespace hb;

static unsigned long long* g_pf_prof = nullptr;

extern "C" {

// Cycle counters of the prefill kernel's roles: `buf` = 16 zeroed uint64 on the device (null switches it off).
// [0] softmax waits for scores, [1] softmax waits for the previous O update, [3] issuer waits for P,
// [4] issuer waits for V, [5] issuer waits for K, [6] / [7] producer waits for a free K / V stage,
// [8] producer issues copies, [9] producer waits for landed copies, [10] softmax loop total, [11] tiles,
// [12] softmax score load, [13] softmax math incl. the wait for the previous O update, [14] publish P.
void hb_attn_prefill_profile(void* buf) { g_pf_prof = static_cast<unsigned long long*>(buf); }

// bf16 KV, head dim 64 or 128, group size hq / hkv <= 128. `max_rows` bounds the new rows of any sequence.
int hb_attn_prefill(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                    long long head_stride,
                    const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len,
                    const void* q_indptr, void* out, int batch, int max_rows, int hq, int hkv, int d, float scale,
                    int causal, long long pool_slots, void* status, void* stream) {
  if (batch <= 0 || max_rows <= 0) return 0;
  if (hq % hkv != 0 || hq / hkv > PF_ROWS) return 1;
  PfParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pool = static_cast<const __nv_bfloat16*>(k_pool);
  p.v_pool = static_cast<const __nv_bfloat16*>(v_pool);
  p.pool_stride = pool_stride;
  p.head_stride = head_stride;
  p.kv_indices = static_cast<const int*>(kv_indices);
  p.ld_idx = ld_idx;
  p.seq_rows = static_cast<const int*>(seq_rows);
  p.ctx_len = static_cast<const int*>(ctx_len);
  p.q_indptr = static_cast<const int*>(q_indptr);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.hq = hq; p.hkv = hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = static_cast<int*>(status);
  p.prof = g_pf_prof;
  const int tok_per_blk = PF_ROWS / (hq / hkv);
  const int qblocks = (max_rows + tok_per_blk - 1) / tok_per_blk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static const CUtensorMap dummy = {};
  const CUtensorMap *tk = &dummy, *tv = &dummy;
  const KvTma t = make_kv_tma(k_pool, v_pool, pool_stride, head_stride, pool_slots, hkv, d, 32);
  p.use_tma = t.ok;
  p.tma_xh = t.xh;
  p.tma_yh = t.yh;
  if (t.ok) {
    tk = &t.k;
    tv = &t.v;
  }
  if (d == 64) return launch_prefill<64>(p, tk, tv, qblocks, batch, st);
  if (d == 128) return launch_prefill<128>(p, tk, tv, qblocks, batch, st);
  if (d == 256) return launch_prefill<256>(p, tk, tv, qblocks, batch, st);
  return 1;
}

}  // extern "C"
