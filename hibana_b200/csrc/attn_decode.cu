// Flash-decoding for paged GQA attention with up to 16 query rows per (sequence, kv head): decode (one token x
// GQA group <= 16) and short speculative verify blocks. Bandwidth-bound by design:
//
//   * K / V tiles of KT keys live in shared memory as 128-byte-swizzled column blocks ([KT rows x 128 bytes] per
//     64 head-dim elements), the layout a bulk tensor copy produces. The pool hands a sequence its slots in
//     ascending runs, so most tiles are KT consecutive pool rows and travel as one TMA box per column block
//     (row pitch = one pool slot): the TMA unit keeps far more bytes in flight than the LSU path, which tops out
//     near 16 KB outstanding per SM (~3.5 TB/s over the chip). Tiles that are not one run (fragmented pool, the
//     tail of the context) are gathered row by row with 16-byte cp.async into the same layout;
//   * each of the 4 warps of a CTA owns a private 3-stage ring of KT-key tiles and walks its own share of the keys,
//     so the main loop has no block-wide barrier and no flag wait: a warp waits only on its own cp.async groups;
//   * S = Q K^T and O += P V run on the tensor cores (m16n8k16 bf16, fp32 accumulate) with the query rows padded to
//     one 16-row tile; the online softmax lives in registers; the 4 warps' partial (m, l, O) merge through shared
//     memory at the end, and KV splits merge through the LSE kernel of attn.cu.
//
// The KV range of a split is derived on the device from ctx_len, so one captured launch serves any context.
// Replaces the FlashInfer decode wrapper the reference plans per step (hibana/engine/graphs.py:55,
// hibana/engine/executor.py:161-169) and the multi-row verify kernel (hibana/kernels/csrc/verify_attn.cu:469).
#include "kv_tma.cuh"
#include "hb_api.h"
#include "hb_common.cuh"
#include "rownorm.cuh"

namespace hb {
namespace {

constexpr int DEC_WARPS = 2;   // two CTAs share an SM: one streams while the other runs its prologue or merge
constexpr int DEC_STAGES = 3;

struct DecParams {
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
  float* part_o;
  float* part_lse;
  int hq, hkv, splits;
  float scale_log2;
  int causal;
  int use_tma;
  int* status;
  unsigned long long* prof;   // optional cycle counters of warp 0 (null = off)
  // Fused split merge: one int per (sequence, kv head), zero between launches. The CTA that finds splits - 1
  // earlier arrivals merges the partials of its (sequence, kv head) itself, so no merge kernel follows.
  int* split_counter;
  // Optional NVFP4 output of the merged (or unsplit) rows, the activation operand of the o projection:
  // q_out [rows, hq * D / 2] packed e2m1, q_sf swizzled ue4m3 scales, *q_gscale the static per-tensor scale.
  uint8_t* q_out;
  uint8_t* q_sf;
  const float* q_gscale;
  int q_ka;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Transposes an 8x8 matrix of 16-bit elements held one 32-bit pair per lane (the mma fragment layout).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

__device__ __forceinline__ void cp16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_wait2() { asm volatile("cp.async.wait_group 2;" ::: "memory"); }

template <int D>
struct DecCfg {
  static constexpr int KT = D >= 256 ? 16 : 32;        // keys per warp tile
  static constexpr int HALVES = D / 64;                 // 128-byte column blocks per row
  static constexpr int BLOCK_BYTES = KT * 128;          // one column block of a tile
  static constexpr int TILE_BYTES = KT * D * 2;         // one of K or V
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int WARP_BYTES = DEC_STAGES * STAGE_BYTES;
  static constexpr int QROWB = D * 2 + 16;              // padded Q row: conflict-free ldmatrix
  static constexpr int Q_BYTES = 16 * QROWB;
  static constexpr int BAR_OFF = DEC_WARPS * WARP_BYTES + Q_BYTES;
  static constexpr int SMEM = BAR_OFF + 256 + 1024;
  static_assert(16 * D * 4 + 16 * 8 <= WARP_BYTES, "merge scratch must fit a warp's ring");
  static_assert(BLOCK_BYTES % 1024 == 0, "column blocks must keep the swizzle atom alignment");
};

// Byte offset of 16-byte chunk c of row `row` in a swizzled tile of KT rows.
template <int KT>
__device__ __forceinline__ uint32_t dsw(int row, int c) {
  return static_cast<uint32_t>((c >> 3) * (KT * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

template <int D, bool T8>
__global__ void __launch_bounds__(DEC_WARPS * 32, 2)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv, const DecParams p) {
  using C = DecCfg<D>;
  grid_dep_wait();     // may run as a programmatic dependent of the RoPE + KV-write kernel
  grid_dep_launch();
  constexpr int KT = C::KT, ROWB = C::QROWB;
  constexpr int NB = KT / 8;     // score n-blocks per tile
  constexpr int KS = D / 16;     // k-steps of Q K^T
  constexpr int ONB = D / 8;     // output n-blocks
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g4 = lane >> 2, t4 = lane & 3;
  uint8_t* ring = smem + warp * C::WARP_BYTES;
  uint8_t* qs = smem + DEC_WARPS * C::WARP_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF) + warp * DEC_STAGES;   // this warp's barriers
  volatile int* abort = reinterpret_cast<volatile int*>(smem + C::BAR_OFF + DEC_WARPS * DEC_STAGES * 8) + warp;
  if (lane == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) mbar_init(&full[s], 1);
    *abort = 0;
    fence_mbar_init();
  }

  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int g = p.hq / p.hkv;
  const int row0 = p.q_indptr ? ldg_keep(p.q_indptr + b) : b;
  const int R = p.q_indptr ? ldg_keep(p.q_indptr + b + 1) - row0 : 1;
  const int nq = R * g;   // <= 16 guaranteed by the host
  const int ctx = ldg_keep(p.ctx_len + b);
  const int per = (((ctx + p.splits - 1) / p.splits + KT - 1) / KT) * KT;
  const int k0 = split * per;
  const int k1 = min(ctx, k0 + per);
  const int ntiles = k1 > k0 ? (k1 - k0 + KT - 1) / KT : 0;

  // Q rows (zero padded to 16) into shared memory.
  for (int i = tid; i < 16 * (D / 8); i += DEC_WARPS * 32) {
    const int qi = i / (D / 8), c = i % (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (qi < nq) {
      const int rr = qi / g, gg = qi % g;
      v = *reinterpret_cast<const uint4*>(p.q + (static_cast<long long>(row0 + rr) * p.hq + kvh * g + gg) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(qs + qi * ROWB + c * 16) = v;
  }
  __syncthreads();

  // Up to 8 query rows (T8): the tile math runs transposed, S^T = K Q^T and O^T = V^T P^T, so the keys (resp. the
  // head dim) take the 16-row side of m16n8k16 and the query rows its 8 columns: half the MMAs of the 16-row
  // form. Q is then the B operand (n = query row, k = head dim).
  uint32_t qf[T8 ? 1 : KS][4];
  uint32_t qb[T8 ? KS : 1][2];
  if constexpr (!T8) {
    const uint32_t base = smem_u32(qs) + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldsm_x4(qf[ks], base + ks * 32);
  } else {
    const uint32_t base = smem_u32(qs) + (lane & 7) * ROWB + (lane >> 3) * 16;
#pragma unroll
    for (int ks = 0; ks < KS; ks += 2) {
      uint32_t r[4];
      ldsm_x4(r, base + ks * 32);
      qb[ks][0] = r[0];
      qb[ks][1] = r[1];
      qb[ks + 1][0] = r[2];
      qb[ks + 1][1] = r[3];
    }
  }

  const int* idx_row = p.kv_indices + static_cast<long long>(p.seq_rows ? ldg_keep(p.seq_rows + b) : b) * p.ld_idx;

  // Issues the copies of this warp's `it`-th tile into its ring stage: one bulk tensor copy per column block of
  // K and of V when the tile's slots are KT consecutive pool rows, else a row-by-row cp.async gather. `tma_mode`
  // remembers per stage which way the tile in flight travels, `tma_phase` the parity of the stage's barrier.
  uint32_t tma_mode = 0, tma_phase = 0;
  // Slot id of key `lane` of this warp's tile `it` (-1 beyond the split). Fetched one tile ahead of its use so
  // that the index load's latency is not on the issue path.
  auto fetch_slot = [&](int it) -> int {
    const int base = k0 + (warp + it * DEC_WARPS) * KT;
    int slot = (warp + it * DEC_WARPS < ntiles && lane < KT && base + lane < k1) ? ldg_keep(idx_row + base + lane) : -1;
    if (slot >= 0 && !index_ok(slot, kBoundKvSlots, kKerAttnDecode)) slot = 0;   // reported; the dummy slot is read
    return slot;
  };
  auto issue = [&](int it, int my_slot) {
    const int tile = warp + it * DEC_WARPS;
    if (tile < ntiles) {
      const int st = it % DEC_STAGES;
      const int base = k0 + tile * KT;
      uint8_t* kt = ring + st * C::STAGE_BYTES;
      const uint32_t kdst = smem_u32(kt);
      const uint32_t vdst = kdst + C::TILE_BYTES;
      constexpr int CPR = D / 8;            // 16-byte chunks per row
      constexpr int RPI = 32 / CPR > 0 ? 32 / CPR : 1;   // rows per warp instruction
      const int slot0 = __shfl_sync(0xffffffffu, my_slot, 0);
      const bool run = p.use_tma && __all_sync(0xffffffffu, lane >= KT || (my_slot >= 0 && my_slot == slot0 + lane));
      if (run) {
        tma_mode |= 1u << st;
        // lane 0 posts the byte count, then 2 * HALVES lanes issue one box each (K / V x column block)
        if (lane == 0) mbar_expect_tx(&full[st], 2 * C::TILE_BYTES);
        __syncwarp();
        if (lane < 2 * C::HALVES) {
          const int h = lane >> 1, is_v = lane & 1;
          tma_load_2d(kt + is_v * C::TILE_BYTES + h * C::BLOCK_BYTES, is_v ? &tmv : &tmk, &full[st],
                      kvh * p.tma_xh + h * 64, kvh * p.tma_yh + slot0);
        }
      } else {
        tma_mode &= ~(1u << st);
        if constexpr (CPR <= 32) {
          const int part = lane % CPR, sub = lane / CPR;
#pragma unroll
          for (int r = 0; r < KT; r += RPI) {
            const int key = r + sub;
            const int slot = __shfl_sync(0xffffffffu, my_slot, key);
            const uint32_t so = dsw<KT>(key, part);
            if (slot >= 0) {
              const __nv_bfloat16* src = p.k_pool + static_cast<long long>(slot) * p.pool_stride +
                                         static_cast<long long>(kvh) * p.head_stride + part * 8;
              cp16(kdst + so, src);
              cp16(vdst + so, p.v_pool + (src - p.k_pool));
            } else {
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(kdst + so), "r"(0) : "memory");
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(vdst + so), "r"(0) : "memory");
            }
          }
        }
      }
    }
    cp_commit();
  };

  // 16-row form: o[n-block][4], rows g4 / g4 + 8. Transposed form: o[16-wide head-dim block][4] = (d g4 | g4 + 8)
  // x (query rows 2 t4, 2 t4 + 1); "lo" / "hi" then name those two query rows.
  constexpr int OB = T8 ? D / 16 : ONB;
  float o[OB][4];
#pragma unroll
  for (int i = 0; i < OB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  // Causal limits of this thread's two rows (keys [0, limit) visible).
  const int row_lo = T8 ? 2 * t4 : g4, row_hi = T8 ? 2 * t4 + 1 : g4 + 8;
  const int lim_lo = p.causal ? ctx - R + (row_lo / g) + 1 : ctx;
  const int lim_hi = p.causal ? ctx - R + (row_hi / g) + 1 : ctx;

  const bool prof = p.prof != nullptr && tid == 0;
  const long long t_start = prof ? clock64() : 0;
  long long c_issue = 0, c_wait = 0, c_math = 0;
  issue(0, fetch_slot(0));
  issue(1, fetch_slot(1));
  int slot_next = fetch_slot(2);
  for (int it = 0; warp + it * DEC_WARPS < ntiles; ++it) {
    // Stage (it + 2) % 3 was read in iteration it - 1: every lane is past it, order it before the async writes.
    __syncwarp();
    long long t0 = prof ? clock64() : 0;
    issue(it + 2, slot_next);
    slot_next = fetch_slot(it + 3);
    long long t1 = prof ? clock64() : 0;
    cp_wait2();
    const int st = it % DEC_STAGES;
    if (tma_mode & (1u << st)) {
      const bool got = mbar_wait(&full[st], (tma_phase >> st) & 1u, abort, p.status, kTimeoutFull);
      tma_phase ^= 1u << st;
      if (!__all_sync(0xffffffffu, got)) break;
    }
    __syncwarp();
    const long long t2 = prof ? clock64() : 0;
    c_issue += t1 - t0;
    c_wait += t2 - t1;
    c_math -= t2;
    const uint32_t kbase = smem_u32(ring + st * C::STAGE_BYTES);
    const uint32_t vbase = kbase + C::TILE_BYTES;
    const int tile = warp + it * DEC_WARPS;
    const int kpos0 = k0 + tile * KT;

    if constexpr (!T8) {
    float s[NB][4];
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ks += 2) {
          uint32_t kb[4];
          ldsm_x4(kb, kbase + dsw<KT>(j * 8 + (lane & 7), ks * 2 + (lane >> 3)));
          mma_bf16(s[j], qf[ks], kb[0], kb[1]);
          mma_bf16(s[j], qf[ks + 1], kb[2], kb[3]);
        }
      }
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int j = 0; j < NB; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kp = kpos0 + j * 8 + 2 * t4 + e;
          const bool in = kp < k1;
          s[j][e] = (in && kp < lim_lo) ? s[j][e] * p.scale_log2 : -INFINITY;
          s[j][2 + e] = (in && kp < lim_hi) ? s[j][2 + e] * p.scale_log2 : -INFINITY;
          mx_lo = fmaxf(mx_lo, s[j][e]);
          mx_hi = fmaxf(mx_hi, s[j][2 + e]);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float a_lo = mn_lo == -INFINITY ? 1.f : exp2f(m_lo - mn_lo);
      const float a_hi = mn_hi == -INFINITY ? 1.f : exp2f(m_hi - mn_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      l_lo *= a_lo;
      l_hi *= a_hi;
      uint32_t pf[NB / 2][4];
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const float p0 = mn_lo == -INFINITY ? 0.f : exp2f(s[j][0] - mn_lo);
        const float p1 = mn_lo == -INFINITY ? 0.f : exp2f(s[j][1] - mn_lo);
        const float p2 = mn_hi == -INFINITY ? 0.f : exp2f(s[j][2] - mn_hi);
        const float p3 = mn_hi == -INFINITY ? 0.f : exp2f(s[j][3] - mn_hi);
        l_lo += p0 + p1;
        l_hi += p2 + p3;
        pf[j >> 1][(j & 1) * 2] = pack_bf16(p0, p1);
        pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int nb = 0; nb < ONB; ++nb) {
        o[nb][0] *= a_lo;
        o[nb][1] *= a_lo;
        o[nb][2] *= a_hi;
        o[nb][3] *= a_hi;
      }
#pragma unroll
      for (int kk = 0; kk < KT / 16; ++kk) {
#pragma unroll
        for (int nb = 0; nb < ONB; nb += 2) {
          uint32_t vb[4];
          ldsm_x4_t(vb, vbase + dsw<KT>(kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), nb + (lane >> 4)));
          mma_bf16(o[nb], pf[kk], vb[0], vb[1]);
          mma_bf16(o[nb + 1], pf[kk], vb[2], vb[3]);
        }
      }
    } else {
      constexpr int MT = KT / 16;   // 16-key blocks of the tile
      float st[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        st[mt][0] = st[mt][1] = st[mt][2] = st[mt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint32_t ka[4];
          ldsm_x4(ka, kbase + dsw<KT>(mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
          mma_bf16(st[mt], ka, qb[ks][0], qb[ks][1]);
        }
      }
      // st[mt] = {key g4: rows lo, hi | key g4 + 8: rows lo, hi} of key block mt
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kp = kpos0 + mt * 16 + g4 + 8 * e;
          const bool in = kp < k1;
          st[mt][2 * e] = (in && kp < lim_lo) ? st[mt][2 * e] * p.scale_log2 : -INFINITY;
          st[mt][2 * e + 1] = (in && kp < lim_hi) ? st[mt][2 * e + 1] * p.scale_log2 : -INFINITY;
          mx_lo = fmaxf(mx_lo, st[mt][2 * e]);
          mx_hi = fmaxf(mx_hi, st[mt][2 * e + 1]);
        }
      }
#pragma unroll
      for (int sh = 4; sh < 32; sh <<= 1) {   // keys live across the g4 lane groups
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, sh));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, sh));
      }
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float a_lo = mn_lo == -INFINITY ? 1.f : exp2f(m_lo - mn_lo);
      const float a_hi = mn_hi == -INFINITY ? 1.f : exp2f(m_hi - mn_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      l_lo *= a_lo;
      l_hi *= a_hi;
      uint32_t pb[MT][2];   // P^T as B operand: (k = key, n = query row)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float p0 = mn_lo == -INFINITY ? 0.f : exp2f(st[mt][2 * e] - mn_lo);
          const float p1 = mn_hi == -INFINITY ? 0.f : exp2f(st[mt][2 * e + 1] - mn_hi);
          l_lo += p0;
          l_hi += p1;
          pb[mt][e] = movmatrix_trans(pack_bf16(p0, p1));
        }
      }
#pragma unroll
      for (int ob = 0; ob < OB; ++ob) {
        o[ob][0] *= a_lo;
        o[ob][1] *= a_hi;
        o[ob][2] *= a_lo;
        o[ob][3] *= a_hi;
      }
#pragma unroll
      for (int kk = 0; kk < MT; ++kk) {
#pragma unroll
        for (int ob = 0; ob < OB; ++ob) {
          uint32_t va[4];   // V^T block (16 head-dim x 16 keys) through transposing loads
          ldsm_x4_t(va, vbase + dsw<KT>(kk * 16 + ((lane >> 4) & 1) * 8 + (lane & 7), ob * 2 + ((lane >> 3) & 1)));
          mma_bf16(o[ob], va, pb[kk][0], pb[kk][1]);
        }
      }
    }
    if (prof) c_math += clock64();
  }
  const long long t_loop_end = prof ? clock64() : 0;
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
  // ---- merge the 4 warps through each warp's own (now idle) ring
  float* mo = reinterpret_cast<float*>(ring);          // [16][D]
  float* ml = mo + 16 * D;                             // [16][2] (m, l)
  if constexpr (!T8) {
    // Row sums live split over the 4 threads of a row group.
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
#pragma unroll
    for (int nb = 0; nb < OB; ++nb) {
      *reinterpret_cast<float2*>(mo + g4 * D + nb * 8 + 2 * t4) = make_float2(o[nb][0], o[nb][1]);
      *reinterpret_cast<float2*>(mo + (g4 + 8) * D + nb * 8 + 2 * t4) = make_float2(o[nb][2], o[nb][3]);
    }
    if (t4 == 0) {
      ml[g4 * 2] = m_lo;
      ml[g4 * 2 + 1] = l_lo;
      ml[(g4 + 8) * 2] = m_hi;
      ml[(g4 + 8) * 2 + 1] = l_hi;
    }
  } else {
    // Row sums live split over the 8 lane groups that hold different keys.
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
      l_lo += __shfl_xor_sync(0xffffffffu, l_lo, sh);
      l_hi += __shfl_xor_sync(0xffffffffu, l_hi, sh);
    }
#pragma unroll
    for (int ob = 0; ob < OB; ++ob) {
      mo[row_lo * D + ob * 16 + g4] = o[ob][0];
      mo[row_hi * D + ob * 16 + g4] = o[ob][1];
      mo[row_lo * D + ob * 16 + g4 + 8] = o[ob][2];
      mo[row_hi * D + ob * 16 + g4 + 8] = o[ob][3];
    }
    if (g4 == 0) {
      ml[row_lo * 2] = m_lo;
      ml[row_lo * 2 + 1] = l_lo;
      ml[row_hi * 2] = m_hi;
      ml[row_hi * 2 + 1] = l_hi;
    }
  }
  __syncthreads();
  const bool fused_merge = p.splits > 1 && p.split_counter != nullptr;
  const bool direct = p.splits == 1;
  // NVFP4 output goes through `fin` (the Q tile's shared memory: Q lives in registers by now) so that one thread
  // owns a whole 16-element group; values are rounded to bf16 first, as the separate quantiser would see them.
  __nv_bfloat16* fin = reinterpret_cast<__nv_bfloat16*>(qs);
  {
    for (int i = tid; i < nq * D; i += DEC_WARPS * 32) {
      const int qi = i / D, d = i % D;
      float mt = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w)
        mt = fmaxf(mt, reinterpret_cast<const float*>(smem + w * C::WARP_BYTES)[16 * D + qi * 2]);
      float acc = 0.f, lt = 0.f;
      if (mt > -INFINITY) {
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
          const float* wo = reinterpret_cast<const float*>(smem + w * C::WARP_BYTES);
          const float mw = wo[16 * D + qi * 2];
          const float sc = mw == -INFINITY ? 0.f : exp2f(mw - mt);
          acc += sc * wo[qi * D + d];
          lt += sc * wo[16 * D + qi * 2 + 1];
        }
      }
      const float val = lt > 0.f ? acc / lt : 0.f;
      const int rr = qi / g, gg = qi % g;
      const long long rh = static_cast<long long>(row0 + rr) * p.hq + kvh * g + gg;
      if (direct) {
        if (p.q_out == nullptr) p.out[rh * D + d] = __float2bfloat16(val);
        else fin[i] = __float2bfloat16(val);
      } else {
        p.part_o[(rh * p.splits + split) * D + d] = val;
        if (d == 0) p.part_lse[rh * p.splits + split] = lt > 0.f ? mt + log2f(lt) : -INFINITY;
      }
    }
  }
  bool finish = direct && p.q_out != nullptr;
  if (fused_merge) {
    // Last arriver of this (sequence, kv head) merges: every CTA publishes its partial (fence, then one counted
    // arrival); the one that counts splits - 1 before it re-arms the counter and reads all partials back from L2.
    int* last_flag = reinterpret_cast<int*>(smem + C::BAR_OFF + 192);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* cnt = p.split_counter + b * p.hkv + kvh;
      const int old = atomicAdd(cnt, 1);
      const int last = old == p.splits - 1;
      if (last) *cnt = 0;
      *last_flag = last;
    }
    __syncthreads();
    if (*last_flag) {
      __threadfence();
      // The merge is latency-bound (a few hundred values per CTA, every one a chain of L2 reads), so the reads are
      // batched: all log-sum-exps of this (sequence, kv head) land in shared memory in one round trip, then every
      // thread keeps four outputs in flight per pass over the splits.
      float* lse_s = reinterpret_cast<float*>(smem);          // [nq][splits], the rings are idle
      const int S = p.splits;
      for (int i = tid; i < nq * S; i += DEC_WARPS * 32) {
        const int qi = i / S, s2 = i - qi * S;
        const long long rh = static_cast<long long>(row0 + qi / g) * p.hq + kvh * g + qi % g;
        lse_s[i] = __ldcg(p.part_lse + rh * S + s2);
      }
      __syncthreads();
      constexpr int V = 4;
      for (int base = 0; base < nq * D; base += V * DEC_WARPS * 32) {
        float o[V], mx[V], wsum[V];
        long long rhv[V];
        int qv[V], dv[V];
        bool live[V];
#pragma unroll
        for (int v = 0; v < V; ++v) {
          const int i = base + v * DEC_WARPS * 32 + tid;
          live[v] = i < nq * D;
          qv[v] = live[v] ? i / D : 0;
          dv[v] = live[v] ? i % D : 0;
          rhv[v] = static_cast<long long>(row0 + qv[v] / g) * p.hq + kvh * g + qv[v] % g;
          float m = -INFINITY;
          for (int s2 = 0; s2 < S; ++s2) m = fmaxf(m, lse_s[qv[v] * S + s2]);
          mx[v] = m;
          o[v] = 0.f;
          wsum[v] = 0.f;
        }
#pragma unroll 2
        for (int s2 = 0; s2 < S; ++s2) {
          float x[V];
#pragma unroll
          for (int v = 0; v < V; ++v) x[v] = live[v] ? __ldcg(p.part_o + (rhv[v] * S + s2) * D + dv[v]) : 0.f;
#pragma unroll
          for (int v = 0; v < V; ++v) {
            const float w = mx[v] > -INFINITY ? exp2f(lse_s[qv[v] * S + s2] - mx[v]) : 0.f;
            if (w > 0.f) o[v] += w * x[v];
            wsum[v] += w;
          }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
          if (!live[v]) continue;
          const float r = wsum[v] > 0.f ? o[v] / wsum[v] : 0.f;
          const int i = base + v * DEC_WARPS * 32 + tid;
          if (p.q_out == nullptr) p.out[rhv[v] * D + dv[v]] = __float2bfloat16(r);
          else fin[i] = __float2bfloat16(r);
        }
      }
      finish = p.q_out != nullptr;
    }
  }
  if (finish) {
    __syncthreads();
    const float inv_gs = 1.f / *p.q_gscale;
    constexpr int GPR = D / 16;   // groups per (row, head)
    for (int it = tid; it < nq * GPR; it += DEC_WARPS * 32) {
      const int qi = it / GPR, gi = it % GPR;
      float x[16];
      load16(fin + qi * D + gi * 16, x);
      uint2 packed;
      const uint32_t sfb = quant16(x, inv_gs, &packed);
      const int rr = qi / g, gg = qi % g;
      const int row = row0 + rr, head = kvh * g + gg;
      *reinterpret_cast<uint2*>(p.q_out + (static_cast<size_t>(row) * p.hq + head) * (D / 2) + gi * 8) = packed;
      p.q_sf[row_sf_off(row, head * GPR + gi, p.q_ka)] = static_cast<uint8_t>(sfb);
    }
  }
  if (prof) {
    const long long t_end = clock64();
    atomicAdd(p.prof + 0, static_cast<unsigned long long>(c_issue));
    atomicAdd(p.prof + 1, static_cast<unsigned long long>(c_wait));
    atomicAdd(p.prof + 2, static_cast<unsigned long long>(c_math));
    atomicAdd(p.prof + 3, static_cast<unsigned long long>(t_loop_end - t_start));
    atomicAdd(p.prof + 4, static_cast<unsigned long long>(t_end - t_loop_end));
    atomicAdd(p.prof + 5, static_cast<unsigned long long>((ntiles + DEC_WARPS - 1 - warp) / DEC_WARPS));
    atomicAdd(p.prof + 6, 1ull);
  }
}

template <int D, bool T8>
int launch_decode(const DecParams& p0, const void* k_pool, const void* v_pool, long long pool_slots, int batch,
                  cudaStream_t st) {
  DecParams p = p0;
  using C = DecCfg<D>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_decode_kernel<D, T8>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) !=
        cudaSuccess)
      return 3;
    attr = true;
  }
  static const CUtensorMap dummy = {};
  const CUtensorMap *tk = &dummy, *tv = &dummy;
  const KvTma t = make_kv_tma(k_pool, v_pool, p.pool_stride, p.head_stride, pool_slots, p.hkv, D, C::KT);
  p.use_tma = t.ok;
  p.tma_xh = t.xh;
  p.tma_yh = t.yh;
  if (t.ok) {
    tk = &t.k;
    tv = &t.v;
  }
  launch_dep(attn_decode_kernel<D, T8>, dim3(batch, p.hkv, p.splits), dim3(DEC_WARPS * 32), C::SMEM, st, *tk, *tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace
}  // namespace hb

using namespace hb;

static unsigned long long* g_dec_prof = nullptr;
struct DecFuse {
  int* counter = nullptr;
  void* q_out = nullptr;
  void* q_sf = nullptr;
  const void* q_gscale = nullptr;
  int q_ka = 0;
};
static thread_local DecFuse g_dec_fuse;

extern "C" {

// Cycle counters of warp 0 of every CTA, summed: `buf` = 8 zeroed uint64 on the device (null switches it off).
// [0] issuing copies, [1] waiting for a tile, [2] tile math, [3] main loop, [4] merge + store, [5] tiles of warp 0,
// [6] CTAs.
void hb_attn_decode_profile(void* buf) { g_dec_prof = static_cast<unsigned long long*>(buf); }

// Arms the fused tail for the NEXT hb_attn_decode call of this thread (consumed by that call): `split_counter`
// (one zeroed int per sequence x kv head, re-armed by the kernel) makes the last-arriving split CTA merge the
// partials, so no hb_attn_merge follows; q_out / q_sf / q_gscale (may be null) make the kernel write the rows as
// NVFP4 instead of bf16 (`out` is then not written).
void hb_attn_decode_fuse(void* split_counter, void* q_out, void* q_sf, const void* q_gscale, int q_ka) {
  g_dec_fuse.counter = static_cast<int*>(split_counter);
  g_dec_fuse.q_out = q_out; g_dec_fuse.q_sf = q_sf; g_dec_fuse.q_gscale = q_gscale; g_dec_fuse.q_ka = q_ka;
}

// bf16 KV only; rows_per_seq * (hq / hkv) must be <= 16. Partials go through hb_attn_merge when splits > 1 unless
// hb_attn_decode_fuse armed the in-kernel merge.
int hb_attn_decode(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                   long long head_stride,
                   const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len,
                   const void* q_indptr, void* out, void* part_o, void* part_lse, int batch, int max_rows, int hq,
                   int hkv, int d, int splits, float scale, int causal, long long pool_slots, void* status,
                   void* stream) {
  if (batch <= 0) return 0;
  if (hq % hkv != 0 || max_rows * (hq / hkv) > 16) return 1;
  DecParams p;
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
  p.part_o = static_cast<float*>(part_o);
  p.part_lse = static_cast<float*>(part_lse);
  p.hq = hq; p.hkv = hkv; p.splits = splits < 1 ? 1 : splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = static_cast<int*>(status);
  p.prof = g_dec_prof;
  p.split_counter = g_dec_fuse.counter;
  p.q_out = static_cast<uint8_t*>(g_dec_fuse.q_out);
  p.q_sf = static_cast<uint8_t*>(g_dec_fuse.q_sf);
  p.q_gscale = static_cast<const float*>(g_dec_fuse.q_gscale);
  p.q_ka = g_dec_fuse.q_ka;
  g_dec_fuse = DecFuse{};
  if (p.q_out != nullptr && p.splits > 1 && p.split_counter == nullptr) return 1;
  if (p.splits > 1 && (part_o == nullptr || part_lse == nullptr)) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool t8 = max_rows * (hq / hkv) <= 8;
  if (d == 64) return t8 ? launch_decode<64, true>(p, k_pool, v_pool, pool_slots, batch, st)
                         : launch_decode<64, false>(p, k_pool, v_pool, pool_slots, batch, st);
  if (d == 128) return t8 ? launch_decode<128, true>(p, k_pool, v_pool, pool_slots, batch, st)
                          : launch_decode<128, false>(p, k_pool, v_pool, pool_slots, batch, st);
  if (d == 256) return t8 ? launch_decode<256, true>(p, k_pool, v_pool, pool_slots, batch, st)
                          : launch_decode<256, false>(p, k_pool, v_pool, pool_slots, batch, st);
  return 1;
}

}  // extern "C"
