// Paged GQA prefill attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA owns one (sequence, kv head, block of query tokens). The block's query rows are packed as
// (token, group member) pairs, 128 rows = floor(128 / g) tokens x g query heads of the kv head, so a K / V tile
// gathered once from the token-granular pool serves the whole GQA group. Per 128-key tile:
//
//   producers (3 warps)   gather K and V rows by slot id with 16-byte cp.async into 128-byte-swizzled tiles
//                         (the layout TMA would produce; rows of a paged pool are not a TMA box), 2 stages;
//   issuer (1 lane)       S = Q K^T (kind::f16, both operands K-major) into TMEM columns [0, 128); after the
//                         softmax warps have published P, PV = P V (V as MN-major B operand) into [128, 128 + D);
//   softmax (4 warps)     thread r owns query row r = TMEM lane r: two passes over S (row max, then exp2 and the
//                         bf16 P tile into swizzled shared memory), then O = O * alpha + PV in registers.
//
// S for tile t + 1 is issued right after PV for tile t, so it overlaps the O update. Causal masking follows the
// ragged-batch rule of the engine: row token j of a sequence with R new rows and context ctx sees keys
// [0, ctx - R + j]. All waits are bounded; a timeout raises the status word and every role leaves.
//
// Replaces the reference's FlashInfer ragged-prefill wrapper + prefix kernel + LSE merge
// (hibana/kernels/ops.py:131-161, hibana/model/attention.py:73-96, hibana/kernels/csrc/verify_attn.cu prefix_kernel).
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int PF_THREADS = 256;
constexpr int PF_ROWS = 128;      // packed query rows per CTA
constexpr int PF_KT = 128;        // keys per tile
constexpr int PF_STAGES = 2;
constexpr int PF_PRODUCERS = 96;  // warps 4, 5, 6

struct PfParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  long long pool_stride;
  const int* kv_indices;
  long long ld_idx;
  const int* seq_rows;
  const int* ctx_len;
  const int* q_indptr;
  __nv_bfloat16* out;
  int hq, hkv;
  float scale_log2;
  int causal;
  int* status;
};

template <int D>
struct PfCfg {
  static constexpr int HALVES = D / 64;                      // 64-element (128-byte) column blocks of a row
  static constexpr int Q_BYTES = PF_ROWS * D * 2;
  static constexpr int KV_TILE = PF_KT * D * 2;              // one of K or V
  static constexpr int STAGE_BYTES = 2 * KV_TILE;
  static constexpr int P_BYTES = PF_ROWS * PF_KT * 2;
  static constexpr int BAR_OFF = Q_BYTES + PF_STAGES * STAGE_BYTES + P_BYTES;
  static constexpr int SMEM = BAR_OFF + 256 + 1024;
  static constexpr int TMEM_COLS = PF_KT + D <= 256 ? 256 : 512;
};

__device__ __forceinline__ void cp16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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
__global__ void __launch_bounds__(PF_THREADS, 1) attn_prefill_kernel(const PfParams p) {
  using C = PfCfg<D>;
  constexpr int CPR = D / 8;   // 16-byte chunks per row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + C::Q_BYTES;
  uint8_t* p_s = kv_s + PF_STAGES * C::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  uint64_t* empty = full + PF_STAGES;
  uint64_t* s_ready = empty + PF_STAGES;
  uint64_t* p_ready = s_ready + 1;
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
  const int ntiles = (kmax + PF_KT - 1) / PF_KT;

  if (tid == 0) {
    for (int s = 0; s < PF_STAGES; ++s) {
      mbar_init(&full[s], PF_PRODUCERS);
      mbar_init(&empty[s], 1);
    }
    mbar_init(s_ready, 1);
    mbar_init(p_ready, PF_ROWS);
    mbar_init(pv_ready, 1);
    *abort = 0;
    fence_mbar_init();
  }
  if (warp == 7) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t s_tmem = tmem_base;
  const uint32_t pv_tmem = tmem_base + PF_KT;

  if (warp >= 4 && warp < 7) {
    // ------------------------------------------------------------------ producers
    const int ptid = tid - 128;
    const int* idx_row = p.kv_indices + static_cast<long long>(p.seq_rows ? p.seq_rows[b] : b) * p.ld_idx;
    // Q rows (zero padded), covered by the first stage's barrier.
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
    bool live = true;
    // Thread layout of a tile copy: 16 consecutive threads move one 256-byte (D = 128) row, so a thread keeps its
    // 16-byte column `part` and walks rows rg, rg + RG, ...; the rows' slot ids are fetched (one broadcast load
    // per row) before the stage wait, so their latency hides behind it.
    constexpr int RG = PF_PRODUCERS / CPR;                    // rows per pass over the producer threads
    constexpr int NR = (PF_KT + RG - 1) / RG;                 // rows per thread and tile
    const int part = ptid % CPR, rg = ptid / CPR;
    const uint32_t part_off = static_cast<uint32_t>((part >> 3) * PF_KT * 128);
    const long long col = static_cast<long long>(kvh) * D + part * 8;
    for (int t = 0; t < ntiles; ++t) {
      const int s = t % PF_STAGES;
      const int k0 = t * PF_KT;
      int slot[NR];
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = rg + i * RG;
        slot[i] = (r < PF_KT && k0 + r < kmax) ? __ldg(idx_row + k0 + r) : -1;
      }
      if (t >= 1) {
        // Tile t - 1 was issued a whole tile period ago: it has landed. Make it visible to the tensor-core proxy
        // and signal it before (possibly) sleeping on this tile's stage.
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        fence_proxy_async_smem();
        mbar_arrive(&full[(t - 1) % PF_STAGES]);
      }
      if (t >= PF_STAGES && !mbar_wait(&empty[s], ((t / PF_STAGES) - 1) & 1, abort, p.status, kTimeoutEmpty)) {
        live = false;
        break;
      }
      const uint32_t kdst = smem_u32(kv_s + s * C::STAGE_BYTES) + part_off;
      const uint32_t vdst = kdst + C::KV_TILE;
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int r = rg + i * RG;
        if (r < PF_KT) {
          const uint32_t off = static_cast<uint32_t>(r * 128 + (((part & 7) ^ (r & 7)) << 4));
          if (slot[i] >= 0) {
            const long long src = static_cast<long long>(slot[i]) * p.pool_stride + col;
            cp16(kdst + off, p.k_pool + src);
            cp16(vdst + off, p.v_pool + src);
          } else {
            st_zero16(kdst + off);
            st_zero16(vdst + off);
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");   // nothing may land after the CTA has gone
    fence_proxy_async_smem();
    if (live && ntiles > 0) mbar_arrive(&full[(ntiles - 1) % PF_STAGES]);
  } else if (warp == 7) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(PF_ROWS, PF_KT);
      constexpr uint32_t idesc_pv = make_idesc_bf16(PF_ROWS, D, 0, 1);
      const uint32_t q_a = smem_u32(q_s), p_a = smem_u32(p_s);
      auto issue_qk = [&](int t) {
        const uint32_t k_a = smem_u32(kv_s + (t % PF_STAGES) * C::STAGE_BYTES);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t in_row = (ks & 3) * 32;   // 16 elements = 32 bytes inside the 128-byte swizzled row
          mma_f16(s_tmem, make_desc_sw128(q_a + (ks >> 2) * (PF_ROWS * 128) + in_row),
                  make_desc_sw128(k_a + (ks >> 2) * (PF_KT * 128) + in_row), idesc_qk, ks > 0 ? 1u : 0u);
        }
        tc_commit(s_ready);
      };
      bool ok = ntiles > 0 && mbar_wait(&full[0], 0, abort, p.status, kTimeoutFull);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int t = 0; ok && t < ntiles; ++t) {
        if (!mbar_wait(p_ready, t & 1, abort, p.status, kTimeoutAccum)) break;
        tc_fence_after();
        const uint32_t v_a = smem_u32(kv_s + (t % PF_STAGES) * C::STAGE_BYTES) + C::KV_TILE;
#pragma unroll
        for (int kk = 0; kk < PF_KT / 16; ++kk) {
          const uint64_t adesc = make_desc_sw128(p_a + (kk >> 2) * (PF_ROWS * 128) + (kk & 3) * 32);
          // 16 keys = two 8-row groups 1024 bytes apart; the D / 64 column blocks are PF_KT * 128 bytes apart
          const uint64_t bdesc = make_desc_sw128_mn(v_a + kk * 2048, PF_KT * 128, 1024);
          mma_f16(pv_tmem, adesc, bdesc, idesc_pv, kk > 0 ? 1u : 0u);
        }
        tc_commit(pv_ready);
        tc_commit(&empty[t % PF_STAGES]);
        if (t + 1 < ntiles) {
          if (!mbar_wait(&full[(t + 1) % PF_STAGES], ((t + 1) / PF_STAGES) & 1, abort, p.status, kTimeoutFull)) break;
          tc_fence_after();
          issue_qk(t + 1);
        }
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
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const uint32_t p_row = smem_u32(p_s) + r * 128;
    bool ok = true;
    for (int t = 0; t < ntiles; ++t) {
      if (!mbar_wait(s_ready, t & 1, abort, p.status, kTimeoutAccum)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int k0 = t * PF_KT;
      // A tile entirely at or before the row's last visible key needs no masking (the common case); four
      // independent accumulators keep the dependency chains short (one softmax warp per scheduler: no other
      // warp hides ALU latency).
      const bool full_vis = k0 + PF_KT - 1 <= lim;
      // pass 1: row maximum of the visible scores
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c0 = 0; c0 < PF_KT; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_tmem + tlane + c0, v);
        tmem_ld_wait();
        if (full_vis) {
#pragma unroll
          for (int j = 0; j < 32; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(v[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (k0 + c0 + j <= lim) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(v[j]));
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float alpha = m_new == -INFINITY ? 1.f : ex2(m - m_new);
      const float neg_m = m_new == -INFINITY ? 0.f : -m_new;
      m = m_new;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      // pass 2: probabilities, row sum, bf16 P tile (K-major, swizzled) for the second MMA
#pragma unroll
      for (int c0 = 0; c0 < PF_KT; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_tmem + tlane + c0, v);
        tmem_ld_wait();
        uint32_t w[16];
        if (full_vis) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float p0 = ex2(fmaf(__uint_as_float(v[j]), p.scale_log2, neg_m));
            const float p1 = ex2(fmaf(__uint_as_float(v[j + 1]), p.scale_log2, neg_m));
            sum4[(j >> 1) & 3] += p0 + p1;
            w[j >> 1] = pack_bf16(p0, p1);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float p0 = k0 + c0 + j <= lim ? ex2(fmaf(__uint_as_float(v[j]), p.scale_log2, neg_m)) : 0.f;
            const float p1 = k0 + c0 + j + 1 <= lim ? ex2(fmaf(__uint_as_float(v[j + 1]), p.scale_log2, neg_m)) : 0.f;
            sum4[(j >> 1) & 3] += p0 + p1;
            w[j >> 1] = pack_bf16(p0, p1);
          }
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
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l = l * alpha + sum;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(p_ready);
      if (!mbar_wait(pv_ready, t & 1, abort, p.status, kTimeoutAccum)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(pv_tmem + tlane + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) o[c0 + j] = fmaf(o[c0 + j], alpha, __uint_as_float(v[j]));
      }
      tc_fence_before();
    }
    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (static_cast<long long>(row0 + tok) * p.hq + kvh * g + r % g) * D;
#pragma unroll
      for (int c = 0; c < D; c += 8)
        *reinterpret_cast<uint4*>(dst + c) =
            make_uint4(pack_bf16(o[c] * inv, o[c + 1] * inv), pack_bf16(o[c + 2] * inv, o[c + 3] * inv),
                       pack_bf16(o[c + 4] * inv, o[c + 5] * inv), pack_bf16(o[c + 6] * inv, o[c + 7] * inv));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 7) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D>
int launch_prefill(const PfParams& p, int qblocks, int batch, cudaStream_t st) {
  using C = PfCfg<D>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) !=
        cudaSuccess)
      return 3;
    attr = true;
  }
  attn_prefill_kernel<D><<<dim3(qblocks, p.hkv, batch), PF_THREADS, C::SMEM, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

// bf16 KV, head dim 64 or 128, group size hq / hkv <= 128. `max_rows` bounds the new rows of any sequence.
int hb_attn_prefill(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                    const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len,
                    const void* q_indptr, void* out, int batch, int max_rows, int hq, int hkv, int d, float scale,
                    int causal, void* status, void* stream) {
  if (batch <= 0 || max_rows <= 0) return 0;
  if (hq % hkv != 0 || hq / hkv > PF_ROWS) return 1;
  PfParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pool = static_cast<const __nv_bfloat16*>(k_pool);
  p.v_pool = static_cast<const __nv_bfloat16*>(v_pool);
  p.pool_stride = pool_stride;
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
  const int tok_per_blk = PF_ROWS / (hq / hkv);
  const int qblocks = (max_rows + tok_per_blk - 1) / tok_per_blk;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d == 64) return launch_prefill<64>(p, qblocks, batch, st);
  if (d == 128) return launch_prefill<128>(p, qblocks, batch, st);
  return 1;
}

}  // extern "C"
