// Paged GQA attention over the token-granular KV pool (split-KV, CUDA-core path).
//
// The KV pool stores one row per token slot: k_pool / v_pool [slots, kv_heads, D] (bf16 or e4m3). A sequence's
// context is a row of the block table `kv_indices[b, 0..ctx)` (slot of every position), so radix-tree prefix
// sharing is token-granular. One CTA owns (sequence, kv head, query-row chunk, KV split): it streams K/V tiles
// of 64 keys through a cp.async double buffer, scores them for all query rows that share the kv head (GQA
// group x up to a few tokens), keeps an online softmax, and writes either the final output or a partial with
// its log-sum-exp for the merge kernel. The KV range of a split is computed on the device from ctx_len, so one
// captured launch serves any context length.
//
// Rows per sequence R >= 1 covers decode (R = 1), speculative verify (R = k + 1 <= 16, causal inside the block)
// and, as a slow general fallback, chunked prefill. Reference counterparts: FlashInfer decode / paged prefill
// wrappers planned in hibana/engine/executor.py:161-169 and hibana/kernels/csrc/verify_attn.cu:299-660.
#include "hb_api.h"
#include "hb_common.cuh"
#include "rownorm.cuh"

namespace hb {
namespace {

constexpr int TK = 64;         // keys per tile
constexpr int ATT_THREADS = 128;

struct AttnParams {
  const __nv_bfloat16* q;      // [T, Hq, D]
  const void* k_pool;
  const void* v_pool;
  long long pool_stride;       // elements between slots
  long long head_stride;       // elements between kv heads
  const int* kv_indices;       // [B, ld_idx]
  long long ld_idx;
  const int* ctx_len;          // [B] keys visible to the last query row of the sequence
  const int* seq_rows;         // [B] row of each sequence in kv_indices (null = identity)
  const int* q_indptr;         // [B + 1] query row offsets; null = one row per sequence
  __nv_bfloat16* out;          // [T, Hq, D]
  float* part_o;               // [T, Hq, S, D]
  float* part_lse;             // [T, Hq, S]
  int hq, hkv, splits, rows_per_cta;
  float scale_log2;            // softmax scale * log2(e)
  float kv_scale;              // dequant scale of fp8 / nvfp4 KV
  int causal;
  // NVFP4 KV (format 2): k_pool / v_pool hold packed e2m1 rows (D / 2 bytes, strides in bytes); these hold the
  // ue4m3 scale of every 16 elements, rows of D / 16 bytes
  const uint8_t* k_sf;
  const uint8_t* v_sf;
  long long sf_pool_stride, sf_head_stride;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void cp_async_small(void* smem, const void* gmem) {   // N = 4, 8 or 16 bytes
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(smem_u32(smem)), "l"(gmem), "n"(N) : "memory");
}

// 16 e2m1 codes (8 bytes) times their block scale -> floats.
__device__ __forceinline__ void unpack_fp4_block(const uint8_t* p, float sf, float* f) {
  const uint2 a = *reinterpret_cast<const uint2*>(p);
  const uint32_t w[2] = {a.x, a.y};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t h2;
      const uint16_t in = static_cast<uint16_t>((w[i] >> (8 * j)) & 0xFFu);
      asm("{\n\t.reg .b8 t;\n\tcvt.u8.u16 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h2) : "h"(in));
      const __half2 hv = *reinterpret_cast<const __half2*>(&h2);
      f[8 * i + 2 * j] = __low2float(hv) * sf;
      f[8 * i + 2 * j + 1] = __high2float(hv) * sf;
    }
  }
}

template <int FMT>
__device__ __forceinline__ void unpack16(const uint8_t* p, float* f, int* n) {
  constexpr bool FP8 = FMT == 1;
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
  if constexpr (FP8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) f[4 * i + j] = e4m3_to_float((w[i] >> (8 * j)) & 0xFF);
    }
    *n = 16;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = bf16_lo(w[i]);
      f[2 * i + 1] = bf16_hi(w[i]);
    }
    *n = 8;
  }
}

template <int D, int FMT>
struct AttRow {
  static constexpr bool FP4 = FMT == 2;
  static constexpr int ESZ = FMT == 0 ? 2 : 1;              // bytes per element of the copied row (fp4: per BYTE)
  static constexpr int VAL_BYTES = FP4 ? D / 2 : D * ESZ;   // packed values of a row
  static constexpr int SF_BYTES = FP4 ? D / 16 : 0;         // block scales of a row (fp4)
  static constexpr int ROWB = ((VAL_BYTES + SF_BYTES + 15) / 16) * 16 + 16;   // padded: conflict-free 16-byte reads
  static constexpr int CHUNKS = VAL_BYTES / 16;
};

template <int D, int MAXQ, int FMT>
__global__ void __launch_bounds__(ATT_THREADS) attn_splitkv_kernel(const AttnParams p) {
  using RL = AttRow<D, FMT>;
  constexpr bool FP8 = FMT == 1, FP4 = FMT == 2, SCALED = FMT != 0;
  constexpr int ESZ = RL::ESZ;
  constexpr int ROWB = RL::ROWB;
  constexpr int CHUNKS = RL::CHUNKS;
  constexpr int EPC = FP4 ? 16 : 16 / ESZ;   // elements handled per score step (fp4: one 16-element scale block)
  constexpr int STEPS = FP4 ? D / 16 : CHUNKS;
  constexpr int HALFQ = (MAXQ + 1) / 2;
  constexpr int DPT = D > 128 ? D / 128 : 1;  // dims per thread in the PV phase

  extern __shared__ uint8_t smem_raw[];
  uint8_t* kbuf = smem_raw;                              // [2][TK][ROWB]
  uint8_t* vbuf = kbuf + 2 * TK * ROWB;                  // [2][TK][ROWB]
  float* qs = reinterpret_cast<float*>(vbuf + 2 * TK * ROWB);  // [MAXQ][D]
  float* sc = qs + MAXQ * D;                             // [MAXQ][TK + 1]
  float* pt = sc + MAXQ * (TK + 1);                      // [TK][MAXQ]
  float* m_s = pt + TK * MAXQ;                           // [MAXQ]
  float* l_s = m_s + MAXQ;
  float* a_s = l_s + MAXQ;
  int* idx_s = reinterpret_cast<int*>(a_s + MAXQ);       // [2][TK]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;
  const int kvh = blockIdx.y % p.hkv;
  const int rchunk = blockIdx.y / p.hkv;
  const int split = blockIdx.z;
  const int g = p.hq / p.hkv;
  const int row0 = p.q_indptr ? p.q_indptr[b] : b;
  const int R = p.q_indptr ? p.q_indptr[b + 1] - row0 : 1;
  const int r0 = rchunk * p.rows_per_cta;
  if (r0 >= R) return;
  const int nrows = min(p.rows_per_cta, R - r0);
  const int nq = nrows * g;
  const int ctx = p.ctx_len[b];
  // Keys this CTA needs: causal limit of its last row, then the split's slice.
  const int need = p.causal ? ctx - R + r0 + nrows : ctx;
  const int per = (((ctx + p.splits - 1) / p.splits + TK - 1) / TK) * TK;
  const int k0 = split * per;
  const int k1 = min(need, k0 + per);
  const int ntiles = k1 > k0 ? (k1 - k0 + TK - 1) / TK : 0;

  for (int i = tid; i < MAXQ * D; i += ATT_THREADS) {
    const int qi = i / D, d = i % D;
    float v = 0.f;
    if (qi < nq) {
      const int rr = qi / g, gg = qi % g;
      v = __bfloat162float(p.q[(static_cast<long long>(row0 + r0 + rr) * p.hq + kvh * g + gg) * D + d]) * p.scale_log2;
    }
    qs[i] = v;
  }
  if (tid < MAXQ) {
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
  }
  float acc[MAXQ][DPT];
#pragma unroll
  for (int i = 0; i < MAXQ; ++i)
#pragma unroll
    for (int j = 0; j < DPT; ++j) acc[i][j] = 0.f;

  const int* idx_row = p.kv_indices + static_cast<long long>(p.seq_rows ? p.seq_rows[b] : b) * p.ld_idx;
  const uint8_t* kp = static_cast<const uint8_t*>(p.k_pool);
  const uint8_t* vp = static_cast<const uint8_t*>(p.v_pool);

  auto load_tile = [&](int t, int buf) {
    const int base = k0 + t * TK;
    // Slot ids are read straight from global by every thread for its own chunks (L1/L2 hits).
    constexpr int PARTS = CHUNKS + (FP4 ? 1 : 0);      // fp4: one more copy per row for its block scales
    for (int c = tid; c < TK * PARTS; c += ATT_THREADS) {
      const int key = c / PARTS, part = c % PARTS;
      const int kpos = base + key;
      uint8_t* kd = kbuf + (buf * TK + key) * ROWB + part * 16;
      uint8_t* vd = vbuf + (buf * TK + key) * ROWB + part * 16;
      if (kpos < k1) {
        if (FP4 && part == CHUNKS) {
          const long long so = static_cast<long long>(idx_row[kpos]) * p.sf_pool_stride +
                               static_cast<long long>(kvh) * p.sf_head_stride;
          cp_async_small<RL::SF_BYTES ? RL::SF_BYTES : 4>(kd, p.k_sf + so);
          cp_async_small<RL::SF_BYTES ? RL::SF_BYTES : 4>(vd, p.v_sf + so);
        } else {
          const long long off = (static_cast<long long>(idx_row[kpos]) * p.pool_stride + static_cast<long long>(kvh) * p.head_stride) * ESZ + part * 16;
          cp_async16(kd, kp + off);
          cp_async16(vd, vp + off);
        }
      } else {
        *reinterpret_cast<uint4*>(kd) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(vd) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };

  if (ntiles > 0) load_tile(0, 0);
  for (int t = 0; t < ntiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < ntiles) {
      load_tile(t + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // ---- scores: two threads per key, each takes every other query row
    {
      const int key = tid & (TK - 1);
      const int qpar = tid >> 6;  // 0 or 1
      float s[HALFQ];
#pragma unroll
      for (int i = 0; i < HALFQ; ++i) s[i] = 0.f;
      const uint8_t* krow = kbuf + (buf * TK + key) * ROWB;
#pragma unroll 2
      for (int c = 0; c < STEPS; ++c) {
        float kf[16];
        int n;
        if constexpr (FP4) unpack_fp4_block(krow + c * 8, e4m3_to_float(krow[RL::VAL_BYTES + c]), kf);
        else unpack16<FMT>(krow + c * 16, kf, &n);
#pragma unroll
        for (int i = 0; i < HALFQ; ++i) {
          const int qi = 2 * i + qpar;
          if (qi < nq) {
            const float4* qv = reinterpret_cast<const float4*>(qs + qi * D + c * EPC);
#pragma unroll
            for (int e = 0; e < EPC / 4; ++e) {
              const float4 qq = qv[e];
              s[i] += kf[4 * e] * qq.x + kf[4 * e + 1] * qq.y + kf[4 * e + 2] * qq.z + kf[4 * e + 3] * qq.w;
            }
          }
        }
      }
      const int kpos = k0 + t * TK + key;
#pragma unroll
      for (int i = 0; i < HALFQ; ++i) {
        const int qi = 2 * i + qpar;
        if (qi < nq) {
          const int rr = qi / g;
          const int limit = p.causal ? ctx - R + r0 + rr + 1 : ctx;  // keys [0, limit) are visible
          float v = s[i];
          if (SCALED) v *= p.kv_scale;
          sc[qi * (TK + 1) + key] = (kpos < limit && kpos < k1) ? v : -INFINITY;
        }
      }
    }
    __syncthreads();
    // ---- online softmax: one warp per query row
    for (int qi = warp; qi < nq; qi += ATT_THREADS / 32) {
      const float s0 = sc[qi * (TK + 1) + lane], s1 = sc[qi * (TK + 1) + lane + 32];
      const float mx = warp_max(fmaxf(s0, s1));
      const float m_old = m_s[qi];
      const float m_new = fmaxf(m_old, mx);
      float p0 = 0.f, p1 = 0.f, alpha = 1.f;
      if (m_new > -INFINITY) {
        p0 = exp2f(s0 - m_new);
        p1 = exp2f(s1 - m_new);
        alpha = exp2f(m_old - m_new);
      }
      const float sum = warp_sum(p0 + p1);
      pt[lane * MAXQ + qi] = p0;
      pt[(lane + 32) * MAXQ + qi] = p1;
      if (lane == 0) {
        m_s[qi] = m_new;
        l_s[qi] = l_s[qi] * alpha + sum;
        a_s[qi] = alpha;
      }
    }
    __syncthreads();
    // ---- PV: thread owns output dims, loops over keys
    if (tid < D || D >= 128) {
#pragma unroll
      for (int i = 0; i < MAXQ; ++i) {
        if (i < nq) {
          const float a = a_s[i];
#pragma unroll
          for (int j = 0; j < DPT; ++j) acc[i][j] *= a;
        }
      }
      const uint8_t* vb = vbuf + buf * TK * ROWB;
      for (int key = 0; key < TK; ++key) {
        float vv[DPT];
#pragma unroll
        for (int j = 0; j < DPT; ++j) {
          const int d = tid + j * 128;
          if constexpr (FP4) {
            const uint8_t byte = vb[key * ROWB + (d >> 1)];
            vv[j] = e2m1_to_float((byte >> ((d & 1) * 4)) & 0xF) * e4m3_to_float(vb[key * ROWB + RL::VAL_BYTES + (d >> 4)]);
          } else if constexpr (FP8) vv[j] = e4m3_to_float(vb[key * ROWB + d]);
          else vv[j] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(vb + key * ROWB + d * 2));
        }
        const float* pr = pt + key * MAXQ;
#pragma unroll
        for (int i = 0; i < MAXQ; i += 4) {
          const float4 pp = *reinterpret_cast<const float4*>(pr + i);
          const float pv[4] = {pp.x, pp.y, pp.z, pp.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (i + e < MAXQ) {
#pragma unroll
              for (int j = 0; j < DPT; ++j) acc[i + e][j] += pv[e] * vv[j];
            }
        }
      }
    }
    __syncthreads();
  }

  // ---- epilogue
  if (tid < D || D >= 128) {
#pragma unroll
    for (int i = 0; i < MAXQ; ++i) {
      if (i < nq) {
        const int rr = i / g, gg = i % g;
        const long long row = row0 + r0 + rr;
        const int head = kvh * g + gg;
        const float l = l_s[i];
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int j = 0; j < DPT; ++j) {
          const int d = tid + j * 128;
          float o = acc[i][j] * inv;
          if (SCALED) o *= p.kv_scale;
          if (p.splits == 1) p.out[(row * p.hq + head) * D + d] = __float2bfloat16(o);
          else p.part_o[((row * p.hq + head) * p.splits + split) * D + d] = o;
        }
        if (p.splits > 1 && tid == 0)
          p.part_lse[(row * p.hq + head) * p.splits + split] = l > 0.f ? m_s[i] + log2f(l) : -INFINITY;
      }
    }
  }
}

// Merge of split partials: o = sum_s 2^(lse_s - m) o_s / sum_s 2^(lse_s - m). One CTA per (row, head).
// With q_out the merged row is written as NVFP4 (the activation operand of the output projection) instead of
// bf16: values are rounded to bf16 first, as a separate quantiser would see them, then one thread per 16-element
// group packs them and writes the group's scale into the swizzled block layout.
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                  __nv_bfloat16* __restrict__ out, int splits, int d, int hq,
                                  uint8_t* __restrict__ q_out, uint8_t* __restrict__ q_sf,
                                  const float* __restrict__ q_gscale, int q_ka) {
  grid_dep_wait();     // may run as a programmatic dependent of the split kernel
  grid_dep_launch();
  __shared__ __align__(32) __nv_bfloat16 fin[256];
  const long long rh = blockIdx.x;
  const float* lse = part_lse + rh * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, lse[s]);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float o = 0.f, wsum = 0.f;
    if (m > -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float w = exp2f(lse[s] - m);
        if (w > 0.f) o += w * part_o[(rh * splits + s) * d + i];
        wsum += w;
      }
      o /= wsum;
    }
    if (q_out == nullptr) out[rh * d + i] = __float2bfloat16(o);
    else fin[i] = __float2bfloat16(o);
  }
  if (q_out != nullptr) {
    __syncthreads();
    const int gpr = d >> 4;
    if (static_cast<int>(threadIdx.x) < gpr) {
      const int gi = threadIdx.x;
      const int row = static_cast<int>(rh / hq), head = static_cast<int>(rh % hq);
      float x[16];
      load16(fin + gi * 16, x);
      uint2 packed;
      const uint32_t sfb = quant16(x, 1.f / *q_gscale, &packed);
      *reinterpret_cast<uint2*>(q_out + static_cast<size_t>(rh) * (d >> 1) + gi * 8) = packed;
      q_sf[row_sf_off(row, head * gpr + gi, q_ka)] = static_cast<uint8_t>(sfb);
    }
  }
}

template <int D, int MAXQ, int FP8>
size_t attn_smem_bytes() {
  constexpr int ROWB = AttRow<D, FP8>::ROWB;
  return static_cast<size_t>(4) * TK * ROWB + sizeof(float) * (MAXQ * D + MAXQ * (TK + 1) + TK * MAXQ + 3 * MAXQ) +
         sizeof(int) * 2 * TK;
}

template <int D, int MAXQ, int FP8>
int launch_attn(const AttnParams& p, int batch, int row_chunks, cudaStream_t st) {
  const size_t smem = attn_smem_bytes<D, MAXQ, FP8>();
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_splitkv_kernel<D, MAXQ, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return 3;
    attr = true;
  }
  const dim3 grid(batch, p.hkv * row_chunks, p.splits);
  attn_splitkv_kernel<D, MAXQ, FP8><<<grid, ATT_THREADS, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

template <int D, int FP8>
int dispatch_q(const AttnParams& p, int batch, int row_chunks, int nq, cudaStream_t st) {
  if (nq <= 8) return launch_attn<D, 8, FP8>(p, batch, row_chunks, st);
  if (nq <= 16) return launch_attn<D, 16, FP8>(p, batch, row_chunks, st);
  return launch_attn<D, 32, FP8>(p, batch, row_chunks, st);
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

// NVFP4 KV (kv_fp8 = 2): scale pools for the NEXT hb_attn_paged call of this thread, strides in bytes.
struct AttnSf {
  const uint8_t* k = nullptr;
  const uint8_t* v = nullptr;
  long long pool_stride = 0, head_stride = 0;
};
static thread_local AttnSf g_attn_sf;
void hb_attn_fp4_scales(const void* k_sf, const void* v_sf, long long pool_stride, long long head_stride) {
  g_attn_sf.k = static_cast<const uint8_t*>(k_sf); g_attn_sf.v = static_cast<const uint8_t*>(v_sf);
  g_attn_sf.pool_stride = pool_stride; g_attn_sf.head_stride = head_stride;
}

// max_rows: largest number of query rows of any sequence (1 for decode). Partials are needed when splits > 1.
// kv_fp8: 0 bf16, 1 e4m3 (x = q * kv_scale), 2 NVFP4 (x = code * block scale * kv_scale; hb_attn_fp4_scales first).
int hb_attn_paged(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                  long long head_stride,
                  const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len, const void* q_indptr,
                  void* out, void* part_o, void* part_lse, int batch, int total_rows, int max_rows, int hq, int hkv, int d,
                  int splits, float scale, int kv_fp8, float kv_scale, int causal, void* stream) {
  if (batch <= 0) return 0;
  if (hq % hkv != 0) return 1;
  const int g = hq / hkv;
  if (g > 32) return 1;
  AttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pool = k_pool; p.v_pool = v_pool; p.pool_stride = pool_stride; p.head_stride = head_stride;
  p.kv_indices = static_cast<const int*>(kv_indices); p.ld_idx = ld_idx;
  p.ctx_len = static_cast<const int*>(ctx_len);
  p.seq_rows = static_cast<const int*>(seq_rows);
  p.q_indptr = static_cast<const int*>(q_indptr);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = static_cast<float*>(part_o); p.part_lse = static_cast<float*>(part_lse);
  p.hq = hq; p.hkv = hkv; p.splits = splits < 1 ? 1 : splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.kv_scale = kv_scale; p.causal = causal;
  p.k_sf = g_attn_sf.k; p.v_sf = g_attn_sf.v;
  p.sf_pool_stride = g_attn_sf.pool_stride; p.sf_head_stride = g_attn_sf.head_stride;
  g_attn_sf = AttnSf{};
  if (p.splits > 1 && (part_o == nullptr || part_lse == nullptr)) return 1;
  // Query rows per CTA: as many tokens as fit 32 (group x tokens), at most what the batch needs.
  int rows_per_cta = 32 / g;
  if (rows_per_cta > max_rows) rows_per_cta = max_rows;
  if (rows_per_cta < 1) rows_per_cta = 1;
  p.rows_per_cta = rows_per_cta;
  const int row_chunks = (max_rows + rows_per_cta - 1) / rows_per_cta;
  const int nq = rows_per_cta * g;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = 1;
  if (kv_fp8 == 2) {
    if (p.k_sf == nullptr || p.v_sf == nullptr) return 1;
    if (d == 64) rc = dispatch_q<64, 2>(p, batch, row_chunks, nq, st);
    else if (d == 128) rc = dispatch_q<128, 2>(p, batch, row_chunks, nq, st);
    else if (d == 256) rc = dispatch_q<256, 2>(p, batch, row_chunks, nq, st);
  } else if (kv_fp8) {
    if (d == 64) rc = dispatch_q<64, 1>(p, batch, row_chunks, nq, st);
    else if (d == 128) rc = dispatch_q<128, 1>(p, batch, row_chunks, nq, st);
    else if (d == 256) rc = dispatch_q<256, 1>(p, batch, row_chunks, nq, st);
  } else {
    if (d == 64) rc = dispatch_q<64, 0>(p, batch, row_chunks, nq, st);
    else if (d == 128) rc = dispatch_q<128, 0>(p, batch, row_chunks, nq, st);
    else if (d == 256) rc = dispatch_q<256, 0>(p, batch, row_chunks, nq, st);
  }
  if (rc != 0) return rc;
  if (p.splits > 1) {
    attn_merge_kernel<<<static_cast<unsigned>(static_cast<long long>(total_rows) * hq), 128, 0, st>>>(
        p.part_o, p.part_lse, p.out, p.splits, d, hq, nullptr, nullptr, nullptr, 0);
    if (cudaGetLastError() != cudaSuccess) return 2;
  }
  return 0;
}

int hb_attn_merge(const void* part_o, const void* part_lse, void* out, long long rows_heads, int splits, int d,
                  void* stream) {
  if (rows_heads <= 0) return 0;
  launch_dep(attn_merge_kernel, dim3(static_cast<unsigned>(rows_heads)), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const float*>(part_o), static_cast<const float*>(part_lse), static_cast<__nv_bfloat16*>(out), splits,
      d, 1, static_cast<uint8_t*>(nullptr), static_cast<uint8_t*>(nullptr), static_cast<const float*>(nullptr), 0);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Split merge with NVFP4 output: rows [rows, hq * d] packed e2m1 into q_out, swizzled ue4m3 scales into q_sf
// (q_ka K atoms per row block), static per-tensor scale *q_gscale. d <= 256, a multiple of 16.
int hb_attn_merge_quant(const void* part_o, const void* part_lse, long long rows, int hq, int splits, int d,
                        void* q_out, void* q_sf, const void* q_gscale, int q_ka, void* stream) {
  if (rows <= 0) return 0;
  if (d > 256 || d % 16 != 0 || q_out == nullptr || q_sf == nullptr || q_gscale == nullptr) return 1;
  launch_dep(attn_merge_kernel, dim3(static_cast<unsigned>(rows * hq)), dim3(128), 0, static_cast<cudaStream_t>(stream),
      static_cast<const float*>(part_o), static_cast<const float*>(part_lse), static_cast<__nv_bfloat16*>(nullptr),
      splits, d, hq, static_cast<uint8_t*>(q_out), static_cast<uint8_t*>(q_sf), static_cast<const float*>(q_gscale),
      q_ka);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
