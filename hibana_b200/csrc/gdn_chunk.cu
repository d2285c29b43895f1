// State pass of the chunked gated delta rule (prefill): walks the 64-token chunks of one sequence carrying the
// recurrent state, with the chunk-local factors (computed for all chunks in parallel beforehand) as inputs.
//
// Per chunk c and value head h, with S^T [K, V] the state transposed and gamma = exp(g_end[c]):
//     V' = U - W S^T                      [64, V]
//     O  = Qg S^T + M V'                  [64, V]      (M = masked, decayed Q K^T)
//     S^T <- gamma S^T + Kd^T V'          [K, V]
// One CTA per (head, 32 columns of V): the columns of the state are independent, so 4 CTAs share a head. The
// three products run on mma.sync m16n8k16 (bf16 operands, fp32 accumulate; the tiles are 64 x 32 x 128 and the
// chain is serial in the chunk, so the win over a token-serial scan is the 64-fold shorter chain, not tensor
// throughput). The fp32 master copy of the state lives in accumulator registers for the whole sequence; a bf16
// copy in shared memory feeds the products. Chunk inputs are double-buffered with cp.async.
// Reference: hibana/kernels/fla/chunk_delta_h.py (state recurrence over chunks), hibana/kernels/fla/chunk_o.py.
#include "hb_api.h"
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int GC = 64;            // tokens per chunk
constexpr int GK = 128;           // key dim
constexpr int VS = 32;            // value columns per CTA
constexpr int P_K = GK * 2 + 16;  // row pitch (bytes) of the [64, 128] bf16 tiles
constexpr int P_M = GC * 2 + 16;  // [64, 64] bf16
constexpr int P_U = VS * 4 + 16;  // [64, 32] fp32
constexpr int P_V = VS * 2 + 16;  // [*, 32] bf16 (V' and S^T)
constexpr int OFF_W = 0;
constexpr int OFF_Q = OFF_W + GC * P_K;
constexpr int OFF_KD = OFF_Q + GC * P_K;
constexpr int OFF_M = OFF_KD + GC * P_K;
constexpr int OFF_U = OFF_M + GC * P_M;
constexpr int STAGE = OFF_U + GC * P_U;
constexpr int OFF_VN = 2 * STAGE;
constexpr int OFF_ST = OFF_VN + GC * P_V;
constexpr int G_SMEM = OFF_ST + GK * P_V;

struct ChunkParams {
  const __nv_bfloat16* w;     // [H, NC, 64, 128]; null: no W term (V' = U, the Mamba-2 / SSD recurrence)
  const __nv_bfloat16* qg;
  const __nv_bfloat16* kd;
  const __nv_bfloat16* m;     // [H, NC, 64, 64]
  const float* u;             // [H, NC, 64, 128]
  const float* g_end;         // [H, NC]
  const float* s_in;          // [H, 128 (v), 128 (k)] or null (zero state)
  float* s_out;               // same layout, may be null
  __nv_bfloat16* o;           // rows of this sequence: o[row * ldo + h * 128 + v]
  long long ldo;
  int nc, n;
  int vdim;                   // value columns of a head (multiple of 32): 128 for the delta rule, head dim for SSD
};

__device__ __forceinline__ void cp16g(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&t);
}

// B fragments of a [K, 32] row-major bf16 tile (pitch P_V) for k rows k0..k0+15: b[j][0..1] for n-tile j.
__device__ __forceinline__ void load_b32(uint32_t (&b)[4][2], uint32_t tile, int k0, int lane) {
  uint32_t r[4];
  const uint32_t row = tile + (k0 + (lane & 15)) * P_V + (lane >> 4) * 16;
  ldsm_x4_t(r, row);
  b[0][0] = r[0]; b[0][1] = r[1]; b[1][0] = r[2]; b[1][1] = r[3];
  ldsm_x4_t(r, row + 32);
  b[2][0] = r[0]; b[2][1] = r[1]; b[3][0] = r[2]; b[3][1] = r[3];
}

__global__ void __launch_bounds__(128) gdn_chunk_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) uint8_t g_smem[];
  const uint32_t sb = smem_u32(g_smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.x, v0 = blockIdx.y * VS;
  const int qr = lane >> 2, qc = (lane & 3) * 2;   // accumulator row / first column of this lane inside a tile
  const int GV = p.vdim;

  auto load_chunk = [&](int c, int stage) {
    const long long tile = static_cast<long long>(h) * p.nc + c;
    const uint8_t* gw = reinterpret_cast<const uint8_t*>(p.w + tile * GC * GK);
    const uint8_t* gq = reinterpret_cast<const uint8_t*>(p.qg + tile * GC * GK);
    const uint8_t* gk = reinterpret_cast<const uint8_t*>(p.kd + tile * GC * GK);
    const uint8_t* gm = reinterpret_cast<const uint8_t*>(p.m + tile * GC * GC);
    const uint8_t* gu = reinterpret_cast<const uint8_t*>(p.u + tile * GC * GV + v0);
    const bool has_w = p.w != nullptr;
    const uint32_t st = sb + stage * STAGE;
    for (int i = tid; i < GC * 16; i += 128) {
      const int r = i >> 4, ch = (i & 15) * 16;
      if (has_w) cp16g(st + OFF_W + r * P_K + ch, gw + r * (GK * 2) + ch);
      cp16g(st + OFF_Q + r * P_K + ch, gq + r * (GK * 2) + ch);
      cp16g(st + OFF_KD + r * P_K + ch, gk + r * (GK * 2) + ch);
    }
    for (int i = tid; i < GC * 8; i += 128) {
      const int r = i >> 3, ch = (i & 7) * 16;
      cp16g(st + OFF_M + r * P_M + ch, gm + r * (GC * 2) + ch);
      cp16g(st + OFF_U + r * P_U + ch, gu + r * (GV * 4) + ch);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // fp32 master copy of S^T: warp w owns key rows 32w .. 32w + 31 (two 16-row tiles), all 32 value columns
  float acc_s[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kr = 32 * warp + 16 * i + qr + (e >> 1) * 8, vc = 8 * j + qc + (e & 1);
        acc_s[i][j][e] =
            p.s_in != nullptr ? p.s_in[(static_cast<long long>(h) * GV + v0 + vc) * GK + kr] : 0.f;
      }
  auto publish_state = [&]() {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
          const int kr = 32 * warp + 16 * i + qr + (e >> 1) * 8, vc = 8 * j + qc;
          *reinterpret_cast<uint32_t*>(g_smem + OFF_ST + kr * P_V + vc * 2) =
              pack_bf16(acc_s[i][j][e], acc_s[i][j][e + 1]);
        }
  };
  publish_state();
  if (p.nc > 0) load_chunk(0, 0);
  __syncthreads();

  for (int c = 0; c < p.nc; ++c) {
    const int stage = c & 1;
    if (c + 1 < p.nc) {
      load_chunk(c + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const uint32_t st = sb + stage * STAGE;
    // ---- W S^T and Qg S^T (same B fragments): rows 16 warp .. 16 warp + 15 of the chunk
    float a1[4][4] = {}, a2[4][4] = {};
    const uint32_t a_off = (16 * warp + (lane & 15)) * P_K + (lane >> 4) * 16;
#pragma unroll
    for (int ks = 0; ks < GK / 16; ++ks) {
      uint32_t fw[4], fq[4], b[4][2];
      ldsm_x4(fq, st + OFF_Q + a_off + ks * 32);
      load_b32(b, sb + OFF_ST, ks * 16, lane);
      if (p.w != nullptr) {
        ldsm_x4(fw, st + OFF_W + a_off + ks * 32);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma16816(a1[j], fw, b[j][0], b[j][1]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) mma16816(a2[j], fq, b[j][0], b[j][1]);
    }
    // ---- V' = U - W S^T, to shared memory as bf16
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int r = 16 * warp + qr + (e >> 1) * 8, vc = 8 * j + qc;
        const float2 u = *reinterpret_cast<const float2*>(g_smem + stage * STAGE + OFF_U + r * P_U + vc * 4);
        *reinterpret_cast<uint32_t*>(g_smem + OFF_VN + r * P_V + vc * 2) = pack_bf16(u.x - a1[j][e], u.y - a1[j][e + 1]);
      }
    __syncthreads();
    // ---- O += M V'
    const uint32_t m_off = (16 * warp + (lane & 15)) * P_M + (lane >> 4) * 16;
#pragma unroll
    for (int ks = 0; ks < GC / 16; ++ks) {
      uint32_t fm[4], b[4][2];
      ldsm_x4(fm, st + OFF_M + m_off + ks * 32);
      load_b32(b, sb + OFF_VN, ks * 16, lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) mma16816(a2[j], fm, b[j][0], b[j][1]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int tok = c * GC + 16 * warp + qr + (e >> 1) * 8, vc = 8 * j + qc;
        if (tok < p.n)
          *reinterpret_cast<uint32_t*>(p.o + tok * p.ldo + h * GV + v0 + vc) = pack_bf16(a2[j][e], a2[j][e + 1]);
      }
    // ---- S^T <- gamma S^T + Kd^T V'
    const float gamma = __expf(p.g_end[static_cast<long long>(h) * p.nc + c]);
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_s[i][j][e] *= gamma;
#pragma unroll
    for (int ks = 0; ks < GC / 16; ++ks) {
      uint32_t b[4][2];
      load_b32(b, sb + OFF_VN, ks * 16, lane);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        // A = Kd^T: element (key row, token) sits at Kd[token][key row]; the four 8x8 blocks of the fragment are
        // (keys 0-7, tokens 0-7), (keys 8-15, tokens 0-7), (keys 0-7, tokens 8-15), (keys 8-15, tokens 8-15)
        const int mi = lane >> 3;
        const int row = ks * 16 + (mi >> 1) * 8 + (lane & 7), col = 32 * warp + 16 * i + (mi & 1) * 8;
        uint32_t fa[4];
        ldsm_x4_t(fa, st + OFF_KD + row * P_K + col * 2);
#pragma unroll
        for (int j = 0; j < 4; ++j) mma16816(acc_s[i][j], fa, b[j][0], b[j][1]);
      }
    }
    publish_state();     // every read of the old copy happened before the barrier above
    __syncthreads();
  }
  if (p.s_out != nullptr) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kr = 32 * warp + 16 * i + qr + (e >> 1) * 8, vc = 8 * j + qc + (e & 1);
          p.s_out[(static_cast<long long>(h) * GV + v0 + vc) * GK + kr] = acc_s[i][j][e];
        }
  }
}

}  // namespace
}  // namespace hb

extern "C" {

// w (may be null: V' = U), qg, kd bf16 [heads, nc, 64, 128]; m bf16 [heads, nc, 64, 64]; u fp32 [heads, nc, 64, vdim];
// g_end fp32 [heads, nc]; s_in / s_out fp32 [heads, vdim, 128] (value row, key column; s_in null = zero state, s_out null = do
// not store); o bf16 rows of the sequence (pitch ldo elements), only rows < n are written.
int hb_gdn_chunk_pass(const void* w, const void* qg, const void* kd, const void* m, const void* u, const void* g_end,
                      const void* s_in, void* s_out, void* o, long long ldo, int heads, int nc, int n, int kdim,
                      int vdim, void* stream) {
  using namespace hb;
  if (kdim != GK || vdim < VS || vdim % VS != 0) return 1;
  if (heads <= 0 || nc <= 0) return 0;
  ChunkParams p;
  p.w = static_cast<const __nv_bfloat16*>(w); p.qg = static_cast<const __nv_bfloat16*>(qg);
  p.kd = static_cast<const __nv_bfloat16*>(kd); p.m = static_cast<const __nv_bfloat16*>(m);
  p.u = static_cast<const float*>(u); p.g_end = static_cast<const float*>(g_end);
  p.s_in = static_cast<const float*>(s_in); p.s_out = static_cast<float*>(s_out);
  p.o = static_cast<__nv_bfloat16*>(o); p.ldo = ldo; p.nc = nc; p.n = n; p.vdim = vdim;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM) != cudaSuccess)
      return 3;
    attr = true;
  }
  gdn_chunk_kernel<<<dim3(heads, vdim / VS), 128, G_SMEM, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Phase 1 of the chunked gated delta rule: everything of a 64-token chunk that does not depend on the incoming
// state, for all chunks and heads in parallel (one CTA per (chunk, value head), 128 threads, 4 warps of 16 rows).
//   Kn, Qn  = l2norm(k), l2norm(q) * scale                    (bf16 in shared memory)
//   gamma_t = running sum of g inside the chunk
//   A[t,i]  = beta_t e^(gamma_t - gamma_i) <Kn_t, Kn_i>  (i < t)      T = (I + A)^-1   (fp32, forward substitution)
//   M[t,i]  = e^(gamma_t - gamma_i) <Qn_t, Kn_i>         (i <= t)
//   U = T (beta V)     W = T (beta e^gamma Kn)     Qg = e^gamma Qn     Kd = e^(gamma_C - gamma) Kn
// The four 64-wide products run on mma.sync with bf16 operands (as the reference's chunk kernels do); the
// triangular inverse stays in fp32 (one thread per column, the column in registers). Outputs are laid out [head, chunk, 64, *] for gdn_chunk_kernel.
namespace hb {
namespace {

constexpr int P1_PK = GK * 2 + 16;     // pitch of the [64, 128] bf16 tiles
constexpr int P1_PA = GC + 4;          // floats per row of A / T
constexpr int P1_PT = GC * 2 + 16;     // pitch of T in bf16
constexpr int P1_KN = 0;
constexpr int P1_QN = P1_KN + GC * P1_PK;
constexpr int P1_VB = P1_QN + GC * P1_PK;
constexpr int P1_KB = P1_VB + GC * P1_PK;
constexpr int P1_A = P1_KB + GC * P1_PK;
constexpr int P1_TB = P1_A + GC * P1_PA * 4;
constexpr int P1_G = P1_TB + GC * P1_PT;          // gamma[64], beta[64]
constexpr int P1_SMEM = P1_G + 2 * GC * 4;

struct Phase1Params {
  const __nv_bfloat16* q;   // [n, k_heads * 128] (pitch ldq)
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;   // [n, v_heads * 128] (pitch ldv)
  const float* g;           // [n, v_heads]
  const float* beta;
  long long ldq, ldv;
  __nv_bfloat16 *w, *qg, *kd, *m;   // outputs, see gdn_chunk_kernel
  float* u;
  float* g_end;
  int n, nc, k_heads, v_heads;
  float scale;
  int l2norm;
};

__global__ void __launch_bounds__(128, 2) gdn_phase1_kernel(const Phase1Params p) {
  extern __shared__ __align__(16) uint8_t sm[];
  const uint32_t sb = smem_u32(sm);
  float* a_s = reinterpret_cast<float*>(sm + P1_A);
  float* gam = reinterpret_cast<float*>(sm + P1_G);
  float* bet = gam + GC;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  const int hk = h / (p.v_heads / p.k_heads);
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  const int t0 = c * GC;

  // ---- gamma, beta
  if (warp == 0) {
    float g0 = 0.f, g1 = 0.f;
    const int ta = t0 + lane, tb = t0 + 32 + lane;
    if (ta < p.n) g0 = p.g[static_cast<long long>(ta) * p.v_heads + h];
    if (tb < p.n) g1 = p.g[static_cast<long long>(tb) * p.v_heads + h];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float x0 = __shfl_up_sync(0xffffffffu, g0, o), x1 = __shfl_up_sync(0xffffffffu, g1, o);
      if (lane >= o) {
        g0 += x0;
        g1 += x1;
      }
    }
    g1 += __shfl_sync(0xffffffffu, g0, 31);
    gam[lane] = g0;
    gam[32 + lane] = g1;
    bet[lane] = ta < p.n ? p.beta[static_cast<long long>(ta) * p.v_heads + h] : 0.f;
    bet[32 + lane] = tb < p.n ? p.beta[static_cast<long long>(tb) * p.v_heads + h] : 0.f;
  }
  // ---- q, k rows: (l2norm,) scale, to shared memory; 16 rows per warp, a lane holds 4 of a row's 128 values.
  // (restrict-qualified views and an unroll hint let the loads of several rows be in flight at once)
  const __nv_bfloat16* __restrict__ gq = p.q;
  const __nv_bfloat16* __restrict__ gk = p.k;
  const __nv_bfloat16* __restrict__ gv = p.v;
#pragma unroll 4
  for (int r = warp * 16; r < warp * 16 + 16; ++r) {
    const int t = t0 + r;
    float qv[4] = {0, 0, 0, 0}, kv[4] = {0, 0, 0, 0};
    if (t < p.n) {
      const uint2 qq = *reinterpret_cast<const uint2*>(gq + t * p.ldq + hk * GK + lane * 4);
      const uint2 kk = *reinterpret_cast<const uint2*>(gk + t * p.ldq + hk * GK + lane * 4);
      qv[0] = bf16_lo(qq.x); qv[1] = bf16_hi(qq.x); qv[2] = bf16_lo(qq.y); qv[3] = bf16_hi(qq.y);
      kv[0] = bf16_lo(kk.x); kv[1] = bf16_hi(kk.x); kv[2] = bf16_lo(kk.y); kv[3] = bf16_hi(kk.y);
    }
    float qs = p.scale, ks = 1.f;
    if (p.l2norm) {
      float q2 = qv[0] * qv[0] + qv[1] * qv[1] + qv[2] * qv[2] + qv[3] * qv[3];
      float k2 = kv[0] * kv[0] + kv[1] * kv[1] + kv[2] * kv[2] + kv[3] * kv[3];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        q2 += __shfl_xor_sync(0xffffffffu, q2, o);
        k2 += __shfl_xor_sync(0xffffffffu, k2, o);
      }
      qs *= rsqrtf(q2 + 1e-6f);
      ks = rsqrtf(k2 + 1e-6f);
    }
    *reinterpret_cast<uint2*>(sm + P1_QN + r * P1_PK + lane * 8) =
        make_uint2(pack_bf16(qv[0] * qs, qv[1] * qs), pack_bf16(qv[2] * qs, qv[3] * qs));
    *reinterpret_cast<uint2*>(sm + P1_KN + r * P1_PK + lane * 8) =
        make_uint2(pack_bf16(kv[0] * ks, kv[1] * ks), pack_bf16(kv[2] * ks, kv[3] * ks));
  }
  __syncthreads();
  const float g_last = gam[GC - 1];
  // ---- beta V, beta e^gamma Kn, and the decayed copies that go straight to global memory
  const long long tile = static_cast<long long>(h) * p.nc + c;
#pragma unroll 4
  for (int r = warp * 16; r < warp * 16 + 16; ++r) {
    const int t = t0 + r;
    const float b = bet[r], eg = __expf(gam[r]), ed = __expf(g_last - gam[r]);
    float vv[4] = {0, 0, 0, 0};
    if (t < p.n) {
      const uint2 x = *reinterpret_cast<const uint2*>(gv + t * p.ldv + h * GK + lane * 4);
      vv[0] = bf16_lo(x.x); vv[1] = bf16_hi(x.x); vv[2] = bf16_lo(x.y); vv[3] = bf16_hi(x.y);
    }
    const uint2 kn = *reinterpret_cast<const uint2*>(sm + P1_KN + r * P1_PK + lane * 8);
    const uint2 qn = *reinterpret_cast<const uint2*>(sm + P1_QN + r * P1_PK + lane * 8);
    const float k0 = bf16_lo(kn.x), k1 = bf16_hi(kn.x), k2 = bf16_lo(kn.y), k3 = bf16_hi(kn.y);
    *reinterpret_cast<uint2*>(sm + P1_VB + r * P1_PK + lane * 8) =
        make_uint2(pack_bf16(vv[0] * b, vv[1] * b), pack_bf16(vv[2] * b, vv[3] * b));
    const float be = b * eg;
    *reinterpret_cast<uint2*>(sm + P1_KB + r * P1_PK + lane * 8) =
        make_uint2(pack_bf16(k0 * be, k1 * be), pack_bf16(k2 * be, k3 * be));
    const long long o = (tile * GC + r) * GK + lane * 4;
    *reinterpret_cast<uint2*>(p.kd + o) = make_uint2(pack_bf16(k0 * ed, k1 * ed), pack_bf16(k2 * ed, k3 * ed));
    *reinterpret_cast<uint2*>(p.qg + o) =
        make_uint2(pack_bf16(bf16_lo(qn.x) * eg, bf16_hi(qn.x) * eg), pack_bf16(bf16_lo(qn.y) * eg, bf16_hi(qn.y) * eg));
  }
  if (tid == 0) p.g_end[tile] = g_last;
  // ---- Kn Kn^T and Qn Kn^T for this warp's 16 rows
  {
    float akk[8][4] = {}, aqk[8][4] = {};
    const uint32_t a_off = (16 * warp + (lane & 15)) * P1_PK + (lane >> 4) * 16;
    const int mi = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < GK / 16; ++ks) {
      uint32_t fk[4], fq[4];
      ldsm_x4(fk, sb + P1_KN + a_off + ks * 32);
      ldsm_x4(fq, sb + P1_QN + a_off + ks * 32);
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {     // two 8-column tiles of the other tokens per load
        uint32_t fb[4];
        ldsm_x4(fb, sb + P1_KN + (16 * jp + (mi >> 1) * 8 + (lane & 7)) * P1_PK + ks * 32 + (mi & 1) * 16);
        mma16816(akk[2 * jp], fk, fb[0], fb[1]);
        mma16816(akk[2 * jp + 1], fk, fb[2], fb[3]);
        mma16816(aqk[2 * jp], fq, fb[0], fb[1]);
        mma16816(aqk[2 * jp + 1], fq, fb[2], fb[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = 16 * warp + qr + (e >> 1) * 8, i = 8 * j + qc + (e & 1);
        const float d = i <= t ? __expf(gam[t] - gam[i]) : 0.f;
        a_s[t * P1_PA + i] = i < t ? bet[t] * d * akk[j][e] : 0.f;
        aqk[j][e] *= d;
      }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int t = 16 * warp + qr + (e >> 1) * 8, i = 8 * j + qc;
        *reinterpret_cast<uint32_t*>(p.m + (tile * GC + t) * GC + i) = pack_bf16(aqk[j][e], aqk[j][e + 1]);
      }
  }
  __syncthreads();
  // ---- T = (I + A)^-1 by forward substitution. Column j of T depends only on A and on the earlier rows of the
  // same column (T[i][j] = delta_ij - sum_{k<i} A[i][k] T[k][j], with T[k][j] = 0 for k < j), so thread j keeps its
  // column in registers and nobody waits for anybody; A is only read (broadcast loads) until all columns are done.
  if (tid < GC) {
    float tcol[GC];
#pragma unroll
    for (int i = 0; i < GC; ++i) {
      float acc = i == tid ? 1.f : 0.f;
#pragma unroll
      for (int k2 = 0; k2 < i; ++k2) acc -= a_s[i * P1_PA + k2] * tcol[k2];
      tcol[i] = acc;
    }
    asm volatile("bar.sync 2, 64;" ::: "memory");
#pragma unroll
    for (int i = 0; i < GC; ++i) a_s[i * P1_PA + tid] = tcol[i];
  }
  __syncthreads();
  // bf16 copy of T as the A operand of the two products
  for (int x = tid; x < GC * GC / 2; x += 128) {
    const int t = x / (GC / 2), i = (x % (GC / 2)) * 2;
    *reinterpret_cast<uint32_t*>(sm + P1_TB + t * P1_PT + i * 2) = pack_bf16(a_s[t * P1_PA + i], a_s[t * P1_PA + i + 1]);
  }
  __syncthreads();
  // ---- U = T (beta V) (fp32 out) and W = T (beta e^gamma Kn) (bf16 out): 16 rows per warp, 128 columns, K = 64
  const uint32_t t_off = (16 * warp + (lane & 15)) * P1_PT + (lane >> 4) * 16;
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const uint32_t bsrc = sb + (which == 0 ? P1_VB : P1_KB);
    float acc[16][4] = {};
#pragma unroll
    for (int ks = 0; ks < GC / 16; ++ks) {
      uint32_t ft[4];
      ldsm_x4(ft, sb + P1_TB + t_off + ks * 32);
#pragma unroll
      for (int jp = 0; jp < 8; ++jp) {     // B = [64 tokens, 128] row-major: transposed loads, two 8-column tiles each
        uint32_t fb[4];
        ldsm_x4_t(fb, bsrc + (ks * 16 + (lane & 15)) * P1_PK + jp * 32 + (lane >> 4) * 16);
        mma16816(acc[2 * jp], ft, fb[0], fb[1]);
        mma16816(acc[2 * jp + 1], ft, fb[2], fb[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int t = 16 * warp + qr + (e >> 1) * 8, col = 8 * j + qc;
        const long long o = (tile * GC + t) * GK + col;
        if (which == 0) *reinterpret_cast<float2*>(p.u + o) = make_float2(acc[j][e], acc[j][e + 1]);
        else *reinterpret_cast<uint32_t*>(p.w + o) = pack_bf16(acc[j][e], acc[j][e + 1]);
      }
  }
}

}  // namespace
}  // namespace hb

extern "C" {

// Phase 1 for the n rows of one sequence (value and key dim 128). Outputs [v_heads, nc, 64, *] with nc = ceil(n / 64):
// w, qg, kd bf16 [.., 128], m bf16 [.., 64], u fp32 [.., 128], g_end fp32 [v_heads, nc].
int hb_gdn_phase1(const void* q, const void* k, const void* v, const void* g, const void* beta, long long ldq,
                  long long ldv, int n, int k_heads, int v_heads, float scale, int l2norm, void* w, void* qg, void* kd,
                  void* m, void* u, void* g_end, void* stream) {
  using namespace hb;
  if (n <= 0) return 0;
  if (k_heads <= 0 || v_heads % k_heads != 0 || (ldq & 3) || (ldv & 3)) return 1;
  Phase1Params p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v); p.g = static_cast<const float*>(g);
  p.beta = static_cast<const float*>(beta); p.ldq = ldq; p.ldv = ldv;
  p.w = static_cast<__nv_bfloat16*>(w); p.qg = static_cast<__nv_bfloat16*>(qg); p.kd = static_cast<__nv_bfloat16*>(kd);
  p.m = static_cast<__nv_bfloat16*>(m); p.u = static_cast<float*>(u); p.g_end = static_cast<float*>(g_end);
  p.n = n; p.nc = (n + GC - 1) / GC; p.k_heads = k_heads; p.v_heads = v_heads; p.scale = scale; p.l2norm = l2norm;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(gdn_phase1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P1_SMEM) != cudaSuccess)
      return 3;
    attr = true;
  }
  gdn_phase1_kernel<<<dim3(p.nc, v_heads), 128, P1_SMEM, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Phase 1 of the chunked Mamba-2 (SSD) scan: the chunk-local factors for gdn_chunk_kernel without its W term. One CTA
// per (chunk, head), 128 threads. With dt_t = softplus(dt + bias), a_t = -exp(a_log) dt_t and gamma its running sum:
//   U = dt * X     M[t,i] = e^(gamma_t - gamma_i) <C_t, B_i> (i <= t)     Qg = e^gamma C     Kd = e^(gamma_C - gamma) B
// B and C are shared by the heads of a group; the 64 x 64 x 128 product is simply recomputed per head (1 MFLOP).
namespace hb {
namespace {

struct SsdP1Params {
  const __nv_bfloat16* x;    // [n, heads * P]   (pitch ldx)
  const __nv_bfloat16* b;    // [n, groups * 128] (pitch ldb)
  const __nv_bfloat16* c;
  const __nv_bfloat16* dt;   // [n, heads]        (pitch lddt)
  const float* a_log;        // [heads]
  const float* dt_bias;      // [heads] or null
  long long ldx, ldb, lddt;
  __nv_bfloat16 *qg, *kd, *m;
  float* u;                  // [heads, nc, 64, P]
  float* g_end;
  int n, nc, heads, groups, p;
};

__global__ void __launch_bounds__(128, 2) ssd_phase1_kernel(const SsdP1Params p) {
  extern __shared__ __align__(16) uint8_t sm[];
  const uint32_t sb = smem_u32(sm);
  constexpr int S_C = 0, S_B = GC * P1_PK, S_G = 2 * GC * P1_PK;
  float* gam = reinterpret_cast<float*>(sm + S_G);
  float* dtv = gam + GC;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y;
  const int grp = h / (p.heads / p.groups);
  const int qr = lane >> 2, qc = (lane & 3) * 2;
  const int t0 = c * GC;
  if (warp == 0) {
    const float a = -__expf(p.a_log[h]);
    const float bias = p.dt_bias ? p.dt_bias[h] : 0.f;
    float d0 = 0.f, d1 = 0.f;
    const int ta = t0 + lane, tb = t0 + 32 + lane;
    if (ta < p.n) {
      const float z = __bfloat162float(p.dt[ta * p.lddt + h]) + bias;
      d0 = z > 20.f ? z : log1pf(__expf(z));
    }
    if (tb < p.n) {
      const float z = __bfloat162float(p.dt[tb * p.lddt + h]) + bias;
      d1 = z > 20.f ? z : log1pf(__expf(z));
    }
    float g0 = d0 * a, g1 = d1 * a;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float x0 = __shfl_up_sync(0xffffffffu, g0, o), x1 = __shfl_up_sync(0xffffffffu, g1, o);
      if (lane >= o) {
        g0 += x0;
        g1 += x1;
      }
    }
    g1 += __shfl_sync(0xffffffffu, g0, 31);
    gam[lane] = g0; gam[32 + lane] = g1;
    dtv[lane] = d0; dtv[32 + lane] = d1;
  }
  const __nv_bfloat16* __restrict__ gb = p.b;
  const __nv_bfloat16* __restrict__ gc = p.c;
  const __nv_bfloat16* __restrict__ gx = p.x;
#pragma unroll 4
  for (int r = warp * 16; r < warp * 16 + 16; ++r) {     // raw B and C rows of the group (zero rows past the end)
    const int t = t0 + r;
    uint2 bb = make_uint2(0, 0), cc = make_uint2(0, 0);
    if (t < p.n) {
      bb = *reinterpret_cast<const uint2*>(gb + t * p.ldb + grp * GK + lane * 4);
      cc = *reinterpret_cast<const uint2*>(gc + t * p.ldb + grp * GK + lane * 4);
    }
    *reinterpret_cast<uint2*>(sm + S_B + r * P1_PK + lane * 8) = bb;
    *reinterpret_cast<uint2*>(sm + S_C + r * P1_PK + lane * 8) = cc;
  }
  __syncthreads();
  const float g_last = gam[GC - 1];
  const long long tile = static_cast<long long>(h) * p.nc + c;
#pragma unroll 4
  for (int r = warp * 16; r < warp * 16 + 16; ++r) {
    const int t = t0 + r;
    const float eg = __expf(gam[r]), ed = __expf(g_last - gam[r]), d = dtv[r];
    const uint2 bb = *reinterpret_cast<const uint2*>(sm + S_B + r * P1_PK + lane * 8);
    const uint2 cc = *reinterpret_cast<const uint2*>(sm + S_C + r * P1_PK + lane * 8);
    const long long o = (tile * GC + r) * GK + lane * 4;
    *reinterpret_cast<uint2*>(p.kd + o) = make_uint2(pack_bf16(bf16_lo(bb.x) * ed, bf16_hi(bb.x) * ed),
                                                     pack_bf16(bf16_lo(bb.y) * ed, bf16_hi(bb.y) * ed));
    *reinterpret_cast<uint2*>(p.qg + o) = make_uint2(pack_bf16(bf16_lo(cc.x) * eg, bf16_hi(cc.x) * eg),
                                                     pack_bf16(bf16_lo(cc.y) * eg, bf16_hi(cc.y) * eg));
    for (int col = lane * 2; col < p.p; col += 64) {       // U = dt * x, two values per lane
      float2 xv = make_float2(0.f, 0.f);
      if (t < p.n) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(gx + t * p.ldx + h * p.p + col);
        xv = make_float2(bf16_lo(w) * d, bf16_hi(w) * d);
      }
      *reinterpret_cast<float2*>(p.u + (tile * GC + r) * p.p + col) = xv;
    }
  }
  if (tid == 0) p.g_end[tile] = g_last;
  // C B^T for this warp's 16 rows, masked and decayed
  float acc[8][4] = {};
  const uint32_t a_off = (16 * warp + (lane & 15)) * P1_PK + (lane >> 4) * 16;
  const int mi = lane >> 3;
#pragma unroll
  for (int ks = 0; ks < GK / 16; ++ks) {
    uint32_t fc[4];
    ldsm_x4(fc, sb + S_C + a_off + ks * 32);
#pragma unroll
    for (int jp = 0; jp < 4; ++jp) {
      uint32_t fb[4];
      ldsm_x4(fb, sb + S_B + (16 * jp + (mi >> 1) * 8 + (lane & 7)) * P1_PK + ks * 32 + (mi & 1) * 16);
      mma16816(acc[2 * jp], fc, fb[0], fb[1]);
      mma16816(acc[2 * jp + 1], fc, fb[2], fb[3]);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; e += 2) {
      const int t = 16 * warp + qr + (e >> 1) * 8, i = 8 * j + qc;
      const float v0 = i <= t ? acc[j][e] * __expf(gam[t] - gam[i]) : 0.f;
      const float v1 = i + 1 <= t ? acc[j][e + 1] * __expf(gam[t] - gam[i + 1]) : 0.f;
      *reinterpret_cast<uint32_t*>(p.m + (tile * GC + t) * GC + i) = pack_bf16(v0, v1);
    }
}

}  // namespace
}  // namespace hb

extern "C" {

// Phase 1 of the chunked SSD scan for the n rows of one sequence; state dim 128, head dim `p` (even, <= 128 pitch
// rules as below). Outputs [heads, nc, 64, *]: qg, kd bf16 [.., 128], m bf16 [.., 64], u fp32 [.., p], g_end fp32.
int hb_ssd_phase1(const void* x, const void* b, const void* c, const void* dt, const void* a_log, const void* dt_bias,
                  long long ldx, long long ldb, long long lddt, int n, int heads, int groups, int p, void* qg, void* kd,
                  void* m, void* u, void* g_end, void* stream) {
  using namespace hb;
  if (n <= 0) return 0;
  if (groups <= 0 || heads % groups != 0 || (p & 1) || (ldx & 1) || (ldb & 3)) return 1;
  SsdP1Params q;
  q.x = static_cast<const __nv_bfloat16*>(x); q.b = static_cast<const __nv_bfloat16*>(b);
  q.c = static_cast<const __nv_bfloat16*>(c); q.dt = static_cast<const __nv_bfloat16*>(dt);
  q.a_log = static_cast<const float*>(a_log); q.dt_bias = static_cast<const float*>(dt_bias);
  q.ldx = ldx; q.ldb = ldb; q.lddt = lddt;
  q.qg = static_cast<__nv_bfloat16*>(qg); q.kd = static_cast<__nv_bfloat16*>(kd); q.m = static_cast<__nv_bfloat16*>(m);
  q.u = static_cast<float*>(u); q.g_end = static_cast<float*>(g_end);
  q.n = n; q.nc = (n + GC - 1) / GC; q.heads = heads; q.groups = groups; q.p = p;
  const int smem = 2 * GC * P1_PK + 2 * GC * 4;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(ssd_phase1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 3;
    attr = true;
  }
  ssd_phase1_kernel<<<dim3(q.nc, heads), 128, smem, static_cast<cudaStream_t>(stream)>>>(q);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
