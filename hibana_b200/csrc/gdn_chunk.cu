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
