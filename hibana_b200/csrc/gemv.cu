// NVFP4 weight-streaming GEMV for one to eight activation rows (single-request decode, speculative verify blocks).
//
// y[m][n] = sum_k W[n][k] * x[m][k], W in the served NVFP4 layout (two e2m1 codes per byte along K, one e4m3 scale per
// 16 elements in 128 x 4 swizzled blocks, one fp32 scale per tensor), x in bf16 and NOT quantised. At these row
// counts the tcgen05 GEMM is bound by its fixed cost (TMEM allocation, tensor maps, cluster reduction: ~12 us for a
// 15 MB projection whose stream takes 2.3 us); this kernel has none of that state. A warp owns a 16-row weight
// tile and one K slice: every lane reads 2 x 32 contiguous bytes (64 codes of rows g and g + 8) plus the 4 scale
// bytes of that 64-element atom, converts with `cvt.rn.f16x2.e2m1x2`, scales in half2 (exact: 2 x 4 significant
// bits) and feeds `mma.sync.m16n8k16` with the weights as the A operand and up to 8 activation rows as B. The K
// index inside a 256-element chunk is permuted (the same way for W and x, which a dot product allows) so that a
// lane's contiguous bytes ARE its A fragments: no shuffles, no shared-memory staging of weights.
// The activation rows live in shared memory as f16; the prologue can apply RMSNorm on the way in (the sum of
// squares is recomputed by every CTA: 10 KB of L2 reads), and the epilogue can add the result to the residual
// stream in place (every element is read and written by its one owner) or apply SiLU-mul on interleaved gate / up
// rows. Weight loads of the first chunks are issued before `griddepcontrol.wait`, so as a programmatic dependent the
// kernel fills its pipeline while the producer of x drains.
// Reference counterpart: the M <= 4 FP8 / NVFP4 GEMV (hibana/kernels/ops.py:19-21, hibana/kernels/csrc/gemv.cu).
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int kGemvWarps = 4;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kChunk = 256;           // K elements per warp step: 4 lanes (t) x 64 codes
constexpr int kPrefetch = 3;          // chunks in flight per warp (registers)
constexpr int kXPad = 16;             // halfs of padding per activation row: rows start 8 banks apart

enum { kGemvStore = 0, kGemvResidual = 1, kGemvSiluMul = 2 };

struct GemvParams {
  const uint8_t* wq;        // [N, K / 2]
  const uint8_t* wsf;       // swizzled scale blocks [ceil(N / 128) (even), ka, 512]
  const float* wscale;      // per-tensor scale
  const __nv_bfloat16* x;   // [M, ldx]
  const __nv_bfloat16* norm_w;   // nullable: RMSNorm weight [K]
  const __nv_bfloat16* residual; // nullable (kGemvResidual): [M, ldr]; may alias `out`
  __nv_bfloat16* out;       // [M, ldo]
  int n, k, ka, m, ldx, ldr, ldo, epi, gemma;
  float eps;
};

struct Chunk {
  uint4 a[2], b[2];     // 64 codes of row g and of row g + 8
  uint32_t sa, sb;      // their 4 block scales (e4m3)
};

// 16-byte streaming load: weights are read once, so they bypass L1
__device__ __forceinline__ uint4 ld_nc_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t cvt_e2m1x2(uint32_t byte) {
  uint32_t h2;
  const uint16_t in = static_cast<uint16_t>(byte);
  asm("{\n\t.reg .b8 t;\n\tcvt.u8.u16 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h2) : "h"(in));
  return h2;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// one e4m3 byte -> half2 with the value in both halves
__device__ __forceinline__ uint32_t scale_h2(uint32_t byte) {
  uint32_t h2;
  const uint16_t in = static_cast<uint16_t>((byte & 0xFFu) * 0x0101u);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
  return h2;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Position of element k of an activation row in shared memory: chunks of 256, inside a chunk ordered
// [step i (16)][lane t (4)][4 elements], where k % 256 = t * 64 + i * 4 + e.
__device__ __forceinline__ int x_pos(int k) {
  const int c = k >> 8, r = k & 255;
  return (c << 8) + (((r & 63) >> 2) << 4) + ((r >> 6) << 2) + (r & 3);
}

template <int KSPLIT, int DEQ>
__global__ void __launch_bounds__(kGemvThreads, 4) nvfp4_gemv_kernel(const GemvParams p) {
  constexpr int TPC = kGemvWarps / KSPLIT;      // 16-row tiles per CTA
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int xs_ld = p.k + kXPad;
  __half* xs = reinterpret_cast<__half*>(smem_raw);                               // [m][k + pad], permuted
  float* red = reinterpret_cast<float*>(smem_raw + static_cast<size_t>(p.m) * xs_ld * 2);   // [warps][16][8]
  __shared__ float s_part[kGemvWarps][8];
  __shared__ float s_rstd[8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x * TPC + warp / KSPLIT;
  const int ks = warp % KSPLIT;
  const int ntiles = p.n >> 4;
  const bool live = tile < ntiles;
  const int nchunks = p.k / kChunk;
  const int mine = live ? (nchunks - ks + KSPLIT - 1) / KSPLIT : 0;      // this warp's chunks: ks, ks + KSPLIT, ...

  const int row_a = live ? (tile << 4) + g : 0, row_b = row_a + 8;
  const uint8_t* wa = p.wq + static_cast<size_t>(row_a) * (p.k >> 1) + t * 32;
  const uint8_t* wb = p.wq + static_cast<size_t>(row_b) * (p.k >> 1) + t * 32;
  auto sf_ptr = [&](int row) {
    const int r = row & 127;
    return p.wsf + static_cast<size_t>(row >> 7) * p.ka * 512 + (((r & 31) << 2) + (r >> 5)) * 4 + t * 512;
  };
  const uint8_t* sfa = sf_ptr(row_a);
  const uint8_t* sfb = sf_ptr(row_b);

  auto load_chunk = [&](Chunk& c, int j) {            // j-th chunk of this warp
    const int ck = ks + j * KSPLIT;
    const uint4* pa = reinterpret_cast<const uint4*>(wa + ck * (kChunk / 2));
    const uint4* pb = reinterpret_cast<const uint4*>(wb + ck * (kChunk / 2));
    c.a[0] = ld_nc_v4(pa);
    c.a[1] = ld_nc_v4(pa + 1);
    c.b[0] = ld_nc_v4(pb);
    c.b[1] = ld_nc_v4(pb + 1);
    c.sa = __ldg(reinterpret_cast<const uint32_t*>(sfa + static_cast<size_t>(ck) * 4 * 512));
    c.sb = __ldg(reinterpret_cast<const uint32_t*>(sfb + static_cast<size_t>(ck) * 4 * 512));
  };
  Chunk ring[kPrefetch];
#pragma unroll
  for (int j = 0; j < kPrefetch; ++j)
    if (j < mine) load_chunk(ring[j], j);

  // ---- activations: everything above touched only weights; what follows reads the producer's output
  grid_dep_wait();
  const int vecs = p.k >> 3;                       // 8-element vectors per row
  if (p.norm_w != nullptr) {
    float ss[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) ss[m] = 0.f;
    for (int v = threadIdx.x; v < vecs; v += kGemvThreads) {
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        if (m < p.m) {
          const uint4 raw = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.ldx + v * 8);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            ss[m] += f.x * f.x + f.y * f.y;
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      float v = ss[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
      if (lane == 0) s_part[warp][m] = v;
    }
    __syncthreads();
    if (threadIdx.x < 8) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) v += s_part[w][threadIdx.x];
      s_rstd[threadIdx.x] = rsqrtf(v / static_cast<float>(p.k) + p.eps);
    }
    __syncthreads();
  }
  for (int v = threadIdx.x; v < vecs; v += kGemvThreads) {
    float nw[8];
    if (p.norm_w != nullptr) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p.norm_w + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        nw[2 * e] = p.gemma ? 1.f + f.x : f.x;
        nw[2 * e + 1] = p.gemma ? 1.f + f.y : f.y;
      }
    }
    const int pos = x_pos(v * 8);
    for (int m = 0; m < p.m; ++m) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.ldx + v * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      __half2 o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        if (p.norm_w != nullptr) {
          const float r = s_rstd[m];
          // the normed row is rounded to bf16 first, like the stand-alone norm kernel's output
          f.x = __bfloat162float(__float2bfloat16(f.x * r * nw[2 * e]));
          f.y = __bfloat162float(__float2bfloat16(f.y * r * nw[2 * e + 1]));
        }
        f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
        f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
        o[e] = __floats2half2_rn(f.x, f.y);
      }
      __half* dst = xs + static_cast<size_t>(m) * xs_ld + pos;
      if (DEQ == 1) {     // shift-and-mask decode pairs element e with e + 4 of a word: steps hold (0,4,1,5), (2,6,3,7)
        const __half2 lo0 = __lows2half2(o[0], o[2]), lo1 = __highs2half2(o[0], o[2]);
        const __half2 hi0 = __lows2half2(o[1], o[3]), hi1 = __highs2half2(o[1], o[3]);
        o[0] = lo0; o[1] = lo1; o[2] = hi0; o[3] = hi1;
      }
      *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(&o[0]);        // elements 0..3: step i
      *reinterpret_cast<uint2*>(dst + 16) = *reinterpret_cast<const uint2*>(&o[2]);   // elements 4..7: step i + 1
    }
  }
  __syncthreads();

  const __half* xrow = xs + static_cast<size_t>(g < p.m ? g : 0) * xs_ld + (t << 2);
  const bool has_x = g < p.m;
  const float wscale = *p.wscale * (DEQ == 1 ? 128.f : 1.f);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  auto compute = [&](const Chunk& c, int j) {
    const int ck = ks + j * KSPLIT;
    const __half* xc = xrow + (ck << 8);
    const uint32_t wa_[8] = {c.a[0].x, c.a[0].y, c.a[0].z, c.a[0].w, c.a[1].x, c.a[1].y, c.a[1].z, c.a[1].w};
    const uint32_t wb_[8] = {c.b[0].x, c.b[0].y, c.b[0].z, c.b[0].w, c.b[1].x, c.b[1].y, c.b[1].z, c.b[1].w};
    if constexpr (DEQ == 1) {
      // e2m1 code s|e e|m placed at f16 bits 15 | 11:9 is the value times 2^-14 (0.5 lands on an f16 subnormal), so
      // two shifts and two masks decode two codes at once; the block scale carries 2^7, the epilogue the other 2^7
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t k128 = 0x58005800u;        // half2(128, 128)
        const uint32_t sa = hmul2(scale_h2(c.sa >> (8 * q)), k128), sb = hmul2(scale_h2(c.sb >> (8 * q)), k128);
#pragma unroll
        for (int hw = 0; hw < 2; ++hw) {          // word 2 q + hw: elements 8 (2 q + hw) .. + 7, steps 2 w, 2 w + 1
          const int wi = 2 * q + hw;
          const uint32_t u = wa_[wi], v = wb_[wi];
          const uint32_t a_h0 = ((u << 9) & 0x0E000E00u) | ((u << 12) & 0x80008000u);
          const uint32_t a_h1 = ((u << 5) & 0x0E000E00u) | ((u << 8) & 0x80008000u);
          const uint32_t a_h2 = ((u << 1) & 0x0E000E00u) | ((u << 4) & 0x80008000u);
          const uint32_t a_h3 = ((u >> 3) & 0x0E000E00u) | (u & 0x80008000u);
          const uint32_t b_h0 = ((v << 9) & 0x0E000E00u) | ((v << 12) & 0x80008000u);
          const uint32_t b_h1 = ((v << 5) & 0x0E000E00u) | ((v << 8) & 0x80008000u);
          const uint32_t b_h2 = ((v << 1) & 0x0E000E00u) | ((v << 4) & 0x80008000u);
          const uint32_t b_h3 = ((v >> 3) & 0x0E000E00u) | (v & 0x80008000u);
          uint2 x0 = make_uint2(0u, 0u), x1 = make_uint2(0u, 0u);
          if (has_x) {
            x0 = *reinterpret_cast<const uint2*>(xc + ((2 * wi) << 4));
            x1 = *reinterpret_cast<const uint2*>(xc + ((2 * wi + 1) << 4));
          }
          mma_16816(acc, hmul2(a_h0, sa), hmul2(b_h0, sb), hmul2(a_h1, sa), hmul2(b_h1, sb), x0.x, x0.y);
          mma_16816(acc, hmul2(a_h2, sa), hmul2(b_h2, sb), hmul2(a_h3, sa), hmul2(b_h3, sb), x1.x, x1.y);
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {                 // 16-element scale group
        const uint32_t sa = scale_h2(c.sa >> (8 * q)), sb = scale_h2(c.sb >> (8 * q));
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {            // mma step i = 4 q + ii: bytes 2 i, 2 i + 1 of the 32
          const int i = 4 * q + ii;
          const uint32_t word_a = wa_[i >> 1], word_b = wb_[i >> 1];
          const int sh = (i & 1) * 16;
          const uint32_t a0 = hmul2(cvt_e2m1x2((word_a >> sh) & 0xFFu), sa);
          const uint32_t a2 = hmul2(cvt_e2m1x2((word_a >> (sh + 8)) & 0xFFu), sa);
          const uint32_t a1 = hmul2(cvt_e2m1x2((word_b >> sh) & 0xFFu), sb);
          const uint32_t a3 = hmul2(cvt_e2m1x2((word_b >> (sh + 8)) & 0xFFu), sb);
          uint2 b = make_uint2(0u, 0u);
          if (has_x) b = *reinterpret_cast<const uint2*>(xc + (i << 4));
          mma_16816(acc, a0, a1, a2, a3, b.x, b.y);
        }
      }
    }
  };

  for (int j0 = 0; j0 < mine; j0 += kPrefetch) {
#pragma unroll
    for (int pf = 0; pf < kPrefetch; ++pf) {
      const int j = j0 + pf;
      if (j < mine) {
        compute(ring[pf], j);
        if (j + kPrefetch < mine) load_chunk(ring[pf], j + kPrefetch);
      }
    }
  }
  grid_dep_launch();      // the next kernel may become resident (and fetch its weights) while this one drains

  // ---- reduce the K slices of a tile in a fixed order, then the epilogue
  float* mine_red = red + warp * 128;
  mine_red[g * 8 + 2 * t] = acc[0];
  mine_red[g * 8 + 2 * t + 1] = acc[1];
  mine_red[(g + 8) * 8 + 2 * t] = acc[2];
  mine_red[(g + 8) * 8 + 2 * t + 1] = acc[3];
  __syncthreads();
  if (ks != 0 || !live) return;
  const float* base = red + (warp / KSPLIT) * KSPLIT * 128;
  const int row0 = tile << 4;
  if (p.epi == kGemvSiluMul) {
    for (int idx = lane; idx < 8 * p.m; idx += 32) {
      const int m = idx >> 3, pr = idx & 7;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int s = 0; s < KSPLIT; ++s) {
        gate += base[s * 128 + (2 * pr) * 8 + m];
        up += base[s * 128 + (2 * pr + 1) * 8 + m];
      }
      gate *= wscale;
      up *= wscale;
      const float y = gate / (1.f + __expf(-gate)) * up;
      p.out[static_cast<size_t>(m) * p.ldo + (row0 >> 1) + pr] = __float2bfloat16(y);
    }
    return;
  }
  for (int idx = lane; idx < 16 * p.m; idx += 32) {
    const int m = idx >> 4, r = idx & 15;
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < KSPLIT; ++s) v += base[s * 128 + r * 8 + m];
    v *= wscale;
    if (p.epi == kGemvResidual)
      v += __bfloat162float(p.residual[static_cast<size_t>(m) * p.ldr + row0 + r]);
    p.out[static_cast<size_t>(m) * p.ldo + row0 + r] = __float2bfloat16(v);
  }
}

template <int KSPLIT, int DEQ>
cudaError_t launch_gemv(const GemvParams& p, int ctas, size_t smem, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(nvfp4_gemv_kernel<KSPLIT, DEQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = hb_gemm_get_pdl() >= 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, nvfp4_gemv_kernel<KSPLIT, DEQ>, p);
}

int g_gemv_deq = 1;      // 0: hardware e2m1 -> f16 conversion, 1: shift-and-mask decode

}  // namespace
}  // namespace hb

extern "C" {

// Largest row count this kernel takes for a given K (two CTAs per SM must still fit their activation rows), 0 when
// the shape is not supported at all.
int hb_nvfp4_gemv_max_rows(int n, int k) {
  if (n <= 0 || k <= 0 || n % 16 != 0 || k % hb::kChunk != 0) return 0;
  const int per_row = (k + hb::kXPad) * 2;
  const int fit = (100 * 1024 - hb::kGemvWarps * 128 * 4) / per_row;      // two CTAs per SM hold their rows
  return fit > 8 ? 8 : fit;
}

// Which code-to-f16 decode the kernel uses (0: `cvt`, 1: shift and mask); for measurements.
void hb_nvfp4_gemv_set_decode(int mode) { hb::g_gemv_deq = mode ? 1 : 0; }

// out[m][n] (+)= W x. `norm_w` != null: x is RMS-normalised (weight norm_w, `gemma`: 1 + w) on the way in.
// epi 0: store; 1: out = residual + y (out may be the residual itself); 2: SiLU-mul of interleaved (gate, up) rows,
// out is [m, n / 2].
int hb_nvfp4_gemv(const void* wq, const void* wsf, const void* wscale, int n, int k, int ka, const void* x, int ldx,
                  int m, const void* norm_w, float eps, int gemma, const void* residual, int ldr, void* out, int ldo,
                  int epi, void* stream) {
  using namespace hb;
  if (m < 1 || m > hb_nvfp4_gemv_max_rows(n, k) || epi < 0 || epi > 2 || (ldx & 7) != 0) return 1;
  if (epi == kGemvResidual && residual == nullptr) return 1;
  if (epi == kGemvSiluMul && (n & 1)) return 1;
  GemvParams p;
  p.wq = static_cast<const uint8_t*>(wq);
  p.wsf = static_cast<const uint8_t*>(wsf);
  p.wscale = static_cast<const float*>(wscale);
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.n = n; p.k = k; p.ka = ka; p.m = m; p.ldx = ldx; p.ldr = ldr; p.ldo = ldo; p.epi = epi; p.gemma = gemma;
  p.eps = eps;
  const size_t smem = static_cast<size_t>(m) * (k + kXPad) * 2 + kGemvWarps * 128 * 4;
  // K slices per tile: as many as keep every CTA resident at once (four per SM while their rows fit)
  const int ntiles = n / 16, nchunks = k / kChunk;
  int per_sm = static_cast<int>((220 * 1024) / (smem + 1024));
  per_sm = per_sm > 4 ? 4 : per_sm < 1 ? 1 : per_sm;
  const int slots = 148 * per_sm;
  int ksplit = 1;
  for (int cand = 4; cand >= 1; cand >>= 1) {
    const int c = (ntiles * cand + kGemvWarps - 1) / kGemvWarps;
    if ((c <= slots && nchunks >= 2 * cand) || cand == 1) { ksplit = cand; break; }
  }
  const int ctas = (ntiles * ksplit + kGemvWarps - 1) / kGemvWarps;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
#define HB_GEMV_LAUNCH(D)                                                                       \
  (ksplit == 4 ? launch_gemv<4, D>(p, ctas, smem, st)                                         \
   : ksplit == 2 ? launch_gemv<2, D>(p, ctas, smem, st) : launch_gemv<1, D>(p, ctas, smem, st))
  e = g_gemv_deq == 1 ? HB_GEMV_LAUNCH(1) : HB_GEMV_LAUNCH(0);
#undef HB_GEMV_LAUNCH
  return e == cudaSuccess ? 0 : 2;
}

}  // extern "C"
