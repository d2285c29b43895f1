// tcgen05 GEMM for sm_100a: D[ra, rb] = A[ra, K] * B[rb, K]^T with fp32 accumulation in TMEM.
//
//   * kind bf16  : tcgen05.mma kind::f16, 64-element (128-byte) K tiles.
//   * kind nvfp4 : tcgen05.mma kind::mxf4nvf4.block_scale (e2m1 values, ue4m3 scale per 16 elements),
//                  256-element (128-byte) K tiles; scale factors travel global -> shared by bulk copies of the
//                  128x4-swizzled blocks and shared -> TMEM by tcgen05.cp.
//
//   * kind fp8   : tcgen05.mma kind::f8f6f4 on e4m3 operands, 128-element (128-byte) K tiles; per-tensor scales
//                  fold into alpha, a per-token scale vector (dynamic activation quantisation) into the epilogue.
//   * kind w3    : the A operand is a 3-bit weight copy (asymmetric integer codes, groups of 64 along K, bf16 scale
//                  and zero per row and group) stored as one 4096-byte tile per (128 rows, 64 columns). A bulk copy
//                  brings the tile into the stage, the four epilogue warps (one thread per row) expand it to the
//                  128-byte-swizzled bf16 A tile of the same stage - two codes per logic op through the bf16 bit
//                  pattern of 128 + code, then one packed subtract and one packed fma - and the MMA is kind::f16.
//                  HBM sees 4 bits per weight; the tensor cores see bf16.
//
// One CTA computes a 128 x BN tile. Warp 0 issues TMA loads into a ring of 128-byte-swizzled stages, one lane
// of warp 1 issues the MMAs and commits stage releases, warps 2-5 read the accumulator back with tcgen05.ld
// and run the epilogue. With `swap` the 128-row operand is the weight matrix and the (few) tokens sit on the
// N side, which keeps decode-sized problems on the tensor cores while streaming each weight byte once.
// Split-K runs as one thread-block cluster per output tile (cluster dims 1 x 1 x splits): every CTA parks its raw
// fp32 partial in its own shared memory, and after a cluster barrier each CTA sums a slice of the tile's columns
// over all partials through distributed shared memory, in split order (deterministic), and applies the epilogue.
// No global workspace, counters or fences are involved.
// The producer issues the weight-side loads of the first ring of stages before `griddepcontrol.wait`, so with
// programmatic dependent launch the weight stream starts while the kernel that produces the activations is
// still running.
//
// Replaces the reference's library GEMM dispatch (hibana/kernels/ops.py:56-128) for bf16 and NVFP4.
#include "gemm.cuh"

#include <mutex>
#include <unordered_map>
#include <memory>
#include <cstring>

#include "hb_common.cuh"
#include "rownorm.cuh"

namespace hb {
namespace {

constexpr int BM = 128;
constexpr int ROW_BYTES = 128;
constexpr int A_TILE_BYTES = BM * ROW_BYTES;
constexpr int NUM_THREADS = 192;

template <int KIND, int BN>
struct Cfg {
  static constexpr int B_TILE_BYTES = BN * ROW_BYTES;
  static constexpr int NRB = (BN + 127) / 128;
  static constexpr int SFA_BYTES = KIND == kGemmNvfp4 ? 4 * 512 : 0;
  static constexpr int SFB_BYTES = KIND == kGemmNvfp4 ? NRB * 4 * 512 : 0;
  static constexpr int PACK_BYTES = KIND == kGemmW3 ? 4096 : 0;   // packed 3-bit tile, behind the operand tiles
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES + SFA_BYTES + SFB_BYTES + PACK_BYTES;
  static constexpr int TX_BYTES = KIND == kGemmW3 ? B_TILE_BYTES + PACK_BYTES : STAGE_BYTES;   // bytes copies deliver
  // Token tiles of up to 64 (decode) keep the ring under ~100 KB so that two CTAs share an SM: the second CTA's
  // prologue and epilogue overlap the first one's streaming, and grids of up to 2 x 148 CTAs are one wave.
  // 128-token tiles (the grouped MoE GEMMs at prefill) get three stages for the same reason: thousands of short
  // CTAs whose fixed cost would otherwise be paid one after the other on every SM.
  static constexpr int SMEM_BUDGET = BN <= 64 ? 100 * 1024 : BN == 128 ? 110 * 1024 : 200 * 1024;
  static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_NEED = BN + (KIND == kGemmNvfp4 ? 16 + 16 * NRB : 0);
  static constexpr int TMEM_COLS =
      TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int CH = BN >= 32 ? 32 : 16;  // accumulator columns per tcgen05.ld
};

struct DevParams {
  const uint8_t* sfa;
  const uint8_t* sfb;
  int ra, rb, k_tiles;
  void* out;
  long long ldo;
  const __nv_bfloat16* residual;
  float alpha;
  const float* alpha_ptr;
  int epilogue, swap, splits;
  float* workspace;
  int* counters;
  int* status;
  int ka_a, ka_b;
  int out_rows, out_cols;
  // grouped (MoE) mode: grid.z = expert, grid.y = chunk of BN tokens of that expert's segment
  const int* grp_start;   // [E] first row of the expert's segment in the sorted activation buffer (multiple of 128)
  const int* grp_cnt;     // [E] rows routed to the expert
  int grp_rows_a;         // weight rows per expert (multiple of 128)
  const int* grp_tiles;   // optional work list: expert * 4096 + chunk (then grid.y = list slot, grid.z = 1)
  const int* grp_ntiles;
  int early_launch;       // release the next kernel's launch at the start of this one (programmatic launch level 2)
  // peer fusion
  int peer_on, world, rank, rows_per_rank;
  uint8_t* peer_base[8];
  long long stage_offset, counter_offset, flag_offset, seq_offset;
  unsigned long long limit_ns;
  // expert-parallel fusion (grouped mode)
  const int* ep_gate_flags;
  const int* ep_seq_ptr;
  const int* ep_row_ret;
  long long ep_ret_offset, ep_ret_flag_offset;
  int* ep_done;
  const float* tok_scale;
  const uint8_t* w3_tiles;   // kind w3: [row blocks][k_tiles][4096]
  // kEpiSiluMulQuant
  uint8_t* q_out;
  uint8_t* q_sf;
  const float* q_gscale;
  int q_ka;
  long long q_ld;
  unsigned long long* prof;   // optional phase timers (hb_gemm_profile), null = off
  int local_reduce;           // unsplit tiles with the weights on the 128-row side go through the parked-partial path
};

// Phase timers of one epilogue thread per CTA, summed over CTAs: nanoseconds since kernel entry at
// [0] set-up done, [1] predecessor complete, [2] accumulator complete, [3] partial parked, [4] cluster barrier 1,
// [5] reduce + stores done, [6] cluster barrier 2; [7] counts CTAs.
__device__ __forceinline__ void prof_mark(const DevParams& p, int slot, unsigned long long t0) {
  if (p.prof != nullptr && threadIdx.x == 64)
    atomicAdd(p.prof + slot, slot == 7 ? 1ull : static_cast<unsigned long long>(globaltimer_ns() - t0));
}

// x * sigmoid(x) with the approximate divide (two special-function ops): the result is rounded to bf16 anyway
__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.f + __expf(-x)); }

// Applies the epilogue to CH accumulator values of one thread: `row` indexes the A operand, columns
// [col0, col0 + CH) the B operand.
template <int CH>
__device__ __forceinline__ void epilogue_chunk(const DevParams& p, float (&v)[CH], int row, int row_lim, int col0,
                                               int col_lim, float alpha, int lane) {
  const bool row_ok = row < row_lim;
  if (p.swap) {
    if (p.tok_scale != nullptr) {   // tokens are the columns here
#pragma unroll
      for (int j = 0; j < CH; ++j) v[j] *= col0 + j < col_lim ? p.tok_scale[col0 + j] : 0.f;
    }
    // out[token = col][feature = row]; lanes are consecutive features -> coalesced per token.
    if (p.epilogue == kEpiSiluMul) {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const float x = v[j] * alpha;
        const float other = __shfl_xor_sync(0xffffffffu, x, 1);
        const int col = col0 + j;
        if (row_ok && col < col_lim && (lane & 1) == 0)
          out[static_cast<long long>(col) * p.ldo + (row >> 1)] = __float2bfloat16(silu(x) * other);
      }
    } else if (p.epilogue == kEpiStoreF32) {
      float* out = static_cast<float*>(p.out);
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int col = col0 + j;
        if (row_ok && col < col_lim) out[static_cast<long long>(col) * p.ldo + row] = v[j] * alpha;
      }
    } else if (p.epilogue == kEpiReturn) {
      // column = one routed row; it goes home to the rank it came from (plain stores over NVLink, lanes are
      // consecutive features of that row)
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int col = col0 + j;
        if (row_ok && col < col_lim) {
          const int meta = p.ep_row_ret[col];
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.peer_base[(meta >> 24) & 7] + p.ep_ret_offset) +
                               static_cast<long long>(meta & 0xFFFFFF) * p.ldo + row;
          *dst = __float2bfloat16(v[j] * alpha);
        }
      }
    } else {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
      for (int j = 0; j < CH; ++j) {
        const int col = col0 + j;
        if (row_ok && col < col_lim) {
          const long long o = static_cast<long long>(col) * p.ldo + row;
          float x = v[j] * alpha;
          if (p.epilogue == kEpiResidual) x += __bfloat162float(p.residual[o]);
          if (p.epilogue == kEpiRelu2) x = x > 0.f ? x * x : 0.f;
          out[o] = __float2bfloat16(x);
        }
      }
    }
    return;
  }
  if (!row_ok) return;
  // out[token = row][feature = col]; each thread owns CH consecutive features of its row.
  const long long base = static_cast<long long>(row) * p.ldo;
  if (p.epilogue == kEpiSiluMul) {
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + base + (col0 >> 1);
    const bool full = (col0 + CH <= col_lim) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    if (full) {
      uint32_t w[CH / 4];
#pragma unroll
      for (int j = 0; j < CH / 4; ++j)
        w[j] = pack_bf16(silu(v[4 * j] * alpha) * (v[4 * j + 1] * alpha),
                         silu(v[4 * j + 2] * alpha) * (v[4 * j + 3] * alpha));
#pragma unroll
      for (int j = 0; j < CH / 16; ++j)
        reinterpret_cast<uint4*>(out)[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < CH / 2; ++j)
        if (col0 + 2 * j + 1 < col_lim)
          out[j] = __float2bfloat16(silu(v[2 * j] * alpha) * (v[2 * j + 1] * alpha));
    }
  } else if (p.epilogue == kEpiStoreF32) {
    float* out = static_cast<float*>(p.out) + base + col0;
#pragma unroll
    for (int j = 0; j < CH; ++j)
      if (col0 + j < col_lim) out[j] = v[j] * alpha;
  } else {
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + base + col0;
    const __nv_bfloat16* res = p.epilogue == kEpiResidual ? p.residual + base + col0 : nullptr;
    const bool full = (col0 + CH <= col_lim) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                      (res == nullptr || (reinterpret_cast<uintptr_t>(res) & 15) == 0);
    if (full) {
#pragma unroll
      for (int j = 0; j < CH / 8; ++j) {
        float x[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) x[t] = v[8 * j + t] * alpha;
        if (res != nullptr) {
          const uint4 r = reinterpret_cast<const uint4*>(res)[j];
          x[0] += bf16_lo(r.x); x[1] += bf16_hi(r.x); x[2] += bf16_lo(r.y); x[3] += bf16_hi(r.y);
          x[4] += bf16_lo(r.z); x[5] += bf16_hi(r.z); x[6] += bf16_lo(r.w); x[7] += bf16_hi(r.w);
        }
        reinterpret_cast<uint4*>(out)[j] =
            make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < CH; ++j)
        if (col0 + j < col_lim) {
          float x = v[j] * alpha;
          if (res != nullptr) x += __bfloat162float(res[j]);
          out[j] = __float2bfloat16(x);
        }
    }
  }
}

// Epilogue of four consecutive features (rows grow0 .. grow0 + 3 of the weight operand, grow0 a multiple of 4) of one
// token with the weights on the 128-row side: out[tok][grow0 ..]. The split-K reduce hands its sums over in this
// shape (one 16-byte distributed-shared-memory load per partial), so gate / up pairs sit in one thread and every
// store is 4 to 16 bytes wide and contiguous across the warp.
template <int NC>
__device__ __forceinline__ void epilogue_rows4(const DevParams& p, const float4 (&v)[NC], const bool (&live)[NC],
                                               const int (&tok)[NC], int grow0, int row_lim, float alpha,
                                               float q_inv_gs) {
  // NC independent columns per call, every stage written as a loop over them: the work per column is a chain of
  // dependent special-function and conversion instructions, and with four epilogue warps per CTA nothing else
  // hides their latency, so the columns' chains are interleaved.
  float x[NC][4];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const float a = p.tok_scale != nullptr && live[c] ? alpha * p.tok_scale[tok[c]] : alpha;
    x[c][0] = v[c].x * a; x[c][1] = v[c].y * a; x[c][2] = v[c].z * a; x[c][3] = v[c].w * a;
  }
  const bool full = grow0 + 3 < row_lim && (p.ldo & 3) == 0;
  if (p.epilogue == kEpiSiluMulQuant) {
    // This thread holds output features f0, f0 + 1 (f0 = grow0 / 2) of each token; the 8 lanes that share lane / 8
    // hold one 16-feature NVFP4 group. Group maximum and the 8 packed bytes travel by shuffles (every lane of the
    // warp is here: the column loop is warp-uniform); lane 0 of the group writes the 8 bytes, lane 0 of the warp
    // the four scale bytes of the token, which are one aligned 32-bit word of the swizzled block.
    float y0[NC], y1[NC], amax[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      y0[c] = __bfloat162float(__float2bfloat16(silu(x[c][0]) * x[c][1]));   // rounded as a bf16 store would
      y1[c] = __bfloat162float(__float2bfloat16(silu(x[c][2]) * x[c][3]));
      amax[c] = fmaxf(fabsf(y0[c]), fabsf(y1[c]));
    }
#pragma unroll
    for (int sh = 1; sh <= 4; sh <<= 1)
#pragma unroll
      for (int c = 0; c < NC; ++c) amax[c] = fmaxf(amax[c], __shfl_xor_sync(0xffffffffu, amax[c], sh));
    uint32_t sfb[NC], pk[NC], hi[NC], sfw[NC];
    const int j = threadIdx.x & 7;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      sfb[c] = float_to_e4m3(amax[c] * (1.f / 6.f) * q_inv_gs);
      const float sf = e4m3_to_float(sfb[c]);
      const float inv = sf > 0.f ? 1.f / (sf * (1.f / q_inv_gs)) : 0.f;
      pk[c] = e2m1x2(y0[c] * inv, y1[c] * inv) << (8 * (j & 3));
      sfw[c] = sfb[c] << (8 * ((threadIdx.x >> 3) & 3));
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) pk[c] |= __shfl_xor_sync(0xffffffffu, pk[c], 1);
#pragma unroll
    for (int c = 0; c < NC; ++c) pk[c] |= __shfl_xor_sync(0xffffffffu, pk[c], 2);
#pragma unroll
    for (int c = 0; c < NC; ++c) hi[c] = __shfl_xor_sync(0xffffffffu, pk[c], 4);
#pragma unroll
    for (int c = 0; c < NC; ++c) sfw[c] |= __shfl_xor_sync(0xffffffffu, sfw[c], 8);
#pragma unroll
    for (int c = 0; c < NC; ++c) sfw[c] |= __shfl_xor_sync(0xffffffffu, sfw[c], 16);
    const int grp = grow0 >> 5;                        // 16-feature group index within a token's row
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      if (!live[c]) continue;
      if (j == 0)
        *reinterpret_cast<uint2*>(p.q_out + static_cast<size_t>(tok[c]) * p.q_ld + grp * 8) = make_uint2(pk[c], hi[c]);
      if ((threadIdx.x & 31) == 0)
        *reinterpret_cast<uint32_t*>(p.q_sf + row_sf_off(tok[c], grp, p.q_ka)) = sfw[c];
    }
  } else if (p.epilogue == kEpiSiluMul) {
    uint32_t w[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) w[c] = pack_bf16(silu(x[c][0]) * x[c][1], silu(x[c][2]) * x[c][3]);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      if (!live[c]) continue;
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(tok[c]) * p.ldo + (grow0 >> 1);
      if (full) {
        *reinterpret_cast<uint32_t*>(out) = w[c];
      } else {
        if (grow0 + 1 < row_lim) out[0] = __float2bfloat16(bf16_lo(w[c]));
        if (grow0 + 3 < row_lim) out[1] = __float2bfloat16(bf16_hi(w[c]));
      }
    }
  } else if (p.epilogue == kEpiStoreF32) {
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      if (!live[c]) continue;
      float* out = static_cast<float*>(p.out) + static_cast<long long>(tok[c]) * p.ldo + grow0;
      if (full) {
        *reinterpret_cast<float4*>(out) = make_float4(x[c][0], x[c][1], x[c][2], x[c][3]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (grow0 + i < row_lim) out[i] = x[c][i];
      }
    }
  } else {
    uint2 r[NC];
    if (p.epilogue == kEpiResidual && full) {
#pragma unroll
      for (int c = 0; c < NC; ++c)
        r[c] = live[c] ? *reinterpret_cast<const uint2*>(p.residual + static_cast<long long>(tok[c]) * p.ldo + grow0)
                       : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      if (!live[c]) continue;
      const long long o = static_cast<long long>(tok[c]) * p.ldo + grow0;
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + o;
      if (full) {
        if (p.epilogue == kEpiResidual) {
          x[c][0] += bf16_lo(r[c].x); x[c][1] += bf16_hi(r[c].x); x[c][2] += bf16_lo(r[c].y); x[c][3] += bf16_hi(r[c].y);
        }
        if (p.epilogue == kEpiRelu2) {
#pragma unroll
          for (int i = 0; i < 4; ++i) x[c][i] = x[c][i] > 0.f ? x[c][i] * x[c][i] : 0.f;
        }
        *reinterpret_cast<uint2*>(out) = make_uint2(pack_bf16(x[c][0], x[c][1]), pack_bf16(x[c][2], x[c][3]));
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (grow0 + i < row_lim) {
            float y = x[c][i];
            if (p.epilogue == kEpiResidual) y += __bfloat162float(p.residual[o + i]);
            if (p.epilogue == kEpiRelu2) y = y > 0.f ? y * y : 0.f;
            out[i] = __float2bfloat16(y);
          }
      }
    }
  }
}

// kEpiReturn: one thread per CTA reports in after its stores are fenced system-wide; the last CTA of the grid
// publishes this rank's sequence number on every rank's return flag and re-arms the counter.
// A CTA that wrote nothing (`wrote` false: an expert chunk past the expert's rows) skips the system-wide fence,
// which costs microseconds over NVLink and would otherwise be paid by every empty chunk of the grid.
__device__ __forceinline__ void ep_publish_returned(const DevParams& p) {
  const int seq = *reinterpret_cast<const volatile int*>(p.ep_seq_ptr) + 1;
  __threadfence_system();
  for (int r = 0; r < p.world; ++r) {
    int* f = reinterpret_cast<int*>(p.peer_base[r] + p.ep_ret_flag_offset) + p.rank;
    asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(f), "r"(seq) : "memory");
  }
}
// With a work list only the CTAs of list slots that exist take part in the count (grid.x of them per slot): the
// thousands of CTAs beyond the list return without touching the counter, which otherwise serialised them all on
// one address.
__device__ __forceinline__ void ep_cta_done(const DevParams& p, bool wrote = true) {
  if (wrote) __threadfence_system();
  const int total = p.grp_tiles != nullptr ? static_cast<int>(gridDim.x) * *p.grp_ntiles
                                           : static_cast<int>(gridDim.x * gridDim.y * gridDim.z);
  if (atomicAdd(p.ep_done, 1) == total - 1) {
    *p.ep_done = 0;
    ep_publish_returned(p);
  }
}

template <int KIND, int BN>
__global__ void __launch_bounds__(NUM_THREADS, BN <= 64 ? 2 : 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma, const __grid_constant__ CUtensorMap tmb, const DevParams p) {
  using C = Cfg<KIND, BN>;
  constexpr int S = C::STAGES;
  constexpr int CH = C::CH;
  const unsigned long long t_entry = p.prof != nullptr ? globaltimer_ns() : 0ull;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S * C::STAGE_BYTES);
  uint64_t* empty = full + S;
  uint64_t* dq = empty + S;       // kind w3: the A tile of the stage has been expanded (128 arrivals)
  uint64_t* accum = dq + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x;
  int tile_b = blockIdx.y, split = blockIdx.z;
  int a_row0 = tile_a * BM, b_row0 = tile_b * BN, row_lim = p.ra, col_lim = p.rb;
  const float* alpha_ptr = p.alpha_ptr;
  if (p.grp_cnt != nullptr) {
    int e = blockIdx.z, chunk = blockIdx.y;
    if (p.grp_tiles != nullptr) {
      if (static_cast<int>(blockIdx.y) >= *p.grp_ntiles) {   // uniform, before any barrier or TMEM allocation
        // an empty list (no rows routed to this rank) still owes every rank its "returned" flag: one CTA says so
        if (p.epilogue == kEpiReturn && *p.grp_ntiles == 0 && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0)
          ep_publish_returned(p);
        return;
      }
      const int code = p.grp_tiles[blockIdx.y];
      e = code >> 12;
      chunk = code & 4095;
    }
    const int cnt = p.grp_cnt[e];
    if (chunk * BN >= cnt) {   // uniform: before any barrier or TMEM allocation
      if (p.epilogue == kEpiReturn && threadIdx.x == 0) ep_cta_done(p, false);
      return;
    }
    a_row0 = e * p.grp_rows_a + tile_a * BM;
    b_row0 = p.grp_start[e] + chunk * BN;
    row_lim = p.grp_rows_a;
    col_lim = b_row0 + min(BN, cnt - chunk * BN);
    if (alpha_ptr != nullptr) alpha_ptr += e;
    split = 0;
    tile_b = 0;
  }
  // unsplit, ungrouped tiles with the weights on the 128-row side reduce "over one partial" (see below)
  const bool local_reduce = p.splits == 1 && p.swap && p.grp_cnt == nullptr && p.epilogue != kEpiReturn &&
                            (p.local_reduce || p.epilogue == kEpiSiluMulQuant);
  const int kt_per = (p.k_tiles + p.splits - 1) / p.splits;
  const int kt0 = split * kt_per;
  const int kt1 = min(kt0 + kt_per, p.k_tiles);
  const int nkt = max(kt1 - kt0, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&dq[s], 128);
    }
    mbar_init(accum, 1);
    *abort = 0;
    fence_mbar_init();
    prefetch_tmap(&tma);
    prefetch_tmap(&tmb);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  prof_mark(p, 0, t_entry);
  // Let the kernel after this one be scheduled now (it waits for this grid's completion before it reads anything
  // this grid writes): its launch latency and prologue overlap this grid's main loop.
  if (p.early_launch) grid_dep_launch();

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      // side 0 = A operand (+ its scales), side 1 = B operand (+ its scales) of K tile i into stage i % S
      auto load_side = [&](int i, int side) {
        const int s = i % S;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        const int kt = kt0 + i;
        const int kx = (KIND == kGemmBf16 || KIND == kGemmW3) ? kt * 64 : kt * 128;
        if (side == 0) {
          if constexpr (KIND == kGemmW3) {
            bulk_load(st + A_TILE_BYTES + C::B_TILE_BYTES,
                      p.w3_tiles + (static_cast<size_t>(a_row0 >> 7) * p.k_tiles + kt) * 4096, 4096, &full[s]);
            return;
          }
          tma_load_2d(st, &tma, &full[s], kx, a_row0);
          if constexpr (KIND == kGemmNvfp4)
            bulk_load(st + A_TILE_BYTES + C::B_TILE_BYTES,
                      p.sfa + (static_cast<size_t>(a_row0 >> 7) * p.ka_a + kt * 4) * 512, 2048, &full[s]);
        } else {
          tma_load_2d(st + A_TILE_BYTES, &tmb, &full[s], kx, b_row0);
          if constexpr (KIND == kGemmNvfp4) {
#pragma unroll
            for (int rb = 0; rb < C::NRB; ++rb)
              bulk_load(st + A_TILE_BYTES + C::B_TILE_BYTES + C::SFA_BYTES + rb * 2048,
                        p.sfb + (static_cast<size_t>((b_row0 >> 7) + rb) * p.ka_b + kt * 4) * 512, 2048, &full[s]);
          }
        }
      };
      // First ring of stages (their `empty` barriers are trivially free): the weights go first; they depend on
      // nothing. Then the waits for whoever produces the activations: the preceding grid (programmatic
      // dependent launch), the source rank of a gathered row tile, or every sender of an expert-parallel
      // dispatch. Then the activations.
      const int wside = p.swap ? 0 : 1;
      const int pre = min(S, nkt);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], C::TX_BYTES);
        load_side(i, wside);
      }
      grid_dep_wait();
      bool ready = true;
      if (p.peer_on && p.flag_offset >= 0) {
        // all-gather -> GEMM: the rows of this A tile were pushed into local memory by rank `src`
        const int src = a_row0 / p.rows_per_rank;
        const int* flag = reinterpret_cast<const int*>(p.peer_base[p.rank] + p.flag_offset) + src;
        const int want = *reinterpret_cast<const volatile int*>(p.peer_base[p.rank] + p.seq_offset);
        const uint64_t t0 = globaltimer_ns();
        ready = false;
        for (unsigned long long it = 0, cap = spin_cap(p.limit_ns); it < cap; ++it) {
          int v;
          asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
          if (v - want >= 0) {
            ready = true;
            break;
          }
          if ((it & 63u) == 63u && (globaltimer_ns() - t0 > p.limit_ns || *reinterpret_cast<volatile int*>(p.status) != 0)) break;
        }
      } else if (p.ep_gate_flags != nullptr) {
        // expert-parallel dispatch -> grouped GEMM: every sender has published its rows
        const int want = *reinterpret_cast<const volatile int*>(p.ep_seq_ptr) + 1;
        const uint64_t t0 = globaltimer_ns();
        for (int r = 0; r < p.world && ready; ++r) {
          ready = false;
          for (unsigned long long it = 0, cap = spin_cap(p.limit_ns); it < cap; ++it) {
            int v;
            asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p.ep_gate_flags + r) : "memory");
            if (v - want >= 0) {
              ready = true;
              break;
            }
            if ((it & 63u) == 63u && (globaltimer_ns() - t0 > p.limit_ns || *reinterpret_cast<volatile int*>(p.status) != 0)) break;
          }
        }
      }
      if (!ready) {
        *abort = 1;
        set_status(p.status, kTimeoutGate);
      }
      // On a failed wait the activation side is still loaded (whatever is there): the stages then complete, the
      // barriers balance and no copy is left in flight; the status word tells the host the result is void.
      for (int i = 0; i < pre; ++i) {
        load_side(i, wside ^ 1);
        ++issued;
      }
      for (int i = pre; i < nkt && !*abort; ++i) {
        const int s = i % S;
        const uint32_t ph = (i / S) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort, p.status, kTimeoutEmpty)) break;
        mbar_expect_tx(&full[s], C::TX_BYTES);
        load_side(i, 0);
        load_side(i, 1);
        ++issued;
      }
      if (*abort) {
        // Wait (bounded) for the copies still in flight so that none lands after the CTA has gone.
        volatile int ignore = 0;
        for (int j = max(issued - S, 0); j < issued; ++j)
          mbar_wait(&full[j % S], (j / S) & 1, &ignore, nullptr, kTimeoutDrain);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = KIND == kGemmNvfp4 ? make_idesc_nvf4(BM, BN)
                                 : KIND == kGemmFp8 ? make_idesc_e4m3(BM, BN) : make_idesc_bf16(BM, BN);
      const uint32_t sfa_t = tmem_base + BN;
      const uint32_t sfb_t = sfa_t + 16;
      bool ok = true;
      for (int i = 0; i < nkt; ++i) {
        const int s = i % S;
        const uint32_t ph = (i / S) & 1;
        if (!mbar_wait(&full[s], ph, abort, p.status, kTimeoutFull)) {
          ok = false;
          break;
        }
        if constexpr (KIND == kGemmW3) {
          if (!mbar_wait(&dq[s], ph, abort, p.status, kTimeoutFull)) {
            ok = false;
            break;
          }
        }
        tc_fence_after();
        uint8_t* st = smem + s * C::STAGE_BYTES;
        const uint64_t adesc = make_desc_sw128(smem_u32(st));
        const uint64_t bdesc = make_desc_sw128(smem_u32(st + A_TILE_BYTES));
        if constexpr (KIND == kGemmNvfp4) {
          const uint32_t sf = smem_u32(st + A_TILE_BYTES + C::B_TILE_BYTES);
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            tmem_cp_32x128b_x4(sfa_t + kb * 4, make_desc_sf(sf + kb * 512));
#pragma unroll
            for (int rb = 0; rb < C::NRB; ++rb)
              tmem_cp_32x128b_x4(sfb_t + kb * 4 * C::NRB + rb * 4,
                                 make_desc_sf(sf + C::SFA_BYTES + rb * 2048 + kb * 512));
          }
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            mma_nvf4(tmem_base, adesc + kb * 2, bdesc + kb * 2, idesc, (i > 0 || kb > 0) ? 1u : 0u,
                     sfa_t + kb * 4, sfb_t + kb * 4 * C::NRB);
        } else if constexpr (KIND == kGemmFp8) {
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            mma_f8(tmem_base, adesc + kb * 2, bdesc + kb * 2, idesc, (i > 0 || kb > 0) ? 1u : 0u);
        } else {
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            mma_f16(tmem_base, adesc + kb * 2, bdesc + kb * 2, idesc, (i > 0 || kb > 0) ? 1u : 0u);
        }
        tc_commit(&empty[s]);
      }
      if (ok) tc_commit(accum);
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    if constexpr (KIND == kGemmW3) {
      // Expand the packed tile of every stage into its bf16 A tile: thread = row. Word w of the row's 28 code
      // bytes holds codes 10 w + 2 i (low half, bits 3 i ..) and 10 w + 2 i + 1 (high half); OR-ing 0x4300 into
      // both halves makes the bf16 numbers 128 + code, exact, so (x - 128) * scale + bias is two packed ops.
      const int r = q * 32 + lane;
      const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
      for (int i = 0; i < nkt; ++i) {
        const int s = i % S;
        if (!mbar_wait(&full[s], (i / S) & 1, abort, p.status, kTimeoutFull)) break;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        const uint8_t* pk = st + A_TILE_BYTES + C::B_TILE_BYTES;
        const uint32_t sz = *reinterpret_cast<const uint32_t*>(pk + 128 * 28 + r * 4);
        __nv_bfloat162 sc2, bias2;
        *reinterpret_cast<uint32_t*>(&sc2) = (sz & 0xFFFFu) | (sz << 16);
        *reinterpret_cast<uint32_t*>(&bias2) = (sz >> 16) | (sz & 0xFFFF0000u);
        uint32_t o[32];
#pragma unroll
        for (int w = 0; w < 7; ++w) {
          const uint32_t x = *reinterpret_cast<const uint32_t*>(pk + r * 28 + w * 4);
#pragma unroll
          for (int j = 0; j < 5; ++j) {
            if (w * 5 + j < 32) {
              uint32_t m = ((x >> (3 * j)) & 0x00070007u) | 0x43004300u;
              __nv_bfloat162 v = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&m), k128);
              v = __hfma2(v, sc2, bias2);
              o[w * 5 + j] = *reinterpret_cast<uint32_t*>(&v);
            }
          }
        }
        const uint32_t row_addr = smem_u32(st) + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + ((c ^ (r & 7)) << 4)),
                       "r"(o[4 * c]), "r"(o[4 * c + 1]), "r"(o[4 * c + 2]), "r"(o[4 * c + 3])
                       : "memory");
        fence_proxy_async_smem();
        mbar_arrive(&dq[s]);
      }
    }
    grid_dep_wait();
    prof_mark(p, 1, t_entry);
    const bool ok = nkt > 0 ? mbar_wait(accum, 0, abort, p.status, kTimeoutAccum) : true;
    tc_fence_after();
    prof_mark(p, 2, t_entry);
    const int row = tile_a * BM + q * 32 + lane;   // feature index (within the expert in grouped mode)
    const uint32_t tlane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    float alpha = p.alpha;
    if (alpha_ptr != nullptr) alpha *= *alpha_ptr;
    if (p.tok_scale != nullptr && !p.swap && row < row_lim) alpha *= p.tok_scale[row];   // tokens are the rows
    if (ok && p.splits == 1 && !p.swap && p.epilogue != kEpiStoreF32 && BN >= 64 && (p.rb & 7) == 0 &&
        (p.ldo & 7) == 0) {
      // Staged epilogue (tokens on the 128-row side): every thread parks its row chunk as bf16 in shared memory
      // (the stage ring is idle once the accumulator is complete), then each warp writes its 32 rows with
      // fully coalesced 16-byte stores: to the local output, or (scatter) to the staging rows of the rank that
      // owns them, over NVLink.
      const bool silu_mul = p.epilogue == kEpiSiluMul;
      const bool quant = p.epilogue == kEpiSiluMulQuant;
      const float q_inv_gs = quant ? 1.f / *p.q_gscale : 0.f;
      constexpr int PITCH = BN * 2 + 16;
      uint8_t* tile = smem + static_cast<size_t>(q) * 32 * PITCH;
      uint8_t* my_row = tile + lane * PITCH;
      for (int c0 = 0; c0 < BN; c0 += CH) {
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_32x32(tlane + c0, r);
        else tmem_ld_32x16(tlane + c0, r);
        tmem_ld_wait();
        if (quant) {
          // SiLU-mul + NVFP4 requantisation: a thread's 32 accumulator columns are 16 gate / up pairs, exactly one
          // 16-feature group of its token: 8 packed bytes at [c0 / 4] of the parked row and one scale byte behind
          // the BN / 4 packed bytes. Same arithmetic, in the same order, as the swapped epilogue (epilogue_rows4)
          // and the stand-alone quantiser.
          if constexpr (CH == 32) {
            float y[16];
#pragma unroll
            for (int t = 0; t < 16; ++t)
              y[t] = __bfloat162float(__float2bfloat16(silu(__uint_as_float(r[2 * t]) * alpha) *
                                                       (__uint_as_float(r[2 * t + 1]) * alpha)));
            const uint32_t sfb = quant16(y, q_inv_gs, reinterpret_cast<uint2*>(my_row + c0 / 4));
            my_row[BN / 4 + c0 / 32] = static_cast<uint8_t>(sfb);
          }
        } else if (silu_mul) {
          uint32_t w[CH / 4];
#pragma unroll
          for (int t = 0; t < CH / 4; ++t)
            w[t] = pack_bf16(silu(__uint_as_float(r[4 * t]) * alpha) * (__uint_as_float(r[4 * t + 1]) * alpha),
                             silu(__uint_as_float(r[4 * t + 2]) * alpha) * (__uint_as_float(r[4 * t + 3]) * alpha));
#pragma unroll
          for (int t = 0; t < CH / 16; ++t)
            *reinterpret_cast<uint4*>(my_row + c0 + 16 * t) = make_uint4(w[4 * t], w[4 * t + 1], w[4 * t + 2], w[4 * t + 3]);
        } else {
          uint32_t w[CH / 2];
#pragma unroll
          for (int t = 0; t < CH / 2; ++t)
            w[t] = pack_bf16(__uint_as_float(r[2 * t]) * alpha, __uint_as_float(r[2 * t + 1]) * alpha);
#pragma unroll
          for (int t = 0; t < CH / 8; ++t)
            *reinterpret_cast<uint4*>(my_row + c0 * 2 + 16 * t) = make_uint4(w[4 * t], w[4 * t + 1], w[4 * t + 2], w[4 * t + 3]);
        }
      }
      __syncwarp();
      if (quant) {
        // packed bytes: BN / 4 per row = BN / 64 16-byte chunks of two groups each, whole rows per store instruction
        constexpr int QCH = BN >= 64 ? BN / 64 : 1;     // (this branch runs with BN >= 64 only)
        constexpr int ROWS = 32 / QCH;
        for (int r0 = 0; r0 < 32; r0 += ROWS) {
          const int lr = r0 + lane / QCH;
          const int ch = lane % QCH;
          const int grow = tile_a * BM + q * 32 + lr;
          if (grow < row_lim && b_row0 + ch * 64 + 64 <= col_lim)
            *reinterpret_cast<uint4*>(p.q_out + static_cast<size_t>(grow) * p.q_ld + (b_row0 >> 2) + ch * 16) =
                *reinterpret_cast<const uint4*>(tile + lr * PITCH + ch * 16);
        }
        // scale bytes: each lane writes its own row's BN / 32 groups (four groups of a K atom are one 32-bit word
        // of the swizzled block; the feature count is a multiple of 64, so groups come in valid pairs)
        const int grow = tile_a * BM + q * 32 + lane;
        if (grow < row_lim) {
#pragma unroll
          for (int g2 = 0; g2 < BN / 64; ++g2) {
            if (b_row0 + g2 * 64 + 64 <= col_lim)
              *reinterpret_cast<uint16_t*>(p.q_sf + row_sf_off(grow, (b_row0 >> 5) + 2 * g2, p.q_ka)) =
                  *reinterpret_cast<const uint16_t*>(my_row + BN / 4 + 2 * g2);
          }
        }
      }
      const int out_cols = silu_mul ? BN / 2 : BN;            // columns this tile produces
      const int chunks = out_cols / 8;                          // 16-byte chunks per row
      const int rows_per_instr = 32 / chunks > 0 ? 32 / chunks : 1;
      const int col_base = silu_mul ? (b_row0 >> 1) : b_row0;   // first output column of the tile
      const int col_end = silu_mul ? (col_lim >> 1) : col_lim;
      for (int r0 = quant ? 32 : 0; r0 < 32; r0 += rows_per_instr) {   // (the quantising epilogue has stored)
        for (int cc = 0; cc < chunks; cc += 32) {
          const int lr = r0 + (chunks >= 32 ? 0 : lane / chunks);
          const int ch = chunks >= 32 ? cc + lane : lane % chunks;
          const int grow = tile_a * BM + q * 32 + lr;
          const int gcol = col_base + ch * 8;
          if (lr < 32 && grow < row_lim && gcol + 8 <= col_end) {
            uint4 v = *reinterpret_cast<const uint4*>(tile + lr * PITCH + ch * 16);
            __nv_bfloat16* dst;
            if (p.epilogue == kEpiScatter) {
              const int owner = grow / p.rows_per_rank;
              dst = reinterpret_cast<__nv_bfloat16*>(p.peer_base[owner] + p.stage_offset) +
                    (static_cast<long long>(p.rank) * p.rows_per_rank + (grow - owner * p.rows_per_rank)) * p.ldo + gcol;
            } else {
              dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(grow) * p.ldo + gcol;
              if (p.epilogue == kEpiResidual) {
                const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(grow) * p.ldo + gcol);
                v.x = pack_bf16(bf16_lo(v.x) + bf16_lo(rr.x), bf16_hi(v.x) + bf16_hi(rr.x));
                v.y = pack_bf16(bf16_lo(v.y) + bf16_lo(rr.y), bf16_hi(v.y) + bf16_hi(rr.y));
                v.z = pack_bf16(bf16_lo(v.z) + bf16_lo(rr.z), bf16_hi(v.z) + bf16_hi(rr.z));
                v.w = pack_bf16(bf16_lo(v.w) + bf16_lo(rr.w), bf16_hi(v.w) + bf16_hi(rr.w));
              }
            }
            *reinterpret_cast<uint4*>(dst) = v;
          }
        }
      }
      if (p.epilogue == kEpiScatter) {
        // make the tile visible system-wide, then one arrival on the owner's counter for this source
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int owner0 = min(a_row0 / p.rows_per_rank, p.world - 1);
          int* cnt = reinterpret_cast<int*>(p.peer_base[owner0] + p.counter_offset) + p.rank;
          asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
        }
      }
    } else if (ok && p.splits == 1 && !local_reduce) {
      for (int c0 = 0; c0 < BN; c0 += CH) {
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_32x32(tlane + c0, r);
        else tmem_ld_32x16(tlane + c0, r);
        tmem_ld_wait();
        float v[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) v[j] = nkt > 0 ? __uint_as_float(r[j]) : 0.f;
        epilogue_chunk<CH>(p, v, row, row_lim, b_row0 + c0, col_lim, alpha, lane);
      }
    } else if (ok) {
      // Split-K: park the raw partial in this CTA's shared memory as [column][row] fp32 (the stage ring is idle
      // once the accumulator is complete); lanes are consecutive rows, so the stores are conflict-free.
      float* part = reinterpret_cast<float*>(smem);
      const int lrow = q * 32 + lane;
      for (int c0 = 0; c0 < BN; c0 += CH) {
        uint32_t r[CH];
        if constexpr (CH == 32) tmem_ld_32x32(tlane + c0, r);
        else tmem_ld_32x16(tlane + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CH; ++j) part[(c0 + j) * BM + lrow] = nkt > 0 ? __uint_as_float(r[j]) : 0.f;
      }
    }
  }
  prof_mark(p, 3, t_entry);
  if (p.splits > 1 || local_reduce) {
    // Every thread of every CTA of the cluster arrives, whatever happened to its pipeline (all waits above are
    // bounded), so the barrier cannot hang; a timed-out CTA has already raised the status word. An unsplit tile
    // with the weights on the 128-row side takes the same path with one partial (its own): the [column][row]
    // layout in shared memory is what makes its stores wide and its gate / up pairs thread-local.
    __syncwarp();
    if (p.splits > 1) cluster_sync_all();
    else if (warp >= 2) asm volatile("bar.sync 1, 128;" ::: "memory");
    prof_mark(p, 4, t_entry);
    if (warp >= 2) {
      const int q = warp & 3;
      const int lrow = q * 32 + lane;
      const int row = tile_a * BM + lrow;
      float alpha = p.alpha;
      if (alpha_ptr != nullptr) alpha *= *alpha_ptr;
      if (p.tok_scale != nullptr && !p.swap && row < row_lim) alpha *= p.tok_scale[row];
      const int ncols = min(BN, col_lim - b_row0);
      int per = (ncols + p.splits - 1) / p.splits;
      if (!p.swap) per = (per + 15) & ~15;      // feature pairs and 16-byte stores stay inside one slice
      const int c_begin = split * per;
      const int c_end = min(ncols, c_begin + per);
      const uint32_t part_local = smem_u32(smem);
      const float q_inv_gs = p.epilogue == kEpiSiluMulQuant ? 1.f / *p.q_gscale : 0.f;
      if (p.swap) {
        // Weights on the 128-row side: the partials are [token column][128 rows] fp32, so four consecutive rows of
        // one column are one 16-byte load. A thread owns rows 4 r4 .. 4 r4 + 3 of every fourth column of the
        // slice and keeps the loads of two columns over all splits in flight (the reduce is a chain of
        // distributed-shared-memory round trips otherwise), then sums in split order (deterministic).
        const int et = static_cast<int>(threadIdx.x) - 64;
        const int lrow0 = (et & 31) * 4, cg = et >> 5;
        const int grow0 = tile_a * BM + lrow0;
        uint32_t base[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) base[s] = s < p.splits ? map_to_cta(part_local, static_cast<uint32_t>(s)) : part_local;
        if (p.splits == 1) {
          // one partial, this CTA's own: plain shared-memory loads (no cluster addressing), four columns in flight
          const float* part = reinterpret_cast<const float*>(smem);
          constexpr int NC = BN >= 64 ? 8 : 4;      // columns in flight per thread (latency hiding, see epilogue_rows4)
          for (int c = c_begin + cg; c < c_end; c += 4 * NC) {
            float4 v[NC];
            bool live[NC];
            int tok[NC];
#pragma unroll
            for (int i = 0; i < NC; ++i) {
              live[i] = c + 4 * i < c_end;
              tok[i] = b_row0 + c + 4 * i;
              v[i] = live[i] ? *reinterpret_cast<const float4*>(part + (c + 4 * i) * BM + lrow0)
                             : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            epilogue_rows4<NC>(p, v, live, tok, grow0, row_lim, alpha, q_inv_gs);
          }
        } else
        for (int c = c_begin + cg; c < c_end; c += 8) {
          const bool two = c + 4 < c_end;
          float4 a[8], b[8];
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s < p.splits) {
              a[s] = ld_dsmem_v4(base[s] + (c * BM + lrow0) * 4);
              if (two) b[s] = ld_dsmem_v4(base[s] + ((c + 4) * BM + lrow0) * 4);
            }
          float4 sa = make_float4(0.f, 0.f, 0.f, 0.f), sb = sa;
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s < p.splits) {
              sa.x += a[s].x; sa.y += a[s].y; sa.z += a[s].z; sa.w += a[s].w;
              if (two) { sb.x += b[s].x; sb.y += b[s].y; sb.z += b[s].z; sb.w += b[s].w; }
            }
          const float4 vs[2] = {sa, sb};
          const bool live[2] = {true, two};
          const int tok[2] = {b_row0 + c, b_row0 + c + 4};
          epilogue_rows4<2>(p, vs, live, tok, grow0, row_lim, alpha, q_inv_gs);
        }
      } else {
      for (int c0 = c_begin; c0 < c_end; c0 += 16) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
        for (int s = 0; s < p.splits; ++s) {
          const uint32_t src = map_to_cta(part_local, static_cast<uint32_t>(s)) + (c0 * BM + lrow) * 4;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < c_end) v[j] += ld_dsmem_f32(src + j * BM * 4);
        }
        epilogue_chunk<16>(p, v, row, row_lim, b_row0 + c0, b_row0 + c_end, alpha, lane);
      }
      }
    }
    prof_mark(p, 5, t_entry);
    __syncwarp();
    if (p.splits > 1) cluster_sync_all();   // nobody leaves while a peer may still read its partial
    prof_mark(p, 6, t_entry);
  }
  prof_mark(p, 7, t_entry);
  if (p.epilogue == kEpiReturn && warp >= 2) __threadfence_system();   // this thread's remote stores
  tc_fence_before();
  __syncthreads();
  if (p.epilogue == kEpiReturn && threadIdx.x == 0) ep_cta_done(p);
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------- host side
struct KeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.rows); mix(k.cols); mix(k.pitch_bytes); mix(k.box_rows); mix(k.box_cols); mix(k.dtype);
    return h;
  }
};

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
    return reinterpret_cast<EncodeFn>(f);
  }();
  return fn;
}

std::mutex g_tmap_mu;
std::unordered_map<TmapKey, std::unique_ptr<CUtensorMap>, KeyHash> g_tmaps;

unsigned long long* g_gemm_prof = nullptr;
int g_local_reduce = 1;
int g_pdl = 0;   // launch with programmatic stream serialisation (set through hb_gemm_set_pdl)

template <int KIND, int BN>
cudaError_t launch_t(const GemmArgs& a, DevParams& p, dim3 grid, const CUtensorMap* ta, const CUtensorMap* tb,
                     cudaStream_t stream) {
  using C = Cfg<KIND, BN>;
  static bool attr_done = false;
  static int max_clusters[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};   // co-resident clusters per cluster size (0 = unknown)
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_done = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  int splits = p.splits;
  if (splits > 1) {
    // One cluster per output tile; shrink the split count until all clusters of the grid are co-resident
    // (clusters live inside one GPC, so odd sizes can strand SMs).
    const int tiles = grid.x * grid.y;
    for (; splits > 1; --splits) {
      if (splits > 1 && (splits - 1) * ((p.k_tiles + splits - 1) / splits) >= p.k_tiles) continue;
      if (max_clusters[splits] == 0) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(1, 1, splits);
        q.blockDim = dim3(NUM_THREADS);
        q.dynamicSmemBytes = C::SMEM_BYTES;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = 1; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = splits;
        q.attrs = qa; q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_kernel<KIND, BN>, &q) != cudaSuccess || n < 1) {
          (void)cudaGetLastError();
          n = -1;
        }
        max_clusters[splits] = n;
      }
      if (max_clusters[splits] >= tiles) break;
    }
    p.splits = splits;
    grid.z = splits;
    if (splits > 1) {
      attrs[na].id = cudaLaunchAttributeClusterDimension;
      attrs[na].val.clusterDim.x = 1; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = splits;
      ++na;
    }
  }
  if (g_pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.gridDim = grid;
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, gemm_kernel<KIND, BN>, *ta, *tb, static_cast<const DevParams&>(p));
}

}  // namespace

// Copies the (cached) tensor map of `key` into *out. The copy matters: the cache is dropped when it grows past its
// limit, so nothing outside this function may hold a pointer into it.
bool get_tmap_2d(const TmapKey& key, CUtensorMap* out_map) {
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) {
    *out_map = *it->second;
    return true;
  }
  if (g_tmaps.size() > 8192) g_tmaps.clear();
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return false;
  auto m = std::make_unique<CUtensorMap>();
  const cuuint64_t dims[2] = {key.cols, key.rows};
  const cuuint64_t strides[1] = {key.pitch_bytes};
  const cuuint32_t box[2] = {key.box_cols, key.box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = key.dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUresult r = fn(m.get(), dt, 2, const_cast<void*>(key.ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  *out_map = *m;
  g_tmaps.emplace(key, std::move(m));
  return true;
}

void clear_tmap_cache() {
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  g_tmaps.clear();
}

static void out_dims(const GemmArgs& a, int* rows, int* cols) {
  *rows = a.swap ? a.rb : a.ra;
  *cols = a.swap ? a.ra : a.rb;
}

size_t gemm_workspace_bytes(const GemmArgs& a) {
  if (a.splits <= 1) return 0;
  int r, c;
  out_dims(a, &r, &c);
  return static_cast<size_t>(a.splits) * r * c * sizeof(float);
}

int gemm_num_tiles(const GemmArgs& a) { return ((a.ra + BM - 1) / BM) * ((a.rb + a.bn - 1) / a.bn); }

cudaError_t gemm_launch(const GemmArgs& a, cudaStream_t stream) {
  const bool fp4 = a.kind == kGemmNvfp4;
  const bool fp8 = a.kind == kGemmFp8;
  const bool w3 = a.kind == kGemmW3;
  if (a.ra <= 0 || a.rb <= 0 || a.k <= 0) return cudaErrorInvalidValue;
  if (fp4 ? (a.k % 32 != 0) : fp8 ? (a.k % 16 != 0) : w3 ? (a.k % 64 != 0) : (a.k % 8 != 0)) return cudaErrorInvalidValue;
  if (w3 && (!a.swap || a.peer != nullptr)) return cudaErrorInvalidValue;   // grouped (3-bit experts) is fine
  const int kt_elems = fp4 ? 256 : fp8 ? 128 : 64;
  const int k_tiles = (a.k + kt_elems - 1) / kt_elems;
  const int tiles_a = (a.ra + BM - 1) / BM;
  const int tiles_b = (a.rb + a.bn - 1) / a.bn;
  const bool grouped = a.grp_cnt != nullptr;
  if (grouped && (!a.swap || a.grp_rows_a % BM != 0 || a.grp_experts < 1 || a.grp_chunks < 1))
    return cudaErrorInvalidValue;
  if (fp4 && a.bn < 128 && tiles_b != 1 && !grouped) return cudaErrorInvalidValue;
  if (fp4 && grouped && a.bn < 128 && a.grp_chunks != 1) return cudaErrorInvalidValue;
  if (fp4 && (a.sf_k_atoms_a < k_tiles * 4 || a.sf_k_atoms_b < k_tiles * 4)) return cudaErrorInvalidValue;
  int splits = a.splits < 1 || grouped ? 1 : a.splits;
  if (splits > k_tiles) splits = k_tiles;
  // Every split must own at least one K tile.
  while (splits > 1 && (splits - 1) * ((k_tiles + splits - 1) / splits) >= k_tiles) --splits;
  if (splits > 8) splits = 8;   // portable cluster size

  // byte-typed maps (packed e2m1 or e4m3): inner extent and pitch in bytes, 128-byte boxes
  const bool bytes = fp4 || fp8;
  TmapKey ka{a.a, static_cast<uint64_t>(a.ra), static_cast<uint64_t>(fp4 ? a.k / 2 : a.k),
             static_cast<uint64_t>(fp4 ? a.lda / 2 : fp8 ? a.lda : a.lda * 2), static_cast<uint32_t>(BM),
             static_cast<uint32_t>(bytes ? 128 : 64), bytes ? 1 : 0};
  TmapKey kb{a.b, static_cast<uint64_t>(a.rb), static_cast<uint64_t>(fp4 ? a.k / 2 : a.k),
             static_cast<uint64_t>(fp4 ? a.ldb / 2 : fp8 ? a.ldb : a.ldb * 2), static_cast<uint32_t>(a.bn),
             static_cast<uint32_t>(bytes ? 128 : 64), bytes ? 1 : 0};
  CUtensorMap map_a, map_b;
  if (!get_tmap_2d(kb, &map_b)) return cudaErrorInvalidValue;
  if (w3) map_a = map_b;                                  // the w3 A operand arrives by bulk copies, not through a map
  else if (!get_tmap_2d(ka, &map_a)) return cudaErrorInvalidValue;
  const CUtensorMap *ta = &map_a, *tb = &map_b;

  DevParams p;
  p.sfa = static_cast<const uint8_t*>(a.sfa);
  p.sfb = static_cast<const uint8_t*>(a.sfb);
  p.ra = a.ra; p.rb = a.rb; p.k_tiles = k_tiles;
  p.out = a.out; p.ldo = a.ldo;
  p.residual = static_cast<const __nv_bfloat16*>(a.residual);
  p.alpha = a.alpha; p.alpha_ptr = a.alpha_ptr;
  p.epilogue = a.epilogue; p.swap = a.swap; p.splits = splits;
  p.workspace = a.workspace; p.counters = a.counters; p.status = a.status;
  p.ka_a = a.sf_k_atoms_a; p.ka_b = a.sf_k_atoms_b;
  out_dims(a, &p.out_rows, &p.out_cols);
  p.grp_start = a.grp_start; p.grp_cnt = a.grp_cnt; p.grp_rows_a = a.grp_rows_a;
  p.grp_tiles = grouped ? a.grp_tiles : nullptr; p.grp_ntiles = a.grp_ntiles;
  p.peer_on = a.peer != nullptr;
  p.flag_offset = -1;
  if (a.peer != nullptr) {
    if (a.swap || grouped || splits != 1 || a.peer->rows_per_rank % BM != 0) return cudaErrorInvalidValue;
    if (a.epilogue == kEpiScatter && (a.bn < 64 || a.rb % 8 != 0 || a.ldo % 8 != 0)) return cudaErrorInvalidValue;
    p.world = a.peer->world; p.rank = a.peer->rank; p.rows_per_rank = a.peer->rows_per_rank;
    for (int i = 0; i < 8; ++i) p.peer_base[i] = static_cast<uint8_t*>(a.peer->base[i]);
    p.stage_offset = a.peer->stage_offset; p.counter_offset = a.peer->counter_offset;
    p.flag_offset = a.peer->flag_offset; p.seq_offset = a.peer->seq_offset; p.limit_ns = a.peer->limit_ns;
  } else if (a.epilogue == kEpiScatter) {
    return cudaErrorInvalidValue;
  }
  p.tok_scale = a.tok_scale;
  p.q_out = static_cast<uint8_t*>(a.q_out); p.q_sf = static_cast<uint8_t*>(a.q_sf); p.q_gscale = a.q_gscale;
  p.q_ka = a.q_ka; p.q_ld = a.q_ld;
  p.prof = g_gemm_prof;
  p.local_reduce = g_local_reduce;
  if (a.epilogue == kEpiSiluMulQuant) {
    // tokens on the N side, whole 128-row feature tiles, no grouped / peer variants; the staging tile of a split-K
    // CTA sits behind its fp32 partial, which the smallest ring must still hold
    if (grouped || a.peer != nullptr || a.tok_scale != nullptr || a.q_out == nullptr || a.q_sf == nullptr ||
        a.q_gscale == nullptr)
      return cudaErrorInvalidValue;
    if (a.swap && (a.ra % BM != 0 || a.q_ka * 64 < a.ra / 2 || a.bn > 128)) return cudaErrorInvalidValue;
    // tokens on the 128-row side: the staged epilogue (output tiles of 128 or 256 columns, no split-K) writes the
    // packed bytes as aligned 16-byte chunks of two groups: feature count a multiple of 64
    if (!a.swap && (a.rb % 64 != 0 || a.q_ka * 64 < a.rb / 2 || a.splits != 1 || (a.bn != 128 && a.bn != 256) ||
                    a.q_ld % 16 != 0 || (reinterpret_cast<uintptr_t>(a.q_out) & 15) != 0))
      return cudaErrorInvalidValue;
  }
  p.early_launch = g_pdl >= 2;
  p.w3_tiles = w3 ? static_cast<const uint8_t*>(a.a) : nullptr;
  p.ep_gate_flags = nullptr; p.ep_seq_ptr = nullptr; p.ep_row_ret = nullptr; p.ep_done = nullptr;
  p.ep_ret_offset = 0; p.ep_ret_flag_offset = 0;
  if (a.ep != nullptr) {
    if (!grouped || a.peer != nullptr) return cudaErrorInvalidValue;
    if (a.epilogue == kEpiReturn && (a.ep->row_ret == nullptr || a.ep->done_counter == nullptr)) return cudaErrorInvalidValue;
    p.world = a.ep->world; p.rank = a.ep->rank; p.limit_ns = a.ep->limit_ns;
    for (int i = 0; i < 8; ++i) p.peer_base[i] = static_cast<uint8_t*>(a.ep->base[i]);
    p.ep_gate_flags = a.ep->gate_flags; p.ep_seq_ptr = a.ep->seq_ptr; p.ep_row_ret = a.ep->row_ret;
    p.ep_ret_offset = a.ep->ret_offset; p.ep_ret_flag_offset = a.ep->ret_flag_offset; p.ep_done = a.ep->done_counter;
  } else if (a.epilogue == kEpiReturn) {
    return cudaErrorInvalidValue;
  }
  const dim3 grid = !grouped ? dim3(tiles_a, tiles_b, splits)
                    : p.grp_tiles != nullptr ? dim3(a.grp_rows_a / BM, a.grp_tile_cap > 0 ? a.grp_tile_cap : 1, 1)
                                             : dim3(a.grp_rows_a / BM, a.grp_chunks, a.grp_experts);

#define HB_DISPATCH(KIND)                                                        \
  switch (a.bn) {                                                                \
    case 16: return launch_t<KIND, 16>(a, p, grid, ta, tb, stream);              \
    case 32: return launch_t<KIND, 32>(a, p, grid, ta, tb, stream);              \
    case 64: return launch_t<KIND, 64>(a, p, grid, ta, tb, stream);              \
    case 128: return launch_t<KIND, 128>(a, p, grid, ta, tb, stream);            \
    case 256: return launch_t<KIND, 256>(a, p, grid, ta, tb, stream);            \
    default: return cudaErrorInvalidValue;                                       \
  }
  if (fp4) {
    HB_DISPATCH(kGemmNvfp4)
  } else if (fp8) {
    HB_DISPATCH(kGemmFp8)
  } else if (w3) {
    HB_DISPATCH(kGemmW3)
  } else {
    HB_DISPATCH(kGemmBf16)
  }
#undef HB_DISPATCH
}

}  // namespace hb

#include "hb_api.h"

extern "C" {

int hb_gemm(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int ra, int rb, int k,
            long long lda, long long ldb, void* out, long long ldo, const void* residual, float alpha,
            const void* alpha_ptr, int epilogue, int swap, int splits, void* workspace, void* counters,
            void* status, int bn, int ka_a, int ka_b, void* stream) {
  hb::GemmArgs g;
  g.kind = kind; g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.ra = ra; g.rb = rb; g.k = k;
  g.lda = lda; g.ldb = ldb; g.out = out; g.ldo = ldo; g.residual = residual; g.alpha = alpha;
  g.alpha_ptr = static_cast<const float*>(alpha_ptr); g.epilogue = epilogue; g.swap = swap; g.splits = splits;
  g.workspace = static_cast<float*>(workspace); g.counters = static_cast<int*>(counters);
  g.status = static_cast<int*>(status); g.bn = bn; g.sf_k_atoms_a = ka_a; g.sf_k_atoms_b = ka_b;
  g.grp_start = nullptr; g.grp_cnt = nullptr; g.grp_rows_a = 0; g.grp_experts = 0; g.grp_chunks = 0;
  g.peer = nullptr;
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Weights on the 128-row side (a = weights [n, k], b = activations [m, k]) with the SiLU-mul + NVFP4 requant
// epilogue: writes packed e2m1 [m, n / 4 bytes] to q_out and swizzled scales to q_sf (see hb::kEpiSiluMulQuant).
int hb_gemm_silu_quant(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int n, int m, int k,
                       long long lda, long long ldb, const void* alpha_ptr, void* q_out, void* q_sf,
                       const void* q_gscale, int q_ka, int splits, void* status, int bn, int ka_a, int ka_b,
                       void* stream) {
  hb::GemmArgs g;
  g.kind = kind; g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.ra = n; g.rb = m; g.k = k;
  g.lda = lda; g.ldb = ldb; g.out = nullptr; g.ldo = 0; g.residual = nullptr; g.alpha = 1.f;
  g.alpha_ptr = static_cast<const float*>(alpha_ptr); g.epilogue = hb::kEpiSiluMulQuant; g.swap = 1; g.splits = splits;
  g.workspace = nullptr; g.counters = nullptr; g.status = static_cast<int*>(status); g.bn = bn;
  g.sf_k_atoms_a = ka_a; g.sf_k_atoms_b = ka_b;
  g.grp_start = nullptr; g.grp_cnt = nullptr; g.grp_rows_a = 0; g.grp_experts = 0; g.grp_chunks = 0;
  g.peer = nullptr;
  g.q_out = q_out; g.q_sf = q_sf; g.q_gscale = static_cast<const float*>(q_gscale); g.q_ka = q_ka; g.q_ld = n / 4;
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// The same epilogue with the tokens on the 128-row side (a = activations [m, k], b = weights [n, k]): prefill-sized
// calls. n a multiple of 64, no split-K.
int hb_gemm_silu_quant_rows(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int m, int n,
                            int k, long long lda, long long ldb, const void* alpha_ptr, void* q_out, void* q_sf,
                            const void* q_gscale, int q_ka, void* status, int bn, int ka_a, int ka_b, void* stream) {
  hb::GemmArgs g;
  g.kind = kind; g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.ra = m; g.rb = n; g.k = k;
  g.lda = lda; g.ldb = ldb; g.out = nullptr; g.ldo = 0; g.residual = nullptr; g.alpha = 1.f;
  g.alpha_ptr = static_cast<const float*>(alpha_ptr); g.epilogue = hb::kEpiSiluMulQuant; g.swap = 0; g.splits = 1;
  g.workspace = nullptr; g.counters = nullptr; g.status = static_cast<int*>(status); g.bn = bn;
  g.sf_k_atoms_a = ka_a; g.sf_k_atoms_b = ka_b;
  g.grp_start = nullptr; g.grp_cnt = nullptr; g.grp_rows_a = 0; g.grp_experts = 0; g.grp_chunks = 0;
  g.peer = nullptr;
  g.q_out = q_out; g.q_sf = q_sf; g.q_gscale = static_cast<const float*>(q_gscale); g.q_ka = q_ka; g.q_ld = n / 4;
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Peer-fused GEMM (normal orientation, M tokens on the 128-row side):
//   epilogue 4 (scatter): GEMM -> reduce-scatter, partial tiles stored into the row owner's staging area;
//   flag_offset >= 0    : all-gather -> GEMM, A row tiles wait for their source rank's arrival flag.
int hb_gemm_peer(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int m, int n, int k,
                 void* out, long long ldo, const void* alpha_ptr, int epilogue, const void* const* peer_bases,
                 int world, int rank, int rows_per_rank, long long stage_offset, long long counter_offset,
                 long long flag_offset, long long seq_offset, long long limit_ns, void* status, int ka_a, int ka_b,
                 void* stream) {
  hb::GemmArgs g;
  hb::GemmPeer peer;
  for (int i = 0; i < 8; ++i) peer.base[i] = i < world ? const_cast<void*>(peer_bases[i]) : nullptr;
  peer.world = world; peer.rank = rank; peer.rows_per_rank = rows_per_rank;
  peer.stage_offset = stage_offset; peer.counter_offset = counter_offset; peer.flag_offset = flag_offset;
  peer.seq_offset = seq_offset; peer.limit_ns = static_cast<unsigned long long>(limit_ns);
  g.kind = kind; g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.ra = m; g.rb = n; g.k = k; g.lda = k; g.ldb = k;
  g.out = out; g.ldo = ldo; g.residual = nullptr; g.alpha = 1.f; g.alpha_ptr = static_cast<const float*>(alpha_ptr);
  g.epilogue = epilogue; g.swap = 0; g.splits = 1; g.workspace = nullptr; g.counters = nullptr;
  g.status = static_cast<int*>(status); g.bn = n >= 256 ? 256 : 128; g.sf_k_atoms_a = ka_a; g.sf_k_atoms_b = ka_b;
  g.grp_start = nullptr; g.grp_cnt = nullptr; g.grp_rows_a = 0; g.grp_experts = 0; g.grp_chunks = 0;
  g.peer = &peer;
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Grouped (mixture-of-experts) GEMM, weights on the 128-row side: for expert e and its `cnt[e]` rows starting at
// `start[e]` (a multiple of 128) of the sorted activation buffer b [rows, K]:
//   out[start[e] + j, n] = sum_k b[start[e] + j, k] * a[e * n_per_expert + n, k]      (n < n_per_expert)
// `max_rows_per_expert` bounds cnt[] (it sizes the grid); alpha_ptr holds one scale per expert (may be null).
int hb_gemm_grouped(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int experts,
                    int n_per_expert, int b_rows, int k, void* out, long long ldo, const void* alpha_ptr,
                    int epilogue, const void* start, const void* cnt, int max_rows_per_expert, void* status, int ka_a,
                    int ka_b, int bn_hint, const void* tiles, const void* n_tiles, int tile_cap, void* stream) {
  hb::GemmArgs g;
  // `bn_hint` (0 = none) sizes the token tile for the EXPECTED rows per expert; the grid still covers
  // max_rows_per_expert, chunks beyond an expert's rows exit at once.
  int bn = 16;
  while (bn < max_rows_per_expert && bn < 256) bn *= 2;
  if (bn_hint >= 16 && bn_hint <= 256 && (bn_hint & (bn_hint - 1)) == 0 && bn_hint < bn) bn = bn_hint;
  g.kind = kind; g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb;
  g.ra = experts * n_per_expert; g.rb = b_rows; g.k = k; g.lda = k; g.ldb = k;
  g.out = out; g.ldo = ldo; g.residual = nullptr; g.alpha = 1.f;
  g.alpha_ptr = static_cast<const float*>(alpha_ptr); g.epilogue = epilogue; g.swap = 1; g.splits = 1;
  g.workspace = nullptr; g.counters = nullptr; g.status = static_cast<int*>(status); g.bn = bn;
  g.sf_k_atoms_a = ka_a; g.sf_k_atoms_b = ka_b;
  g.grp_start = static_cast<const int*>(start); g.grp_cnt = static_cast<const int*>(cnt);
  g.grp_rows_a = n_per_expert; g.grp_experts = experts; g.grp_chunks = (max_rows_per_expert + bn - 1) / bn;
  // the work list was built for one tile width (hb_moe_plan's `bn`); it is used only when that is the width chosen
  if (tiles != nullptr && n_tiles != nullptr && tile_cap > 0 && bn == bn_hint && g.grp_chunks <= 4096) {
    g.grp_tiles = static_cast<const int*>(tiles); g.grp_ntiles = static_cast<const int*>(n_tiles);
    g.grp_tile_cap = tile_cap;
  }
  g.peer = nullptr;
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Grouped GEMM with expert-parallel fusion: `gate_flags` (may be null) delays the activation loads until every
// sender's flag has reached *seq_ptr + 1; epilogue 5 sends every output row back to its source rank (see
// hb::GemmEp) and raises this rank's flag on every rank when the whole grid is done.
int hb_gemm_grouped_ep(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int experts,
                       int n_per_expert, int b_rows, int k, void* out, long long ldo, const void* alpha_ptr,
                       int epilogue, const void* start, const void* cnt, int max_rows_per_expert, void* status,
                       int ka_a, int ka_b, const void* const* bases, int world, int rank, const void* gate_flags,
                       const void* seq_ptr, const void* row_ret, long long ret_offset, void* done_counter,
                       long long ret_flag_offset, long long limit_ns, int bn_hint, const void* tiles,
                       const void* n_tiles, int tile_cap, void* stream) {
  hb::GemmArgs g;
  hb::GemmEp ep;
  int bn = 16;
  while (bn < max_rows_per_expert && bn < 256) bn *= 2;
  if (bn_hint >= 16 && bn_hint <= 256 && (bn_hint & (bn_hint - 1)) == 0 && bn_hint < bn) bn = bn_hint;
  for (int i = 0; i < 8; ++i) ep.base[i] = i < world ? const_cast<void*>(bases[i]) : nullptr;
  ep.world = world; ep.rank = rank;
  ep.gate_flags = static_cast<const int*>(gate_flags); ep.seq_ptr = static_cast<const int*>(seq_ptr);
  ep.row_ret = static_cast<const int*>(row_ret); ep.ret_offset = ret_offset;
  ep.done_counter = static_cast<int*>(done_counter); ep.ret_flag_offset = ret_flag_offset;
  ep.limit_ns = static_cast<unsigned long long>(limit_ns);
  g.kind = kind; g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb;
  g.ra = experts * n_per_expert; g.rb = b_rows; g.k = k; g.lda = k; g.ldb = k;
  g.out = out; g.ldo = ldo; g.residual = nullptr; g.alpha = 1.f;
  g.alpha_ptr = static_cast<const float*>(alpha_ptr); g.epilogue = epilogue; g.swap = 1; g.splits = 1;
  g.workspace = nullptr; g.counters = nullptr; g.status = static_cast<int*>(status); g.bn = bn;
  g.sf_k_atoms_a = ka_a; g.sf_k_atoms_b = ka_b;
  g.grp_start = static_cast<const int*>(start); g.grp_cnt = static_cast<const int*>(cnt);
  g.grp_rows_a = n_per_expert; g.grp_experts = experts; g.grp_chunks = (max_rows_per_expert + bn - 1) / bn;
  if (tiles != nullptr && n_tiles != nullptr && tile_cap > 0 && bn == bn_hint && g.grp_chunks <= 4096) {
    g.grp_tiles = static_cast<const int*>(tiles); g.grp_ntiles = static_cast<const int*>(n_tiles);
    g.grp_tile_cap = tile_cap;
  }
  g.peer = nullptr;
  g.ep = &ep;
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// e4m3 x e4m3 GEMM: out = alpha * (*alpha_ptr) * tok_scale[token] * A B^T. lda / ldb in elements (= bytes).
int hb_gemm_fp8(const void* a, const void* b, int ra, int rb, int k, long long lda, long long ldb, void* out,
                long long ldo, const void* residual, float alpha, const void* alpha_ptr, const void* tok_scale,
                int epilogue, int swap, int splits, void* status, int bn, void* stream) {
  hb::GemmArgs g;
  g.kind = hb::kGemmFp8; g.a = a; g.b = b; g.sfa = nullptr; g.sfb = nullptr; g.ra = ra; g.rb = rb; g.k = k;
  g.lda = lda; g.ldb = ldb; g.out = out; g.ldo = ldo; g.residual = residual; g.alpha = alpha;
  g.alpha_ptr = static_cast<const float*>(alpha_ptr); g.epilogue = epilogue; g.swap = swap; g.splits = splits;
  g.workspace = nullptr; g.counters = nullptr; g.status = static_cast<int*>(status); g.bn = bn;
  g.sf_k_atoms_a = 0; g.sf_k_atoms_b = 0;
  g.grp_start = nullptr; g.grp_cnt = nullptr; g.grp_rows_a = 0; g.grp_experts = 0; g.grp_chunks = 0;
  g.peer = nullptr;
  g.tok_scale = static_cast<const float*>(tok_scale);
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Dequant-fused 3-bit GEMM: out[m, n] = alpha * sum_k x[m, k] * w[n, k] with w given as 4096-byte tiles
// [ceil(n / 128)][k / 64] (see hibana_b200/weights/w3.py); x bf16 [m, k], m <= 256 (weights on the 128-row side).
int hb_gemm_w3(const void* tiles, const void* x, int n, int m, int k, long long ldx, void* out, long long ldo,
               const void* residual, float alpha, int epilogue, int splits, void* status, int bn, void* stream) {
  hb::GemmArgs g;
  g.kind = hb::kGemmW3; g.a = tiles; g.b = x; g.sfa = nullptr; g.sfb = nullptr; g.ra = n; g.rb = m; g.k = k;
  g.lda = k; g.ldb = ldx; g.out = out; g.ldo = ldo; g.residual = residual; g.alpha = alpha; g.alpha_ptr = nullptr;
  g.epilogue = epilogue; g.swap = 1; g.splits = splits; g.workspace = nullptr; g.counters = nullptr;
  g.status = static_cast<int*>(status); g.bn = bn; g.sf_k_atoms_a = 0; g.sf_k_atoms_b = 0;
  g.grp_start = nullptr; g.grp_cnt = nullptr; g.grp_rows_a = 0; g.grp_experts = 0; g.grp_chunks = 0;
  g.peer = nullptr;
  const cudaError_t e = hb::gemm_launch(g, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Phase timers (see prof_mark): `buf` = 8 zeroed uint64 on the device, null switches them off.
void hb_gemm_profile(void* buf) { hb::g_gemm_prof = static_cast<unsigned long long*>(buf); }

// Unsplit tiles with the weights on the 128-row side: 1 = epilogue through the parked [column][row] partial (wide
// stores, thread-local gate / up pairs), 0 = straight from the accumulator (one thread per row).
void hb_gemm_set_local_reduce(int on) { hb::g_local_reduce = on != 0; }

void hb_clear_tmap_cache(void) { hb::clear_tmap_cache(); }

void hb_gemm_set_pdl(int on) { hb::g_pdl = on < 0 ? 0 : on > 2 ? 2 : on; }
int hb_gemm_get_pdl(void) { return hb::g_pdl; }

}  // extern "C"
