// Recurrent state (Mamba-2, and the gated delta rule in mode 1) as a quantised window record: an int8 boundary
// state plus the tokens committed since.
//
//   S_t = G(1..t) * dequant(Z) + sum_j G(j+1..t) * u_j (x) B_j          G(a..b) = exp(sum of the rows' dt * A)
//
// Per (layer, slot, head): Z int8 [P, N] with one fp32 scale per value row; per head a log of up to `cap` records
// u_j = dt_j * x_j [P] (fp16) and c_j = running sum of dt * A since the boundary (fp32); per group the records' B_j [N]
// (fp16) and the record count. A decode / verify / replay step never rewrites the boundary state: it reads Z once
// (a quarter of the fp32 state's bytes, no write-back), forms y_t = C_t . S_t through the expansion above, and a
// committing call appends its rows' records. A committing call that finds `window` or more records first folds them
// into a new boundary state and quantises once, so quantisation error enters once per window of committed tokens
// instead of once per token (the plain int8 format requantises every step). A verify call (commit = 0) writes
// nothing at all: the accepted rows are replayed later by a committing call, which needs no scratch slot.
// One CTA per (sequence, group): thread (head of the group, value row p); the records of a call's earlier rows live
// in shared memory, so later rows of the same call see them whether or not the call commits.
// `mamba2_window_io_kernel` converts between the record and a plain fp32 state (prefill chunks run the fp32 kernels
// on a temporary state and fold the result back).
// Reference: hibana/cache/ssm_format.py:1-60 (the record), hibana/kernels/ssm_window.py:182-391 (verify / commit /
// materialise); this build keeps the record without the smoothing factors and low-rank compensators.
#include "hb_common.cuh"

namespace hb {
namespace {

constexpr int kWinExtra = 16;        // records a call may append beyond `window` before the next call folds
constexpr int kWinMaxRows = 16;      // rows of one sequence in one call (decode 1, verify / replay k + 1)
constexpr int kWinMaxCap = 64 + kWinExtra;

struct WinParams {
  const __nv_bfloat16 *x, *bmat, *cmat, *dt;      // [T, H*P], [T, G*N], [T, G*N], [T, H] (row strides below)
  long long ldx, ldb, lddt;
  const float *a_log, *dt_bias, *dskip;           // [H] each (dt_bias / dskip nullable)
  __nv_bfloat16* y;
  long long ldy;
  int8_t* z;            // [slots, H, P, N]
  float* zscale;        // [slots, H, P]
  __half* win_b;        // [slots, G, cap, N]
  __half* win_u;        // [slots, H, cap, P]
  float* win_c;         // [slots, H, cap]
  int* win_len;         // [slots, G]
  const int *q_indptr, *slot_in, *has_init;       // q_indptr / has_init nullable
  int batch, heads, groups, p, n, window, cap, commit;
  int* status;
  // mode 1, gated delta rule: x = v [T, H*P], bmat = k, cmat = q [T, G*N]; log decay and beta fp32 [T, H]
  int mode, l2norm;
  float scale;
  const float *g_log, *beta;
};

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(__expf(v)); }

// dot of a shared-memory fp16 record row with the shared fp32 C row, by one warp
__device__ __forceinline__ float warp_dot(const __half* b, const float* c, int n, int lane) {
  float s = 0.f;
  for (int i = lane; i < n; i += 32) s += __half2float(b[i]) * c[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  return s;
}

__global__ void __launch_bounds__(1024) mamba2_window_kernel(const WinParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int hg = p.heads / p.groups;                       // heads per group
  const int P = p.p, N = p.n, cap = p.cap;
  const int rec_cap = cap + kWinMaxRows;                   // stored records + this call's rows
  __half* sB = reinterpret_cast<__half*>(smem_raw);                              // [rec_cap][N]
  float* sC = reinterpret_cast<float*>(sB + static_cast<size_t>(rec_cap) * N);   // [N]   the row's C
  float* sCum = sC + N;                                                          // [hg][rec_cap] c_j per head
  float* sW = sCum + hg * rec_cap;                                               // [hg][rec_cap] weight of record j
  float* sDot = sW + hg * rec_cap;                                               // [rec_cap] B_j . C
  float* sK = sDot + rec_cap;                                                    // [N]   delta rule: the row's k
  float* sDotK = sK + N;                                                         // [rec_cap] k_j . k_t
  float* sWk = sDotK + rec_cap;                                                  // [hg][rec_cap]
  float* sNorm = sWk + hg * rec_cap;                                             // [2]
  __half* sU = reinterpret_cast<__half*>(sNorm + 2);                             // [kWinMaxRows][threads]: this call's u
  const int b = blockIdx.x, g = blockIdx.y;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int hl = tid / P, pv = tid % P;                    // head within the group, value row
  const int h = g * hg + hl;
  const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
  const int slot = p.slot_in[b];
  if (!index_ok(slot, kBoundStateSlots, kKerMambaScan)) return;
  const int r0 = p.q_indptr ? p.q_indptr[b] : b;
  const int r1 = p.q_indptr ? p.q_indptr[b + 1] : b + 1;
  const int rows = min(r1 - r0, kWinMaxRows);
  if (r1 - r0 > kWinMaxRows) set_status(p.status, kBadShape);
  const bool fresh = p.has_init != nullptr && p.has_init[b] == 0;

  int8_t* zrow = p.z + ((static_cast<size_t>(slot) * p.heads + h) * P + pv) * N;
  float* zs_ptr = p.zscale + (static_cast<size_t>(slot) * p.heads + h) * P + pv;
  __half* gB = p.win_b + (static_cast<size_t>(slot) * p.groups + g) * cap * N;
  __half* gU = p.win_u + (static_cast<size_t>(slot) * p.heads + h) * cap * P;
  float* gC = p.win_c + (static_cast<size_t>(slot) * p.heads + h) * cap;
  int* glen = p.win_len + static_cast<size_t>(slot) * p.groups + g;

  int len = fresh ? 0 : min(*glen, cap);
  float zs = fresh ? 0.f : *zs_ptr;
  // ---- stored records into shared memory (B rows, running sums) and registers (this thread's u values)
  for (int i = tid; i < len * N; i += nthreads) sB[i] = gB[i];
  if (pv < len) sCum[hl * rec_cap + pv] = gC[pv];
  for (int j = pv + P; j < len; j += P) sCum[hl * rec_cap + j] = gC[j];
  __syncthreads();
  int stored = len;          // records [0, stored) live in global memory, [stored, len) are this call's (shared memory)
  auto u_of = [&](int j) -> float {
    return __half2float(j < stored ? gU[static_cast<size_t>(j) * P + pv] : sU[(j - stored) * nthreads + tid]);
  };

  // ---- a committing call that finds a full window folds it into a new boundary state first
  if (p.commit && (len >= p.window || fresh)) {
    const float clast = len > 0 ? sCum[hl * rec_cap + len - 1] : 0.f;
    const float gain = __expf(clast) * zs;
    float amax = 0.f;
    for (int pass = 0; pass < 2; ++pass) {
      const float inv = pass == 1 ? (amax > 0.f ? 127.f / amax : 0.f) : 0.f;
      for (int n0 = 0; n0 < N; n0 += 16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(zrow + n0);
        const int8_t* zq = reinterpret_cast<const int8_t*>(&raw);
        float sv[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) sv[e] = gain * static_cast<float>(zq[e]);
        for (int j = 0; j < len; ++j) {
          const float wj = __expf(clast - sCum[hl * rec_cap + j]) * u_of(j);
          const __half* bj = sB + static_cast<size_t>(j) * N + n0;
#pragma unroll
          for (int e = 0; e < 16; ++e) sv[e] += wj * __half2float(bj[e]);
        }
        if (pass == 0) {
#pragma unroll
          for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(sv[e]));
        } else {
          uint32_t packed[4] = {0u, 0u, 0u, 0u};
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int q = max(-127, min(127, __float2int_rn(sv[e] * inv)));
            packed[e >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(q))) << (8 * (e & 3));
          }
          *reinterpret_cast<uint4*>(zrow + n0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
    zs = amax / 127.f;
    *zs_ptr = zs;
    len = 0;
    stored = 0;
    __syncthreads();          // every thread is done with the old records before new ones overwrite them
  } else if (len >= cap) {
    set_status(p.status, kOverflow);       // a read-only call found a record it cannot extend: nothing to do but report
  }

  // ---- the call's rows
  float cum = len > 0 ? sCum[hl * rec_cap + len - 1] : 0.f;
  const float a_h = p.mode == 0 ? -__expf(p.a_log[h]) : 0.f;
  const float d_h = (p.mode == 0 && p.dskip) ? p.dskip[h] : 0.f;
  for (int r = 0; r < rows; ++r) {
    const long long row = r0 + r;
    float xv, u_val = 0.f;
    if (p.mode == 0) {
      // this row's C and B (B becomes record `len`), the head's step size
      for (int i = tid; i < N; i += nthreads) {
        sC[i] = __bfloat162float(p.cmat[row * p.ldb + g * N + i]);
        sB[static_cast<size_t>(len) * N + i] = __float2half(__bfloat162float(p.bmat[row * p.ldb + g * N + i]));
      }
      const float dtv = softplus_f(__bfloat162float(p.dt[row * p.lddt + h]) + (p.dt_bias ? p.dt_bias[h] : 0.f));
      xv = __bfloat162float(p.x[row * p.ldx + h * P + pv]);
      cum += dtv * a_h;
      u_val = __half2float(__float2half(dtv * xv));
      sU[(len - stored) * nthreads + tid] = __float2half(u_val);
    } else {
      // delta rule: q (scaled) and k of this key head, both L2-normalised; k (rounded to fp16) becomes record `len`
      for (int i = tid; i < N; i += nthreads) {
        sC[i] = __bfloat162float(p.cmat[row * p.ldb + g * N + i]);
        sK[i] = __bfloat162float(p.bmat[row * p.ldb + g * N + i]);
      }
      __syncthreads();
      if (warp < 2) {
        const float* src = warp == 0 ? sC : sK;
        float ss = 0.f;
        for (int i = lane; i < N; i += 32) ss += src[i] * src[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) sNorm[warp] = p.l2norm ? rsqrtf(ss + 1e-6f) : 1.f;
      }
      __syncthreads();
      const float nq = sNorm[0] * p.scale, nk = sNorm[1];
      __syncthreads();
      for (int i = tid; i < N; i += nthreads) {
        sC[i] *= nq;
        const __half kh = __float2half(sK[i] * nk);
        sK[i] = __half2float(kh);
        sB[static_cast<size_t>(len) * N + i] = kh;
      }
      xv = __bfloat162float(p.x[row * p.ldx + h * P + pv]);
      cum += p.g_log[row * p.heads + h];
    }
    if (pv == 0) sCum[hl * rec_cap + len] = cum;
    __syncthreads();
    for (int j = warp; j <= len; j += nwarps) {
      const float d = warp_dot(sB + static_cast<size_t>(j) * N, sC, N, lane);
      if (lane == 0) sDot[j] = d;
      if (p.mode == 1 && j < len) {
        const float dk = warp_dot(sB + static_cast<size_t>(j) * N, sK, N, lane);
        if (lane == 0) sDotK[j] = dk;
      }
    }
    __syncthreads();
    for (int i = tid; i < hg * (len + 1); i += nthreads) {
      const int hh = i / (len + 1), j = i % (len + 1);
      const float decay = __expf(sCum[hh * rec_cap + len] - sCum[hh * rec_cap + j]);
      sW[hh * rec_cap + j] = decay * sDot[j];
      if (p.mode == 1 && j < len) sWk[hh * rec_cap + j] = decay * sDotK[j];
    }
    // boundary term: this thread's int8 row against C (and against k for the delta rule)
    float acc = 0.f, acck = 0.f;
    if (zs != 0.f) {
      for (int n0 = 0; n0 < N; n0 += 16) {
        const uint4 raw = *reinterpret_cast<const uint4*>(zrow + n0);
        const int8_t* zq = reinterpret_cast<const int8_t*>(&raw);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float zf = static_cast<float>(zq[e]);
          acc += zf * sC[n0 + e];
          if (p.mode == 1) acck += zf * sK[n0 + e];
        }
      }
      const float gain = zs * __expf(cum);
      acc *= gain;
      acck *= gain;
    }
    __syncthreads();
    if (p.mode == 1) {
      for (int j = 0; j < len; ++j) acck += sWk[hl * rec_cap + j] * u_of(j);
      u_val = __half2float(__float2half(p.beta[row * p.heads + h] * (xv - acck)));
      sU[(len - stored) * nthreads + tid] = __float2half(u_val);
      for (int j = 0; j < len; ++j) acc += sW[hl * rec_cap + j] * u_of(j);
      acc += sW[hl * rec_cap + len] * u_val;
    } else {
      for (int j = 0; j <= len; ++j) acc += sW[hl * rec_cap + j] * u_of(j);
      acc += d_h * xv;
    }
    p.y[row * p.ldy + h * P + pv] = __float2bfloat16(acc);
    if (p.commit) {
      gU[static_cast<size_t>(len) * P + pv] = __float2half(u_val);
      if (pv == 0) gC[len] = cum;
      if (hl == 0)
        for (int i = pv; i < N; i += P) gB[static_cast<size_t>(len) * N + i] = sB[static_cast<size_t>(len) * N + i];
    }
    ++len;
    __syncthreads();
  }
  if (p.commit && tid == 0) *glen = len;
}

struct WinIoParams {
  float* dense;         // [batch, H, P, N] fp32
  int8_t* z;
  float* zscale;
  __half *win_b, *win_u;
  float* win_c;
  int* win_len;
  const int* slots;
  int batch, heads, groups, p, n, cap, to_dense;
};

// to_dense = 1: dense[b] = the state the record of slot slots[b] stands for. to_dense = 0: the record becomes a
// fresh boundary state quantised from dense[b] (no records).
__global__ void __launch_bounds__(256) mamba2_window_io_kernel(const WinIoParams p) {
  const int b = blockIdx.x, h = blockIdx.y;
  const int P = p.p, N = p.n, cap = p.cap;
  const int hg = p.heads / p.groups, g = h / hg;
  const int slot = p.slots[b];
  if (!index_ok(slot, kBoundStateSlots, kKerMambaScan)) return;
  float* dense = p.dense + (static_cast<size_t>(b) * p.heads + h) * P * N;
  int8_t* z = p.z + (static_cast<size_t>(slot) * p.heads + h) * P * N;
  float* zsc = p.zscale + (static_cast<size_t>(slot) * p.heads + h) * P;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (p.to_dense) {
    const __half* gB = p.win_b + (static_cast<size_t>(slot) * p.groups + g) * cap * N;
    const __half* gU = p.win_u + (static_cast<size_t>(slot) * p.heads + h) * cap * P;
    const float* gC = p.win_c + (static_cast<size_t>(slot) * p.heads + h) * cap;
    const int len = min(p.win_len[static_cast<size_t>(slot) * p.groups + g], cap);
    const float clast = len > 0 ? gC[len - 1] : 0.f;
    for (int pv = warp; pv < P; pv += nwarps) {
      const float gain = __expf(clast) * zsc[pv];
      for (int n = lane; n < N; n += 32) {
        float s = gain * static_cast<float>(z[pv * N + n]);
        for (int j = 0; j < len; ++j)
          s += __expf(clast - gC[j]) * __half2float(gU[static_cast<size_t>(j) * P + pv]) *
               __half2float(gB[static_cast<size_t>(j) * N + n]);
        dense[pv * N + n] = s;
      }
    }
    return;
  }
  for (int pv = warp; pv < P; pv += nwarps) {
    float amax = 0.f;
    for (int n = lane; n < N; n += 32) amax = fmaxf(amax, fabsf(dense[pv * N + n]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    for (int n = lane; n < N; n += 32)
      z[pv * N + n] = static_cast<int8_t>(max(-127, min(127, __float2int_rn(dense[pv * N + n] * inv))));
    if (lane == 0) zsc[pv] = amax / 127.f;
  }
  if (threadIdx.x == 0 && h % hg == 0) p.win_len[static_cast<size_t>(slot) * p.groups + g] = 0;
}

}  // namespace
}  // namespace hb

extern "C" {

int hb_mamba2_window_extra(void) { return hb::kWinExtra; }

// The NEXT hb_mamba2_window call of this thread runs the gated delta rule over the same record format: x = v rows,
// bmat = k rows, cmat = q rows (heads = value heads, groups = key heads, head_dim = V, d_state = K), with the rows'
// log decay and beta (fp32 [T, heads]).
struct WinDelta {
  bool on = false;
  int l2norm = 1;
  float scale = 1.f;
  const float *g_log = nullptr, *beta = nullptr;
};
static thread_local WinDelta g_win_delta;
void hb_window_delta_rule(const void* g_log, const void* beta, float scale, int l2norm) {
  g_win_delta.on = true; g_win_delta.g_log = static_cast<const float*>(g_log);
  g_win_delta.beta = static_cast<const float*>(beta); g_win_delta.scale = scale; g_win_delta.l2norm = l2norm;
}

// One decode / verify / replay call over the window records (`commit` = 0: read only). State tensors are the layer's
// [slots, ...] views with the strides of contiguous tensors.
int hb_mamba2_window(const void* x, const void* bmat, const void* cmat, const void* dt, long long ldx, long long ldb,
                     long long lddt, const void* a_log, const void* dt_bias, const void* dskip, void* y, long long ldy,
                     void* z, void* zscale, void* win_b, void* win_u, void* win_c, void* win_len, const void* q_indptr,
                     const void* slot_in, const void* has_init, int batch, int heads, int groups, int head_dim,
                     int d_state, int window, int cap, int commit, void* status, void* stream) {
  using namespace hb;
  if (batch <= 0) return 0;
  const int hg = groups > 0 ? heads / groups : 0;
  if (groups <= 0 || heads % groups || hg * head_dim > 1024 || (hg * head_dim) % 32 || d_state % 16 ||
      cap != window + kWinExtra || cap > kWinMaxCap)
    return 1;
  WinParams p;
  p.x = static_cast<const __nv_bfloat16*>(x); p.bmat = static_cast<const __nv_bfloat16*>(bmat);
  p.cmat = static_cast<const __nv_bfloat16*>(cmat); p.dt = static_cast<const __nv_bfloat16*>(dt);
  p.ldx = ldx; p.ldb = ldb; p.lddt = lddt;
  p.a_log = static_cast<const float*>(a_log); p.dt_bias = static_cast<const float*>(dt_bias);
  p.dskip = static_cast<const float*>(dskip);
  p.y = static_cast<__nv_bfloat16*>(y); p.ldy = ldy;
  p.z = static_cast<int8_t*>(z); p.zscale = static_cast<float*>(zscale);
  p.win_b = static_cast<__half*>(win_b); p.win_u = static_cast<__half*>(win_u);
  p.win_c = static_cast<float*>(win_c); p.win_len = static_cast<int*>(win_len);
  p.q_indptr = static_cast<const int*>(q_indptr); p.slot_in = static_cast<const int*>(slot_in);
  p.has_init = static_cast<const int*>(has_init);
  p.batch = batch; p.heads = heads; p.groups = groups; p.p = head_dim; p.n = d_state; p.window = window; p.cap = cap;
  p.commit = commit; p.status = static_cast<int*>(status);
  p.mode = g_win_delta.on ? 1 : 0; p.l2norm = g_win_delta.l2norm; p.scale = g_win_delta.scale;
  p.g_log = g_win_delta.g_log; p.beta = g_win_delta.beta;
  g_win_delta = WinDelta{};
  const int rec_cap = cap + kWinMaxRows;
  const size_t smem = static_cast<size_t>(rec_cap) * d_state * 2 +
                      (2 * d_state + 3 * hg * rec_cap + 2 * rec_cap + 2) * 4 +
                      static_cast<size_t>(kWinMaxRows) * hg * head_dim * 2;
  static size_t attr = 0;
  if (smem > 48 * 1024 && smem > attr) {
    if (cudaFuncSetAttribute(mamba2_window_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return 3;
    attr = smem;
  }
  mamba2_window_kernel<<<dim3(batch, groups), hg * head_dim, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int hb_mamba2_window_io(void* dense, void* z, void* zscale, void* win_b, void* win_u, void* win_c, void* win_len,
                        const void* slots, int batch, int heads, int groups, int head_dim, int d_state, int cap,
                        int to_dense, void* stream) {
  using namespace hb;
  if (batch <= 0) return 0;
  if (groups <= 0 || heads % groups) return 1;
  WinIoParams p;
  p.dense = static_cast<float*>(dense); p.z = static_cast<int8_t*>(z); p.zscale = static_cast<float*>(zscale);
  p.win_b = static_cast<__half*>(win_b); p.win_u = static_cast<__half*>(win_u);
  p.win_c = static_cast<float*>(win_c); p.win_len = static_cast<int*>(win_len);
  p.slots = static_cast<const int*>(slots);
  p.batch = batch; p.heads = heads; p.groups = groups; p.p = head_dim; p.n = d_state; p.cap = cap; p.to_dense = to_dense;
  mamba2_window_io_kernel<<<dim3(batch, heads), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
