// Host-visible interface of the tcgen05 GEMM family (no torch headers here: plain C++ launchers).
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace hb {

enum GemmKind : int {
  kGemmBf16 = 0,
  kGemmNvfp4 = 1,
  kGemmFp8 = 2,   // e4m3 x e4m3, 128-element K tiles
  kGemmW3 = 3,    // A = 3-bit asymmetric codes (groups of 64, bf16 scale + zero) in 4096-byte tiles, dequantised to
                  // bf16 in shared memory by the CTA; B = bf16 activations; weights on the 128-row side only
};
enum GemmEpilogue : int {
  kEpiStore = 0,      // out = alpha * acc                      (bf16)
  kEpiResidual = 1,   // out = alpha * acc + residual           (bf16)
  kEpiSiluMul = 2,    // out[.., j] = silu(acc[2j]) * acc[2j+1] (bf16, gate/up rows interleaved pairwise)
  kEpiStoreF32 = 3,   // out = alpha * acc                      (fp32)
  kEpiScatter = 4,    // row-parallel GEMM -> reduce-scatter: the bf16 partial tile is stored straight into the
                      // staging area of the rank that owns its rows (peer memory), then that rank's arrival
                      // counter for this source is bumped (normal orientation only)
  kEpiReturn = 5,     // expert-parallel fc2 (grouped, weights on the 128-row side): column j of the output (one
                      // routed row) is stored into the return buffer of the rank the row came from, at the row
                      // that rank asked for; when every CTA is done the kernel raises a flag on every rank
  kEpiRelu2 = 6,      // out = max(alpha * acc, 0)^2            (bf16; weights on the 128-row side only)
  kEpiSiluMulQuant = 7,  // SiLU-mul as in kEpiSiluMul, then requantised to NVFP4 in the same epilogue: packed e2m1
                         // rows go to q_out, ue4m3 scales to q_sf (128x4-swizzled blocks) with the static per-tensor
                         // scale *q_gscale of the consuming projection. Weights on the 128-row side only; the next
                         // GEMM reads the result as its activation operand with no kernel in between.
};

// Peer-memory fusion arguments (all ranks pass the same offsets; pointers are this process's mappings).
struct GemmPeer {
  void* base[8];            // heap base of every rank
  int world, rank;
  int rows_per_rank;        // owner of output row m is m / rows_per_rank (multiple of 128)
  long long stage_offset;   // scatter: byte offset of staging [world][rows_per_rank][ldo] bf16 in every heap
  long long counter_offset; // scatter: byte offset of int counters[world] (arrivals per source) in every heap
  // gather gating (all-gather -> GEMM): A row tiles of source rank s may be loaded once flags[s] >= *seq_ptr
  long long flag_offset;    // byte offset of int flags[world] in this rank's heap (-1 = no gating)
  long long seq_offset;     // byte offset of the int holding the expected sequence number
  unsigned long long limit_ns;
};

// Expert-parallel fusion of the grouped GEMM (all-to-all dispatch -> fc1, fc2 -> return).
struct GemmEp {
  void* base[8];              // heap base of every rank
  int world, rank;
  const int* gate_flags;      // this rank's int flags[world]: activations may be read once every flag has reached
                              // *seq_ptr + 1 (the senders' rows have landed); null = no gating
  const int* seq_ptr;         // this rank's count of completed expert-parallel calls
  const int* row_ret;         // kEpiReturn: per sorted row (source rank << 24) | row in that rank's return buffer
  long long ret_offset;       // kEpiReturn: byte offset of the return buffer [rows, ldo] bf16 in every heap
  int* done_counter;          // kEpiReturn: this rank's int, zero between launches
  long long ret_flag_offset;  // kEpiReturn: byte offset of int flags[world] in every heap
  unsigned long long limit_ns;
};

// D[ra, rb] = sum_k A[ra, k] * B[rb, k]; both operands K-major. `swap` tells the epilogue that A rows are
// output *columns* (weights on the 128-row side, tokens on the N side): out[rb * ldo + ra].
struct GemmArgs {
  int kind;
  const void* a;        // [RA, K]  (bf16, or packed e2m1 with K/2 bytes per row)
  const void* b;        // [RB, K]
  const void* sfa;      // nvfp4 only: scale factors of A, 128x4-swizzled blocks [ceil(RA/128)][KA][512 B]
  const void* sfb;      // nvfp4 only: scale factors of B
  int ra, rb, k;
  int64_t lda, ldb;     // row pitch in elements
  void* out;
  int64_t ldo;
  const void* residual; // bf16, same indexing as out (may be null)
  float alpha;
  const float* alpha_ptr;  // optional device scalar multiplied into alpha (dynamic activation scale)
  int epilogue;
  int swap;
  int splits;           // split-K factor (>= 1)
  float* workspace;     // splits > 1: fp32 [splits][out rows][out cols]
  int* counters;        // splits > 1: one int per output tile, zero before the first launch, self-resetting
  int* status;          // device status word (may be null)
  int bn;               // N tile: 16, 32, 64, 128 or 256
  int sf_k_atoms_a;     // nvfp4: number of 64-element K atoms per row block in sfa (padded to a multiple of 4)
  int sf_k_atoms_b;
  // grouped mode (null grp_cnt = off); see hb_gemm_grouped
  const int* grp_start;
  const int* grp_cnt;
  int grp_rows_a, grp_experts, grp_chunks;
  // optional compact work list (see hb_moe_plan): grp_tiles[i] = expert * 4096 + chunk for i < *grp_ntiles; the grid
  // then has grp_tile_cap entries instead of experts * chunks, most of which would find nothing to do
  const int* grp_tiles = nullptr;
  const int* grp_ntiles = nullptr;
  int grp_tile_cap = 0;
  const GemmPeer* peer;     // null = no peer fusion
  const GemmEp* ep = nullptr;   // null = no expert-parallel fusion (grouped mode only)
  // kEpiSiluMulQuant outputs: q_out [tokens, q_ld bytes] packed e2m1, q_sf swizzled scales with q_ka K atoms per
  // row block, q_gscale the device scalar x ~= q * sf * gscale. Scale bytes of padding rows / groups are not written.
  void* q_out = nullptr;
  void* q_sf = nullptr;
  const float* q_gscale = nullptr;
  int q_ka = 0;
  long long q_ld = 0;
  const float* tok_scale = nullptr;   // optional per-token factor (dynamic per-row activation scale): indexed by
                                      // the token, i.e. the B row with `swap`, else the A row
};

// Returns cudaSuccess or the launch error. Tensor maps are built (and cached) inside.
cudaError_t gemm_launch(const GemmArgs& args, cudaStream_t stream);

// Bytes of fp32 workspace and number of counters a launch with these arguments needs.
size_t gemm_workspace_bytes(const GemmArgs& args);
int gemm_num_tiles(const GemmArgs& args);

// Tensor-map cache (host). 2-D row-major tensor, box = {box_inner elements, box_rows}, 128-byte swizzle.
struct TmapKey {
  const void* ptr;
  uint64_t rows, cols;   // cols = inner extent in elements
  uint64_t pitch_bytes;
  uint32_t box_rows, box_cols;
  int dtype;             // 0 = bf16, 1 = u8
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && pitch_bytes == o.pitch_bytes &&
           box_rows == o.box_rows && box_cols == o.box_cols && dtype == o.dtype;
  }
};
bool get_tmap_2d(const TmapKey& key, CUtensorMap* out_map);   // copies the cached map (never hand out cache pointers)
void clear_tmap_cache();

}  // namespace hb
