// C ABI of the hibana_b200 native library (loaded from Python with ctypes; callable from any C program).
// Every function returns 0 on success. Pointers are device pointers unless stated; `stream` is a cudaStream_t.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- GEMM (gemm.cu) ------------------------------------------------------------------------------------
// kind: 0 bf16, 1 nvfp4. D[ra, rb] = A[ra, K] . B[rb, K]^T; swap != 0 stores D transposed (out[rb][ra]).
// epilogue: 0 store bf16, 1 + residual, 2 silu(gate)*up on pairwise-interleaved rows/cols, 3 store fp32.
int hb_gemm(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int ra, int rb, int k,
            long long lda, long long ldb, void* out, long long ldo, const void* residual, float alpha,
            const void* alpha_ptr, int epilogue, int swap, int splits, void* workspace, void* counters,
            void* status, int bn, int ka_a, int ka_b, void* stream);
// Decode-shaped gate/up projection (a = weights [n, k] with gate / up rows interleaved, b = activations [m, k]):
// SiLU-mul and NVFP4 requantisation in the epilogue; q_out [m, n / 4] packed e2m1, q_sf swizzled ue4m3 scales.
int hb_gemm_silu_quant(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int n, int m, int k,
                       long long lda, long long ldb, const void* alpha_ptr, void* q_out, void* q_sf,
                       const void* q_gscale, int q_ka, int splits, void* status, int bn, int ka_a, int ka_b,
                       void* stream);
// The same epilogue for prefill-sized calls: a = activations [m, k] on the 128-row side, b = weights [n, k];
// n a multiple of 32, no split-K.
int hb_gemm_silu_quant_rows(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int m, int n,
                            int k, long long lda, long long ldb, const void* alpha_ptr, void* q_out, void* q_sf,
                            const void* q_gscale, int q_ka, void* status, int bn, int ka_a, int ka_b, void* stream);
int hb_gemm_grouped(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int experts,
                    int n_per_expert, int b_rows, int k, void* out, long long ldo, const void* alpha_ptr,
                    int epilogue, const void* start, const void* cnt, int max_rows_per_expert, void* status, int ka_a,
                    int ka_b, int bn_hint, const void* tiles, const void* n_tiles, int tile_cap, void* stream);
int hb_gemm_peer(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int m, int n, int k,
                 void* out, long long ldo, const void* alpha_ptr, int epilogue, const void* const* peer_bases,
                 int world, int rank, int rows_per_rank, long long stage_offset, long long counter_offset,
                 long long flag_offset, long long seq_offset, long long limit_ns, void* status, int ka_a, int ka_b,
                 void* stream);
int hb_gemm_grouped_ep(int kind, const void* a, const void* b, const void* sfa, const void* sfb, int experts,
                       int n_per_expert, int b_rows, int k, void* out, long long ldo, const void* alpha_ptr,
                       int epilogue, const void* start, const void* cnt, int max_rows_per_expert, void* status,
                       int ka_a, int ka_b, const void* const* bases, int world, int rank, const void* gate_flags,
                       const void* seq_ptr, const void* row_ret, long long ret_offset, void* done_counter,
                       long long ret_flag_offset, long long limit_ns, int bn_hint, const void* tiles, const void* n_tiles,
                       int tile_cap, void* stream);
// Expert-parallel all-to-all (csrc/ep.cu); heaps come from hb_comm_alloc / hb_comm_ipc_open.
int hb_ep_ctrl_bytes(void);
void hb_ep_ctrl_layout(long long* out4);
int hb_ep_count(const void* ids, int pairs, int experts, const void* const* bases, int world, int rank,
                long long cnt_mat_off, void* stream);
int hb_ep_plan(const void* ids, int pairs, int experts, const void* const* bases, int world, int rank,
               long long cnt_mat_off, int rows_cap, void* grp_cnt, void* grp_start, void* total_rows, void* dst_rank,
               void* dst_row, long long limit_ns, void* status, void* stream);
int hb_ep_dispatch(const void* x, long long ldx, int tokens, int topk, int h, int ka, const void* dst_rank,
                   const void* dst_row, const void* gscale, const void* const* bases, int world, int rank,
                   long long q_off, long long sf_off, long long bf_off, long long row_ret_off, void* stream);
int hb_ep_combine(const void* weights, const void* dst_rank, const void* shared, long long ld_shared, void* out,
                  long long ldo, int tokens, int topk, int h, const void* const* bases, int world, int rank,
                  long long ret_off, long long limit_ns, void* status, void* stream);
int hb_kv_copy(void* pool, void* payload, const void* slots, int tokens, int layers, int kv_heads,
               long long slots_dim, int d, int esize, int to_pool, void* stream);
int hb_gemm_fp8(const void* a, const void* b, int ra, int rb, int k, long long lda, long long ldb, void* out,
                long long ldo, const void* residual, float alpha, const void* alpha_ptr, const void* tok_scale,
                int epilogue, int swap, int splits, void* status, int bn, void* stream);
int hb_gemm_w3(const void* tiles, const void* x, int n, int m, int k, long long ldx, void* out, long long ldo,
               const void* residual, float alpha, int epilogue, int splits, void* status, int bn, void* stream);
// Host row gather over sharded table files (csrc/row_gather.cpp).
void* hb_rows_open(int row_bytes, long long rows_per_shard, int threads);
int hb_rows_add_shard(void* g, const char* path);
long long hb_rows_gather(void* g, const long long* rows, long long n, void* dst, long long* cold);
void hb_rows_close(void* g);
// Hyper-connection steps (csrc/hyper.cu).
int hb_hc_norm(const void* hyper, const void* w, void* normed, int tokens, int hc, int h, float eps, void* stream);
int hb_hc_gate_mean(const void* gate, const void* normed, void* mixed, int tokens, int hc, int h, void* stream);
int hb_hc_inject(const void* hyper, const void* block_out, const void* inject_logits, long long ld_logits, void* out,
                 int tokens, int hc, int h, void* stream);
int hb_hc_low(const void* x, long long ldx, void* low, int rows, int rank, void* stream);
// Sparse-attention indexer (csrc/qsa.cu).
int hb_qsa_compress(const void* raw_k, void* ckey, const void* kv_indices, long long ld_idx, const void* seq_rows,
                    const void* grp_indptr, const void* grp_first, int batch, int total_groups, int ratio,
                    const void* norm_w, float eps, const void* inv_freq, int rot, void* stream);
int hb_qsa_score(const void* q, int rows, int heads, const void* ckey, const void* kv_indices, long long ld_idx,
                 const void* row_seq, const void* row_pos, int ratio, int max_groups, void* scores, void* stream);
int hb_qsa_expand(const void* chosen, const void* chosen_scores, int rows, int width, const void* kv_indices,
                  long long ld_idx, const void* row_seq, const void* row_pos, int ratio, void* sel, long long ld_sel,
                  void* sel_len, void* stream);
void hb_clear_tmap_cache(void);
// GEMM launches use programmatic dependent launch (weight prefetch overlaps the preceding kernel) when on.
void hb_gemm_set_pdl(int on);
int hb_gemm_get_pdl(void);

// ---- quantisers (quant.cu) -----------------------------------------------------------------------------
int hb_quant_nvfp4(const void* x, long long ldx, int m, int k, int ka, const void* gscale, void* q, void* sf,
                   int mode, void* stream);
int hb_quant_nvfp4_rows(const void* x, long long ldx, int m, int k, int ka, const void* gscale, void* q, void* sf,
                        int mode, const void* src_rows, const void* total_rows, void* stream);
int hb_norm_quant_nvfp4(const void* x, void* residual, const void* w, float eps, int gemma, int m, int k, int ka,
                        const void* gscale, void* q, void* sf, void* normed, void* stream);
int hb_quant_fp8_static(const void* x, long long n, const void* scale, void* q, void* stream);
int hb_quant_fp8_rows(const void* x, int m, int k, void* q, void* scales, void* stream);

// ---- pointwise / row kernels (misc.cu) -----------------------------------------------------------------
int hb_rmsnorm(const void* x, void* residual, const void* w, void* y, int rows, int h, long long ldx, long long ldy,
               float eps, int gemma, void* stream);
int hb_gated_rmsnorm(const void* x, const void* z, const void* w, void* y, int rows, int h, int gs, long long ldx,
                     long long ldz, float eps, int norm_first, int sigmoid_gate, int gemma, void* stream);
// KV pools are [slots, kv_heads, D] with `pool_stride` elements between slots and `head_stride` between heads.
int hb_rope_kv_write(const void* qkv, long long ld_qkv, const void* positions, const void* slots,
                     const void* inv_freq, const void* q_norm_w, const void* k_norm_w, float eps, int gemma_norm,
                     void* q_out, void* k_pool, void* v_pool, long long pool_stride, long long head_stride, int tokens,
                     int hq, int hkv, int d, int rot, int kv_fp8, float kv_inv_scale, int q_gate, void* stream);
int hb_act_mul(const void* x, const void* gate, void* out, long long rows, int inter, long long ldx, int mode,
               void* stream);
int hb_embedding(const void* ids, const void* table, void* out, int tokens, int h, long long vocab, void* stream);
int hb_add(const void* a, const void* b, void* out, long long n, void* stream);

// ---- paged attention (attn.cu) -------------------------------------------------------------------------
int hb_attn_paged(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                  long long head_stride,
                  const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len, const void* q_indptr,
                  void* out, void* part_o, void* part_lse, int batch, int total_rows, int max_rows, int hq, int hkv, int d,
                  int splits, float scale, int kv_fp8, float kv_scale, int causal, void* stream);
int hb_attn_merge(const void* part_o, const void* part_lse, void* out, long long rows_heads, int splits, int d,
                  void* stream);
// Tensor-core flash-decoding (attn_decode.cu): bf16 KV, rows_per_sequence * (hq / hkv) <= 16.
// Prefill / chunked-prefill attention on tcgen05 (bf16 KV, head dim 64 or 128); any number of new rows per sequence.
int hb_attn_prefill(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                    long long head_stride,
                    const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len,
                    const void* q_indptr, void* out, int batch, int max_rows, int hq, int hkv, int d, float scale,
                    int causal, long long pool_slots, void* status, void* stream);
int hb_gdn_phase1(const void* q, const void* k, const void* v, const void* g, const void* beta, long long ldq,
                  long long ldv, int n, int k_heads, int v_heads, float scale, int l2norm, void* w, void* qg, void* kd,
                  void* m, void* u, void* g_end, void* stream);
int hb_ssd_phase1(const void* x, const void* b, const void* c, const void* dt, const void* a_log, const void* dt_bias,
                  long long ldx, long long ldb, long long lddt, int n, int heads, int groups, int p, void* qg, void* kd,
                  void* m, void* u, void* g_end, void* stream);
int hb_gdn_chunk_pass(const void* w, const void* qg, const void* kd, const void* m, const void* u, const void* g_end,
                      const void* s_in, void* s_out, void* o, long long ldo, int heads, int nc, int n, int kdim,
                      int vdim, void* stream);
int hb_attn_decode_tc(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                      long long head_stride, const void* kv_indices, long long ld_idx, const void* seq_rows,
                      const void* ctx_len, const void* q_indptr, void* out, void* part_o, void* part_lse, int batch,
                      int max_rows, int hq, int hkv, int d, int splits, float scale, int causal, long long pool_slots,
                      void* status, void* stream);
void hb_attn_decode_tc_profile(void* buf);
void hb_attn_prefill_profile(void* buf);
void hb_attn_decode_profile(void* buf);
int hb_attn_decode(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                   long long head_stride,
                   const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len,
                   const void* q_indptr, void* out, void* part_o, void* part_lse, int batch, int max_rows, int hq,
                   int hkv, int d, int splits, float scale, int causal, long long pool_slots, void* status,
                   void* stream);

// ---- sampling and speculative acceptance (sample.cu) -----------------------------------------------------
int hb_argmax(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* bitmask, int mask_words,
              void* out, void* out_val, void* stream);
int hb_sample(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* temperature,
              const void* top_k, const void* top_p, const void* seeds, const void* offsets, const void* bitmask,
              int mask_words, void* out, void* out_prob, int skip_greedy, void* stream);
int hb_argmax2(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* bitmask, int mask_words,
               int nch, void* scratch_v, void* scratch_i, const void* temperature, void* out, void* out_val,
               void* stream);
int hb_quant_nvfp4_pairs(const void* x, long long ldx, const void* pos, int pairs, int topk, int k, int ka,
                         const void* gscale, void* q, void* sf, void* stream);
int hb_gated_rmsnorm_quant(const void* x, const void* z, const void* w, int rows, int h, int gs, long long ldx,
                           long long ldz, float eps, int norm_first, int sigmoid_gate, int gemma, void* q, void* sf,
                           const void* gscale, int ka, void* stream);
int hb_gdn_gates(const void* ba, long long ld, const void* a_log, const void* dt_bias, int rows, int heads,
                 void* beta, void* g, void* stream);
int hb_moe_share(void* ids, void* weights, int rows, int k, int experts, int keep, int budget, float scale,
                 void* stream);
int hb_ggml_gemv(int type, const void* w, long long row_bytes, int n, int k, const void* x, long long ldx, int m,
                 const void* grid, int relu2, void* y, long long ldy, void* stream);
int hb_ggml_gemv_pairs(int type, const void* w, long long row_bytes, long long expert_bytes, int n, int k,
                       const void* x, long long ldx, const void* grid, const void* pair_expert, const void* pair_row,
                       int pairs, int relu2, void* y, long long ldy, void* stream);
int hb_ggml_dequant(int type, const void* w, long long row_bytes, int row0, int rows, int k, const void* grid,
                    void* out, void* stream);
int hb_bounds_enabled();
int hb_bounds_set(int which, long long value);
int hb_bounds_read(long long* out);
int hb_lattice_walk(const void* cand, const void* scores, const void* temperature, const void* uniforms, int batch,
                    int k, int width, void* tokens, void* chosen, void* probs, void* estimate, void* stream);
int hb_spec_targets(const void* logits, long long ld, int batch, int k, int vocab, int is_f32, const void* drafts,
                    const void* temperature, const void* top_k, const void* top_p, const void* seeds,
                    const void* draws, const void* soft, const void* bitmask, int mask_words,
                    const void* greedy_pick, void* target, void* p_draft, void* stream);
int hb_accept_greedy(const void* target, const void* drafts, const void* stop_ids, int n_stop, const void* budget,
                     const void* depth, int k_max, int batch, void* emitted, void* count, void* accepted,
                     void* stream);
int hb_rank_gap(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* ids, void* rank,
                void* gap, void* stream);

// ---- recurrent layers (ssm.cu) ---------------------------------------------------------------------------
int hb_conv1d(const void* x, long long ldx, const void* w, const void* bias, void* y, long long ldy, void* state,
              long long state_stride, const void* q_indptr, const void* slot_in, const void* slot_out,
              const void* has_init, int batch, int channels, int width, int act_silu, int max_rows, void* stream);
int hb_mamba2_scan_fmt(const void* x, const void* bmat, const void* cmat, const void* dt, long long ldx,
                       long long ldb, long long lddt, const void* a_log, const void* dt_bias, const void* dskip,
                       void* y, long long ldy, void* state, long long state_stride, const void* q_indptr,
                       const void* slot_in, const void* slot_out, const void* has_init, int batch, int heads,
                       int groups, int head_dim, int d_state, int state_fmt, void* state_scale, unsigned sr_seed,
                       void* stream);
int hb_mamba2_scan(const void* x, const void* bmat, const void* cmat, const void* dt, long long ldx, long long ldb,
                   long long lddt, const void* a_log, const void* dt_bias, const void* dskip, void* y, long long ldy,
                   void* state, long long state_stride, const void* q_indptr, const void* slot_in,
                   const void* slot_out, const void* has_init, int batch, int heads, int groups, int head_dim,
                   int d_state, void* stream);
int hb_gdn_scan(const void* q, const void* k, const void* v, const void* g, const void* beta, long long ldq,
                long long ldv, void* o, long long ldo, void* state, long long state_stride, const void* q_indptr,
                const void* slot_in, const void* slot_out, const void* has_init, int batch, int k_heads,
                int v_heads, int kdim, int vdim, float scale, int l2norm, void* stream);

// ---- communicator (comm.cu) ------------------------------------------------------------------------------
int hb_comm_ctrl_bytes(void);
int hb_comm_nslot(void);
int hb_comm_alloc(long long bytes, void** out);
int hb_comm_free(void* p);
int hb_comm_ipc_handle(void* p, void* handle64);
int hb_comm_ipc_open(const void* handle64, void** out);
int hb_comm_ipc_close(void* p);
int hb_ar_norm(const void* const* peer_bases, int world, int rank, int slot, long long data_offset, int rows, int h,
               void* residual, const void* weight, float eps, int gemma, void* out, void* q, void* sf,
               const void* gscale, int ka, long long limit_ns, void* status, long long ll_offset, int ll_rows,
               void* stream);
int hb_comm_sp_layout(long long* out3);
int hb_rs_norm_ag(const void* const* peer_bases, int world, int rank, int rows_per_rank, int h, long long stage_offset,
                  int expected, void* residual, const void* weight, float eps, int gemma, long long gather_q_offset,
                  long long gather_sf_offset, long long gather_bf_offset, const void* gscale, int ka,
                  long long limit_ns, void* status, void* stream);
int hb_barrier(const void* const* peer_bases, int world, int rank, int slot, long long limit_ns, void* status,
               void* stream);

// ---- mixture of experts (moe.cu) -------------------------------------------------------------------------
int hb_moe_route(const void* logits, long long ld, const void* sel_bias, int tokens, int experts, int topk,
                 int sigmoid, int renorm, float scale, void* ids, void* weights, void* stream);
int hb_moe_plan(const void* ids, int tokens, int topk, int experts, int e_lo, int e_n, int id_base, void* cnt,
                void* start,
                void* pos, void* src_row, int rows_cap, void* total_rows, int tile_bn, void* tiles, void* n_tiles,
                int tile_cap, void* stream);
int hb_moe_tiles(const void* cnt, int experts, int tile_bn, void* tiles, void* n_tiles, int tile_cap, void* stream);
int hb_moe_gather(const void* x, long long ldx, const void* src_row, const void* total_rows, void* out, int rows_cap,
                  int h, void* stream);
int hb_moe_combine(const void* y, long long ldy, const void* pos, const void* weights, const void* shared,
                   long long ld_shared, void* out, long long ldo, int tokens, int topk, int h, void* stream);

#ifdef __cplusplus
}
#endif
