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
void hb_clear_tmap_cache(void);

// ---- quantisers (quant.cu) -----------------------------------------------------------------------------
int hb_quant_nvfp4(const void* x, long long ldx, int m, int k, int ka, const void* gscale, void* q, void* sf,
                   int mode, void* stream);
int hb_norm_quant_nvfp4(const void* x, void* residual, const void* w, float eps, int gemma, int m, int k, int ka,
                        const void* gscale, void* q, void* sf, void* normed, void* stream);
int hb_quant_fp8_static(const void* x, long long n, const void* scale, void* q, void* stream);
int hb_quant_fp8_rows(const void* x, int m, int k, void* q, void* scales, void* stream);

// ---- pointwise / row kernels (misc.cu) -----------------------------------------------------------------
int hb_rmsnorm(const void* x, void* residual, const void* w, void* y, int rows, int h, long long ldx, long long ldy,
               float eps, int gemma, void* stream);
int hb_gated_rmsnorm(const void* x, const void* z, const void* w, void* y, int rows, int h, int gs, long long ldx,
                     long long ldz, float eps, int norm_first, int sigmoid_gate, int gemma, void* stream);
int hb_rope_kv_write(const void* qkv, long long ld_qkv, const void* positions, const void* slots,
                     const void* inv_freq, const void* q_norm_w, const void* k_norm_w, float eps, int gemma_norm,
                     void* q_out, void* k_pool, void* v_pool, long long pool_stride, int tokens, int hq, int hkv,
                     int d, int rot, int kv_fp8, float kv_inv_scale, int q_gate, void* stream);
int hb_act_mul(const void* x, const void* gate, void* out, long long rows, int inter, long long ldx, int mode,
               void* stream);
int hb_embedding(const void* ids, const void* table, void* out, int tokens, int h, long long vocab, void* stream);
int hb_add(const void* a, const void* b, void* out, long long n, void* stream);

// ---- paged attention (attn.cu) -------------------------------------------------------------------------
int hb_attn_paged(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                  const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len, const void* q_indptr,
                  void* out, void* part_o, void* part_lse, int batch, int total_rows, int max_rows, int hq, int hkv, int d,
                  int splits, float scale, int kv_fp8, float kv_scale, int causal, void* stream);
int hb_attn_merge(const void* part_o, const void* part_lse, void* out, long long rows_heads, int splits, int d,
                  void* stream);
// Tensor-core flash-decoding (attn_decode.cu): bf16 KV, rows_per_sequence * (hq / hkv) <= 16.
int hb_attn_decode(const void* q, const void* k_pool, const void* v_pool, long long pool_stride,
                   const void* kv_indices, long long ld_idx, const void* seq_rows, const void* ctx_len,
                   const void* q_indptr, void* out, void* part_o, void* part_lse, int batch, int max_rows, int hq,
                   int hkv, int d, int splits, float scale, int causal, void* status, void* stream);

// ---- sampling and speculative acceptance (sample.cu) -----------------------------------------------------
int hb_argmax(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* bitmask, int mask_words,
              void* out, void* out_val, void* stream);
int hb_sample(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* temperature,
              const void* top_k, const void* top_p, const void* seeds, const void* offsets, const void* bitmask,
              int mask_words, void* out, void* out_prob, int skip_greedy, void* stream);
int hb_argmax2(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* bitmask, int mask_words,
               int nch, void* scratch_v, void* scratch_i, const void* temperature, void* out, void* out_val,
               void* stream);
int hb_accept_greedy(const void* target, const void* drafts, const void* stop_ids, int n_stop, const void* budget,
                     const void* depth, int k_max, int batch, void* emitted, void* count, void* accepted,
                     void* stream);
int hb_rank_gap(const void* logits, long long ld, int rows, int vocab, int is_f32, const void* ids, void* rank,
                void* gap, void* stream);

#ifdef __cplusplus
}
#endif
