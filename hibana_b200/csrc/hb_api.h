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

#ifdef __cplusplus
}
#endif
