/*
 * krk_oracle.h -- CPU restatement of Kraken's scalar f32 quantized-weight matmul.
 *
 * TEST INFRASTRUCTURE ONLY. This library is the checker the CUDA path is compared
 * against (tests, the smoke check and the CPU-baseline leg of the benchmark). It is
 * never linked into, imported by, or called from the product library.
 *
 * Parity status: PINNED. Every function here is compared bit-for-bit against the
 * reference's own compiled sources (oracle/_ref/libkrk_ref.so, built by the Makefile
 * in this directory from the reference tree where it lies) and against the
 * known-answer vectors held by the reference's test-suite (tests/test_kraken.cpp:456-469,
 * 563-573, 981-1001, 1026-1042); the outputs of the compiled reference are committed
 * as fixtures under tests/golden/.
 *
 * Each function cites the reference file:line whose arithmetic it follows.
 */
#ifndef KRK_ORACLE_H
#define KRK_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF on-disk type ids (include/krk/quant.hpp:16-30). */
enum {
    KRK_ORACLE_Q4_0 = 2,
    KRK_ORACLE_Q8_0 = 8,
    KRK_ORACLE_Q4_K = 12,
    KRK_ORACLE_Q6_K = 14,
    KRK_ORACLE_Q2_K = 10,
    KRK_ORACLE_Q3_K = 11,
    KRK_ORACLE_IQ4_NL = 20,
    KRK_ORACLE_Q5_0 = 6,
    KRK_ORACLE_Q5_1 = 7,
    KRK_ORACLE_Q5_K = 13
};

/* Geometry (src/quant.cpp:1805-1900). Return 0 for a type outside those above. */
int krk_oracle_block_size(int wt);
int krk_oracle_block_bytes(int wt);
size_t krk_oracle_row_bytes(int wt, int64_t n_in);

/* IEEE half -> float, exact including subnormals (src/common.cpp:161-187). */
float krk_oracle_fp16_to_fp32(uint16_t h);

/* Decode n_rows rows of n_in values each to f32 (src/quant.cpp:1911-1960 over the
 * per-format decoders :331-339, :381-387, :437-460, :491-512). Returns 0, or -1 for
 * an unknown type / n_in not a whole number of blocks. */
int krk_oracle_dequant_rows(float *out, const void *w, int wt, int64_t n_rows, int64_t n_in);

/* out[rows][n_out] = x[rows][n_in] . W[n_out][n_in]^T, one in-order f32 chain per
 * output (src/quant.cpp:5579-5589 driven by src/backend_cpu.cpp:1303-1320).
 * n_threads splits outputs only; bits do not depend on it. */
int krk_oracle_gemm(float *out, const float *x, const void *w, int wt, int64_t n_out,
                    int64_t n_in, int64_t rows, int n_threads);

/* Router: softmax over all experts, k picks of the largest probability with ties to
 * the lower id, weights renormalised over the picks in slot order
 * (src/engine.cpp:11704-11713, 11853-11920). ids/wts are [n_tok][k]. */
int krk_oracle_route(int32_t *ids, float *wts, const float *logits, int64_t n_tok,
                     int n_expert, int k);

/* out[i] = (g/(1+exp(-g))) * u  (src/backend_cpu.cpp:2394-2400). */
void krk_oracle_silu_mul(float *out, const float *gate, const float *up, int64_t n);
int krk_oracle_embed(float *out, const void *table, int wt, int64_t n_vocab, int64_t n_embd,
                     const int32_t *tokens, int64_t n_tok);
int krk_oracle_logits_topk(const float *logits, int64_t n, int k, const uint32_t *pen_mask, float rep_pen,
                           float softcap, float temp, int32_t *ids, float *vals, float *mass_out);

/* dst[rows[i]] += alpha[i] * src[i]  (src/backend_cpu.cpp:3193-3220). */
void krk_oracle_scatter_axpy_rows(float *dst, const float *src, const int32_t *rows,
                                  const float *alpha, int64_t n_rows, int64_t n);

/* Routed-expert FFN for n_tok tokens: per token, experts in ascending id, each
 * gate/up GEMV -> silu_mul -> down GEMV -> y += w_e * down
 * (src/engine.cpp:12353-, per-expert loop; ascending-id order :12215-12248).
 * gate/up/down are arrays of n_expert pointers (NULL for an expert that is not held;
 * a selected expert that is NULL contributes nothing, which is how a shard of the
 * expert bank is expressed). y is [n_tok][n_embd], overwritten. */
int krk_oracle_moe_ffn(float *y, const float *x, const int32_t *ids, const float *wts,
                       const void *const *gate, const void *const *up,
                       const void *const *down, int wt_gate_up, int wt_down,
                       int n_expert, int k, int64_t n_tok, int64_t n_embd, int64_t n_ff,
                       int n_threads);

#ifdef __cplusplus
}
#endif
#endif
