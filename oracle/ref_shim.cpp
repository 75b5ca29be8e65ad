// ref_shim.cpp -- a C face on the UNMODIFIED reference sources, for checking the
// restatement in krk_oracle.c and for timing Kraken's own CPU path.
//
// TEST INFRASTRUCTURE ONLY. This file holds no arithmetic of its own: every entry
// forwards to a function the reference exports (krk::dequant_row, krk::vec_dot,
// krk::Backend::gemm / silu_mul / scatter_axpy_rows of make_cpu_backend()). It is
// compiled together with the reference's own translation units, in place, by the
// Makefile beside it; the result (oracle/_ref/libkrk_ref.so) is never committed.

#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "krk/backend.hpp"
#include "krk/common.hpp"
#include "krk/quant.hpp"

namespace {

krk::Backend *cpu_backend() {
    static krk::Backend *be = krk::make_cpu_backend();
    return be;
}

struct TierDefaults {
    bool int8, fast, avx2, wide;
};

// The switches as the reference leaves them on this host (include/krk/quant.hpp:245-284).
const TierDefaults &tier_defaults() {
    static const TierDefaults d = {krk::vec_dot_int8(), krk::vec_dot_fast(),
                                   krk::vec_dot_avx2(), krk::vec_dot_wide()};
    return d;
}

// tier 0: the scalar oracle, one in-order f32 chain (include/krk/quant.hpp:208-227).
// tier 1: whatever a user of the reference's CPU backend gets by default.
void select_tier(int tier) {
    const TierDefaults &d = tier_defaults();
    if (tier == 0) {
        krk::set_vec_dot_int8(false);
        krk::set_vec_dot_fast(false);
        krk::set_vec_dot_avx2(false);
        krk::set_vec_dot_wide(false);
    } else {
        krk::set_vec_dot_int8(d.int8);
        krk::set_vec_dot_fast(d.fast);
        krk::set_vec_dot_avx2(d.avx2);
        krk::set_vec_dot_wide(d.wide);
    }
}

} // namespace

extern "C" {

float krk_ref_fp16_to_fp32(uint16_t h) { return krk::fp16_to_fp32(h); }
uint16_t krk_ref_fp32_to_fp16(float f) { return krk::fp32_to_fp16(f); }

int krk_ref_block_size(int wt) { return krk::dtype_block_size(static_cast<krk::DType>(wt)); }
int krk_ref_block_bytes(int wt) { return krk::dtype_block_bytes(static_cast<krk::DType>(wt)); }
size_t krk_ref_row_bytes(int wt, int64_t n) {
    return krk::dtype_row_bytes(static_cast<krk::DType>(wt), n);
}

int krk_ref_dequant_rows(float *out, const void *w, int wt, int64_t n_rows, int64_t n_in) {
    const krk::DType t = static_cast<krk::DType>(wt);
    const size_t rb = krk::dtype_row_bytes(t, n_in);
    const uint8_t *p = static_cast<const uint8_t *>(w);
    for (int64_t r = 0; r < n_rows; r++)
        krk::dequant_row(t, p + static_cast<size_t>(r) * rb, out + r * n_in, n_in);
    return 0;
}

float krk_ref_vec_dot(int wt, const void *row, const float *x, int64_t n, int tier) {
    tier_defaults();
    select_tier(tier);
    return krk::vec_dot(static_cast<krk::DType>(wt), row, x, n);
}

// out[rows][n_out] through CpuBackend::gemm (src/backend_cpu.cpp:914-1321).
int krk_ref_gemm(float *out, const float *x, const void *w, int wt, int64_t n_out,
                 int64_t n_in, int64_t rows, int tier) {
    tier_defaults();
    select_tier(tier);
    cpu_backend()->gemm(out, x, w, static_cast<krk::DType>(wt), n_out, n_in, rows);
    return 0;
}

void krk_ref_silu_mul(float *out, const float *gate, const float *up, int64_t n) {
    cpu_backend()->silu_mul(out, gate, up, n);
}

void krk_ref_scatter_axpy_rows(float *dst, const float *src, const int32_t *rows,
                               const float *alpha, int64_t n_rows, int64_t n) {
    cpu_backend()->scatter_axpy_rows(dst, src, rows, alpha, n_rows, n);
}

// CpuBackend::embed (src/backend_cpu.cpp:746-778) and CpuBackend::logits_topk (:862-912).
void krk_ref_embed(float *out, const void *table, int wt, int64_t n_vocab, int64_t n_embd,
                   const int32_t *tokens, int64_t n_tok) {
    cpu_backend()->embed(out, table, static_cast<krk::DType>(wt), n_vocab, n_embd, tokens, n_tok);
}

void krk_ref_logits_topk(const float *logits, int64_t n, int k, const uint32_t *pen_mask, float rep_pen,
                         float softcap, float temp, int32_t *ids, float *vals, float *mass_out) {
    int64_t count = 0;
    cpu_backend()->logits_topk(logits, n, k, pen_mask, rep_pen, softcap, temp, ids, vals, mass_out, nullptr, 0, &count);
}

// Bit 0: int8 tier on by default; bit 1: four-lane order; bit 2: fused AVX2; bit 3: wide.
int krk_ref_default_tiers(void) {
    const TierDefaults &d = tier_defaults();
    return (d.int8 ? 1 : 0) | (d.fast ? 2 : 0) | (d.avx2 ? 4 : 0) | (d.wide ? 8 : 0);
}

} // extern "C"
