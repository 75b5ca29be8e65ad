// krk_cuda_kraken_binding.hpp -- the file a Kraken maintainer adds to the Kraken tree (as
// src/cuda/backend_cuda.cpp or a header included from it) to get an sm_100a backend for the
// quantized-weight matmul path: `class CudaBackend final : public krk::Backend` over the C ABI of
// krk_cuda.h, plus the factory `make_cuda_backend` with make_hip_backend's contract
// (include/krk/backend.hpp:1886).
//
// It includes Kraken's own header, so it only compiles inside a Kraken tree (or with -I <kraken>/include);
// every pure virtual of krk::Backend is overridden, with the reference's exact signature, so the class
// instantiates. Members on the path forward to libkrk_cuda.so. Members that are NOT on the path (norms,
// rope, attention, KV append, plain element-wise ops) log what was asked and abort, like the reference's
// own answer to an operation a backend cannot run (src/hip/backend_hip.hip:3186-3190): a Kraken build that
// wants whole-model inference on this backend has to supply those kernels; the matmul path does not.
#pragma once

#include <cstdio>
#include <cstdlib>
#include <string>

#include "krk/backend.hpp"
#include "krk_cuda.h"

namespace krk {

class CudaBackend final : public Backend {
public:
    explicit CudaBackend(void *impl) : impl_(impl) {
        caps_.name = krk_cuda_backend_describe(impl_);
        caps_.gfx = "sm_100a";
        caps_.wave_size = 32;
    }
    ~CudaBackend() override { krk_cuda_backend_free(impl_); }

    // ---- identity and memory (include/krk/backend.hpp:341-362, 720-805, 1505) ----
    BackendKind kind() const override { return BackendKind::HIP; }   // "a discrete device"; add a CUDA value beside HIP to tell them apart
    const DeviceCaps &caps() const override { return caps_; }
    DType act_type() const override { return DType::F32; }           // f32 activations, as on the CPU backend
    size_t act_size() const override { return sizeof(f32); }
    void *alloc(size_t bytes) override { return krk_cuda_backend_alloc(impl_, bytes); }
    void release(void *p) override { krk_cuda_backend_release(impl_, p); }
    void upload(void *dst, const void *src, size_t bytes, size_t off = 0) override {
        krk_cuda_backend_upload(impl_, dst, src, bytes, off);
    }
    void download(void *dst, const void *src, size_t bytes, size_t off = 0) override {
        krk_cuda_backend_download(impl_, dst, src, bytes, off);
    }
    void fill0(void *dst, size_t bytes) override { krk_cuda_backend_fill0(impl_, dst, bytes); }
    void sync() override { krk_cuda_backend_sync(impl_); }
    void download_f32(f32 *dst, const void *src, i64 n) override { krk_cuda_backend_download_f32(impl_, dst, src, n); }
    void upload_i32(i32 *dst, const i32 *src, i64 n) override { krk_cuda_backend_upload_i32(impl_, dst, src, n); }
    std::string describe() const override { return krk_cuda_backend_describe(impl_); }

    // ---- the matmul path (include/krk/backend.hpp:858-900, 1040-1056) ----
    bool gemm_k_ok(i64 k) const override { return k > 0 && k % 32 == 0; }
    void gemm(void *out, const void *x, const void *w, DType wt, i64 n_out, i64 n_in, i64 rows) override {
        krk_cuda_backend_gemm(impl_, out, x, w, static_cast<int>(wt), n_out, n_in, rows);
    }
    bool gemm_accumulate(void *dst, const void *x, const void *w, DType wt, i64 n_out, i64 n_in, i64 rows,
                         const i32 *rexp = nullptr) override {
        return rexp == nullptr &&
               krk_cuda_backend_gemm_accumulate(impl_, dst, x, w, static_cast<int>(wt), n_out, n_in, rows) != 0;
    }
    bool gemm_group(void *const out[], const void *x, const void *const w[], DType wt, const i64 n_out[], i64 n_in,
                    int n_mat, i64 rows, bool silu = false, bool *silu_fused = nullptr, bool row_parallel_only = false,
                    const DType *wts = nullptr, const void *const xs[] = nullptr) override {
        (void)row_parallel_only;   // every matrix is one row-parallel pass on this backend
        int fused = 0;
        int types[64];
        if (wts && n_mat > 64)
            return Backend::gemm_group(out, x, w, wt, n_out, n_in, n_mat, rows, silu, silu_fused, row_parallel_only, wts, xs);
        if (wts)
            for (int m = 0; m < n_mat; m++) types[m] = static_cast<int>(wts[m]);
        const bool ran = krk_cuda_backend_gemm_group_ex(impl_, out, x, w, static_cast<int>(wt), n_out, n_in, n_mat, rows,
                                                        silu ? 1 : 0, &fused, wts ? types : nullptr, xs) != 0;
        if (silu_fused) *silu_fused = fused != 0;
        return ran;
    }

    // ---- the steps either side of the matmuls (backend.hpp:838, 902-922, 1309, 1451, 1473) ----
    void embed(void *out, const void *tok_embd, DType tt, i64 n_vocab, i64 n_embd, const i32 *tokens, i64 n_tok) override {
        krk_cuda_backend_embed(impl_, out, tok_embd, static_cast<int>(tt), n_vocab, n_embd, tokens, n_tok);
    }
    void logits_topk(const void *logits, i64 n, i32 k, const void *pen_mask, f32 rep_pen, f32 softcap, f32 temp, i32 *ids,
                     f32 *vals, f32 *mass_out, void *scratch, i32 cand_cap, i64 *count_out) override {
        krk_cuda_backend_logits_topk(impl_, logits, n, k, pen_mask, rep_pen, softcap, temp, ids, vals, mass_out, scratch,
                                     cand_cap, count_out);
    }
    void silu_mul(void *out, const void *gate, const void *up, i64 n, i64 row_len = 0, f32 *row_scale = nullptr) override {
        krk_cuda_backend_silu_mul(impl_, out, gate, up, n, row_len, row_scale);
    }
    using Backend::gather_rows;   // the i64-index byte-row overload (backend.hpp:1254) keeps the base class's body
    void gather_rows(void *dst, const void *src, const i32 *rows, i64 n_rows, i64 n) override {
        krk_cuda_backend_gather_rows(impl_, dst, src, rows, n_rows, n);
    }
    void scatter_axpy_rows(void *dst, const void *src, const i32 *rows, const f32 *alpha, i64 n_rows, i64 n,
                           const f32 *row_scale = nullptr, i32 *row_exp = nullptr) override {
        (void)row_scale;   // f32 activations carry no storage exponent (backend.hpp:1306-1308)
        (void)row_exp;
        krk_cuda_backend_scatter_axpy_rows(impl_, dst, src, rows, alpha, n_rows, n);
    }

    // ---- the router on the device (backend.hpp:934-986) ----
    bool router_softmax_supported() const override { return true; }
    void router_softmax(void *probs, const void *logits, i64 n_rows, i32 n_expert) override {
        krk_cuda_backend_router_softmax(impl_, probs, logits, n_rows, n_expert);
    }
    bool router_topk_supported() const override { return true; }
    void router_topk(const void *probs, i64 n_rows, i32 n_expert, i32 k, void *ids, void *wts, i32 normalize,
                     f32 scale) override {
        krk_cuda_backend_router_topk(impl_, probs, n_rows, n_expert, k, ids, wts, normalize, scale);
    }
    void moe_plan_build(const void *ids, i64 n_rows, i32 k, i32 n_expert, void *off, void *rows, void *wt,
                        const void *wts) override {
        krk_cuda_backend_moe_plan_build(impl_, ids, n_rows, k, n_expert, off, rows, wt, wts);
    }

    // ---- not on the quantized-weight matmul path: a Kraken build supplies these ----
    void rmsnorm(void *, const void *, const f32 *, i64, i64, f32, const i32 * = nullptr) override { off_path("rmsnorm"); }
    void rope(void *, void *, i64, i64, i64, i64, i64, const f32 *, f32, f32, bool) override { off_path("rope"); }
    void kv_append(void *, void *, const void *, const void *, const AttnDesc &) override { off_path("kv_append"); }
    void attention(void *, const void *, const void *, const void *, const AttnDesc &) override { off_path("attention"); }
    void swiglu_oai(void *, const void *, const void *, i64) override { off_path("swiglu_oai"); }
    void add_bias_rows(void *, const f32 *, i64, i64) override { off_path("add_bias_rows"); }
    void add_inplace(void *, const void *, i64) override { off_path("add_inplace"); }
    void copy_act(void *, const void *, i64) override { off_path("copy_act"); }
    void axpy(void *, const void *, f32, i64) override { off_path("axpy"); }

private:
    [[noreturn]] static void off_path(const char *op) {
        std::fprintf(stderr, "[krk-cuda] ERROR %s is not part of the quantized-weight matmul path this backend provides\n", op);
        std::abort();
    }
    void *impl_;
    DeviceCaps caps_;
};

inline Backend *make_cuda_backend(int device_index, std::string *err) {
    char msg[256] = "";
    void *impl = krk_cuda_backend_make(device_index, msg, sizeof msg);
    if (!impl) {
        if (err) *err = msg;
        return nullptr;
    }
    return new CudaBackend(impl);
}

} // namespace krk
