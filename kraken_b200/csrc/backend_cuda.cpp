// CudaBackend: the krk::Backend-shaped host class over the C ABI, plus a C shim so that
// a non-C++ host (the Python tests, the benchmark) can drive the very same object.
#include "krk_cuda_backend.hpp"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "krk_cuda.h"

namespace krk_cuda {

namespace {

// The reference routes every HIP call through KRK_HIP(expr) -> hip_check, which logs and
// aborts (src/hip/krk_hip.hpp:104-115). Same rule here.
void cuda_check(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return;
    std::fprintf(stderr, "[krk-cuda] ERROR %s: %s\n", what, cudaGetErrorString(e));
    std::abort();
}
#define KRK_CUDA_CHECK(expr) cuda_check((expr), #expr)

[[noreturn]] void die(const char *op, int rc, i64 n_out, i64 n_in, i64 rows, int wt) {
    std::fprintf(stderr, "[krk-cuda] ERROR %s refused: %s (wt=%d n_out=%lld n_in=%lld rows=%lld) %s\n", op,
                 krk_cuda_strerror(rc), wt, (long long)n_out, (long long)n_in, (long long)rows,
                 krk_cuda_last_cuda_error());
    std::abort();
}

} // namespace

CudaBackend *CudaBackend::make(int device_index, std::string *err) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || device_index < 0 || device_index >= n) {
        if (err) *err = e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range";
        return nullptr;
    }
    cudaDeviceProp prop;
    if ((e = cudaSetDevice(device_index)) != cudaSuccess ||
        (e = cudaGetDeviceProperties(&prop, device_index)) != cudaSuccess) {
        if (err) *err = cudaGetErrorString(e);
        return nullptr;
    }
    if (prop.major != 10) {
        if (err) *err = std::string("device is sm_") + std::to_string(prop.major * 10 + prop.minor) +
                        "; this backend is built for sm_100a only";
        return nullptr;
    }
    CudaBackend *be = new CudaBackend();
    be->device_ = device_index;
    be->stream_ = nullptr;   // the default stream, like the reference (backend.hpp:775-779)
    char buf[256];
    std::snprintf(buf, sizeof buf, "cuda:%d %s sm_%d%d %d SMs %.0f GiB", device_index, prop.name, prop.major,
                  prop.minor, prop.multiProcessorCount, (double)prop.totalGlobalMem / (1 << 30));
    be->describe_ = buf;
    return be;
}

CudaBackend::~CudaBackend() {
    if (ws_) cudaFree(ws_);
}

void CudaBackend::use() const {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != device_) KRK_CUDA_CHECK(cudaSetDevice(device_));
}

void *CudaBackend::alloc(size_t bytes) {
    use();
    void *p = nullptr;
    if (bytes == 0) bytes = 16;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;   // caller checks, as with the reference
    return p;
}
void CudaBackend::release(void *p) {
    if (p) KRK_CUDA_CHECK(cudaFree(p));
}
void CudaBackend::upload(void *dst, const void *host_src, size_t bytes, size_t off) {
    use();
    if (bytes)
        KRK_CUDA_CHECK(cudaMemcpyAsync(static_cast<char *>(dst) + off, host_src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream_));
}
void CudaBackend::download(void *host_dst, const void *src, size_t bytes, size_t off) {
    use();
    if (bytes)
        KRK_CUDA_CHECK(cudaMemcpyAsync(host_dst, static_cast<const char *>(src) + off, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream_));
    KRK_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream_));
}
void CudaBackend::download_f32(f32 *host_dst, const void *src, i64 n) {
    download(host_dst, src, sizeof(f32) * (size_t)n);   // activations are f32 already
}
void CudaBackend::upload_i32(i32 *dst, const i32 *host_src, i64 n) { upload(dst, host_src, sizeof(i32) * (size_t)n); }
void CudaBackend::fill0(void *p, size_t bytes) {
    use();
    if (bytes) KRK_CUDA_CHECK(cudaMemsetAsync(p, 0, bytes, (cudaStream_t)stream_));
}
void CudaBackend::sync() {
    use();
    KRK_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream_));
}

bool CudaBackend::gemm_k_ok(DType wt, i64 k) const { return krk_cuda_gemm_k_ok((int)wt, k) != 0; }

void *CudaBackend::workspace(size_t bytes) {
    if (bytes > ws_bytes_) {
        // Grows only; a grow first drains the stream so no kernel still reads the old block.
        if (ws_) {
            KRK_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream_));
            KRK_CUDA_CHECK(cudaFree(ws_));
        }
        KRK_CUDA_CHECK(cudaMalloc(&ws_, bytes));
        ws_bytes_ = bytes;
    }
    return ws_;
}

void CudaBackend::gemm(void *out, const void *x, const void *w, DType wt, i64 n_out, i64 n_in, i64 rows) {
    use();
    int rc;
    if (rows <= KRK_CUDA_MAX_ROWS) {
        rc = krk_cuda_gemv(out, x, w, (int)wt, n_out, n_in, rows, 0, stream_);
    } else {
        const size_t need = krk_cuda_gemm_workspace_bytes(KRK_CUDA_X_F32, n_out, n_in, rows);
        rc = krk_cuda_gemm(out, x, KRK_CUDA_X_F32, w, (int)wt, n_out, n_in, rows, workspace(need), need, stream_);
    }
    if (rc != KRK_CUDA_OK) die("gemm", rc, n_out, n_in, rows, (int)wt);
}

bool CudaBackend::gemm_accumulate(void *dst, const void *x, const void *w, DType wt, i64 n_out, i64 n_in,
                                  i64 rows, const i32 *rexp) {
    // A storage exponent belongs to f16 residual streams (backend.hpp:882-893); activations are
    // f32 here, so only the null form is taken and anything else is "do it the long way".
    if (rexp != nullptr || rows > KRK_CUDA_MAX_ROWS || rows < 1) return false;
    if (!krk_cuda_gemm_k_ok((int)wt, n_in)) return false;
    use();
    const int rc = krk_cuda_gemv(dst, x, w, (int)wt, n_out, n_in, rows, 1, stream_);
    if (rc != KRK_CUDA_OK) die("gemm_accumulate", rc, n_out, n_in, rows, (int)wt);
    return true;
}

bool CudaBackend::gemm_group(void *const out[], const void *x, const void *const w[], DType wt,
                             const i64 n_out[], i64 n_in, int n_mat, i64 rows, bool silu, bool *silu_fused,
                             bool row_parallel_only, const DType *wts, const void *const xs[]) {
    (void)row_parallel_only;   // every matrix is one row-parallel pass here; there is no split-K
    use();
    if (silu_fused) *silu_fused = false;
    const bool fold = silu && n_mat >= 2 && n_out[0] == n_out[1] && !xs &&
                      (!wts || wts[0] == wts[1]);
    if (rows == 1 && n_mat >= 1 && n_mat <= KRK_CUDA_MAX_GROUP) {
        const void *xv[KRK_CUDA_MAX_GROUP];
        int wtv[KRK_CUDA_MAX_GROUP];
        for (int m = 0; m < n_mat; m++) {
            xv[m] = xs ? xs[m] : x;
            wtv[m] = (int)(wts ? wts[m] : wt);
        }
        int rc;
        if (fold && n_mat == 2) {
            rc = krk_cuda_gemv_group(out, xv, w, wtv, n_out, n_in, 2, 1, stream_);
            if (rc == KRK_CUDA_OK && silu_fused) *silu_fused = true;
        } else {
            rc = krk_cuda_gemv_group(out, xv, w, wtv, n_out, n_in, n_mat, 0, stream_);
        }
        if (rc != KRK_CUDA_OK) die("gemm_group", rc, n_out[0], n_in, rows, wtv[0]);
        return true;
    }
    for (int m = 0; m < n_mat; m++) gemm(out[m], xs ? xs[m] : x, w[m], wts ? wts[m] : wt, n_out[m], n_in, rows);
    return false;
}

void CudaBackend::router_softmax(void *probs, const void *logits, i64 n_rows, i32 n_expert) {
    use();
    const int rc = krk_cuda_router_softmax(probs, logits, n_rows, n_expert, stream_);
    if (rc != KRK_CUDA_OK) die("router_softmax", rc, n_rows, n_expert, 0, 0);
}

void CudaBackend::router_topk(const void *probs, i64 n_rows, i32 n_expert, i32 k, void *ids, void *wts, i32 normalize,
                              f32 scale) {
    use();
    const int rc = krk_cuda_router_topk(probs, n_rows, n_expert, k, ids, wts, normalize, scale, stream_);
    if (rc != KRK_CUDA_OK) die("router_topk", rc, n_rows, n_expert, k, 0);
}

void CudaBackend::moe_plan_build(const void *ids, i64 n_rows, i32 k, i32 n_expert, void *off, void *rows, void *wt,
                                 const void *wts) {
    use();
    const int rc = krk_cuda_moe_plan_build(ids, n_rows, k, n_expert, off, rows, wt, wts, stream_);
    if (rc != KRK_CUDA_OK) die("moe_plan_build", rc, n_rows, n_expert, k, 0);
}

void CudaBackend::silu_mul(void *out, const void *gate, const void *up, i64 n, i64 row_len, f32 *row_scale) {
    use();
    const int rc = krk_cuda_silu_mul(out, gate, up, n, stream_);
    if (rc != KRK_CUDA_OK) die("silu_mul", rc, n, 0, 0, 0);
    // f32 activations carry no storage exponent: one scale of 1.0 per row, as the CPU backend
    // answers (src/backend_cpu.cpp:2401-2408). row_scale is a host array there and here.
    if (row_scale && row_len > 0 && n % row_len == 0)
        for (i64 r = 0; r < n / row_len; r++) row_scale[r] = 1.0f;
}

void CudaBackend::silu_mul_rows(void *const out[], const void *const gate[], const void *const up[], i64 row_len,
                                int count, f32 *const scale[]) {
    // The reference's default is `count` silu_mul calls and a batched form has to match them bit for bit
    // (backend.hpp:1312-1319); the element-wise kernel has no per-launch state, so the calls are the form.
    for (int i = 0; i < count; i++) silu_mul(out[i], gate[i], up[i], row_len, row_len, scale ? scale[i] : nullptr);
}

void CudaBackend::gather_rows(void *dst, const void *src, const i32 *rows, i64 n_rows, i64 n) {
    use();
    const int rc = krk_cuda_gather_rows(dst, src, rows, n_rows, n, stream_);
    if (rc != KRK_CUDA_OK) die("gather_rows", rc, n_rows, n, 0, 0);
}

void CudaBackend::scatter_axpy_rows(void *dst, const void *src, const i32 *rows, const f32 *alpha, i64 n_rows,
                                    i64 n, const f32 *row_scale, i32 *row_exp) {
    (void)row_scale;   // f32 backends fill it with 1.0 and ignore the exponent (backend.hpp:1306-1308)
    (void)row_exp;
    use();
    const int rc = krk_cuda_scatter_axpy_rows(dst, src, rows, alpha, n_rows, n, stream_);
    if (rc != KRK_CUDA_OK) die("scatter_axpy_rows", rc, n_rows, n, 0, 0);
}

void CudaBackend::embed(void *out, const void *tok_embd, DType tt, i64 n_vocab, i64 n_embd, const i32 *tokens,
                        i64 n_tok) {
    if (n_tok <= 0) return;
    use();
    const size_t need = (size_t)n_tok * sizeof(i32);
    void *dev_tokens = workspace(need);
    KRK_CUDA_CHECK(cudaMemcpyAsync(dev_tokens, tokens, need, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream_)));
    const int rc = krk_cuda_embed(out, tok_embd, (int)tt, n_vocab, n_embd, dev_tokens, n_tok, stream_);
    if (rc != KRK_CUDA_OK) die("embed", rc, n_vocab, n_embd, n_tok, (int)tt);
}

void CudaBackend::logits_topk(const void *logits, i64 n, i32 k, const void *pen_mask, f32 rep_pen, f32 softcap,
                              f32 temp, i32 *ids, f32 *vals, f32 *mass_out, void *scratch, i32 cand_cap,
                              i64 *count_out) {
    (void)scratch;
    (void)cand_cap;
    if (n <= 0 || k <= 0) return;
    use();
    const size_t need = krk_cuda_logits_topk_workspace_bytes(n, k);
    const int rc = krk_cuda_logits_topk(logits, n, k, pen_mask, rep_pen, softcap, temp, ids, vals, mass_out,
                                        workspace(need), need, stream_);
    if (rc != KRK_CUDA_OK) die("logits_topk", rc, n, k, 0, 0);
    if (count_out) {   // min(n, k) <= 64 as a little-endian i64, without a host buffer that must outlive the copy
        const i64 keep = n < k ? n : k;
        KRK_CUDA_CHECK(cudaMemsetAsync(count_out, 0, sizeof(i64), static_cast<cudaStream_t>(stream_)));
        KRK_CUDA_CHECK(cudaMemsetAsync(count_out, (int)keep, 1, static_cast<cudaStream_t>(stream_)));
    }
}

} // namespace krk_cuda

// ---- C shim over the class (declared in krk_cuda.h) -------------------------------------------
using krk_cuda::CudaBackend;
using krk_cuda::DType;

extern "C" {

void *krk_cuda_backend_make(int device_index, char *err, size_t err_len) {
    std::string e;
    CudaBackend *be = CudaBackend::make(device_index, &e);
    if (!be && err && err_len) {
        std::strncpy(err, e.c_str(), err_len - 1);
        err[err_len - 1] = 0;
    }
    return be;
}
void krk_cuda_backend_free(void *be) { delete static_cast<CudaBackend *>(be); }
const char *krk_cuda_backend_describe(void *be) { return static_cast<CudaBackend *>(be)->describe(); }
void *krk_cuda_backend_alloc(void *be, size_t bytes) { return static_cast<CudaBackend *>(be)->alloc(bytes); }
void krk_cuda_backend_release(void *be, void *p) { static_cast<CudaBackend *>(be)->release(p); }
void krk_cuda_backend_upload(void *be, void *dst, const void *host_src, size_t bytes, size_t off) {
    static_cast<CudaBackend *>(be)->upload(dst, host_src, bytes, off);
}
void krk_cuda_backend_download(void *be, void *host_dst, const void *src, size_t bytes, size_t off) {
    static_cast<CudaBackend *>(be)->download(host_dst, src, bytes, off);
}
void krk_cuda_backend_download_f32(void *be, float *host_dst, const void *src, int64_t n) {
    static_cast<CudaBackend *>(be)->download_f32(host_dst, src, n);
}
void krk_cuda_backend_upload_i32(void *be, int32_t *dst, const int32_t *host_src, int64_t n) {
    static_cast<CudaBackend *>(be)->upload_i32(dst, host_src, n);
}
void krk_cuda_backend_embed(void *be, void *out, const void *tok_embd, int tt, int64_t n_vocab, int64_t n_embd,
                            const int32_t *host_tokens, int64_t n_tok) {
    static_cast<CudaBackend *>(be)->embed(out, tok_embd, static_cast<DType>(tt), n_vocab, n_embd, host_tokens, n_tok);
}
void krk_cuda_backend_logits_topk(void *be, const void *logits, int64_t n, int32_t k, const void *pen_mask, float rep_pen,
                                  float softcap, float temp, int32_t *ids, float *vals, float *mass_out, void *scratch,
                                  int32_t cand_cap, int64_t *count_out) {
    static_cast<CudaBackend *>(be)->logits_topk(logits, n, k, pen_mask, rep_pen, softcap, temp, ids, vals, mass_out, scratch,
                                                cand_cap, count_out);
}
void krk_cuda_backend_silu_mul(void *be, void *out, const void *gate, const void *up, int64_t n, int64_t row_len,
                               float *host_row_scale) {
    static_cast<CudaBackend *>(be)->silu_mul(out, gate, up, n, row_len, host_row_scale);
}
void krk_cuda_backend_gather_rows(void *be, void *dst, const void *src, const int32_t *rows, int64_t n_rows, int64_t n) {
    static_cast<CudaBackend *>(be)->gather_rows(dst, src, rows, n_rows, n);
}
void krk_cuda_backend_scatter_axpy_rows(void *be, void *dst, const void *src, const int32_t *rows, const float *alpha,
                                        int64_t n_rows, int64_t n) {
    static_cast<CudaBackend *>(be)->scatter_axpy_rows(dst, src, rows, alpha, n_rows, n);
}
void krk_cuda_backend_router_softmax(void *be, void *probs, const void *logits, int64_t n_rows, int32_t n_expert) {
    static_cast<CudaBackend *>(be)->router_softmax(probs, logits, n_rows, n_expert);
}
void krk_cuda_backend_router_topk(void *be, const void *probs, int64_t n_rows, int32_t n_expert, int32_t k, void *ids,
                                  void *wts, int32_t normalize, float scale) {
    static_cast<CudaBackend *>(be)->router_topk(probs, n_rows, n_expert, k, ids, wts, normalize, scale);
}
void krk_cuda_backend_moe_plan_build(void *be, const void *ids, int64_t n_rows, int32_t k, int32_t n_expert, void *off,
                                     void *rows, void *wt, const void *wts) {
    static_cast<CudaBackend *>(be)->moe_plan_build(ids, n_rows, k, n_expert, off, rows, wt, wts);
}
int krk_cuda_backend_device(void *be) { return static_cast<CudaBackend *>(be)->device(); }
void krk_cuda_backend_fill0(void *be, void *p, size_t bytes) { static_cast<CudaBackend *>(be)->fill0(p, bytes); }
void krk_cuda_backend_sync(void *be) { static_cast<CudaBackend *>(be)->sync(); }
int krk_cuda_backend_gemm_k_ok(void *be, int wt, int64_t k) {
    return static_cast<CudaBackend *>(be)->gemm_k_ok(static_cast<DType>(wt), k) ? 1 : 0;
}
void krk_cuda_backend_gemm(void *be, void *out, const void *x, const void *w, int wt, int64_t n_out,
                           int64_t n_in, int64_t rows) {
    static_cast<CudaBackend *>(be)->gemm(out, x, w, static_cast<DType>(wt), n_out, n_in, rows);
}
int krk_cuda_backend_gemm_accumulate(void *be, void *dst, const void *x, const void *w, int wt, int64_t n_out,
                                     int64_t n_in, int64_t rows) {
    return static_cast<CudaBackend *>(be)->gemm_accumulate(dst, x, w, static_cast<DType>(wt), n_out, n_in, rows)
               ? 1 : 0;
}
int krk_cuda_backend_gemm_group(void *be, void *const out[], const void *x, const void *const w[], int wt,
                                const int64_t n_out[], int64_t n_in, int n_mat, int64_t rows, int silu,
                                int *silu_fused) {
    bool fused = false;
    const bool ran = static_cast<CudaBackend *>(be)->gemm_group(out, x, w, static_cast<DType>(wt), n_out, n_in,
                                                                n_mat, rows, silu != 0, &fused);
    if (silu_fused) *silu_fused = fused ? 1 : 0;
    return ran ? 1 : 0;
}

int krk_cuda_backend_gemm_group_ex(void *be, void *const out[], const void *x, const void *const w[], int wt,
                                   const int64_t n_out[], int64_t n_in, int n_mat, int64_t rows, int silu,
                                   int *silu_fused, const int wts[], const void *const xs[]) {
    bool fused = false;
    DType types[KRK_CUDA_MAX_GROUP];
    if (wts && n_mat > KRK_CUDA_MAX_GROUP) {   // larger groups than one launch takes: the per-matrix loop
        auto *b = static_cast<CudaBackend *>(be);
        for (int m = 0; m < n_mat; m++) b->gemm(out[m], xs ? xs[m] : x, w[m], static_cast<DType>(wts[m]), n_out[m], n_in, rows);
        if (silu_fused) *silu_fused = 0;
        return 0;
    }
    if (wts)
        for (int m = 0; m < n_mat; m++) types[m] = static_cast<DType>(wts[m]);
    const bool ran = static_cast<CudaBackend *>(be)->gemm_group(out, x, w, static_cast<DType>(wt), n_out, n_in, n_mat, rows,
                                                                silu != 0, &fused, false, wts ? types : nullptr, xs);
    if (silu_fused) *silu_fused = fused ? 1 : 0;
    return ran ? 1 : 0;
}

} // extern "C"
