// krk_cuda_backend.hpp -- the host-side class a Kraken build links to get the sm_100a
// matmul path: the subset of krk::Backend (include/krk/backend.hpp:337-1878) that the
// quantized-weight matmul needs, with the same member names, argument meaning and error
// behaviour, implemented on the C ABI of krk_cuda.h.
//
// In a Kraken tree this class derives from krk::Backend (add the base class and `override`); here it
// stands alone so that it compiles without the reference's headers. All pointers handed to
// the ops are device pointers obtained from alloc(); the caller owns their lifetime
// (include/krk/backend.hpp:361-362). Ops are enqueued on one stream, asynchronous and
// ordered; completion is observed through sync() or download()
// (include/krk/backend.hpp:772-801). The engine calls a backend from one thread.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace krk_cuda {

using i32 = int32_t;
using i64 = int64_t;
using f32 = float;

// GGUF on-disk ids, the values of krk::DType (include/krk/quant.hpp:16-30).
enum class DType : int { F32 = 0, F16 = 1, Q4_0 = 2, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14 };

class CudaBackend {
public:
    // make_hip_backend's contract (include/krk/backend.hpp:1886): nullptr and *err on failure.
    static CudaBackend *make(int device_index, std::string *err);
    ~CudaBackend();

    const char *describe() const { return describe_.c_str(); }   // backend.hpp:805
    DType act_type() const { return DType::F32; }                // backend.hpp:341-358 (CPU: f32)
    size_t act_size() const { return sizeof(f32); }

    void *alloc(size_t bytes);                                   // backend.hpp:361
    void release(void *p);                                       // backend.hpp:362
    // backend.hpp:720 / :755: `off` is a byte offset into the DEVICE side (dst of an upload, src of a
    // download), as in src/backend_cpu.cpp:676-683. An upload from pageable host memory has been staged by
    // the driver when the call returns; from pinned memory it is asynchronous and the source must stay
    // valid until sync() or a download. download synchronises.
    void upload(void *dst, const void *host_src, size_t bytes, size_t off = 0);
    void download(void *host_dst, const void *src, size_t bytes, size_t off = 0);
    void download_f32(f32 *host_dst, const void *src, i64 n);    // backend.hpp:803
    void upload_i32(i32 *dst, const i32 *host_src, i64 n);       // backend.hpp:1505
    void fill0(void *p, size_t bytes);                           // backend.hpp:769
    void sync();                                                 // backend.hpp:770

    // backend.hpp:862-869. The reference's HIP rule is k > 0 && k % 32 == 0; the K-quant
    // formats additionally need whole 256-value super-blocks, which is asked per type.
    bool gemm_k_ok(i64 k) const { return k > 0 && k % 32 == 0; }
    bool gemm_k_ok(DType wt, i64 k) const;

    // out[rows, n_out] = x[rows, n_in] * W[n_out, n_in]^T (backend.hpp:858-860). A shape the
    // kernels cannot address is a logged error followed by std::abort(), as in
    // src/hip/backend_hip.hip:3186-3190; ask gemm_k_ok first.
    void gemm(void *out, const void *x, const void *w, DType wt, i64 n_out, i64 n_in, i64 rows);

    // dst += x * W^T, the residual fold (backend.hpp:894-900). True when the fused form ran;
    // false (nothing launched) for rows > 8 or a non-zero storage exponent.
    bool gemm_accumulate(void *dst, const void *x, const void *w, DType wt, i64 n_out, i64 n_in,
                         i64 rows, const i32 *rexp = nullptr);

    // Up to 16 independent projections in one launch (backend.hpp:1040-1056). True when the
    // single-launch form ran; otherwise every matrix went through gemm() and false is returned.
    bool gemm_group(void *const out[], const void *x, const void *const w[], DType wt,
                    const i64 n_out[], i64 n_in, int n_mat, i64 rows, bool silu = false,
                    bool *silu_fused = nullptr, bool row_parallel_only = false,
                    const DType *wts = nullptr, const void *const xs[] = nullptr);

    void silu_mul(void *out, const void *gate, const void *up, i64 n, i64 row_len = 0,
                  f32 *row_scale = nullptr);                     // backend.hpp:1309
    // silu_mul over `count` one-row buffers (backend.hpp:1320): exactly `count` silu_mul calls, scale[i] = 1.0
    void silu_mul_rows(void *const out[], const void *const gate[], const void *const up[], i64 row_len, int count,
                       f32 *const scale[]);
    void gather_rows(void *dst, const void *src, const i32 *rows, i64 n_rows, i64 n);   // backend.hpp:1451
    void scatter_axpy_rows(void *dst, const void *src, const i32 *rows, const f32 *alpha,
                           i64 n_rows, i64 n, const f32 *row_scale = nullptr,
                           i32 *row_exp = nullptr);              // backend.hpp:1473

    // out[n_tok, n_embd] <- rows of the quantized table selected by tokens (backend.hpp:838). `tokens` is
    // HOST memory, as the Backend contract has it; it is staged into device scratch on the stream. An id
    // outside [0, n_vocab) gives a zero row (src/backend_cpu.cpp:746-778).
    void embed(void *out, const void *tok_embd, DType tt, i64 n_vocab, i64 n_embd, const i32 *tokens, i64 n_tok);
    // Top-k of one f32 logits row on the device (backend.hpp:902-922): ids, vals, mass_out and count_out
    // are device pointers, as on the HIP backend; scratch / cand_cap are accepted and not needed (the
    // candidate buffer is the backend's own workspace, and the set is never truncated: *count_out = min(n, k)).
    void logits_topk(const void *logits, i64 n, i32 k, const void *pen_mask, f32 rep_pen, f32 softcap, f32 temp,
                     i32 *ids, f32 *vals, f32 *mass_out, void *scratch, i32 cand_cap, i64 *count_out);

    // The router on the device, in the interface's three steps (backend.hpp:934-986); all pointers device memory.
    bool router_softmax_supported() const { return true; }
    void router_softmax(void *probs, const void *logits, i64 n_rows, i32 n_expert);
    bool router_topk_supported() const { return true; }
    void router_topk(const void *probs, i64 n_rows, i32 n_expert, i32 k, void *ids, void *wts, i32 normalize, f32 scale);
    void moe_plan_build(const void *ids, i64 n_rows, i32 k, i32 n_expert, void *off, void *rows, void *wt, const void *wts);
    // moe_dispatch (backend.hpp:1002) reads the reference's expert-cache residency table, which this build does
    // not have; the routed-expert FFN over a resident bank is krk_cuda_moe_ffn(_routed) instead.
    bool moe_dispatch_supported() const { return false; }

    void *stream() const { return stream_; }
    int device() const { return device_; }

private:
    CudaBackend() = default;
    void *workspace(size_t bytes);
    void use() const;   // makes this backend's device current (a second backend may have changed it)
    int device_ = 0;
    void *stream_ = nullptr;
    void *ws_ = nullptr;
    size_t ws_bytes_ = 0;
    std::string describe_;
};

} // namespace krk_cuda
