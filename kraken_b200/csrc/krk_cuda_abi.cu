// The extern "C" surface declared in include/krk_cuda.h: argument checks, then a launch.
// Nothing here computes on the host.
#include <atomic>
#include <cstring>
#include <mutex>

#include "krk_common.cuh"

namespace krk_cuda {

namespace {
thread_local char g_cuda_err[256] = "";
std::atomic<int64_t> g_launches{0};
std::atomic<int64_t> g_family[4];

struct DeviceState {
    int *status = nullptr;
    std::atomic<int> sms{0};   // published last (release): a thread that sees it set also sees `status`
};
constexpr int kMaxDevices = 64;
DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mu;

DeviceState *device_state() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    DeviceState &s = g_dev[dev];
    if (s.sms.load(std::memory_order_acquire) == 0) {
        std::lock_guard<std::mutex> lk(g_dev_mu);
        if (s.sms.load(std::memory_order_relaxed) == 0) {
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
            int *p = nullptr;
            if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
            cudaMemset(p, 0, sizeof(int));
            s.status = p;
            s.sms.store(sms, std::memory_order_release);
        }
    }
    return &s;
}
} // namespace

void note_cuda_error(cudaError_t e) {
    std::strncpy(g_cuda_err, cudaGetErrorString(e), sizeof(g_cuda_err) - 1);
    g_cuda_err[sizeof(g_cuda_err) - 1] = 0;
}
void note_launch(int n, int family) {
    g_launches.fetch_add(n, std::memory_order_relaxed);
    if (family > 0 && family < 4) g_family[family].fetch_add(n, std::memory_order_relaxed);
}
int *device_status_word() {
    DeviceState *s = device_state();
    return s ? s->status : nullptr;
}
int sm_count() {
    DeviceState *s = device_state();
    return s ? s->sms.load(std::memory_order_relaxed) : 1;
}

static inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

static int check_matmul_args(const void *y, const void *x, const void *w, int wt, int64_t n_out,
                             int64_t n_in, int64_t rows) {
    if (!krk_cuda_dtype_ok(wt)) return KRK_CUDA_EDTYPE;
    if (n_out < 0 || rows < 0 || !krk_cuda_gemm_k_ok(wt, n_in)) return KRK_CUDA_ESHAPE;
    if (n_out > 0 && rows > 0 && (!y || !x || !w)) return KRK_CUDA_ENULL;
    if (!aligned(w, 16) || !aligned(x, 16) || !aligned(y, 4)) return KRK_CUDA_EALIGN;
    return KRK_CUDA_OK;
}

} // namespace krk_cuda

using namespace krk_cuda;

extern "C" {

const char *krk_cuda_strerror(int rc) {
    switch (rc) {
    case KRK_CUDA_OK: return "ok";
    case KRK_CUDA_EDTYPE: return "unsupported weight type (want Q8_0, Q4_0, Q4_K, Q6_K, Q5_0, Q5_1, Q5_K, Q2_K, Q3_K or IQ4_NL)";
    case KRK_CUDA_ESHAPE: return "shape not addressable (n_in must be a positive whole number of blocks; sizes non-negative; rows in range)";
    case KRK_CUDA_ENULL: return "null pointer";
    case KRK_CUDA_EALIGN: return "misaligned pointer (weights and x 16 bytes, y 4 bytes)";
    case KRK_CUDA_ELAUNCH: return "CUDA launch failed";
    case KRK_CUDA_EWORKSPACE: return "workspace missing or too small";
    case KRK_CUDA_EDEVICE: return "no usable CUDA device is current";
    case KRK_CUDA_EARG: return "bad argument";
    case KRK_CUDA_ETIMEOUT: return "a bounded device-side wait gave up";
    case KRK_CUDA_ETOOBIG: return "problem larger than the fixed scratch array of the no-allocation entry (rows * n_in <= 4194304)";
    default: return "unknown error";
    }
}

const char *krk_cuda_last_cuda_error(void) { return g_cuda_err; }

int krk_cuda_dtype_ok(int wt) { return block_size(wt) != 0; }
int krk_cuda_block_size(int wt) { return block_size(wt); }
int krk_cuda_block_bytes(int wt) { return block_bytes(wt); }
size_t krk_cuda_row_bytes(int wt, int64_t n_in) { return n_in < 0 ? 0 : row_bytes(wt, n_in); }
int krk_cuda_gemm_k_ok(int wt, int64_t k) {
    const int bs = block_size(wt);
    return bs != 0 && k > 0 && k % bs == 0;
}

int krk_cuda_dequant_rows(void *out_f32, const void *w, int wt, int64_t n_rows, int64_t n_in,
                          void *stream) {
    if (!krk_cuda_dtype_ok(wt)) return KRK_CUDA_EDTYPE;
    if (n_rows < 0 || n_in < 0 || n_in % block_size(wt) != 0) return KRK_CUDA_ESHAPE;
    if (n_rows * n_in == 0) return KRK_CUDA_OK;
    if (!out_f32 || !w) return KRK_CUDA_ENULL;
    if (!aligned(out_f32, 4)) return KRK_CUDA_EALIGN;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_dequant_rows(static_cast<float *>(out_f32), static_cast<const uint8_t *>(w), wt,
                               n_rows, n_in, static_cast<cudaStream_t>(stream));
}

int krk_cuda_gemv(void *y_f32, const void *x_f32, const void *w, int wt, int64_t n_out, int64_t n_in,
                  int64_t rows, int accumulate, void *stream) {
    int rc = check_matmul_args(y_f32, x_f32, w, wt, n_out, n_in, rows);
    if (rc != KRK_CUDA_OK) return rc;
    if (rows > KRK_CUDA_MAX_ROWS) return KRK_CUDA_ESHAPE;
    if (n_out == 0 || rows == 0) return KRK_CUDA_OK;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    GemvMat m;
    m.w = static_cast<const uint8_t *>(w);
    m.x = static_cast<const float *>(x_f32);
    m.y = static_cast<float *>(y_f32);
    m.n_out = n_out;
    m.wt = wt;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = launch_gemv_stream(&m, 1, n_in, (int)rows, accumulate, 0, st);
    if (rc != 0) return rc < 0 ? rc : KRK_CUDA_OK;
    return launch_gemv_generic(&m, 1, n_in, (int)rows, accumulate, 0, st);
}

int krk_cuda_gemv_group(void *const host_y[], const void *const host_x[], const void *const host_w[],
                        const int host_wt[], const int64_t host_n_out[], int64_t n_in, int n_mat,
                        int fuse_silu_pair, void *stream) {
    if (n_mat < 0 || n_mat > KRK_CUDA_MAX_GROUP) return KRK_CUDA_EARG;
    if (n_mat == 0) return KRK_CUDA_OK;
    if (!host_y || !host_x || !host_w || !host_wt || !host_n_out) return KRK_CUDA_ENULL;
    if (fuse_silu_pair && (n_mat & 1)) return KRK_CUDA_EARG;
    GemvMat mats[KRK_CUDA_MAX_GROUP];
    for (int m = 0; m < n_mat; m++) {
        const int rc = check_matmul_args(host_y[m], host_x[m], host_w[m], host_wt[m], host_n_out[m], n_in, 1);
        if (rc != KRK_CUDA_OK) return rc;
        if (fuse_silu_pair && (m & 1) &&
            (host_n_out[m] != host_n_out[m - 1] || host_wt[m] != host_wt[m - 1] || host_x[m] != host_x[m - 1]))
            return KRK_CUDA_EARG;
        mats[m].w = static_cast<const uint8_t *>(host_w[m]);
        mats[m].x = static_cast<const float *>(host_x[m]);
        mats[m].y = static_cast<float *>(host_y[m]);
        mats[m].n_out = host_n_out[m];
        mats[m].wt = host_wt[m];
    }
    if (!device_state()) return KRK_CUDA_EDEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // One launch per run of equal weight types (a pair of the silu fold never straddles two runs: its types are
    // equal), each on the streaming kernel where it addresses the shape.
    for (int first = 0; first < n_mat;) {
        int last = first + 1;
        while (last < n_mat && mats[last].wt == mats[first].wt) last++;
        int rc = launch_gemv_stream(mats + first, last - first, n_in, 1, 0, fuse_silu_pair, st);
        if (rc < 0) return rc;
        if (rc == 0) {
            rc = launch_gemv_generic(mats + first, last - first, n_in, 1, 0, fuse_silu_pair, st);
            if (rc != KRK_CUDA_OK) return rc;
        }
        first = last;
    }
    return KRK_CUDA_OK;
}

size_t krk_cuda_gemm_workspace_bytes(int x_dtype, int64_t n_out, int64_t n_in, int64_t rows) {
    if (rows <= 0 || n_in <= 0 || n_out <= 0) return 0;
    if (n_in % 256 != 0) return 0;   // the row-batch rung below needs none
    return gemm_workspace_bytes(x_dtype, n_out, n_in, rows);
}

int krk_cuda_gemm(void *y_f32, const void *x, int x_dtype, const void *w, int wt, int64_t n_out,
                  int64_t n_in, int64_t rows, void *workspace, size_t ws_bytes, void *stream) {
    if (x_dtype != KRK_CUDA_X_F32 && x_dtype != KRK_CUDA_X_F16) return KRK_CUDA_EARG;
    const int rc = check_matmul_args(y_f32, x, w, wt, n_out, n_in, rows);
    if (rc != KRK_CUDA_OK) return rc;
    if (n_in % 256 != 0 || !gemm_tc_takes(wt)) {
        // The fallback rung (the place of gemm_simt_kernel, src/hip/kernels/gemm.hpp:1013-1134): 32-value
        // block formats whose K is a whole number of blocks but not of 256. Correct, not fast: the
        // shape-agnostic GEMV over batches of KRK_CUDA_MAX_ROWS activation rows. f32 activations only.
        if (x_dtype != KRK_CUDA_X_F32) return KRK_CUDA_ESHAPE;
        if (n_out == 0 || rows == 0) return KRK_CUDA_OK;
        if (!device_state()) return KRK_CUDA_EDEVICE;
        for (int64_t r0 = 0; r0 < rows; r0 += KRK_CUDA_MAX_ROWS) {
            const int64_t nr = rows - r0 < KRK_CUDA_MAX_ROWS ? rows - r0 : KRK_CUDA_MAX_ROWS;
            GemvMat m;
            m.w = static_cast<const uint8_t *>(w);
            m.x = static_cast<const float *>(x) + r0 * n_in;
            m.y = static_cast<float *>(y_f32) + r0 * n_out;
            m.n_out = n_out;
            m.wt = wt;
            const int grc = launch_gemv_generic(&m, 1, n_in, (int)nr, 0, 0, static_cast<cudaStream_t>(stream));
            if (grc != KRK_CUDA_OK) return grc;
        }
        return KRK_CUDA_OK;
    }
    if (n_out == 0 || rows == 0) return KRK_CUDA_OK;
    const size_t need = gemm_workspace_bytes(x_dtype, n_out, n_in, rows);
    if (need > 0 && (!workspace || ws_bytes < need || !aligned(workspace, 128))) return KRK_CUDA_EWORKSPACE;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_gemm_tc(static_cast<float *>(y_f32), x, x_dtype, static_cast<const uint8_t *>(w), wt,
                          n_out, n_in, rows, workspace, static_cast<cudaStream_t>(stream));
}

int krk_cuda_route(void *ids_i32, void *wts_f32, const void *logits_f32, int64_t n_tok, int n_expert,
                   int k, void *stream) {
    if (n_tok < 0) return KRK_CUDA_ESHAPE;
    if (n_tok > 0 && (!ids_i32 || !wts_f32 || !logits_f32)) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_route(static_cast<int32_t *>(ids_i32), static_cast<float *>(wts_f32),
                        static_cast<const float *>(logits_f32), n_tok, n_expert, k,
                        static_cast<cudaStream_t>(stream));
}

int krk_cuda_router_softmax(void *probs_f32, const void *logits_f32, int64_t n_rows, int n_expert, void *stream) {
    if (n_rows < 0) return KRK_CUDA_ESHAPE;
    if (n_rows > 0 && (!probs_f32 || !logits_f32)) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_router_softmax(static_cast<float *>(probs_f32), static_cast<const float *>(logits_f32), n_rows, n_expert,
                                 static_cast<cudaStream_t>(stream));
}

int krk_cuda_router_topk(const void *probs_f32, int64_t n_rows, int n_expert, int k, void *ids_i32, void *wts_f32,
                         int normalize, float scale, void *stream) {
    if (n_rows < 0) return KRK_CUDA_ESHAPE;
    if (n_rows > 0 && (!probs_f32 || !ids_i32 || !wts_f32)) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_router_topk(static_cast<const float *>(probs_f32), n_rows, n_expert, k, static_cast<int32_t *>(ids_i32),
                              static_cast<float *>(wts_f32), normalize, scale, static_cast<cudaStream_t>(stream));
}

int krk_cuda_moe_plan_build(const void *ids_i32, int64_t n_rows, int k, int n_expert, void *off_i32, void *rows_i32,
                            void *wt_f32, const void *wts_f32, void *stream) {
    if (n_rows < 0) return KRK_CUDA_ESHAPE;
    if (!off_i32 || (n_rows > 0 && (!ids_i32 || !rows_i32 || !wt_f32))) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_moe_plan_build(static_cast<const int32_t *>(ids_i32), n_rows, k, n_expert, static_cast<int32_t *>(off_i32),
                                 static_cast<int32_t *>(rows_i32), static_cast<float *>(wt_f32),
                                 static_cast<const float *>(wts_f32), static_cast<cudaStream_t>(stream));
}

static int check_bank(const krk_cuda_expert_bank *b) {
    if (!b) return KRK_CUDA_ENULL;
    if (!krk_cuda_dtype_ok(b->wt_gate_up) || !krk_cuda_dtype_ok(b->wt_down)) return KRK_CUDA_EDTYPE;
    if (b->n_local < 0 || !krk_cuda_gemm_k_ok(b->wt_gate_up, b->n_embd) ||
        !krk_cuda_gemm_k_ok(b->wt_down, b->n_ff))
        return KRK_CUDA_ESHAPE;
    if (b->n_local > 0 && (!b->gate || !b->up || !b->down)) return KRK_CUDA_ENULL;
    if (!aligned(b->gate, 16) || !aligned(b->up, 16) || !aligned(b->down, 16)) return KRK_CUDA_EALIGN;
    return KRK_CUDA_OK;
}

size_t krk_cuda_moe_workspace_bytes(const struct krk_cuda_expert_bank *bank, int k, int64_t n_tok) {
    if (check_bank(bank) != KRK_CUDA_OK || k <= 0 || n_tok <= 0) return 0;
    return moe_workspace_bytes(bank, k, n_tok);
}

int krk_cuda_moe_ffn(void *y_f32, const void *x_f32, const void *ids_i32, const void *wts_f32,
                     const struct krk_cuda_expert_bank *bank, int k, int64_t n_tok, void *workspace,
                     size_t ws_bytes, void *stream) {
    const int rc = check_bank(bank);
    if (rc != KRK_CUDA_OK) return rc;
    if (k <= 0 || k > 32) return KRK_CUDA_EARG;
    if (n_tok < 0 || n_tok * k > (1 << 22)) return KRK_CUDA_ESHAPE;
    if (n_tok == 0) return KRK_CUDA_OK;
    if (!y_f32 || !x_f32 || !ids_i32 || !wts_f32) return KRK_CUDA_ENULL;
    if (!aligned(x_f32, 16) || !aligned(y_f32, 4)) return KRK_CUDA_EALIGN;
    if (!workspace || ws_bytes < moe_workspace_bytes(bank, k, n_tok) || !aligned(workspace, n_tok > KRK_CUDA_MAX_ROWS ? 128 : 16))
        return KRK_CUDA_EWORKSPACE;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_moe_ffn_generic(static_cast<float *>(y_f32), static_cast<const float *>(x_f32),
                                  static_cast<const int32_t *>(ids_i32),
                                  static_cast<const float *>(wts_f32), bank, k, n_tok, workspace,
                                  static_cast<cudaStream_t>(stream));
}

int krk_cuda_moe_ffn_routed(void *y_f32, const void *x_f32, const void *router_logits_f32, int n_expert,
                            void *ids_i32, void *wts_f32, const struct krk_cuda_expert_bank *bank, int k,
                            int64_t n_tok, void *workspace, size_t ws_bytes, void *stream) {
    const int rc = check_bank(bank);
    if (rc != KRK_CUDA_OK) return rc;
    if (k <= 0 || k > 32 || n_expert <= 0 || n_expert > 1024 || k > n_expert) return KRK_CUDA_EARG;
    if (n_tok < 0 || n_tok * k > (1 << 22)) return KRK_CUDA_ESHAPE;
    if (n_tok == 0) return KRK_CUDA_OK;
    if (!y_f32 || !x_f32 || !router_logits_f32 || !ids_i32 || !wts_f32) return KRK_CUDA_ENULL;
    if (!aligned(x_f32, 16) || !aligned(y_f32, 4)) return KRK_CUDA_EALIGN;
    if (!workspace || ws_bytes < moe_workspace_bytes(bank, k, n_tok) || !aligned(workspace, n_tok > KRK_CUDA_MAX_ROWS ? 128 : 16))
        return KRK_CUDA_EWORKSPACE;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_moe_ffn_generic(static_cast<float *>(y_f32), static_cast<const float *>(x_f32),
                                  static_cast<const int32_t *>(ids_i32), static_cast<const float *>(wts_f32), bank, k,
                                  n_tok, workspace, static_cast<cudaStream_t>(stream),
                                  static_cast<const float *>(router_logits_f32), n_expert);
}

int krk_cuda_silu_mul(void *out_f32, const void *gate_f32, const void *up_f32, int64_t n, void *stream) {
    if (n < 0) return KRK_CUDA_ESHAPE;
    if (n > 0 && (!out_f32 || !gate_f32 || !up_f32)) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_silu_mul(static_cast<float *>(out_f32), static_cast<const float *>(gate_f32),
                           static_cast<const float *>(up_f32), n, static_cast<cudaStream_t>(stream));
}

int krk_cuda_gather_rows(void *dst_f32, const void *src_f32, const void *rows_i32, int64_t n_rows, int64_t n,
                         void *stream) {
    if (n_rows < 0 || n < 0) return KRK_CUDA_ESHAPE;
    if (n_rows * n > 0 && (!dst_f32 || !src_f32 || !rows_i32)) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_gather_rows(static_cast<float *>(dst_f32), static_cast<const float *>(src_f32),
                              static_cast<const int32_t *>(rows_i32), n_rows, n, static_cast<cudaStream_t>(stream));
}

int krk_cuda_scatter_axpy_rows(void *dst_f32, const void *src_f32, const void *rows_i32,
                               const void *alpha_f32, int64_t n_rows, int64_t n, void *stream) {
    if (n_rows < 0 || n < 0) return KRK_CUDA_ESHAPE;
    if (n_rows * n > 0 && (!dst_f32 || !src_f32 || !rows_i32 || !alpha_f32)) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_scatter_axpy_rows(static_cast<float *>(dst_f32), static_cast<const float *>(src_f32),
                                    static_cast<const int32_t *>(rows_i32),
                                    static_cast<const float *>(alpha_f32), n_rows, n,
                                    static_cast<cudaStream_t>(stream));
}

int krk_cuda_sum_parts(void *out_f32, const void *parts_f32, int n_parts, int64_t n, void *stream) {
    if (n < 0 || n_parts <= 0) return KRK_CUDA_ESHAPE;
    if (n > 0 && (!out_f32 || !parts_f32)) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_sum_parts(static_cast<float *>(out_f32), static_cast<const float *>(parts_f32),
                            n_parts, n, static_cast<cudaStream_t>(stream));
}

int krk_cuda_gemv_allgather(void *const host_y_peers[], void *const host_flag_peers[], int n_peers, int my_rank,
                            int epoch, int wait_in_kernel, int64_t slice_offset, int64_t n_out_total,
                            const void *x_f32, const void *w, int wt, int64_t n_out_local, int64_t n_in,
                            int64_t rows, void *stream) {
    if (epoch < 0) return KRK_CUDA_EARG;
    if (n_peers < 1 || n_peers > KRK_CUDA_MAX_PEERS || my_rank < 0 || my_rank >= n_peers) return KRK_CUDA_EARG;
    if (!host_y_peers || !host_flag_peers) return KRK_CUDA_ENULL;
    if (slice_offset < 0 || n_out_total < slice_offset + n_out_local) return KRK_CUDA_ESHAPE;
    const int rc = check_matmul_args(host_y_peers[my_rank], x_f32, w, wt, n_out_local, n_in, rows);
    if (rc != KRK_CUDA_OK) return rc;
    if (rows < 1 || rows > KRK_CUDA_MAX_ROWS || n_out_local < 1) return KRK_CUDA_ESHAPE;
    PeerScatter ps;
    for (int q = 0; q < n_peers; q++) {
        if (!host_y_peers[q] || !host_flag_peers[q]) return KRK_CUDA_ENULL;
        ps.y[q] = static_cast<float *>(host_y_peers[q]);
        ps.flag[q] = static_cast<int *>(host_flag_peers[q]);
    }
    ps.n_peers = n_peers;
    ps.my_rank = my_rank;
    ps.epoch = epoch;
    ps.wait_peers = wait_in_kernel != 0;
    ps.row_stride = n_out_total;
    ps.offset = slice_offset;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    GemvMat m;
    m.w = static_cast<const uint8_t *>(w);
    m.x = static_cast<const float *>(x_f32);
    m.y = nullptr;
    m.n_out = n_out_local;
    m.wt = wt;
    const int took = launch_gemv_stream_peers(m, n_in, (int)rows, ps, static_cast<cudaStream_t>(stream));
    if (took < 0) return took;
    return took == 1 ? KRK_CUDA_OK : KRK_CUDA_ESHAPE;
}

int krk_cuda_embed(void *out_f32, const void *tok_embd, int wt, int64_t n_vocab, int64_t n_embd,
                   const void *tokens_i32, int64_t n_tok, void *stream) {
    if (!krk_cuda_dtype_ok(wt)) return KRK_CUDA_EDTYPE;
    if (n_vocab < 0 || n_embd < 0 || n_tok < 0 || n_embd % block_size(wt) != 0) return KRK_CUDA_ESHAPE;
    if (n_tok * n_embd == 0) return KRK_CUDA_OK;
    if (!out_f32 || !tok_embd || !tokens_i32) return KRK_CUDA_ENULL;
    if (!aligned(out_f32, 4) || !aligned(tokens_i32, 4)) return KRK_CUDA_EALIGN;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_embed(static_cast<float *>(out_f32), static_cast<const uint8_t *>(tok_embd), wt, n_vocab, n_embd,
                        static_cast<const int32_t *>(tokens_i32), n_tok, static_cast<cudaStream_t>(stream));
}

size_t krk_cuda_logits_topk_workspace_bytes(int64_t n, int k) {
    if (n < 1 || k < 1 || k > 64) return 0;
    return logits_topk_workspace_bytes(n, k);
}

int krk_cuda_logits_topk(const void *logits_f32, int64_t n, int k, const void *pen_mask_u32, float rep_pen,
                         float softcap, float temp, void *ids_i32, void *vals_f32, void *mass_f32,
                         void *workspace, size_t ws_bytes, void *stream) {
    if (n < 1) return KRK_CUDA_ESHAPE;
    if (k < 1 || k > 64) return KRK_CUDA_EARG;
    if (!logits_f32 || !ids_i32 || !vals_f32) return KRK_CUDA_ENULL;
    if (!workspace || ws_bytes < logits_topk_workspace_bytes(n, k) || !aligned(workspace, 16)) return KRK_CUDA_EWORKSPACE;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_logits_topk(static_cast<const float *>(logits_f32), n, k, static_cast<const uint32_t *>(pen_mask_u32),
                              rep_pen, softcap, temp, static_cast<int32_t *>(ids_i32), static_cast<float *>(vals_f32),
                              static_cast<float *>(mass_f32), workspace, static_cast<cudaStream_t>(stream));
}

int krk_cuda_allgather_sum(void *const host_gather_peers[], void *const host_flag_peers[], int n_peers, int my_rank,
                           int64_t slot_stride, const void *part_f32, void *out_f32, int64_t n, void *stream) {
    if (n_peers < 1 || n_peers > KRK_CUDA_MAX_PEERS || my_rank < 0 || my_rank >= n_peers) return KRK_CUDA_EARG;
    if (!host_gather_peers || !host_flag_peers) return KRK_CUDA_ENULL;
    if (n < 0 || n % 4 != 0 || slot_stride < n || slot_stride % 4 != 0) return KRK_CUDA_ESHAPE;
    if (n > 0 && (!part_f32 || !out_f32)) return KRK_CUDA_ENULL;
    if ((reinterpret_cast<uintptr_t>(part_f32) | reinterpret_cast<uintptr_t>(out_f32)) & 15) return KRK_CUDA_EALIGN;
    float *gather[KRK_CUDA_MAX_PEERS];
    int *flag[KRK_CUDA_MAX_PEERS];
    for (int q = 0; q < n_peers; q++) {
        if (!host_gather_peers[q] || !host_flag_peers[q]) return KRK_CUDA_ENULL;
        if (reinterpret_cast<uintptr_t>(host_gather_peers[q]) & 15) return KRK_CUDA_EALIGN;
        gather[q] = static_cast<float *>(host_gather_peers[q]);
        flag[q] = static_cast<int *>(host_flag_peers[q]);
    }
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_allgather_sum(gather, flag, n_peers, my_rank, slot_stride, static_cast<const float *>(part_f32),
                                static_cast<float *>(out_f32), n, static_cast<cudaStream_t>(stream));
}

int krk_cuda_peer_alloc(void **dev_ptr, size_t bytes, unsigned char handle[KRK_CUDA_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == KRK_CUDA_IPC_HANDLE_BYTES, "handle size");
    if (!dev_ptr || !handle) return KRK_CUDA_ENULL;
    if (bytes == 0) return KRK_CUDA_EARG;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        if (p) cudaFree(p);
        return KRK_CUDA_ELAUNCH;
    }
    memcpy(handle, &h, sizeof h);
    *dev_ptr = p;
    return KRK_CUDA_OK;
}

int krk_cuda_peer_open(void **dev_ptr, const unsigned char handle[KRK_CUDA_IPC_HANDLE_BYTES]) {
    if (!dev_ptr || !handle) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    int me = 0;
    cudaGetDevice(&me);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return KRK_CUDA_ELAUNCH;
    }
    // Make sure that kernels of THIS device can store there before anyone launches one.
    cudaPointerAttributes attr;
    e = cudaPointerGetAttributes(&attr, p);
    if (e == cudaSuccess && attr.device != me) {
        int can = 0;
        e = cudaDeviceCanAccessPeer(&can, me, attr.device);
        if (e == cudaSuccess && !can) {
            cudaIpcCloseMemHandle(p);
            return KRK_CUDA_EDEVICE;
        }
        if (e == cudaSuccess) {
            e = cudaDeviceEnablePeerAccess(attr.device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) {
                cudaGetLastError();
                e = cudaSuccess;
            }
        }
    }
    if (e != cudaSuccess) {
        note_cuda_error(e);
        cudaIpcCloseMemHandle(p);
        return KRK_CUDA_ELAUNCH;
    }
    *dev_ptr = p;
    return KRK_CUDA_OK;
}

int krk_cuda_peer_close(void *dev_ptr) {
    if (!dev_ptr) return KRK_CUDA_ENULL;
    const cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return KRK_CUDA_ELAUNCH;
    }
    return KRK_CUDA_OK;
}

int krk_cuda_peer_free(void *dev_ptr) {
    if (!dev_ptr) return KRK_CUDA_ENULL;
    const cudaError_t e = cudaFree(dev_ptr);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return KRK_CUDA_ELAUNCH;
    }
    return KRK_CUDA_OK;
}

int krk_cuda_wait_flags(const void *flags_i32, int n_peers, int epoch, void *stream) {
    if (n_peers < 1 || n_peers > KRK_CUDA_MAX_PEERS) return KRK_CUDA_EARG;
    if (!flags_i32) return KRK_CUDA_ENULL;
    if (!device_state()) return KRK_CUDA_EDEVICE;
    return launch_flag_wait(static_cast<const int *>(flags_i32), n_peers, epoch, static_cast<cudaStream_t>(stream));
}

int krk_cuda_device_status(void) {
    int *p = device_status_word();
    if (!p) return KRK_CUDA_EDEVICE;
    int v = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return KRK_CUDA_ELAUNCH;
    }
    if (v != 0) cudaMemset(p, 0, sizeof(int));
    return v;
}

int64_t krk_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
int64_t krk_cuda_family_count(int family) {
    return (family > 0 && family < 4) ? g_family[family].load(std::memory_order_relaxed) : 0;
}

} // extern "C"
