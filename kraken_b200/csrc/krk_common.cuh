// Shared declarations of the sm_100a backend: error plumbing, block geometry and the
// bit-exact element decoders every kernel family builds on.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "krk_cuda.h"

namespace krk_cuda {

// ---- host-side plumbing ------------------------------------------------------------

void note_cuda_error(cudaError_t e);   // remembers the text for krk_cuda_last_cuda_error()
void note_launch(int n = 1, int family = 0);   // counts kernels for krk_cuda_launch_count() / _family_count()
int *device_status_word();             // per-device int in global memory, 0 unless a wait gave up
int sm_count();                        // multiprocessors of the current device

inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return KRK_CUDA_ELAUNCH;
    }
    return KRK_CUDA_OK;
}

// exp of an f32 the way the host computes it: the host's expf (the reference's std::exp on a float,
// src/engine.cpp:11704-11713, src/backend_cpu.cpp:2394-2400) is the correctly rounded result in all
// but a fraction of a percent of its arguments; the device's own expf is only good to a unit in the
// last place. Going through double gives the correctly rounded f32 here too, so that probabilities
// ranked on the device collide and order exactly as they do on the host.
__device__ __forceinline__ float exp_as_host(float x) { return (float)exp((double)x); }

// ---- geometry (src/quant.cpp:1805-1900) ----------------------------------------------

__host__ __device__ constexpr int block_size(int wt) {
    return (wt == KRK_CUDA_Q8_0 || wt == KRK_CUDA_Q4_0 || wt == KRK_CUDA_Q5_0 || wt == KRK_CUDA_Q5_1 || wt == KRK_CUDA_IQ4_NL) ? 32
           : (wt == KRK_CUDA_Q4_K || wt == KRK_CUDA_Q6_K || wt == KRK_CUDA_Q5_K || wt == KRK_CUDA_Q2_K || wt == KRK_CUDA_Q3_K) ? 256 : 0;
}
__host__ __device__ constexpr int block_bytes(int wt) {
    return wt == KRK_CUDA_Q8_0 ? 34 : wt == KRK_CUDA_Q4_0 ? 18 : wt == KRK_CUDA_Q4_K ? 144
           : wt == KRK_CUDA_Q6_K ? 210 : wt == KRK_CUDA_Q5_0 ? 22 : wt == KRK_CUDA_Q5_1 ? 24
           : wt == KRK_CUDA_Q5_K ? 176 : wt == KRK_CUDA_Q2_K ? 84 : wt == KRK_CUDA_Q3_K ? 110
           : wt == KRK_CUDA_IQ4_NL ? 18 : 0;
}
__host__ __device__ inline size_t row_bytes(int wt, int64_t n_in) {
    const int bs = block_size(wt);
    return bs ? (size_t)((n_in + bs - 1) / bs) * (size_t)block_bytes(wt) : 0;
}

// ---- bit-exact element decode ----------------------------------------------------------
// Every product is rounded on its own (__fmul_rn / __fsub_rn): nvcc would otherwise
// contract a*b-c into one fused operation and the result would differ from the host
// decoders in the last bit.

__device__ __forceinline__ float half_bits_to_float(const uint8_t *p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

// The j-th 6-bit scale and min of a Q4_K super-block (src/quant.cpp:427-435).
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *p, int &sc, int &mn) {
    if (j < 4) {
        sc = p[j] & 63;
        mn = p[j + 4] & 63;
    } else {
        sc = (p[j + 4] & 0xF) | ((p[j - 4] >> 6) << 4);
        mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4);
    }
}

// Value k of a weight row, exactly as the host decoder of that format produces it.
template <int WT>
__device__ __forceinline__ float decode_value(const uint8_t *row, int64_t k);

// src/quant.cpp:381-387
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q8_0>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 5) * 34;
    return __fmul_rn(half_bits_to_float(b), (float)(int8_t)b[2 + (k & 31)]);
}

// src/quant.cpp:331-339
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q4_0>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 5) * 18;
    const int j = (int)(k & 31);
    const int q = j < 16 ? (b[2 + j] & 0xF) : (b[2 + j - 16] >> 4);
    return __fmul_rn(half_bits_to_float(b), (float)(q - 8));
}

// src/quant.cpp:437-460
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q4_K>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 8) * 144;
    const int e = (int)(k & 255), c = e >> 5, l = e & 31;
    const uint8_t byte = b[16 + 32 * (c >> 1) + l];
    const int q = (c & 1) ? (byte >> 4) : (byte & 0xF);
    int sc, mn;
    scale_min_k4(c, b + 4, sc, mn);
    const float dl = __fmul_rn(half_bits_to_float(b), (float)sc);
    const float ml = __fmul_rn(half_bits_to_float(b + 2), (float)mn);
    return __fsub_rn(__fmul_rn(dl, (float)q), ml);
}

// src/quant.cpp:491-512
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q6_K>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 8) * 210;
    const int e = (int)(k & 255), half = e >> 7, r = e & 127, quad = r >> 5, l = r & 31;
    const uint8_t *ql = b + 64 * half + ((quad & 1) ? 32 : 0);
    const uint8_t qh = b[128 + 32 * half + l];
    const int lo = (quad & 2) ? (ql[l] >> 4) : (ql[l] & 0xF);
    const int q = lo | (((qh >> (2 * quad)) & 3) << 4);
    const int sc = (int8_t)b[192 + 8 * half + 2 * quad + (l >> 4)];
    return __fmul_rn(__fmul_rn(half_bits_to_float(b + 208), (float)sc), (float)(q - 32));
}

// src/quant.cpp:352-364: 4 low bits in the nibbles, the fifth in the 32-bit mask after the scale
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q5_0>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 5) * 22;
    const int j = (int)(k & 31);
    const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
    const int lo4 = j < 16 ? (b[6 + j] & 0xF) : (b[6 + j - 16] >> 4);
    const int q = lo4 | (int)(((qh >> j) & 1u) << 4);
    return __fmul_rn(half_bits_to_float(b), (float)(q - 16));
}

// src/quant.cpp:366-379: as Q5_0 with an unsigned quant and a per-block offset m: d * q + m
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q5_1>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 5) * 24;
    const int j = (int)(k & 31);
    const uint32_t qh = (uint32_t)b[4] | ((uint32_t)b[5] << 8) | ((uint32_t)b[6] << 16) | ((uint32_t)b[7] << 24);
    const int lo4 = j < 16 ? (b[8 + j] & 0xF) : (b[8 + j - 16] >> 4);
    const int q = lo4 | (int)(((qh >> j) & 1u) << 4);
    return __fadd_rn(__fmul_rn(half_bits_to_float(b), (float)q), half_bits_to_float(b + 2));
}

// src/quant.cpp:462-489: Q4_K's scales and mins, a fifth quant bit per value in 32 bytes of masks
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q5_K>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 8) * 176;
    const int e = (int)(k & 255), c = e >> 5, l = e & 31;
    const uint8_t byte = b[48 + 32 * (c >> 1) + l];
    const int q = ((c & 1) ? (byte >> 4) : (byte & 0xF)) + (((b[16 + l] >> c) & 1) ? 16 : 0);
    int sc, mn;
    scale_min_k4(c, b + 4, sc, mn);
    const float dl = __fmul_rn(half_bits_to_float(b), (float)sc);
    const float ml = __fmul_rn(half_bits_to_float(b + 2), (float)mn);
    return __fsub_rn(__fmul_rn(dl, (float)q), ml);
}

// src/quant.cpp:398-424: 16 scale bytes (scale low nibble, min high nibble), 64 bytes of 2-bit quants, d, dmin
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q2_K>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 8) * 84;
    const int e = (int)(k & 255), g = e >> 7, r = e & 127, j = r >> 5, l = r & 31;
    const uint8_t sc = b[8 * g + 2 * j + (l >> 4)];
    const int q = (b[16 + 32 * g + l] >> (2 * j)) & 3;
    const float dl = __fmul_rn(half_bits_to_float(b + 80), (float)(sc & 0xF));
    const float ml = __fmul_rn(half_bits_to_float(b + 82), (float)(sc >> 4));
    return __fsub_rn(__fmul_rn(dl, (float)q), ml);
}

// src/quant.cpp:514-553: 32 mask bytes, 64 bytes of 2-bit quants, sixteen 6-bit scales in 12 bytes, d
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_Q3_K>(const uint8_t *row, int64_t k) {
    const uint8_t *b = row + (k >> 8) * 110;
    const int e = (int)(k & 255), nn = e >> 7, r = e & 127, j = r >> 5, l = r & 31;
    const int is = 8 * nn + 2 * j + (l >> 4);
    const uint8_t *sr = b + 96;
    const int lo = is < 8 ? (sr[is] & 0xF) : (sr[is - 8] >> 4);
    const int hi = (sr[8 + (is & 3)] >> (2 * (is >> 2))) & 3;
    const int scale = (lo | (hi << 4)) - 32;
    const int q = (int)((b[32 + 32 * nn + l] >> (2 * j)) & 3) - ((b[l] >> (4 * nn + j)) & 1 ? 0 : 4);
    return __fmul_rn(__fmul_rn(half_bits_to_float(b + 108), (float)scale), (float)q);
}

// src/quant.cpp:88-91, 566-575: d and 16 bytes of indices into the format's non-linear grid
template <>
__device__ __forceinline__ float decode_value<KRK_CUDA_IQ4_NL>(const uint8_t *row, int64_t k) {
    // the sixteen grid values, packed four to a word (signed bytes)
    constexpr uint32_t grid[4] = {0xBFAD9881u, 0xF6EADDCFu, 0x26190D01u, 0x71594535u};
    const uint8_t *b = row + (k >> 5) * 18;
    const int j = (int)(k & 31);
    const int idx = j < 16 ? (b[2 + j] & 0xF) : (b[2 + j - 16] >> 4);
    const int v = (int)(int8_t)((grid[idx >> 2] >> (8 * (idx & 3))) & 0xFF);
    return __fmul_rn(half_bits_to_float(b), (float)v);
}

// Runs the statement(s) with `WT` bound to the compile-time weight type matching `wt`
// (kernels are specialised per format; there is no runtime type switch on the device).
#define KRK_DISPATCH_WT(wt, ...)                                                        \
    switch (wt) {                                                                       \
    case KRK_CUDA_Q8_0: { constexpr int WT = KRK_CUDA_Q8_0; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q4_0: { constexpr int WT = KRK_CUDA_Q4_0; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q4_K: { constexpr int WT = KRK_CUDA_Q4_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q6_K: { constexpr int WT = KRK_CUDA_Q6_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q5_0: { constexpr int WT = KRK_CUDA_Q5_0; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q5_1: { constexpr int WT = KRK_CUDA_Q5_1; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q5_K: { constexpr int WT = KRK_CUDA_Q5_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q2_K: { constexpr int WT = KRK_CUDA_Q2_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q3_K: { constexpr int WT = KRK_CUDA_Q3_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_IQ4_NL: { constexpr int WT = KRK_CUDA_IQ4_NL; __VA_ARGS__; } break;   \
    default: break;                                                                     \
    }

// The formats the tensor-core GEMM stages: every one whose 256-value segment is a whole number of 8-byte
// granules (Q2_K's 84 and Q3_K's 110 bytes are not: those take the row-batch rung).
#define KRK_DISPATCH_WT_GEMM(wt, ...)                                                   \
    switch (wt) {                                                                       \
    case KRK_CUDA_Q8_0: { constexpr int WT = KRK_CUDA_Q8_0; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q4_0: { constexpr int WT = KRK_CUDA_Q4_0; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q4_K: { constexpr int WT = KRK_CUDA_Q4_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q6_K: { constexpr int WT = KRK_CUDA_Q6_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q5_0: { constexpr int WT = KRK_CUDA_Q5_0; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q5_1: { constexpr int WT = KRK_CUDA_Q5_1; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q5_K: { constexpr int WT = KRK_CUDA_Q5_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_IQ4_NL: { constexpr int WT = KRK_CUDA_IQ4_NL; __VA_ARGS__; } break;   \
    case KRK_CUDA_Q2_K: { constexpr int WT = KRK_CUDA_Q2_K; __VA_ARGS__; } break;       \
    case KRK_CUDA_Q3_K: { constexpr int WT = KRK_CUDA_Q3_K; __VA_ARGS__; } break;       \
    default: break;                                                                     \
    }
// (every format this library decodes has a tensor-core prefill arm; the row-batch rung remains for K % 256 != 0)
__host__ __device__ constexpr bool gemm_tc_takes(int wt) { return block_size(wt) != 0; }

// ---- kernel-family entry points (one .cu file each) -------------------------------------

int launch_dequant_rows(float *out, const uint8_t *w, int wt, int64_t n_rows, int64_t n_in,
                        cudaStream_t st);

// One GEMV of a grouped launch.
struct GemvMat {
    const uint8_t *w;
    const float *x;   // [rows][n_in]
    float *y;         // [rows][n_out]
    int64_t n_out;
    int wt;
};

// A list of single-row GEMVs in device memory, for launches whose matrices are chosen on the device
// (the routed experts). Entries are matrices, or gate/up pairs (2 matrices per entry); gran_begin is
// the running count of row granules (see stream_gran) before each entry.
constexpr int kStreamTableEntries = 64;
struct StreamTable {
    GemvMat mat[2 * kStreamTableEntries];
    int gran_begin[kStreamTableEntries + 1];
    int n_entries;
    int total_gran;
};

// Reference-shaped kernel (one warp per output row): takes every legal shape.
int launch_gemv_generic(const GemvMat *mats, int n_mat, int64_t n_in, int rows, int accumulate,
                        int silu_pair, cudaStream_t st);
// Streaming kernel (bulk-async ring + integer tensor-core dot). Returns 1 when it took
// the launch, 0 when the shape is outside what it addresses (nothing launched), < 0 on error.
int launch_gemv_stream(const GemvMat *mats, int n_mat, int64_t n_in, int rows, int accumulate,
                       int silu_pair, cudaStream_t st);

// Destination of a fused GEMV + all-gather: the full output row in every peer's memory.
struct PeerScatter {
    float *y[KRK_CUDA_MAX_PEERS];    // base of the full [rows][row_stride] output on each GPU (own one included)
    int *flag[KRK_CUDA_MAX_PEERS];   // each GPU's flag array, one int per rank
    int n_peers, my_rank, epoch;     // epoch 0: counted on the device, in flag[my_rank][n_peers]
    int wait_peers;                  // the kernel itself waits for every peer's epoch before it ends
    long long row_stride, offset;    // n_out of the whole head; first row of this shard
};
int launch_gemv_stream_peers(const GemvMat &mat, int64_t n_in, int rows, const PeerScatter &ps, cudaStream_t st);
int launch_flag_wait(const int *flags, int n, int epoch, cudaStream_t st);
// All-gather of this GPU's partial sum into every GPU's gather buffer (peer stores), bounded wait for the
// peers, rank-ordered sum into `out`; one kernel, steps counted on the device. n a multiple of 4.
int launch_allgather_sum(float *const gather[], int *const flag[], int n_peers, int my_rank, int64_t slot_stride,
                         const float *part, float *out, int64_t n, cudaStream_t st);

// The stacked banks the matrices of a table lie in (entry matrix j of a pair lies in bank j; single matrices in
// bank 0), `rows` weight rows each: with them a table launch stages weights with tensor copies out of one map per
// bank instead of one copy per row.
struct StreamBanks {
    const uint8_t *base[2];
    int64_t rows;
};
// Rows per granule the streaming kernel splits matrices of this type and width by (1, 8, or a whole tile when the
// launch will use the banks' tensor maps), or 0 when it does not address the shape (then the shape-agnostic kernels
// serve it).
int stream_gran(int wt, int64_t n_in, bool banks = false);
// The streaming kernel over a device-side table (one activation row per matrix; all matrices of type
// wt and width n_in; built with the granule of stream_gran(wt, n_in, banks != nullptr)). Returns 1 when launched, 0
// when the shape is not addressed, < 0 on error.
int launch_gemv_stream_table(const StreamTable *table, int wt, int64_t n_in, int silu_pair, const StreamBanks *banks,
                             cudaStream_t st);

int launch_silu_mul(float *out, const float *gate, const float *up, int64_t n, cudaStream_t st);
int launch_gather_rows(float *dst, const float *src, const int32_t *rows, int64_t n_rows, int64_t n, cudaStream_t st);
int launch_scatter_axpy_rows(float *dst, const float *src, const int32_t *rows, const float *alpha,
                             int64_t n_rows, int64_t n, cudaStream_t st);
int launch_sum_parts(float *out, const float *parts, int n_parts, int64_t n, cudaStream_t st);
// Embedding gather (decoded rows by token id) and device top-k of a logits row.
int launch_embed(float *out, const uint8_t *table, int wt, int64_t n_vocab, int64_t n_embd, const int32_t *tokens,
                 int64_t n_tok, cudaStream_t st);
size_t logits_topk_workspace_bytes(int64_t n, int k);
int launch_logits_topk(const float *logits, int64_t n, int k, const uint32_t *pen_mask, float rep_pen, float softcap,
                       float temp, int32_t *ids, float *vals, float *mass_out, void *workspace, cudaStream_t st);
int launch_route(int32_t *ids, float *wts, const float *logits, int64_t n_tok, int n_expert, int k,
                 cudaStream_t st);
int launch_router_softmax(float *probs, const float *logits, int64_t n_rows, int n_expert, cudaStream_t st);
int launch_router_topk(const float *probs, int64_t n_rows, int n_expert, int k, int32_t *ids, float *wts, int normalize,
                       float scale, cudaStream_t st);
int launch_moe_plan_build(const int32_t *ids, int64_t n_rows, int k, int n_expert, int32_t *off, int32_t *rows, float *wt,
                          const float *wts, cudaStream_t st);
size_t moe_workspace_bytes(const krk_cuda_expert_bank *bank, int k, int64_t n_tok);
// With `logits` (and n_expert) the routing runs first and ids / wts are outputs.
int launch_moe_ffn_generic(float *y, const float *x, const int32_t *ids, const float *wts,
                           const krk_cuda_expert_bank *bank, int k, int64_t n_tok, void *workspace,
                           cudaStream_t st, const float *logits = nullptr, int n_expert = 0);

// Prefill GEMM on tcgen05 (krk_gemm_tc.cu).
size_t gemm_workspace_bytes(int x_dtype, int64_t n_out, int64_t n_in, int64_t rows);
int launch_gemm_tc(float *y, const void *x, int x_dtype, const uint8_t *w, int wt, int64_t n_out,
                   int64_t n_in, int64_t rows, void *workspace, cudaStream_t st);

} // namespace krk_cuda
