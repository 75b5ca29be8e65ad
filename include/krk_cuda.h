/*
 * krk_cuda.h -- C ABI of the B200 (sm_100a) backend for Kraken's quantized-weight
 * matmul path: GGUF Q8_0 / Q4_0 / Q4_K / Q6_K weights that stay quantized in device
 * memory and are decoded inside the GEMV (decode) and GEMM (prefill) kernels.
 *
 * Conventions (they mirror krk::Backend, include/krk/backend.hpp:337):
 *  - every data pointer is a DEVICE pointer unless the parameter is named host_*;
 *  - weights are the unmodified GGUF bytes, row-major [n_out][krk_cuda_row_bytes()],
 *    16-byte aligned at the base, resident and not written while a call is in flight; a kernel may read the
 *    whole 16-byte granule that holds a matrix's last byte (rows whose size is not a multiple of 16 bytes are
 *    fetched in aligned 16-byte pieces), which device allocations always cover;
 *  - activations and outputs are f32 (the CPU backend's activation type,
 *    src/backend_cpu.cpp:584), except the f16 X of the prefill entry;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the default stream, which is
 *    the reference's only stream, include/krk/backend.hpp:775-779); work is enqueued,
 *    ordered, asynchronous;
 *  - every entry returns 0 or a negative KRK_CUDA_E* code, never aborts or throws,
 *    and has launched nothing when it returns an error (the reference's "false =
 *    nothing launched" rule for optional fused ops, include/krk/backend.hpp:876-881).
 * There is no CPU fallback behind any entry.
 */
#ifndef KRK_CUDA_H
#define KRK_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF on-disk type ids, identical to krk::DType (include/krk/quant.hpp:16-30). */
#define KRK_CUDA_Q4_0 2
#define KRK_CUDA_Q8_0 8
#define KRK_CUDA_Q4_K 12
#define KRK_CUDA_Q6_K 14
/* further GGUF formats a Q4_K_M / Q5_K_M file mixes in: decoded bit-exactly and served by the prefill GEMM and,
 * for decode, by the streaming GEMV (the shape-agnostic GEMV when K is not a multiple of 256) */
#define KRK_CUDA_Q5_0 6
#define KRK_CUDA_Q5_1 7
#define KRK_CUDA_Q5_K 13
/* and the low-bit formats of Q2_K / Q3_K_M / IQ4_NL files (src/quant.cpp:398-424, 514-553, 566-575): bit-exact
 * decode, streaming GEMV, embedding gather, prefill GEMM (raw blocks staged by the decode warps, decoded
 * element by element) */
#define KRK_CUDA_Q2_K 10
#define KRK_CUDA_Q3_K 11
#define KRK_CUDA_IQ4_NL 20

/* Activation types accepted by krk_cuda_gemm. */
#define KRK_CUDA_X_F32 0
#define KRK_CUDA_X_F16 1

#define KRK_CUDA_OK 0
#define KRK_CUDA_EDTYPE (-1)    /* weight type is not one of the four above */
#define KRK_CUDA_ESHAPE (-2)    /* n_in not a whole number of blocks, negative size, rows out of range */
#define KRK_CUDA_ENULL (-3)     /* a required pointer is NULL */
#define KRK_CUDA_EALIGN (-4)    /* weight base or x not 16-byte aligned, or y not 4-byte aligned */
#define KRK_CUDA_ELAUNCH (-5)   /* the CUDA runtime refused the launch or call; see krk_cuda_last_cuda_error() */
#define KRK_CUDA_EWORKSPACE (-6)/* workspace missing or smaller than the _workspace_bytes() answer */
#define KRK_CUDA_EDEVICE (-7)   /* no sm_100 device is current */
#define KRK_CUDA_EARG (-8)      /* any other bad argument (n_mat, k, flags) */
#define KRK_CUDA_ETIMEOUT (-9)  /* a bounded device-side wait gave up; see krk_cuda_device_status() */
#define KRK_CUDA_ETOOBIG (-10)  /* larger than the fixed scratch of krk_cuda_gemm_f32_static */

#define KRK_CUDA_MAX_GROUP 16   /* matrices per grouped launch */
#define KRK_CUDA_MAX_ROWS 8     /* activation rows per GEMV launch */
#define KRK_CUDA_MAX_PEERS 8    /* GPUs of one box a fused GEMV + all-gather writes to */

const char *krk_cuda_strerror(int rc);

/* Text of the last CUDA runtime error seen by this library on this thread ("" if none). */
const char *krk_cuda_last_cuda_error(void);

/* 1 if `wt` is one of the formats above (Q8_0, Q4_0, Q4_K, Q6_K, Q5_0, Q5_1, Q5_K, Q2_K, Q3_K, IQ4_NL). Replaces
 * krk::dtype_supported for this path
 * (include/krk/quant.hpp:180-186). */
int krk_cuda_dtype_ok(int wt);

/* Geometry: replaces dtype_block_size / dtype_block_bytes / dtype_row_bytes
 * (src/quant.cpp:1805-1900). 0 for an unsupported type. */
int krk_cuda_block_size(int wt);
int krk_cuda_block_bytes(int wt);
size_t krk_cuda_row_bytes(int wt, int64_t n_in);

/* Can the GEMV/GEMM address a contraction of k columns of type wt? Replaces
 * Backend::gemm_k_ok (include/krk/backend.hpp:862-869): k > 0 and a whole number of
 * blocks. */
int krk_cuda_gemm_k_ok(int wt, int64_t k);

/* out_f32[n_rows][n_in] = decode(w). Bit-exact with the host decoders deq_q8_0 /
 * deq_q4_0 / deq_q4_k / deq_q6_k (src/quant.cpp:331-339, 381-387, 437-460, 491-512)
 * behind krk::dequant_row (src/quant.cpp:1911-1960). */
int krk_cuda_dequant_rows(void *out_f32, const void *w, int wt, int64_t n_rows, int64_t n_in,
                          void *stream);

/* Decode GEMV: y[rows][n_out] (+)= x[rows][n_in] . W^T for rows in 1..8. Replaces
 * Backend::gemm at rows <= 8 (include/krk/backend.hpp:858-860; HIP ladder
 * src/hip/backend_hip.hip:3203-3237) and, with accumulate != 0, Backend::gemm_accumulate
 * with a null rexp (include/krk/backend.hpp:894-900). y must not alias x. */
int krk_cuda_gemv(void *y_f32, const void *x_f32, const void *w, int wt, int64_t n_out,
                  int64_t n_in, int64_t rows, int accumulate, void *stream);

/* Up to KRK_CUDA_MAX_GROUP independent GEMVs of one activation row each, in one launch.
 * Replaces Backend::gemm_group at rows == 1 (include/krk/backend.hpp:1040-1056;
 * src/hip/kernels/fused.hpp:71-126). x[m] is matrix m's activation (the same pointer
 * may repeat: the `x` form; distinct pointers: the `xs` form). All matrices share n_in.
 * With fuse_silu_pair != 0 matrices (0,1), (2,3), ... are gate/up pairs of equal n_out:
 * y[2i] receives silu(gate) * up; y[2i+1] must still be a valid buffer of n_out floats,
 * whose contents are unspecified afterwards (the `silu` fold,
 * src/hip/kernels/fused.hpp:142-169; silu as in src/backend_cpu.cpp:2394-2400).
 * The pointer arrays are HOST arrays, read before the call returns. */
int krk_cuda_gemv_group(void *const host_y[], const void *const host_x[],
                        const void *const host_w[], const int host_wt[],
                        const int64_t host_n_out[], int64_t n_in, int n_mat,
                        int fuse_silu_pair, void *stream);

/* Prefill GEMM on the tensor cores: y[rows][n_out] = x[rows][n_in] . W^T, W decoded to
 * f16 tiles in shared memory, f32 accumulation. Replaces Backend::gemm at rows > 8
 * (src/hip/backend_hip.hip:3284-3325 -> src/hip/kernels/gemm.hpp:621-970). x is f16
 * (KRK_CUDA_X_F16) or f32 (KRK_CUDA_X_F32, converted to f16 into the workspace first).
 * n_in must be a multiple of 256. */
size_t krk_cuda_gemm_workspace_bytes(int x_dtype, int64_t n_out, int64_t n_in, int64_t rows);
int krk_cuda_gemm(void *y_f32, const void *x, int x_dtype, const void *w, int wt, int64_t n_out,
                  int64_t n_in, int64_t rows, void *workspace, size_t ws_bytes, void *stream);

/* The f32-activation prefill GEMM for hosts that must not allocate: no counterpart in the reference.
 * Same result as krk_cuda_gemm(..., KRK_CUDA_X_F32, ...), but the f16 copy of X goes to a fixed 8 MiB
 * array inside the library's device image instead of a caller workspace, and the call performs no
 * device allocation of any kind (krk_cuda_gemm itself allocates a 4-byte status word per device on first
 * use). Meant for an engine that has committed all device memory at load time, or that cannot accept
 * the implicit device-wide synchronisation of an allocation between decode steps.
 *  - Limit: rows * n_in <= 4,194,304 values (e.g. 1024 x 4096); beyond it the call returns
 *    KRK_CUDA_ETOOBIG and launches nothing.
 *  - The first call on each device looks up the array's device address (with that device current);
 *    make that first call outside any stream capture.
 *  - Every device that loads the library carries the 8 MiB until the process exits.
 *  - All calls on one device share the array: a call rewrites the part it uses before reading it, so
 *    back-to-back calls on one stream are fine, but two calls whose kernels can overlap on the GPU
 *    (different streams) race on it. A bounded-wait give-up of this entry's kernels is recorded in a
 *    word of that array, not in krk_cuda_device_status(): krk_cuda_gemm_f32_static_status() reads it. */
int krk_cuda_gemm_f32_static(void *y_f32, const void *x_f32, const void *w, int wt, int64_t n_out,
                             int64_t n_in, int64_t rows, void *stream);

/* Companion of krk_cuda_gemm_f32_static (no counterpart in the reference): 0, or the KRK_CUDA_ETIMEOUT-class
 * code a kernel of that entry left in the array's status word on the current device; a non-zero word is
 * cleared by the read. Synchronises the device; copies four bytes through the symbol and allocates nothing. */
int krk_cuda_gemm_f32_static_status(void);

/* Router on the device: softmax over n_expert logits per token, k picks of the largest
 * probability (ties to the lower id), weights renormalised over the picks. Replaces the
 * host routing of Engine::moe_ffn (src/engine.cpp:11704-11713, 11853-11920) and
 * Backend::router_softmax / router_topk (include/krk/backend.hpp:934-975).
 * ids_i32 and wts_f32 are [n_tok][k]. */
int krk_cuda_route(void *ids_i32, void *wts_f32, const void *logits_f32, int64_t n_tok,
                   int n_expert, int k, void *stream);

/* The router in the three steps of the Backend interface, for an engine that drives them one at a time
 * (Engine::moe_ffn with KRK_DEVICE_SOFTMAX / the device plan). All pointers are device memory.
 *  - krk_cuda_router_softmax replaces Backend::router_softmax (include/krk/backend.hpp:934-937): probs_f32
 *    [n_rows][n_expert] = softmax of the logits rows, maximum subtracted, summed in expert order.
 *  - krk_cuda_router_topk replaces Backend::router_topk (include/krk/backend.hpp:950-954): k picks of the
 *    largest probability per row, a tie keeps the lower id; weights are the picked probabilities, divided by
 *    their slot-order sum when normalize != 0, then multiplied by scale.
 *  - krk_cuda_moe_plan_build replaces Backend::moe_plan_build (include/krk/backend.hpp:975-980; device twin
 *    src/hip/kernels/router.hpp:252-289): off_i32[n_expert + 1], rows_i32[n_rows * k] and wt_f32[n_rows * k]
 *    in expert-major order, entries of one expert in (token, slot) order, exactly the host's plan
 *    (src/engine.cpp:12215-12248). wts_f32 may be NULL (then wt_f32 is zero-filled). */
int krk_cuda_router_softmax(void *probs_f32, const void *logits_f32, int64_t n_rows, int n_expert, void *stream);
int krk_cuda_router_topk(const void *probs_f32, int64_t n_rows, int n_expert, int k, void *ids_i32, void *wts_f32,
                         int normalize, float scale, void *stream);
int krk_cuda_moe_plan_build(const void *ids_i32, int64_t n_rows, int k, int n_expert, void *off_i32, void *rows_i32,
                            void *wt_f32, const void *wts_f32, void *stream);

/* One bank of routed experts held by this device: expert e (global id) is held when
 * expert_base <= e < expert_base + n_local; its matrices are the e-expert_base'th
 * [n_ff][row_bytes(n_embd)] / [n_embd][row_bytes(n_ff)] slices of gate/up/down. */
struct krk_cuda_expert_bank {
    const void *gate;   /* [n_local][n_ff][row_bytes(wt_gate_up, n_embd)] */
    const void *up;     /* same shape as gate */
    const void *down;   /* [n_local][n_embd][row_bytes(wt_down, n_ff)] */
    int wt_gate_up;
    int wt_down;
    int n_local;
    int expert_base;
    int64_t n_embd;
    int64_t n_ff;
};

/* Routed-expert FFN: y[t] = sum over the picks of token t that this bank holds, in
 * ascending expert id, of wts * Wdown_e . (silu(Wgate_e x_t) * (Wup_e x_t)); picks held
 * elsewhere contribute nothing (a shard's partial sum). Replaces the per-expert loop /
 * moe_decode_batch / Backend::moe_dispatch (src/engine.cpp:12353-, 10896-11060;
 * include/krk/backend.hpp:1001-1009). ids/wts come from krk_cuda_route.
 * n_tok 1..8 (decode): the streaming GEMV over device-side matrix tables, ids never leave the device.
 * n_tok > 8 (prefill): expert-major, the reference's grouped form (src/engine.cpp:12353-12690; device twin
 * src/hip/kernels/moe_table.hpp:463-534): the plan is built on the device, its per-expert row counts are read
 * back once (this call synchronises the stream once), then per expert gather_rows -> gate / up / down as
 * tensor-core GEMMs (GEMVs for up to 8 rows) -> silu_mul -> scatter_axpy_rows in ascending expert id.
 * workspace: krk_cuda_moe_workspace_bytes() bytes of device memory, 256-byte aligned. */
size_t krk_cuda_moe_workspace_bytes(const struct krk_cuda_expert_bank *bank, int k, int64_t n_tok);
int krk_cuda_moe_ffn(void *y_f32, const void *x_f32, const void *ids_i32, const void *wts_f32,
                     const struct krk_cuda_expert_bank *bank, int k, int64_t n_tok,
                     void *workspace, size_t ws_bytes, void *stream);

/* The same with the routing folded in (krk_cuda_route + krk_cuda_moe_ffn in one call, one kernel fewer on
 * the streaming path): router_logits_f32 is [n_tok][n_expert] over ALL experts of the layer; ids_i32 and
 * wts_f32 ([n_tok][k], device memory) are OUTPUTS and hold what krk_cuda_route would have written.
 * Replaces the same reference code as the two calls it combines. */
int krk_cuda_moe_ffn_routed(void *y_f32, const void *x_f32, const void *router_logits_f32, int n_expert,
                            void *ids_i32, void *wts_f32, const struct krk_cuda_expert_bank *bank, int k,
                            int64_t n_tok, void *workspace, size_t ws_bytes, void *stream);

/* out = silu(gate) * up elementwise (Backend::silu_mul, include/krk/backend.hpp:1309;
 * src/backend_cpu.cpp:2394-2400). */
int krk_cuda_silu_mul(void *out_f32, const void *gate_f32, const void *up_f32, int64_t n,
                      void *stream);

/* dst[i] = src[rows[i]] over rows of n floats (Backend::gather_rows, include/krk/backend.hpp:1451):
 * the permute that puts the tokens of one expert into a contiguous block. rows: n_rows device i32;
 * dst must not overlap src. */
int krk_cuda_gather_rows(void *dst_f32, const void *src_f32, const void *rows_i32, int64_t n_rows,
                         int64_t n, void *stream);

/* dst[rows[i]] += alpha[i] * src[i] over rows of n floats (Backend::scatter_axpy_rows,
 * include/krk/backend.hpp:1473; src/backend_cpu.cpp:3193-3220). Row indices must be
 * distinct within one call. */
int krk_cuda_scatter_axpy_rows(void *dst_f32, const void *src_f32, const void *rows_i32,
                               const void *alpha_f32, int64_t n_rows, int64_t n, void *stream);

/* Sum n_parts partial outputs [n_parts][n] in part order 0..n_parts-1 into out[n]: the
 * deterministic combine of expert-sharded partial sums after they were gathered. */
int krk_cuda_sum_parts(void *out_f32, const void *parts_f32, int n_parts, int64_t n, void *stream);

/* Row-sharded GEMV fused with its all-gather over NVLink (the reference is single-device, so this has no
 * counterpart there). This GPU holds rows [slice_offset, slice_offset + n_out_local) of a head of
 * n_out_total rows; the kernel's epilogue stores its slice of y straight into the
 * [rows][n_out_total] row of EVERY GPU: host_y_peers[q] is that buffer on GPU q as mapped into this
 * process by krk_cuda_peer_open (this GPU's own buffer at q == my_rank). When all CTAs have stored, the
 * kernel writes the step's epoch into host_flag_peers[q][my_rank] on every GPU. Loads never touch peer
 * memory; only plain stores do.
 *   epoch > 0: the host counts steps (strictly increasing, the same on every GPU).
 *   epoch == 0: the step count lives on the device, in host_flag_peers[my_rank][n_peers]; the launch
 *     carries no per-step value and can be replayed from a CUDA graph.
 *   Each flag array holds n_peers + 2 ints, zero at start: one epoch per peer, the step count, and the
 *   kernel's count of CTAs that have stored (so every exchange object has its own; objects that share a
 *   flag array must not run at the same time).
 *   wait_in_kernel != 0: the last CTA also waits (bounded, about 2 s, then krk_cuda_device_status() is
 *     raised) until every peer's epoch has arrived here, so the end of the kernel is the end of the
 *     all-gather on this GPU. With 0 the host enqueues krk_cuda_wait_flags where it wants the row.
 * Use two output buffers alternately so that a fast GPU's next step cannot overwrite a row a slow GPU
 * is still reading. Shapes the streaming kernel does not address return KRK_CUDA_ESHAPE. */
int krk_cuda_gemv_allgather(void *const host_y_peers[], void *const host_flag_peers[], int n_peers, int my_rank,
                            int epoch, int wait_in_kernel, int64_t slice_offset, int64_t n_out_total,
                            const void *x_f32, const void *w, int wt, int64_t n_out_local, int64_t n_in,
                            int64_t rows, void *stream);

/* ---- the steps either side of the output head ---- */

/* Replaces Backend::embed (include/krk/backend.hpp:838; src/backend_cpu.cpp:746-778): out_f32[t] = decoded
 * row tokens_i32[t] of the quantized table (row-major [n_vocab][row_bytes]); an id outside [0, n_vocab)
 * gives a zero row. tokens_i32 is device memory. Bit-exact with krk::dequant_row. */
int krk_cuda_embed(void *out_f32, const void *tok_embd, int wt, int64_t n_vocab, int64_t n_embd,
                   const void *tokens_i32, int64_t n_tok, void *stream);

/* Replaces Backend::logits_topk (include/krk/backend.hpp:902-922; src/backend_cpu.cpp:862-912) for f32
 * logits: softcap clamp and repetition penalty (pen_mask_u32: one bit per token id, may be NULL) before
 * ranking; k ids and values in descending order, ties toward the lower id, -1 / -FLT_MAX past the row's
 * length; mass_f32 (may be NULL) = sum over the whole row of exp((key - max) / temp). All pointers are
 * device memory; 1 <= k <= 64. The candidate buffer of the reference is the workspace here. */
size_t krk_cuda_logits_topk_workspace_bytes(int64_t n, int k);
int krk_cuda_logits_topk(const void *logits_f32, int64_t n, int k, const void *pen_mask_u32, float rep_pen,
                         float softcap, float temp, void *ids_i32, void *vals_f32, void *mass_f32,
                         void *workspace, size_t ws_bytes, void *stream);

/* Expert-sharded FFN, exchange step: all-gather of partial sums over NVLink peer stores fused with the
 * rank-ordered sum that follows (no counterpart in the reference, which is single-device). part_f32
 * holds this GPU's partial sum (n floats, n % 4 == 0, 16-byte aligned like out_f32); the kernel stores it
 * into slot my_rank of EVERY GPU's gather buffer, publishes the step to every GPU, waits (bounded, about
 * 2 s, then krk_cuda_device_status() is raised) until every peer's slot has arrived here, and writes
 * out = ((slot 0 + slot 1) + slot 2) + ... : the same bits on every GPU. host_gather_peers[q] is GPU q's
 * gather buffer as mapped into this process (krk_cuda_peer_open; own buffer at q == my_rank), laid out
 * [2][n_peers][slot_stride] floats (two steps deep; slot_stride >= n, % 4 == 0); host_flag_peers[q] is
 * GPU q's flag array of n_peers + 2 ints (epochs, step count, CTA count), zero at start. Steps are counted on the device, so the launch
 * replays from a CUDA graph. Every GPU must make the same sequence of calls. */
int krk_cuda_allgather_sum(void *const host_gather_peers[], void *const host_flag_peers[], int n_peers, int my_rank,
                           int64_t slot_stride, const void *part_f32, void *out_f32, int64_t n, void *stream);

/* Buffers that peers store into. The reference is single-device (src/hip/backend_hip.hip:5036-5043), so
 * these have no counterpart there. krk_cuda_peer_alloc: zero-filled device memory on the current device
 * plus its 64-byte inter-process handle, which the host passes to the other processes of the box by any
 * means. krk_cuda_peer_open maps another process's buffer into this one WITH the current device as the
 * accessor: it enables peer access from the current device to the owner's and refuses
 * (KRK_CUDA_EDEVICE) when the two GPUs cannot reach each other, so that a kernel never meets an
 * unmapped address. close unmaps; free releases an own buffer (after every peer closed it). */
#define KRK_CUDA_IPC_HANDLE_BYTES 64
int krk_cuda_peer_alloc(void **dev_ptr, size_t bytes, unsigned char handle[KRK_CUDA_IPC_HANDLE_BYTES]);
int krk_cuda_peer_open(void **dev_ptr, const unsigned char handle[KRK_CUDA_IPC_HANDLE_BYTES]);
int krk_cuda_peer_close(void *dev_ptr);
int krk_cuda_peer_free(void *dev_ptr);

/* The exchange step over NCCL for a C/C++ host (the reference is single-device: no counterpart there):
 * ncclAllGather of slice_bytes bytes from every rank into full (n_ranks * slice_bytes bytes, rank order), on
 * `stream`; in place when slice == full + rank * slice_bytes. nccl_comm is an ncclComm_t of the host's own
 * (ncclCommInitRank) or one made by krk_cuda_nccl_comm_init below. Follow it with krk_cuda_sum_parts for
 * expert-sharded partial sums. The NCCL library is looked up at run time (libnccl.so.2); KRK_CUDA_EDEVICE when
 * it cannot be found, KRK_CUDA_ELAUNCH (text in krk_cuda_nccl_last_error) when NCCL refuses.
 * krk_cuda_nccl_unique_id / _comm_init / _comm_destroy wrap ncclGetUniqueId / ncclCommInitRank /
 * ncclCommDestroy for hosts that do not link NCCL themselves: rank 0 makes the 128-byte id, every rank passes it
 * (by any channel) to _comm_init with its device current. */
#define KRK_CUDA_NCCL_ID_BYTES 128
int krk_cuda_shard_allgather(void *full, const void *slice, size_t slice_bytes, void *nccl_comm, void *stream);
int krk_cuda_nccl_unique_id(unsigned char id[KRK_CUDA_NCCL_ID_BYTES]);
int krk_cuda_nccl_comm_init(void **comm, int n_ranks, int rank, const unsigned char id[KRK_CUDA_NCCL_ID_BYTES]);
int krk_cuda_nccl_comm_destroy(void *comm);
const char *krk_cuda_nccl_last_error(void);

/* Enqueues a bounded wait until flags_i32[q] >= epoch for every q < n_peers (flags_i32 is this GPU's own
 * flag array). A wait that runs out (about 2 s) raises krk_cuda_device_status() instead of hanging. */
int krk_cuda_wait_flags(const void *flags_i32, int n_peers, int epoch, void *stream);

/* Device-side status word of the current device: 0, or a KRK_CUDA_ETIMEOUT-class code
 * written by a kernel whose bounded wait gave up. Synchronises the device. */
int krk_cuda_device_status(void);

/* Kernels launched by this library since the process started (all threads). */
int64_t krk_cuda_launch_count(void);

/* The same count for one kernel family, so that a caller (or a test) can tell which path
 * served a shape: the streaming GEMV, the shape-agnostic GEMV, or the tensor-core GEMM. */
#define KRK_CUDA_FAMILY_GEMV_STREAM 1
#define KRK_CUDA_FAMILY_GEMV_GENERIC 2
#define KRK_CUDA_FAMILY_GEMM_TC 3
int64_t krk_cuda_family_count(int family);

/* Diagnostic, no counterpart in the reference: cycles between two instructions of one kind on one SM
 * sub-partition, measured with every SM busy. kind: 0 mma.sync m16n8k32 s8, 1 m16n8k16 s8, 2 m16n8k16 f16,
 * 3 m16n8k16 bf16, 4 m16n8k32 e4m3, 5 dp4a, 6 mad.lo.s32, 7 fma.rn.f16x2, 8 lop3, 9 fma.rn.f32,
 * 10 m16n8k8 f16. `warps` per CTA (1..32, one CTA per SM); chained != 0 measures the dependent-issue
 * latency instead of the throughput. Allocates and frees its own buffers and synchronises the device;
 * `bench.py --issue-rates` prints the table the kernel formulations were chosen from. */
int krk_cuda_probe_issue(int kind, int warps, int iters, int chained, double *host_cycles_per_instr);

/* ---- host-buffer plumbing: the CudaBackend class of krk_cuda_backend.hpp behind a C face ----
 * These are the calls a host that is not C++ binds. `be` is the object returned by
 * krk_cuda_backend_make (make_hip_backend's contract, include/krk/backend.hpp:1886: NULL and a
 * message in err on failure). alloc/release/upload/download/fill0/sync replace the members of
 * the same names (include/krk/backend.hpp:361-362, 720, 755, 769, 770); gemm, gemm_accumulate and
 * gemm_group replace include/krk/backend.hpp:858-860, 894-900, 1040-1056 and, like the
 * reference, log and abort on a shape they cannot address (ask gemm_k_ok first). host_* pointers
 * are host memory (pinned memory makes upload asynchronous); all others come from alloc. */
void *krk_cuda_backend_make(int device_index, char *err, size_t err_len);
void krk_cuda_backend_free(void *be);
const char *krk_cuda_backend_describe(void *be);
void *krk_cuda_backend_alloc(void *be, size_t bytes);
void krk_cuda_backend_release(void *be, void *p);
/* off: byte offset into the device side (dst of an upload, src of a download), as Backend::upload / download
 * have it (include/krk/backend.hpp:720, 755; src/backend_cpu.cpp:676-683) */
void krk_cuda_backend_upload(void *be, void *dst, const void *host_src, size_t bytes, size_t off);
void krk_cuda_backend_download(void *be, void *host_dst, const void *src, size_t bytes, size_t off);
void krk_cuda_backend_download_f32(void *be, float *host_dst, const void *src, int64_t n);          /* backend.hpp:803 */
void krk_cuda_backend_upload_i32(void *be, int32_t *dst, const int32_t *host_src, int64_t n);       /* backend.hpp:1505 */
/* the members either side of the matmuls, with the reference's argument lists (include/krk/backend.hpp:838,
 * 902-922, 1309, 1451, 1473, 934-986); host_* are host memory, everything else device memory from alloc */
void krk_cuda_backend_embed(void *be, void *out, const void *tok_embd, int tt, int64_t n_vocab, int64_t n_embd,
                            const int32_t *host_tokens, int64_t n_tok);
void krk_cuda_backend_logits_topk(void *be, const void *logits, int64_t n, int32_t k, const void *pen_mask, float rep_pen,
                                  float softcap, float temp, int32_t *ids, float *vals, float *mass_out, void *scratch,
                                  int32_t cand_cap, int64_t *count_out);
void krk_cuda_backend_silu_mul(void *be, void *out, const void *gate, const void *up, int64_t n, int64_t row_len,
                               float *host_row_scale);
void krk_cuda_backend_gather_rows(void *be, void *dst, const void *src, const int32_t *rows, int64_t n_rows, int64_t n);
void krk_cuda_backend_scatter_axpy_rows(void *be, void *dst, const void *src, const int32_t *rows, const float *alpha,
                                        int64_t n_rows, int64_t n);
void krk_cuda_backend_router_softmax(void *be, void *probs, const void *logits, int64_t n_rows, int32_t n_expert);
void krk_cuda_backend_router_topk(void *be, const void *probs, int64_t n_rows, int32_t n_expert, int32_t k, void *ids,
                                  void *wts, int32_t normalize, float scale);
void krk_cuda_backend_moe_plan_build(void *be, const void *ids, int64_t n_rows, int32_t k, int32_t n_expert, void *off,
                                     void *rows, void *wt, const void *wts);
int krk_cuda_backend_device(void *be);
void krk_cuda_backend_fill0(void *be, void *p, size_t bytes);
void krk_cuda_backend_sync(void *be);
int krk_cuda_backend_gemm_k_ok(void *be, int wt, int64_t k);
void krk_cuda_backend_gemm(void *be, void *out, const void *x, const void *w, int wt, int64_t n_out,
                           int64_t n_in, int64_t rows);
int krk_cuda_backend_gemm_accumulate(void *be, void *dst, const void *x, const void *w, int wt,
                                     int64_t n_out, int64_t n_in, int64_t rows);
int krk_cuda_backend_gemm_group(void *be, void *const out[], const void *x, const void *const w[], int wt,
                                const int64_t n_out[], int64_t n_in, int n_mat, int64_t rows, int silu,
                                int *silu_fused);
/* The same with the two optional arrays of Backend::gemm_group (backend.hpp:1040-1056): wts[m] the weight type of
 * matrix m (NULL: all of type wt) and xs[m] its activation (NULL: all read x), e.g. the routed experts' down
 * projections, which read a different silu row each. Both are HOST arrays. */
int krk_cuda_backend_gemm_group_ex(void *be, void *const out[], const void *x, const void *const w[], int wt,
                                   const int64_t n_out[], int64_t n_in, int n_mat, int64_t rows, int silu,
                                   int *silu_fused, const int wts[], const void *const xs[]);

/* ---- the on-disk format either side of the path: a GGUF v2 / v3 tensor reader ----
 * Replaces krk::Gguf for this path (include/krk/gguf.hpp; src/gguf.cpp): one file, mapped read-only; header,
 * key/value block and tensor directory are parsed, tensor data is never copied or repacked on the host.
 * krk_gguf_open returns NULL and a message in err on a file it cannot read (bad magic, version other than 2 or 3,
 * truncated directory, tensor data past the end of the file). Host-only: no device is touched except by
 * krk_gguf_upload_tensor. */
struct krk_gguf_tensor {
    const char *name;        /* valid until krk_gguf_close */
    int type_id;             /* GGUF type id = krk::DType value */
    int supported;           /* 1 when krk_cuda_dtype_ok(type_id) */
    int n_dims;
    int64_t ne[4];           /* ne[0] = row length (n_in), ne[1] = rows (n_out), as GGUF stores them */
    const void *host_data;   /* the tensor's bytes inside the mapping */
    size_t n_bytes;          /* rows * row_bytes; 0 for a type this library does not size */
};
void *krk_gguf_open(const char *path, char *err, size_t err_len);
void krk_gguf_close(void *gguf);
int krk_gguf_version(void *gguf);
int64_t krk_gguf_tensor_count(void *gguf);
int64_t krk_gguf_kv_count(void *gguf);
int64_t krk_gguf_find_tensor(void *gguf, const char *name);                 /* index, or -1 */
int krk_gguf_tensor_info(void *gguf, int64_t index, struct krk_gguf_tensor *out);
int krk_gguf_get_i64(void *gguf, const char *key, int64_t *out);            /* any integer, bool or float value */
int krk_gguf_get_f64(void *gguf, const char *key, double *out);
int64_t krk_gguf_get_str(void *gguf, const char *key, char *buf, size_t buf_len);   /* length, or -1 */
int64_t krk_gguf_get_array_count(void *gguf, const char *key, int *elem_type);       /* count, or -1 */
/* alloc() on the backend + upload of the tensor's unmodified bytes (Backend::upload, include/krk/backend.hpp:720);
 * the caller releases the pointer with krk_cuda_backend_release. NULL for an unsized type or a failed alloc. */
void *krk_gguf_upload_tensor(void *gguf, int64_t index, void *backend);

#ifdef __cplusplus
}
#endif
#endif
