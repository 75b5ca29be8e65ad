// Router and routed-expert FFN for decode batches (1..8 tokens).
//
// The routing result stays on the device: expert ids are read by the kernels themselves,
// so no logits or ids cross PCIe (the reference downloads the logits and routes on the
// host, src/engine.cpp:11678-11920, or reads device ids in its opt-in moe_dispatch,
// src/hip/kernels/moe_table.hpp:67-180).
#include "krk_chunk.cuh"

namespace krk_cuda {

namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxK = 32;

// The sum of v[0..n) in index order (the order the host adds them in), by a whole warp: each lane fetches one value
// of every 32 and the running sum takes them lane by lane through shuffles, so the chain is 4-cycle additions
// instead of one shared-memory round trip per term. Every lane returns the sum.
__device__ __forceinline__ float ordered_sum(const float *v, int n, int lane) {
    float sum = 0.0f;
    for (int base = 0; base < n; base += 32) {
        const float mine = base + lane < n ? v[base + lane] : 0.0f;
        const int m = min(32, n - base);
#pragma unroll 8
        for (int i = 0; i < m; i++) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, mine, i));
    }
    return sum;
}

// The k largest of prob[0..n) in slot order by one warp: strict '>' so equal values keep the lower index
// (src/engine.cpp:11857-11886). Lane s (s < k) returns slot s's index (-1: none left) and value; `sum` is the sum of
// the picked values in slot order. Up to 128 entries live in registers (four per lane) and a round is two warp
// reductions: the maximum over the bit patterns of the (non-negative) values, then the lowest index among the lanes
// that hold it. More entries take rounds over shared memory (prob is then modified: -2 marks a taken entry).
__device__ __forceinline__ void topk_warp(float *prob, int n, int k, int lane, int &my_id, float &my_w, float &sum) {
    my_id = -1;
    my_w = 0.0f;
    sum = 0.0f;
    if (n <= 128) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = lane + 32 * j < n ? prob[lane + 32 * j] : -2.0f;
        for (int s = 0; s < k; s++) {
            float bp = -1.0f;
            int be = 0x7FFFFFFF;
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (v[j] > bp) {
                    bp = v[j];
                    be = lane + 32 * j;
                }
            const unsigned key = bp >= 0.0f ? __float_as_uint(bp) + 1u : 0u;   // bit patterns of values >= 0 order like the values
            const unsigned top = __reduce_max_sync(0xFFFFFFFFu, key);
            const unsigned win = __reduce_min_sync(0xFFFFFFFFu, (key == top && top != 0u) ? (unsigned)be : 0x7FFFFFFFu);
            const bool ok = top != 0u;
            const float w = ok ? __uint_as_float(top - 1u) : 0.0f;
            sum = __fadd_rn(sum, w);
            if (lane == s) {
                my_id = ok ? (int)win : -1;
                my_w = w;
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (ok && lane + 32 * j == (int)win) v[j] = -2.0f;
        }
        return;
    }
    for (int s = 0; s < k; s++) {
        float bp = -1.0f;
        int be = 0x7FFFFFFF;
        for (int e = lane; e < n; e += 32) {
            const float pe = prob[e];
            if (pe > bp) {
                bp = pe;
                be = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float op = __shfl_xor_sync(0xFFFFFFFFu, bp, o);
            const int oe = __shfl_xor_sync(0xFFFFFFFFu, be, o);
            if (op > bp || (op == bp && oe < be)) {
                bp = op;
                be = oe;
            }
        }
        const bool ok = be < n && bp >= 0.0f;
        const float w = ok ? bp : 0.0f;
        sum = __fadd_rn(sum, w);
        if (lane == s) {
            my_id = ok ? be : -1;
            my_w = w;
        }
        if (ok && lane == 0) prob[be] = -2.0f;
        __syncwarp();
    }
}

// One warp per token. Softmax as the reference computes it: subtract the maximum, sum the
// exponentials in expert order, multiply by the reciprocal (src/engine.cpp:11704-11713);
// then k picks of the largest probability, strict '>' so equal probabilities keep the lower
// id (:11857-11886); then the picked weights are divided by their slot-order sum
// (:11913-11918).
__device__ __forceinline__ void route_token(int32_t *__restrict__ ids, float *__restrict__ wts, const float *__restrict__ lg,
                                            int n_expert, int k, float *prob, int *sid, int lane) {
    float mx = -INFINITY;
    for (int e = lane; e < n_expert; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    for (int e = lane; e < n_expert; e += 32) prob[e] = exp_as_host(__fsub_rn(lg[e], mx));
    __syncwarp();
    const float sum = ordered_sum(prob, n_expert, lane);
    const float inv = sum > 0.0f ? __fdiv_rn(1.0f, sum) : 0.0f;
    for (int e = lane; e < n_expert; e += 32) prob[e] = __fmul_rn(prob[e], inv);
    __syncwarp();

    int my_id;
    float my_w, ksum;
    topk_warp(prob, n_expert, k, lane, my_id, my_w, ksum);
    const float kinv = ksum > 0.0f ? __fdiv_rn(1.0f, ksum) : 0.0f;
    if (lane < k) {
        ids[lane] = my_id;
        wts[lane] = __fmul_rn(my_w, kinv);
        if (sid) sid[lane] = my_id;
    }
}

__global__ void __launch_bounds__(32)
route_kernel(int32_t *__restrict__ ids, float *__restrict__ wts, const float *__restrict__ logits,
             int n_expert, int k) {
    __shared__ float prob[kMaxExperts];
    const int64_t t = blockIdx.x;
    route_token(ids + t * k, wts + t * k, logits + t * n_expert, n_expert, k, prob, nullptr, threadIdx.x);
}

// The router in the three steps Backend exposes (include/krk/backend.hpp:934-986): probabilities,
// selection, expert-major plan. Same arithmetic as route_token, split where the interface splits it.
__global__ void __launch_bounds__(32)
router_softmax_kernel(float *__restrict__ probs, const float *__restrict__ logits, int n_expert) {
    const float *lg = logits + (int64_t)blockIdx.x * n_expert;
    float *pr = probs + (int64_t)blockIdx.x * n_expert;
    const int lane = threadIdx.x;
    float mx = -INFINITY;
    for (int e = lane; e < n_expert; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    for (int e = lane; e < n_expert; e += 32) pr[e] = exp_as_host(__fsub_rn(lg[e], mx));
    __syncwarp();
    const float sum = ordered_sum(pr, n_expert, lane);   // in expert order, as the host adds them
    const float inv = sum > 0.0f ? __fdiv_rn(1.0f, sum) : 0.0f;
    for (int e = lane; e < n_expert; e += 32) pr[e] = __fmul_rn(pr[e], inv);
}

// k picks of the largest probability per row (strict '>': a tie keeps the lower id), weights = the picked
// probabilities, divided by their slot-order sum when `normalize`, times `scale`.
__global__ void __launch_bounds__(32)
router_topk_kernel(const float *__restrict__ probs, int n_expert, int k, int32_t *__restrict__ ids, float *__restrict__ wts,
                   int normalize, float scale) {
    __shared__ float prob[kMaxExperts];
    const float *pr = probs + (int64_t)blockIdx.x * n_expert;
    const int lane = threadIdx.x;
    for (int e = lane; e < n_expert; e += 32) prob[e] = pr[e];
    __syncwarp();
    int my_id;
    float my_w, ksum;
    topk_warp(prob, n_expert, k, lane, my_id, my_w, ksum);
    const float kinv = normalize ? (ksum > 0.0f ? __fdiv_rn(1.0f, ksum) : 0.0f) : 1.0f;
    if (lane < k) {
        float w = normalize ? __fmul_rn(my_w, kinv) : my_w;
        if (scale != 1.0f) w = __fmul_rn(w, scale);
        ids[(int64_t)blockIdx.x * k + lane] = my_id;
        wts[(int64_t)blockIdx.x * k + lane] = w;
    }
}

// The expert-major plan of a layer from the selected ids: off[n_expert + 1] prefix offsets, rows[n * k] the
// token of each entry and wt[n * k] its weight, entries of one expert in (token, slot) order: the order of the
// host's plan (src/engine.cpp:12215-12248; device twin src/hip/kernels/router.hpp:252-289). Thread e walks
// the pairs in order for expert e, so the order is prescribed, not left to scheduling. One block.
__global__ void __launch_bounds__(1024)
moe_plan_build_kernel(const int32_t *__restrict__ ids, int n_rows, int k, int n_expert, int32_t *__restrict__ off,
                      int32_t *__restrict__ rows, float *__restrict__ wt, const float *__restrict__ wts) {
    __shared__ int count[kMaxExperts + 1];
    const int nk = n_rows * k;
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
        int c = 0;
        for (int i = 0; i < nk; i++) c += ids[i] == e;
        count[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_expert; e++) {
            const int c = count[e];
            count[e] = run;
            off[e] = run;
            run += c;
        }
        off[n_expert] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
        int at = count[e];
        for (int i = 0; i < nk; i++)
            if (ids[i] == e) {
                rows[at] = i / k;
                wt[at] = wts ? wts[i] : 0.0f;
                at++;
            }
    }
}

struct MoeParams {
    const uint8_t *gate, *up, *down;
    const float *x;        // [n_tok][n_embd]
    const int32_t *ids;    // [n_tok][k]
    const float *wts;      // [n_tok][k]
    float *h;              // [n_tok*k][n_ff]   silu(gate) * up per pick
    float *d;              // [n_tok*k][n_embd] down projection per pick
    float *y;              // [n_tok][n_embd]
    int64_t n_embd, n_ff;
    int n_local, expert_base, k, n_tok;
};

__device__ __forceinline__ int local_expert(const MoeParams &p, int pick) {
    const int e = p.ids[pick] - p.expert_base;
    return (e >= 0 && e < p.n_local) ? e : -1;
}

// h[pick][row] = silu(Wgate_e[row] . x_t) * (Wup_e[row] . x_t); one warp per (pick, row).
template <int WT>
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(const __grid_constant__ MoeParams p) {
    const int pick = blockIdx.y;
    const int e = local_expert(p, pick);
    if (e < 0) return;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= p.n_ff) return;
    const size_t rb = row_bytes(WT, p.n_embd);
    const uint8_t *g = p.gate + ((size_t)e * p.n_ff + row) * rb;
    const uint8_t *u = p.up + ((size_t)e * p.n_ff + row) * rb;
    const float *x = p.x + (int64_t)(pick / p.k) * p.n_embd;
    float sg = 0.0f, su = 0.0f;
    for (int64_t c = lane; c < (p.n_embd >> 5); c += 32) {
        sg += chunk_dot<WT>(g, c, x);
        su += chunk_dot<WT>(u, c, x);
    }
    sg = warp_sum(sg);
    su = warp_sum(su);
    if (lane == 0)
        p.h[(int64_t)pick * p.n_ff + row] = __fmul_rn(__fdiv_rn(sg, __fadd_rn(1.0f, exp_as_host(-sg))), su);
}

// d[pick][row] = Wdown_e[row] . h[pick]
template <int WT>
__global__ void __launch_bounds__(256)
moe_down_kernel(const __grid_constant__ MoeParams p) {
    const int pick = blockIdx.y;
    const int e = local_expert(p, pick);
    if (e < 0) return;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= p.n_embd) return;
    const uint8_t *w = p.down + ((size_t)e * p.n_embd + row) * row_bytes(WT, p.n_ff);
    const float *h = p.h + (int64_t)pick * p.n_ff;
    float s = 0.0f;
    for (int64_t c = lane; c < (p.n_ff >> 5); c += 32) s += chunk_dot<WT>(w, c, h);
    s = warp_sum(s);
    if (lane == 0) p.d[(int64_t)pick * p.n_embd + row] = s;
}

// y[t][j] = sum over the picks of token t held here, ascending expert id, of w * d[pick][j]
// starting from zero: the order and the arithmetic of the reference's per-expert
// scatter_axpy_rows chain (src/engine.cpp:12353-, src/backend_cpu.cpp:3193-3220).
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __grid_constant__ MoeParams p) {
    __shared__ int s_pick[kMaxK];
    __shared__ float s_w[kMaxK];
    __shared__ int s_n;
    // programmatic dependent launch: this grid may start while the one before it drains (it reads nothing before
    // that grid is complete), and lets the one after it start the same way
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int t = blockIdx.y;
    if (threadIdx.x < 32) {
        // lane s looks at slot s of this token: its place among the slots held here, by expert id
        const int s = threadIdx.x;
        int id = 0x7FFFFFFF, e = -1;
        if (s < p.k) {
            id = p.ids[t * p.k + s];
            e = local_expert(p, t * p.k + s);
        }
        int rank = 0, n = 0;
        for (int j = 0; j < p.k; j++) {
            const int idj = __shfl_sync(0xFFFFFFFFu, id, j), ej = __shfl_sync(0xFFFFFFFFu, e, j);
            if (ej >= 0) {
                n++;
                rank += (idj < id || (idj == id && j < s)) ? 1 : 0;
            }
        }
        if (e >= 0) {
            s_pick[rank] = t * p.k + s;
            s_w[rank] = p.wts[t * p.k + s];
        }
        if (s == 0) s_n = n;
    }
    __syncthreads();
    const int n = s_n;
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < p.n_embd;
         j += (int64_t)gridDim.x * blockDim.x) {
        // the loads of a batch of eight go out together; the additions keep their order
        float acc = 0.0f;
        for (int i0 = 0; i0 < n; i0 += 8) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = i0 + i < n ? p.d[(int64_t)s_pick[i0 + i] * p.n_embd + j] : 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (i0 + i < n) acc = __fadd_rn(acc, __fmul_rn(s_w[i0 + i], v[i]));
        }
        p.y[(int64_t)t * p.n_embd + j] = acc;
    }
}

// Builds the two device-side matrix tables of the streaming path from the routed expert ids: one
// gate/up pair and one down matrix per pick this bank holds, ordered by expert id so that an expert
// picked by several tokens is streamed by neighbouring CTAs at about the same time (its second read
// comes from L2). One block; picks <= kStreamTableEntries.
// With `logits` the routing itself runs first, one warp per token (n_tok <= 8), writing p.ids / p.wts.
constexpr int kPlanThreads = 256;
constexpr int kPlanRouteExperts = 1024;   // experts the fused routing holds in shared memory, per token
__global__ void __launch_bounds__(kPlanThreads)
moe_plan_kernel(const __grid_constant__ MoeParams p, StreamTable *gate_up, StreamTable *down, int wt_gate_up, int wt_down,
                size_t rb_gate_up, size_t rb_down, int gran_gate_up, int gran_down, const float *logits, int n_expert) {
    __shared__ int key[kStreamTableEntries];
    __shared__ float prob[KRK_CUDA_MAX_ROWS][kPlanRouteExperts];
    __shared__ int sid[KRK_CUDA_MAX_ROWS][kMaxK];   // the ids the fused routing picked, for the plan below
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // (see moe_combine_kernel)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (logits) {
        const int t = threadIdx.x >> 5;
        if (t < p.n_tok)
            route_token(const_cast<int32_t *>(p.ids) + t * p.k, const_cast<float *>(p.wts) + t * p.k,
                        logits + (int64_t)t * n_expert, n_expert, p.k, prob[t], sid[t], threadIdx.x & 31);
        __syncthreads();   // the ids written above are read below by other threads of this block
    }
    const int n_pick = p.n_tok * p.k, pick = threadIdx.x;
    int e = -1;
    if (pick < n_pick) {
        // (with the routing fused the ids come out of shared memory, not back from global memory)
        const int id = logits ? sid[pick / p.k][pick % p.k] : p.ids[pick];
        const int le = id - p.expert_base;
        e = (le >= 0 && le < p.n_local) ? le : -1;
    }
    if (pick < kStreamTableEntries) key[pick] = e >= 0 ? e * kStreamTableEntries + pick : 0x7FFFFFFF;
    __syncthreads();
    if (e >= 0) {
        int rank = 0;
        for (int j = 0; j < n_pick; j++) rank += key[j] < key[pick];
        const float *x = p.x + (int64_t)(pick / p.k) * p.n_embd;
        float *h = p.h + (int64_t)pick * p.n_ff;
        GemvMat g, u, d;
        g.w = p.gate + (size_t)e * p.n_ff * rb_gate_up;
        u.w = p.up + (size_t)e * p.n_ff * rb_gate_up;
        g.x = u.x = x;
        g.y = u.y = h;            // the pair's fold writes silu(gate) * up through the gate's pointer
        g.n_out = u.n_out = p.n_ff;
        g.wt = u.wt = wt_gate_up;
        d.w = p.down + (size_t)e * p.n_embd * rb_down;
        d.x = h;
        d.y = p.d + (int64_t)pick * p.n_embd;
        d.n_out = p.n_embd;
        d.wt = wt_down;
        gate_up->mat[2 * rank] = g;
        gate_up->mat[2 * rank + 1] = u;
        down->mat[rank] = d;
    }
    if (threadIdx.x == 0) {
        int n = 0;
        for (int j = 0; j < n_pick; j++) n += key[j] != 0x7FFFFFFF;
        const int gu = (int)((p.n_ff + gran_gate_up - 1) / gran_gate_up), dn = (int)((p.n_embd + gran_down - 1) / gran_down);
        for (int i = 0; i <= n; i++) {
            gate_up->gran_begin[i] = i * gu;
            down->gran_begin[i] = i * dn;
        }
        gate_up->n_entries = down->n_entries = n;
        gate_up->total_gran = n * gu;
        down->total_gran = n * dn;
    }
}

// A launch that may overlap the tail of the kernel before it in the stream (the kernel waits for that grid itself).
template <class... KArgs, class... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

} // namespace

int launch_route(int32_t *ids, float *wts, const float *logits, int64_t n_tok, int n_expert, int k,
                 cudaStream_t st) {
    if (n_expert <= 0 || n_expert > kMaxExperts || k <= 0 || k > kMaxK || k > n_expert)
        return KRK_CUDA_EARG;
    if (n_tok == 0) return KRK_CUDA_OK;
    route_kernel<<<(unsigned)n_tok, 32, 0, st>>>(ids, wts, logits, n_expert, k);
    note_launch();
    return check_launch();
}

int launch_router_softmax(float *probs, const float *logits, int64_t n_rows, int n_expert, cudaStream_t st) {
    if (n_expert <= 0 || n_expert > kMaxExperts) return KRK_CUDA_EARG;
    if (n_rows == 0) return KRK_CUDA_OK;
    router_softmax_kernel<<<(unsigned)n_rows, 32, 0, st>>>(probs, logits, n_expert);
    note_launch();
    return check_launch();
}

int launch_router_topk(const float *probs, int64_t n_rows, int n_expert, int k, int32_t *ids, float *wts, int normalize,
                       float scale, cudaStream_t st) {
    if (n_expert <= 0 || n_expert > kMaxExperts || k <= 0 || k > kMaxK || k > n_expert) return KRK_CUDA_EARG;
    if (n_rows == 0) return KRK_CUDA_OK;
    router_topk_kernel<<<(unsigned)n_rows, 32, 0, st>>>(probs, n_expert, k, ids, wts, normalize, scale);
    note_launch();
    return check_launch();
}

int launch_moe_plan_build(const int32_t *ids, int64_t n_rows, int k, int n_expert, int32_t *off, int32_t *rows, float *wt,
                          const float *wts, cudaStream_t st) {
    if (n_expert <= 0 || n_expert > kMaxExperts || k <= 0 || n_rows < 0 || n_rows * k > (1 << 24)) return KRK_CUDA_EARG;
    moe_plan_build_kernel<<<1, n_expert < 1024 ? ((n_expert + 31) / 32) * 32 : 1024, 0, st>>>(ids, (int)n_rows, k, n_expert, off, rows,
                                                                                              wt, wts);
    note_launch();
    return check_launch();
}

static size_t moe_float_bytes(const krk_cuda_expert_bank *bank, int k, int64_t n_tok) {
    const size_t b = sizeof(float) * (size_t)(n_tok * k) * (size_t)(bank->n_ff + bank->n_embd);
    return (b + 255) & ~(size_t)255;
}

// ---- more than eight tokens: expert-major, the tokens of an expert as one matrix (the reference's grouped form,
// src/engine.cpp:12353-12690: gather the expert's rows, gate / up as a GEMM each, silu_mul, down, scatter-add).
struct GroupedLayout {
    size_t off, rows, wt, xg, g, u, dg, gemm, total;
    size_t gemm_bytes;
};
static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
// rung for a [m x n_in] . W^T product by row count: streaming / shape-agnostic GEMV up to 8 rows, tensor cores above
static size_t grouped_gemm_bytes(const krk_cuda_expert_bank *bank, int64_t n_tok) {
    size_t a = 0, b = 0;
    if (bank->n_embd % 256 == 0 && gemm_tc_takes(bank->wt_gate_up)) a = gemm_workspace_bytes(KRK_CUDA_X_F32, bank->n_ff, bank->n_embd, n_tok);
    if (bank->n_ff % 256 == 0 && gemm_tc_takes(bank->wt_down)) b = gemm_workspace_bytes(KRK_CUDA_X_F32, bank->n_embd, bank->n_ff, n_tok);
    return up256(a > b ? a : b);
}
static GroupedLayout grouped_layout(const krk_cuda_expert_bank *bank, int k, int64_t n_tok) {
    GroupedLayout L;
    const size_t picks = (size_t)(n_tok * k);
    size_t at = 0;
    L.off = at; at += up256(sizeof(int32_t) * (kMaxExperts + 1));
    L.rows = at; at += up256(sizeof(int32_t) * picks);
    L.wt = at; at += up256(sizeof(float) * picks);
    L.xg = at; at += up256(sizeof(float) * (size_t)n_tok * bank->n_embd);
    L.g = at; at += up256(sizeof(float) * (size_t)n_tok * bank->n_ff);
    L.u = at; at += up256(sizeof(float) * (size_t)n_tok * bank->n_ff);
    L.dg = at; at += up256(sizeof(float) * (size_t)n_tok * bank->n_embd);
    L.gemm = at;
    L.gemm_bytes = grouped_gemm_bytes(bank, n_tok);
    at += L.gemm_bytes;
    L.total = at;
    return L;
}

size_t moe_workspace_bytes(const krk_cuda_expert_bank *bank, int k, int64_t n_tok) {
    if (n_tok > KRK_CUDA_MAX_ROWS) return grouped_layout(bank, k, n_tok).total;
    // per-pick h and d rows, then the two matrix tables of the streaming path
    return moe_float_bytes(bank, k, n_tok) + 2 * ((sizeof(StreamTable) + 255) & ~(size_t)255);
}

static int grouped_matmul(float *y, const float *x, const uint8_t *w, int wt, int64_t n_out, int64_t n_in, int64_t m, void *ws,
                          cudaStream_t st) {
    if (m > KRK_CUDA_MAX_ROWS && n_in % 256 == 0 && gemm_tc_takes(wt))
        return launch_gemm_tc(y, x, KRK_CUDA_X_F32, w, wt, n_out, n_in, m, ws, st);
    for (int64_t r0 = 0; r0 < m; r0 += KRK_CUDA_MAX_ROWS) {
        const int64_t nr = m - r0 < KRK_CUDA_MAX_ROWS ? m - r0 : KRK_CUDA_MAX_ROWS;
        GemvMat mat;
        mat.w = w;
        mat.x = x + r0 * n_in;
        mat.y = y + r0 * n_out;
        mat.n_out = n_out;
        mat.wt = wt;
        int rc = launch_gemv_stream(&mat, 1, n_in, (int)nr, 0, 0, st);
        if (rc < 0) return rc;
        if (rc == 0) rc = launch_gemv_generic(&mat, 1, n_in, (int)nr, 0, 0, st);
        if (rc != KRK_CUDA_OK && rc != 1) return rc;
    }
    return KRK_CUDA_OK;
}

// y[n_tok][n_embd] = sum over the picks this bank holds, experts in ascending id, of w * down(silu(gate x) * up x).
// One device-to-host copy of the plan's offsets (a stream synchronisation) tells the host how many rows each
// expert has, as the reference's host plan does.
static int launch_moe_ffn_grouped(float *y, const float *x, const int32_t *ids, const float *wts, const krk_cuda_expert_bank *bank,
                                  int k, int64_t n_tok, void *workspace, cudaStream_t st) {
    const int n_expert = bank->expert_base + bank->n_local;   // ids at or above this are held elsewhere
    if (n_expert > kMaxExperts) return KRK_CUDA_EARG;
    const GroupedLayout L = grouped_layout(bank, k, n_tok);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    int32_t *off = reinterpret_cast<int32_t *>(ws + L.off), *rows = reinterpret_cast<int32_t *>(ws + L.rows);
    float *wt = reinterpret_cast<float *>(ws + L.wt), *xg = reinterpret_cast<float *>(ws + L.xg);
    float *g = reinterpret_cast<float *>(ws + L.g), *u = reinterpret_cast<float *>(ws + L.u), *dg = reinterpret_cast<float *>(ws + L.dg);
    int rc = launch_moe_plan_build(ids, n_tok, k, n_expert, off, rows, wt, wts, st);
    if (rc != KRK_CUDA_OK) return rc;
    static thread_local int32_t h_off[kMaxExperts + 1];
    cudaError_t e = cudaMemcpyAsync(h_off, off, sizeof(int32_t) * (size_t)(n_expert + 1), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess) e = cudaMemsetAsync(y, 0, sizeof(float) * (size_t)n_tok * bank->n_embd, st);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        return KRK_CUDA_ELAUNCH;
    }
    const size_t rb_gu = row_bytes(bank->wt_gate_up, bank->n_embd), rb_dn = row_bytes(bank->wt_down, bank->n_ff);
    for (int ex = bank->expert_base; ex < n_expert; ex++) {
        const int64_t m = h_off[ex + 1] - h_off[ex];
        if (m <= 0) continue;
        const int local = ex - bank->expert_base;
        const int32_t *er = rows + h_off[ex];
        const float *ew = wt + h_off[ex];
        const uint8_t *wg = static_cast<const uint8_t *>(bank->gate) + (size_t)local * bank->n_ff * rb_gu;
        const uint8_t *wu = static_cast<const uint8_t *>(bank->up) + (size_t)local * bank->n_ff * rb_gu;
        const uint8_t *wd = static_cast<const uint8_t *>(bank->down) + (size_t)local * bank->n_embd * rb_dn;
        if ((rc = launch_gather_rows(xg, x, er, m, bank->n_embd, st)) != KRK_CUDA_OK) return rc;
        if ((rc = grouped_matmul(g, xg, wg, bank->wt_gate_up, bank->n_ff, bank->n_embd, m, ws + L.gemm, st)) != KRK_CUDA_OK) return rc;
        if ((rc = grouped_matmul(u, xg, wu, bank->wt_gate_up, bank->n_ff, bank->n_embd, m, ws + L.gemm, st)) != KRK_CUDA_OK) return rc;
        if ((rc = launch_silu_mul(g, g, u, m * bank->n_ff, st)) != KRK_CUDA_OK) return rc;
        if ((rc = grouped_matmul(dg, g, wd, bank->wt_down, bank->n_embd, bank->n_ff, m, ws + L.gemm, st)) != KRK_CUDA_OK) return rc;
        if ((rc = launch_scatter_axpy_rows(y, dg, er, ew, m, bank->n_embd, st)) != KRK_CUDA_OK) return rc;
    }
    return KRK_CUDA_OK;
}

int launch_moe_ffn_generic(float *y, const float *x, const int32_t *ids, const float *wts,
                           const krk_cuda_expert_bank *bank, int k, int64_t n_tok, void *workspace,
                           cudaStream_t st, const float *logits, int n_expert) {
    // `logits` set: route first (ids / wts are outputs). The streaming path folds the routing into its plan
    // kernel; every other path runs the routing kernel on its own.
    bool routed = logits == nullptr;
    if (n_tok > KRK_CUDA_MAX_ROWS) {
        if (!routed) {
            const int rc = launch_route(const_cast<int32_t *>(ids), const_cast<float *>(wts), logits, n_tok, n_expert, k, st);
            if (rc != KRK_CUDA_OK) return rc;
        }
        return launch_moe_ffn_grouped(y, x, ids, wts, bank, k, n_tok, workspace, st);
    }
    MoeParams p;
    p.gate = static_cast<const uint8_t *>(bank->gate);
    p.up = static_cast<const uint8_t *>(bank->up);
    p.down = static_cast<const uint8_t *>(bank->down);
    p.x = x;
    p.ids = ids;
    p.wts = wts;
    p.h = static_cast<float *>(workspace);
    p.d = p.h + (size_t)(n_tok * k) * bank->n_ff;
    p.y = y;
    p.n_embd = bank->n_embd;
    p.n_ff = bank->n_ff;
    p.n_local = bank->n_local;
    p.expert_base = bank->expert_base;
    p.k = k;
    p.n_tok = (int)n_tok;
    const int picks = (int)(n_tok * k);
    // Streaming path: the same kernel as the dense decode GEMV, fed from device-side tables.
    // gate and up experts are rows of two stacked banks: their table launch stages weights out of one tensor map each
    StreamBanks gu_banks;
    gu_banks.base[0] = p.gate;
    gu_banks.base[1] = p.up;
    gu_banks.rows = (int64_t)bank->n_local * bank->n_ff;
    const int gran_gu = stream_gran(bank->wt_gate_up, bank->n_embd, true), gran_dn = stream_gran(bank->wt_down, bank->n_ff);
    if (gran_gu > 0 && gran_dn > 0 && picks <= kStreamTableEntries) {
        const bool fuse_route = !routed && n_expert <= kPlanRouteExperts && n_tok * 32 <= kPlanThreads;
        if (!routed && !fuse_route) {
            const int rc = launch_route(const_cast<int32_t *>(ids), const_cast<float *>(wts), logits, n_tok, n_expert, k, st);
            if (rc != KRK_CUDA_OK) return rc;
        }
        routed = true;
        uint8_t *tables = static_cast<uint8_t *>(workspace) + moe_float_bytes(bank, k, n_tok);
        StreamTable *ta = reinterpret_cast<StreamTable *>(tables);
        StreamTable *tb = reinterpret_cast<StreamTable *>(tables + ((sizeof(StreamTable) + 255) & ~(size_t)255));
        cudaError_t le = launch_overlapped(moe_plan_kernel, dim3(1), dim3(kPlanThreads), st, p, ta, tb, bank->wt_gate_up,
                                           bank->wt_down, row_bytes(bank->wt_gate_up, bank->n_embd),
                                           row_bytes(bank->wt_down, bank->n_ff), gran_gu, gran_dn,
                                           fuse_route ? logits : (const float *)nullptr, n_expert);
        note_launch();
        if (le != cudaSuccess) {
            note_cuda_error(le);
            (void)cudaGetLastError();
            return KRK_CUDA_ELAUNCH;
        }
        int rc = check_launch();
        if (rc != KRK_CUDA_OK) return rc;
        rc = launch_gemv_stream_table(ta, bank->wt_gate_up, bank->n_embd, 1, &gu_banks, st);
        if (rc < 0) return rc;
        rc = launch_gemv_stream_table(tb, bank->wt_down, bank->n_ff, 0, nullptr, st);
        if (rc < 0) return rc;
        dim3 grid((unsigned)((bank->n_embd + 255) / 256), (unsigned)n_tok);
        le = launch_overlapped(moe_combine_kernel, grid, dim3(256), st, p);
        note_launch();
        if (le != cudaSuccess) {
            note_cuda_error(le);
            (void)cudaGetLastError();
            return KRK_CUDA_ELAUNCH;
        }
        return check_launch();
    }
    if (!routed) {
        const int rc = launch_route(const_cast<int32_t *>(ids), const_cast<float *>(wts), logits, n_tok, n_expert, k, st);
        if (rc != KRK_CUDA_OK) return rc;
    }
    {
        dim3 grid((unsigned)((bank->n_ff + 7) / 8), (unsigned)picks);
        KRK_DISPATCH_WT(bank->wt_gate_up, moe_gate_up_kernel<WT><<<grid, 256, 0, st>>>(p));
        note_launch();
        const int rc = check_launch();
        if (rc != KRK_CUDA_OK) return rc;
    }
    {
        dim3 grid((unsigned)((bank->n_embd + 7) / 8), (unsigned)picks);
        KRK_DISPATCH_WT(bank->wt_down, moe_down_kernel<WT><<<grid, 256, 0, st>>>(p));
        note_launch();
        const int rc = check_launch();
        if (rc != KRK_CUDA_OK) return rc;
    }
    {
        dim3 grid((unsigned)((bank->n_embd + 255) / 256), (unsigned)n_tok);
        moe_combine_kernel<<<grid, 256, 0, st>>>(p);
        note_launch();
        return check_launch();
    }
}

} // namespace krk_cuda
