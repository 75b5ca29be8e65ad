// The two steps either side of the output-head GEMV: the embedding gather before the first layer and the
// top-k of the logits row after the head, both on the device so that neither token rows nor the 513 KB
// logits row cross PCIe per token.
//
// embed: out[t] = decoded row tokens[t] of the (quantized) embedding table; an id outside [0, n_vocab)
// gives a zero row (src/backend_cpu.cpp:746-778). Bit-exact with the host decoders.
//
// logits_topk: Backend::logits_topk (include/krk/backend.hpp:902-922; CPU twin src/backend_cpu.cpp:862-912):
// key(i) = logits[i], clamped to +-softcap when softcap > 0, then divided (positive) or multiplied
// (negative) by rep_pen where the token's bit is set in pen_mask; the k largest keys in descending order,
// ties toward the lower id; ids past the row's length are -1 / -FLT_MAX; mass = sum over the whole row of
// exp((key - max) / temp). Two kernels. Every block takes a 2048-key slice of the row: each of its 32 warps
// pulls the k best of its own 64 keys out of registers (k rounds of a shuffle arg-max), one warp merges the
// 32 sorted lists into the block's k best, and the slice's (max, sum of exp) is left beside them. One warp of
// the second kernel merges the blocks' lists the same way and the sums are folded. No block-wide barrier
// sits inside a round.
#include "krk_common.cuh"

#include <cfloat>

namespace krk_cuda {

namespace {

template <int WT>
__global__ void __launch_bounds__(256)
embed_kernel(float *__restrict__ out, const uint8_t *__restrict__ table, const int32_t *__restrict__ tokens,
             int64_t n_vocab, int64_t n_embd, int64_t n_tok, size_t rb) {
    const int64_t total = n_tok * n_embd;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / n_embd, k = i - t * n_embd;
        const int32_t id = tokens[t];
        out[i] = (id < 0 || (int64_t)id >= n_vocab) ? 0.0f : decode_value<WT>(table + (size_t)id * rb, k);
    }
}

constexpr int kTopkThreads = 1024;
constexpr int kTopkMaxK = 64;
constexpr int kTopkSlice = 2048;   // keys a block holds in shared memory

struct TopkParams {
    const float *logits;
    const uint32_t *pen_mask;
    float rep_pen, softcap, inv_temp;
    int64_t n;
    int k;
};

__device__ __forceinline__ float topk_key(const TopkParams &p, int64_t i) {
    float v = p.logits[i];
    if (p.softcap > 0.0f) v = v > p.softcap ? p.softcap : (v < -p.softcap ? -p.softcap : v);
    if (p.pen_mask && p.rep_pen > 0.0f && p.rep_pen != 1.0f && ((p.pen_mask[(uint32_t)i >> 5] >> ((uint32_t)i & 31)) & 1u))
        v = v > 0.0f ? __fdiv_rn(v, p.rep_pen) : __fmul_rn(v, p.rep_pen);
    return v;
}

// (value, id) order of the reference: larger value first, then lower id. "Nothing" is (-inf, INT_MAX): it
// loses to every real element, a real -inf key included.
constexpr int kNone = 0x7FFFFFFF;
__device__ __forceinline__ bool better(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

__device__ __forceinline__ void warp_best(float &v, int &i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, i, o);
        if (better(ov, oi, v, i)) {
            v = ov;
            i = oi;
        }
    }
}

// One warp merges `n_lists` lists of `k` (value, id) pairs, each best first, into the k best overall, best
// first: lane l looks after lists l, l + 32, ...; a round takes the best list head and advances that list.
// head[] (one int per list) is scratch in shared memory.
__device__ __forceinline__ void merge_lists(const float *lv, const int *li, int n_lists, int k, int *head, float *out_v,
                                            int *out_i, int lane) {
    for (int l = lane; l < n_lists; l += 32) head[l] = 0;
    __syncwarp();
    for (int r = 0; r < k; r++) {
        float v = -INFINITY;
        int i = kNone, from = -1;
        for (int l = lane; l < n_lists; l += 32) {
            const int h = head[l];
            if (h < k) {
                const float cv = lv[l * k + h];
                const int ci = li[l * k + h];
                if (better(cv, ci, v, i)) {
                    v = cv;
                    i = ci;
                    from = l;
                }
            }
        }
        float bv = v;
        int bi = i;
        warp_best(bv, bi);
        if (from >= 0 && i == bi && bi != kNone) head[from]++;   // ids are distinct: exactly one lane advances
        if (lane == 0) {
            out_v[r] = bv;
            out_i[r] = bi;
        }
        __syncwarp();
    }
}

// cand_v / cand_i: [blocks][k] best first; part: [blocks][2] = (slice max, slice sum of exp((key - slice max) * inv_temp))
__global__ void __launch_bounds__(kTopkThreads)
topk_slices_kernel(const __grid_constant__ TopkParams p, float *__restrict__ cand_v, int *__restrict__ cand_i,
                   float *__restrict__ part) {
    constexpr int kWarps = kTopkThreads / 32, kPerLane = kTopkSlice / kTopkThreads;
    __shared__ float wl_v[kWarps * kTopkMaxK];   // every warp's k best of its 64 keys, best first
    __shared__ int wl_i[kWarps * kTopkMaxK];
    __shared__ float red[kWarps];
    __shared__ int head[kWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t per = (p.n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = (int64_t)blockIdx.x * per, hi = min(p.n, lo + per);
    const int cnt = (int)max((int64_t)0, hi - lo);
    float v[kPerLane];
    int id[kPerLane];
    float mx = -FLT_MAX;
#pragma unroll
    for (int u = 0; u < kPerLane; u++) {
        const int j = warp * (32 * kPerLane) + 32 * u + lane;
        v[u] = -INFINITY;
        id[u] = kNone;
        if (j < cnt) {
            float key = topk_key(p, lo + j);
            if (!(key == key)) key = -INFINITY;   // a NaN key ranks last
            v[u] = key;
            id[u] = (int)(lo + j);
            mx = fmaxf(mx, key);
        }
    }
    // slice max and sum of exponentials for the mass
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < kWarps; w++) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int u = 0; u < kPerLane; u++)
        if (id[u] != kNone) sum += expf((v[u] - mx) * p.inv_temp);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int w = 0; w < kWarps; w++) s += red[w];
        part[2 * blockIdx.x] = mx;
        part[2 * blockIdx.x + 1] = cnt > 0 ? s : 0.0f;
    }
    // every warp: k rounds over its own keys (registers and shuffles only)
    for (int r = 0; r < p.k; r++) {
        float bv = -INFINITY;
        int bi = kNone;
#pragma unroll
        for (int u = 0; u < kPerLane; u++)
            if (better(v[u], id[u], bv, bi)) {
                bv = v[u];
                bi = id[u];
            }
        warp_best(bv, bi);
#pragma unroll
        for (int u = 0; u < kPerLane; u++)
            if (id[u] == bi && bi != kNone) {   // struck
                v[u] = -INFINITY;
                id[u] = kNone;
            }
        if (lane == 0) {
            wl_v[warp * p.k + r] = bv;
            wl_i[warp * p.k + r] = bi;
        }
    }
    __syncthreads();
    // warp 0: the block's k best out of the warps' lists
    if (warp == 0)
        merge_lists(wl_v, wl_i, kWarps, p.k, head, cand_v + (size_t)blockIdx.x * p.k, cand_i + (size_t)blockIdx.x * p.k, lane);
}

__global__ void __launch_bounds__(256)
topk_merge_kernel(const float *__restrict__ cand_v, const int *__restrict__ cand_i, const float *__restrict__ part,
                  int n_blocks, int k, float inv_temp, int32_t *__restrict__ ids, float *__restrict__ vals,
                  float *__restrict__ mass_out) {
    extern __shared__ float sm_v[];                       // [n_blocks * k], then the ids, then one head per list
    int *sm_i = reinterpret_cast<int *>(sm_v + (size_t)n_blocks * k);
    int *head = sm_i + (size_t)n_blocks * k;
    __shared__ float out_v[kTopkMaxK];
    __shared__ int out_i[kTopkMaxK];
    const int total = n_blocks * k;
    for (int j = threadIdx.x; j < total; j += blockDim.x) {
        sm_v[j] = cand_v[j];
        sm_i[j] = cand_i[j];
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        merge_lists(sm_v, sm_i, n_blocks, k, head, out_v, out_i, threadIdx.x);
        for (int r = threadIdx.x; r < k; r += 32) {
            const bool ok = out_i[r] != kNone;
            ids[r] = ok ? out_i[r] : -1;
            vals[r] = ok ? out_v[r] : -FLT_MAX;
        }
    } else if (mass_out && threadIdx.x == 32) {
        float mx = -FLT_MAX;
        for (int b = 0; b < n_blocks; b++) mx = fmaxf(mx, part[2 * b]);
        float m = 0.0f;
        for (int b = 0; b < n_blocks; b++)
            if (part[2 * b + 1] > 0.0f) m += part[2 * b + 1] * expf((part[2 * b] - mx) * inv_temp);
        *mass_out = m;
    }
}

int topk_blocks(int64_t n) {
    const int64_t need = (n + kTopkSlice - 1) / kTopkSlice;   // a slice must fit the block's shared memory
    return (int)(need < 1 ? 1 : need);
}

} // namespace

int launch_embed(float *out, const uint8_t *table, int wt, int64_t n_vocab, int64_t n_embd, const int32_t *tokens,
                 int64_t n_tok, cudaStream_t st) {
    const int64_t total = n_tok * n_embd;
    if (total == 0) return KRK_CUDA_OK;
    const int64_t want = (total + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
    const size_t rb = row_bytes(wt, n_embd);
    KRK_DISPATCH_WT(wt, embed_kernel<WT><<<grid, 256, 0, st>>>(out, table, tokens, n_vocab, n_embd, n_tok, rb));
    note_launch();
    return check_launch();
}

size_t logits_topk_workspace_bytes(int64_t n, int k) {
    const size_t blocks = (size_t)topk_blocks(n);
    return blocks * (size_t)k * 8 + blocks * 8 + 256;
}

int launch_logits_topk(const float *logits, int64_t n, int k, const uint32_t *pen_mask, float rep_pen, float softcap,
                       float temp, int32_t *ids, float *vals, float *mass_out, void *workspace, cudaStream_t st) {
    if (k < 1 || k > kTopkMaxK || n < 1) return KRK_CUDA_EARG;
    const int blocks = topk_blocks(n);
    if ((size_t)blocks * k * 8 + (size_t)blocks * 4 > 200 * 1024) return KRK_CUDA_ESHAPE;   // the merge holds every candidate in shared memory
    float *cand_v = static_cast<float *>(workspace);
    int *cand_i = reinterpret_cast<int *>(cand_v + (size_t)blocks * k);
    float *part = reinterpret_cast<float *>(cand_i + (size_t)blocks * k);
    TopkParams p;
    p.logits = logits;
    p.pen_mask = pen_mask;
    p.rep_pen = rep_pen;
    p.softcap = softcap;
    p.inv_temp = temp > 0.0f ? 1.0f / temp : 1.0f;
    p.n = n;
    p.k = k;
    topk_slices_kernel<<<blocks, kTopkThreads, 0, st>>>(p, cand_v, cand_i, part);
    note_launch();
    int rc = check_launch();
    if (rc != KRK_CUDA_OK) return rc;
    const size_t smem = (size_t)blocks * k * 8 + (size_t)blocks * 4;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[dev])) {
        if (cudaFuncSetAttribute(topk_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return KRK_CUDA_ELAUNCH;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    topk_merge_kernel<<<1, 256, smem, st>>>(cand_v, cand_i, part, blocks, k, p.inv_temp, ids, vals, mass_out);
    note_launch();
    return check_launch();
}

} // namespace krk_cuda
