// Shape-agnostic decode GEMV: one warp per output row, lanes stride over 32-value chunks staged in shared
// memory, f32 accumulation, shuffle reduction. It takes every legal shape (any n_in that is a
// whole number of blocks, any alignment the format allows) and is the path for shapes the
// streaming kernel does not address (K not a multiple of 256, activations too wide for shared
// memory). Same contract as gemv_kernel /
// gemv_m_kernel of the reference (src/hip/kernels/gemm.hpp:76-167) with f32 activations.
#include "krk_chunk.cuh"

namespace krk_cuda {

namespace {

constexpr int kWarpsPerBlock = 8;

struct GenericParams {
    GemvMat mat[KRK_CUDA_MAX_GROUP];
    int block_begin[KRK_CUDA_MAX_GROUP + 1];  // first thread block of each matrix
    int n_mat;
    int rows;
    int accumulate;
    int64_t n_in;
};

// A K segment of 1024 values is staged in shared memory before it is decoded: the activations of every row once
// per block (chunk c at a pitch of 33 floats, so that the 32 lanes of a warp, one chunk each, read different
// banks), and each warp's own weight-row bytes with 16-byte loads from the 16-byte boundary before them. The
// per-value decode then reads shared memory instead of issuing byte loads to global memory. Which lane takes
// which chunk, and the order of the additions, are those of the plain warp-per-row walk.
constexpr int kSegValues = 1024, kSegChunks = kSegValues / 32, kXPitch = 33;
constexpr int kSegBytesMax = kSegValues / 32 * 34;   // Q8_0 is the widest format per value

template <int WT, int ROWS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gemv_generic_kernel(const __grid_constant__ GenericParams p) {
    __shared__ float xs[ROWS][kSegChunks * kXPitch];
    __shared__ __align__(16) uint8_t wbuf[kWarpsPerBlock][kSegBytesMax + 32];
    int m = 0;
    while (m + 1 < p.n_mat && (int)blockIdx.x >= p.block_begin[m + 1]) m++;
    const GemvMat &mat = p.mat[m];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = (int64_t)(blockIdx.x - p.block_begin[m]) * kWarpsPerBlock + warp;
    const bool live = row < mat.n_out;
    const int64_t n_chunks = p.n_in >> 5;
    const size_t rb = row_bytes(WT, p.n_in);
    const uint8_t *wrow = mat.w + (size_t)(live ? row : 0) * rb;
    const uint8_t *w_end = mat.w + (size_t)mat.n_out * rb;
    constexpr int kChunksPerBlock = block_size(WT) / 32;

    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; r++) acc[r] = 0.0f;

    for (int64_t c0 = 0; c0 < n_chunks; c0 += kSegChunks) {
        const int seg_chunks = (int)min((int64_t)kSegChunks, n_chunks - c0);
        __syncthreads();   // everybody is done with the segment before
        for (int r = 0; r < ROWS; r++) {
            if (r >= p.rows) break;
            const float *xr = mat.x + (int64_t)r * p.n_in + c0 * 32;
            for (int i = threadIdx.x; i < seg_chunks * 32; i += kWarpsPerBlock * 32) xs[r][(i >> 5) * kXPitch + (i & 31)] = xr[i];
        }
        const uint8_t *src = wrow + (size_t)(c0 / kChunksPerBlock) * block_bytes(WT);
        const int lead = (int)(reinterpret_cast<uintptr_t>(src) & 15);
        if (live) {
            const int total = lead + seg_chunks / kChunksPerBlock * block_bytes(WT);
            const uint8_t *base = src - lead;   // not before the matrix: its base is 16-byte aligned
            for (int i = lane * 16; i < total; i += 32 * 16) {
                if (base + i + 16 <= w_end) {
                    *reinterpret_cast<uint4 *>(&wbuf[warp][i]) = *reinterpret_cast<const uint4 *>(base + i);
                } else {
                    for (int j = 0; j < 16 && base + i + j < w_end; j++) wbuf[warp][i + j] = base[i + j];
                }
            }
        }
        __syncthreads();
        if (live && lane < seg_chunks) {
            float v[32];
            decode_chunk<WT>(&wbuf[warp][lead], lane, v);
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                if (r < p.rows) {
                    const float *xv = &xs[r][lane * kXPitch];
                    float s = 0.0f;
#pragma unroll
                    for (int k = 0; k < 32; k++) s = fmaf(v[k], xv[k], s);
                    acc[r] += s;
                }
            }
        }
    }
    if (!live) return;
#pragma unroll
    for (int r = 0; r < ROWS; r++) {
        float s = acc[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (lane == 0 && r < p.rows) {
            float *y = mat.y + (int64_t)r * mat.n_out + row;
            *y = p.accumulate ? __fadd_rn(*y, s) : s;
        }
    }
}

} // namespace

int launch_gemv_generic(const GemvMat *mats, int n_mat, int64_t n_in, int rows, int accumulate,
                        int silu_pair, cudaStream_t st) {
    // Matrices of one launch share a weight type here; mixed groups go out as one launch
    // per run of equal types.
    int first = 0;
    while (first < n_mat) {
        int last = first + 1;
        while (last < n_mat && mats[last].wt == mats[first].wt) last++;
        GenericParams p;
        p.n_mat = 0;
        p.rows = rows;
        p.accumulate = accumulate;
        p.n_in = n_in;
        int blocks = 0;
        for (int m = first; m < last; m++) {
            if (mats[m].n_out == 0) continue;
            p.mat[p.n_mat] = mats[m];
            p.block_begin[p.n_mat] = blocks;
            blocks += (int)((mats[m].n_out + kWarpsPerBlock - 1) / kWarpsPerBlock);
            p.n_mat++;
        }
        p.block_begin[p.n_mat] = blocks;
        if (blocks > 0) {
            const int wt = mats[first].wt;
            if (rows <= 1) {
                KRK_DISPATCH_WT(wt, gemv_generic_kernel<WT, 1><<<blocks, kWarpsPerBlock * 32, 0, st>>>(p));
            } else if (rows <= 4) {
                KRK_DISPATCH_WT(wt, gemv_generic_kernel<WT, 4><<<blocks, kWarpsPerBlock * 32, 0, st>>>(p));
            } else {
                KRK_DISPATCH_WT(wt, gemv_generic_kernel<WT, 8><<<blocks, kWarpsPerBlock * 32, 0, st>>>(p));
            }
            note_launch(1, KRK_CUDA_FAMILY_GEMV_GENERIC);
            const int rc = check_launch();
            if (rc != KRK_CUDA_OK) return rc;
        }
        first = last;
    }
    if (silu_pair) {
        // The gate/up fold as a second pass: y[2i] = silu(y[2i]) * y[2i+1].
        for (int m = 0; m + 1 < n_mat; m += 2) {
            for (int r = 0; r < rows; r++) {
                float *g = mats[m].y + (int64_t)r * mats[m].n_out;
                const float *u = mats[m + 1].y + (int64_t)r * mats[m + 1].n_out;
                const int rc = launch_silu_mul(g, g, u, mats[m].n_out, st);
                if (rc != KRK_CUDA_OK) return rc;
            }
        }
    }
    return KRK_CUDA_OK;
}

} // namespace krk_cuda
