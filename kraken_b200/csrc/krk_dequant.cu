// Row decode to f32 and the small elementwise ops that sit beside the matmul path.
#include "krk_common.cuh"

namespace krk_cuda {

// One thread per output value: stores are fully coalesced, the few header bytes a value
// needs are re-read through L1. This kernel is the parity anchor (bit-exact with the host
// decoders), not a hot path.
template <int WT>
__global__ void __launch_bounds__(256)
dequant_rows_kernel(float *__restrict__ out, const uint8_t *__restrict__ w, int64_t n_rows,
                    int64_t n_in, size_t rb) {
    const int64_t total = n_rows * n_in;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n_in, k = i - r * n_in;
        out[i] = decode_value<WT>(w + (size_t)r * rb, k);
    }
}

int launch_dequant_rows(float *out, const uint8_t *w, int wt, int64_t n_rows, int64_t n_in,
                        cudaStream_t st) {
    const int64_t total = n_rows * n_in;
    if (total == 0) return KRK_CUDA_OK;
    const int64_t want = (total + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
    const size_t rb = row_bytes(wt, n_in);
    KRK_DISPATCH_WT(wt, dequant_rows_kernel<WT><<<grid, 256, 0, st>>>(out, w, n_rows, n_in, rb));
    note_launch();
    return check_launch();
}

// silu(g) * u with the reference's formula g / (1 + exp(-g)) (src/backend_cpu.cpp:2394-2400).
__global__ void __launch_bounds__(256)
silu_mul_kernel(float *__restrict__ out, const float *__restrict__ gate,
                const float *__restrict__ up, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float g = gate[i];
        out[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, exp_as_host(-g))), up[i]);
    }
}

int launch_silu_mul(float *out, const float *gate, const float *up, int64_t n, cudaStream_t st) {
    if (n == 0) return KRK_CUDA_OK;
    const int64_t want = (n + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    silu_mul_kernel<<<grid, 256, 0, st>>>(out, gate, up, n);
    note_launch();
    return check_launch();
}

// dst[rows[i]][j] += alpha[i] * src[i][j] (src/backend_cpu.cpp:3193-3220). Row ids are
// distinct within a call, so no two threads touch the same destination.
__global__ void __launch_bounds__(256)
scatter_axpy_rows_kernel(float *__restrict__ dst, const float *__restrict__ src,
                         const int32_t *__restrict__ rows, const float *__restrict__ alpha,
                         int64_t n_rows, int64_t n) {
    const int64_t total = n_rows * n;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n, j = i - r * n;
        float *d = dst + (int64_t)rows[r] * n + j;
        *d = __fadd_rn(*d, __fmul_rn(alpha[r], src[i]));
    }
}

int launch_scatter_axpy_rows(float *dst, const float *src, const int32_t *rows, const float *alpha,
                             int64_t n_rows, int64_t n, cudaStream_t st) {
    const int64_t total = n_rows * n;
    if (total == 0) return KRK_CUDA_OK;
    const int64_t want = (total + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    scatter_axpy_rows_kernel<<<grid, 256, 0, st>>>(dst, src, rows, alpha, n_rows, n);
    note_launch();
    return check_launch();
}

// dst[i][j] = src[rows[i]][j] (Backend::gather_rows, include/krk/backend.hpp:1451): the tokens that picked an
// expert, permuted into one contiguous block. Four floats per thread where the rows allow it.
__global__ void __launch_bounds__(256)
gather_rows_kernel(float *__restrict__ dst, const float *__restrict__ src, const int32_t *__restrict__ rows,
                   int64_t n_rows, int64_t n, int vec) {
    if (vec) {
        const int64_t n4 = n >> 2, total = n_rows * n4;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = i / n4, j = i - r * n4;
            reinterpret_cast<float4 *>(dst)[i] = __ldg(reinterpret_cast<const float4 *>(src + (int64_t)rows[r] * n) + j);
        }
        return;
    }
    const int64_t total = n_rows * n;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n, j = i - r * n;
        dst[i] = src[(int64_t)rows[r] * n + j];
    }
}

int launch_gather_rows(float *dst, const float *src, const int32_t *rows, int64_t n_rows, int64_t n, cudaStream_t st) {
    const int64_t total = n_rows * n;
    if (total == 0) return KRK_CUDA_OK;
    const int vec = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0;
    const int64_t want = ((vec ? total / 4 : total) + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    gather_rows_kernel<<<grid, 256, 0, st>>>(dst, src, rows, n_rows, n, vec);
    note_launch();
    return check_launch();
}

// out[j] = ((parts[0][j] + parts[1][j]) + parts[2][j]) + ... : fixed order, so the combined
// output of an expert-sharded layer has the same bits on every rank and every run.
__global__ void __launch_bounds__(256)
sum_parts_kernel(float *__restrict__ out, const float *__restrict__ parts, int n_parts, int64_t n) {
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n;
         j += (int64_t)gridDim.x * blockDim.x) {
        float s = parts[j];
        for (int p = 1; p < n_parts; p++) s = __fadd_rn(s, parts[(int64_t)p * n + j]);
        out[j] = s;
    }
}

int launch_sum_parts(float *out, const float *parts, int n_parts, int64_t n, cudaStream_t st) {
    if (n == 0) return KRK_CUDA_OK;
    const int64_t want = (n + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
    sum_parts_kernel<<<grid, 256, 0, st>>>(out, parts, n_parts, n);
    note_launch();
    return check_launch();
}

} // namespace krk_cuda
