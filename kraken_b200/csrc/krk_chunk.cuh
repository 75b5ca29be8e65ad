// 32-value chunk decode shared by the shape-agnostic kernels: every format is a whole
// number of 32-value chunks (Q8_0/Q4_0: one block; Q4_K/Q6_K: an eighth of a super-block).
#pragma once

#include "krk_common.cuh"

namespace krk_cuda {

// The 32 values of chunk c of a row, as the host decoder produces them.
template <int WT>
__device__ __forceinline__ void decode_chunk(const uint8_t *row, int64_t c, float (&v)[32]);

template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q8_0>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + c * 34;
    const float d = half_bits_to_float(b);
#pragma unroll
    for (int k = 0; k < 32; k++) v[k] = __fmul_rn(d, (float)(int8_t)b[2 + k]);
}

template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q4_0>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + c * 18;
    const float d = half_bits_to_float(b);
#pragma unroll
    for (int k = 0; k < 16; k++) {
        const uint8_t q = b[2 + k];
        v[k] = __fmul_rn(d, (float)((int)(q & 0xF) - 8));
        v[k + 16] = __fmul_rn(d, (float)((int)(q >> 4) - 8));
    }
}

template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q4_K>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + (c >> 3) * 144;
    const int cc = (int)(c & 7);
    int sc, mn;
    scale_min_k4(cc, b + 4, sc, mn);
    const float dl = __fmul_rn(half_bits_to_float(b), (float)sc);
    const float ml = __fmul_rn(half_bits_to_float(b + 2), (float)mn);
    const uint8_t *q = b + 16 + 32 * (cc >> 1);
    const int shift = (cc & 1) * 4;
#pragma unroll
    for (int k = 0; k < 32; k++)
        v[k] = __fsub_rn(__fmul_rn(dl, (float)((q[k] >> shift) & 0xF)), ml);
}

template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q6_K>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + (c >> 3) * 210;
    const int cc = (int)(c & 7), half = cc >> 2, quad = cc & 3;
    const uint8_t *ql = b + 64 * half + ((quad & 1) ? 32 : 0);
    const uint8_t *qh = b + 128 + 32 * half;
    const int8_t *sc = (const int8_t *)(b + 192) + 8 * half + 2 * quad;
    const float d = half_bits_to_float(b + 208);
    const float d0 = __fmul_rn(d, (float)sc[0]), d1 = __fmul_rn(d, (float)sc[1]);
#pragma unroll
    for (int k = 0; k < 32; k++) {
        const int lo = (quad & 2) ? (ql[k] >> 4) : (ql[k] & 0xF);
        const int q = lo | (((qh[k] >> (2 * quad)) & 3) << 4);
        v[k] = __fmul_rn(k < 16 ? d0 : d1, (float)(q - 32));
    }
}

// The formats below follow decode_value<WT> operation for operation (so the values are the same bits) with
// everything that is common to a chunk taken out of the loop over its 32 values.

// src/quant.cpp:351-364
template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q5_0>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + c * 22;
    const float d = half_bits_to_float(b);
    const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const uint8_t q = b[6 + j];
        v[j] = __fmul_rn(d, (float)(((q & 0xF) | (int)(((qh >> j) & 1u) << 4)) - 16));
        v[j + 16] = __fmul_rn(d, (float)(((q >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4)) - 16));
    }
}

// src/quant.cpp:366-379
template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q5_1>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + c * 24;
    const float d = half_bits_to_float(b), m = half_bits_to_float(b + 2);
    const uint32_t qh = (uint32_t)b[4] | ((uint32_t)b[5] << 8) | ((uint32_t)b[6] << 16) | ((uint32_t)b[7] << 24);
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const uint8_t q = b[8 + j];
        v[j] = __fadd_rn(__fmul_rn(d, (float)((q & 0xF) | (int)(((qh >> j) & 1u) << 4))), m);
        v[j + 16] = __fadd_rn(__fmul_rn(d, (float)((q >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4))), m);
    }
}

// src/quant.cpp:462-489
template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q5_K>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + (c >> 3) * 176;
    const int cc = (int)(c & 7);
    int sc, mn;
    scale_min_k4(cc, b + 4, sc, mn);
    const float dl = __fmul_rn(half_bits_to_float(b), (float)sc);
    const float ml = __fmul_rn(half_bits_to_float(b + 2), (float)mn);
    const uint8_t *q = b + 48 + 32 * (cc >> 1), *qh = b + 16;
    const int shift = (cc & 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; l++) {
        const int quant = ((q[l] >> shift) & 0xF) + (((qh[l] >> cc) & 1) ? 16 : 0);
        v[l] = __fsub_rn(__fmul_rn(dl, (float)quant), ml);
    }
}

// src/quant.cpp:398-424
template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q2_K>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + (c >> 3) * 84;
    const int cc = (int)(c & 7), g = cc >> 2, j = cc & 3;
    const float d = half_bits_to_float(b + 80), dmin = half_bits_to_float(b + 82);
    const uint8_t s0 = b[8 * g + 2 * j], s1 = b[8 * g + 2 * j + 1];
    const float dl0 = __fmul_rn(d, (float)(s0 & 0xF)), ml0 = __fmul_rn(dmin, (float)(s0 >> 4));
    const float dl1 = __fmul_rn(d, (float)(s1 & 0xF)), ml1 = __fmul_rn(dmin, (float)(s1 >> 4));
    const uint8_t *q = b + 16 + 32 * g;
#pragma unroll
    for (int l = 0; l < 32; l++) {
        const int quant = (q[l] >> (2 * j)) & 3;
        v[l] = __fsub_rn(__fmul_rn(l < 16 ? dl0 : dl1, (float)quant), l < 16 ? ml0 : ml1);
    }
}

// src/quant.cpp:514-553
template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_Q3_K>(const uint8_t *row, int64_t c, float (&v)[32]) {
    const uint8_t *b = row + (c >> 3) * 110;
    const int cc = (int)(c & 7), nn = cc >> 2, j = cc & 3;
    const uint8_t *sr = b + 96;
    float dl[2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int is = 8 * nn + 2 * j + h;
        const int lo = is < 8 ? (sr[is] & 0xF) : (sr[is - 8] >> 4);
        const int hi = (sr[8 + (is & 3)] >> (2 * (is >> 2))) & 3;
        dl[h] = __fmul_rn(half_bits_to_float(b + 108), (float)((lo | (hi << 4)) - 32));
    }
    const uint8_t *q = b + 32 + 32 * nn;
#pragma unroll
    for (int l = 0; l < 32; l++) {
        const int quant = (int)((q[l] >> (2 * j)) & 3) - ((b[l] >> (4 * nn + j)) & 1 ? 0 : 4);
        v[l] = __fmul_rn(l < 16 ? dl[0] : dl[1], (float)quant);
    }
}

// src/quant.cpp:88-91, 566-575
template <>
__device__ __forceinline__ void decode_chunk<KRK_CUDA_IQ4_NL>(const uint8_t *row, int64_t c, float (&v)[32]) {
    constexpr uint32_t grid[4] = {0xBFAD9881u, 0xF6EADDCFu, 0x26190D01u, 0x71594535u};
    const uint8_t *b = row + c * 18;
    const float d = half_bits_to_float(b);
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int lo = b[2 + j] & 0xF, hi = b[2 + j] >> 4;
        v[j] = __fmul_rn(d, (float)(int)(int8_t)((grid[lo >> 2] >> (8 * (lo & 3))) & 0xFF));
        v[j + 16] = __fmul_rn(d, (float)(int)(int8_t)((grid[hi >> 2] >> (8 * (hi & 3))) & 0xFF));
    }
}

// Dot of chunk c of a weight row with the matching 32 activations (x 16-byte aligned).
template <int WT>
__device__ __forceinline__ float chunk_dot(const uint8_t *row, int64_t c, const float *x) {
    float v[32];
    decode_chunk<WT>(row, c, v);
    const float4 *xv = reinterpret_cast<const float4 *>(x + c * 32);
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const float4 t = xv[k];
        s = fmaf(v[4 * k + 0], t.x, s);
        s = fmaf(v[4 * k + 1], t.y, s);
        s = fmaf(v[4 * k + 2], t.z, s);
        s = fmaf(v[4 * k + 3], t.w, s);
    }
    return s;
}

__device__ __forceinline__ float warp_sum(float s) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    return s;
}

} // namespace krk_cuda
