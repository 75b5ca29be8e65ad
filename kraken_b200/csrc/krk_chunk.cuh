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

// The 5-bit formats decode element by element (they ride the shape-agnostic kernels only).
#define KRK_CHUNK_BY_ELEMENT(WT_)                                                                                        \
    template <>                                                                                                          \
    __device__ __forceinline__ void decode_chunk<WT_>(const uint8_t *row, int64_t c, float (&v)[32]) {                    \
        _Pragma("unroll") for (int k = 0; k < 32; k++) v[k] = decode_value<WT_>(row, c * 32 + k);                          \
    }
KRK_CHUNK_BY_ELEMENT(KRK_CUDA_Q5_0)
KRK_CHUNK_BY_ELEMENT(KRK_CUDA_Q5_1)
KRK_CHUNK_BY_ELEMENT(KRK_CUDA_Q5_K)
KRK_CHUNK_BY_ELEMENT(KRK_CUDA_Q2_K)
KRK_CHUNK_BY_ELEMENT(KRK_CUDA_Q3_K)
KRK_CHUNK_BY_ELEMENT(KRK_CUDA_IQ4_NL)
#undef KRK_CHUNK_BY_ELEMENT

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
