// Issue-rate probe: how often one SM sub-partition accepts the instructions the decode GEMV could be
// built from (legacy integer and half tensor-core MMAs, dp4a, and the plain integer / half pipes).
// One CTA per SM, `warps` warps, every lane runs `iters` rounds of eight instructions of one kind, either
// on eight independent accumulator sets (throughput) or chained on one (latency); the SM's own clock
// is read on both sides. The numbers choose between formulations of the kernel; nothing on the
// product path calls this.
#include "krk_common.cuh"

namespace krk_cuda {
namespace {

enum ProbeKind {
    kImmaK32 = 0,    // mma.sync m16n8k32 s8 x s8 -> s32
    kImmaK16 = 1,    // mma.sync m16n8k16 s8 x s8 -> s32
    kHmmaK16 = 2,    // mma.sync m16n8k16 f16 x f16 -> f32
    kBmmaK16 = 3,    // mma.sync m16n8k16 bf16 x bf16 -> f32
    kQmmaK32 = 4,    // mma.sync m16n8k32 e4m3 x e4m3 -> f32
    kDp4a = 5,       // dp4a.s32.s32
    kImad = 6,       // mad.lo.s32
    kHfma2 = 7,      // fma.rn.f16x2
    kLop3 = 8,       // lop3.b32
    kFfma = 9,       // fma.rn.f32
    kHmmaK8 = 10,    // mma.sync m16n8k8 f16 x f16 -> f32
    kProbeKinds = 11
};

template <int KIND>
__device__ __forceinline__ void probe_op(uint32_t (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    if (KIND == kImmaK32)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    if (KIND == kImmaK16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
    if (KIND == kHmmaK16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    if (KIND == kBmmaK16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    if (KIND == kQmmaK32)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    if (KIND == kHmmaK8)
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
    if (KIND == kDp4a) asm volatile("dp4a.s32.s32 %0, %1, %2, %0;" : "+r"(c[0]) : "r"(a0), "r"(b0));
    if (KIND == kImad) asm volatile("mad.lo.s32 %0, %1, %2, %0;" : "+r"(c[0]) : "r"(a0), "r"(b0));
    if (KIND == kHfma2) asm volatile("fma.rn.f16x2 %0, %1, %2, %0;" : "+r"(c[0]) : "r"(a0), "r"(b0));
    if (KIND == kLop3) asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(c[0]) : "r"(a0), "r"(b0));
    if (KIND == kFfma) asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(*reinterpret_cast<float *>(&c[0])) : "f"(__uint_as_float(a0)), "f"(__uint_as_float(b0)));
}

template <int KIND, bool CHAIN>
__global__ void __launch_bounds__(1024, 1) probe_kernel(const uint32_t *src, uint32_t *sink, long long *cycles, int iters) {
    // operands that the compiler cannot fold; finite halves (1.0) so that no pipe sees denormals or NaNs
    const uint32_t a0 = src[threadIdx.x & 31], a1 = src[32 + (threadIdx.x & 31)], a2 = src[64 + (threadIdx.x & 31)],
                   a3 = src[96 + (threadIdx.x & 31)], b0 = src[128 + (threadIdx.x & 31)], b1 = src[160 + (threadIdx.x & 31)];
    uint32_t c[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) c[j][i] = 0;
    __syncthreads();
    const long long t0 = clock64();
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int j = 0; j < 8; j++) probe_op<KIND>(c[CHAIN ? 0 : j], a0, a1, a2, a3, b0, b1);
    }
    const long long t1 = clock64();
    uint32_t s = 0;
#pragma unroll
    for (int j = 0; j < 8; j++)
#pragma unroll
        for (int i = 0; i < 4; i++) s ^= c[j][i];
    sink[blockIdx.x * blockDim.x + threadIdx.x] = s;
    if ((threadIdx.x & 31) == 0) cycles[blockIdx.x * 32 + (threadIdx.x >> 5)] = t1 - t0;
}

template <int KIND>
void probe_launch(bool chain, int grid, int warps, const uint32_t *src, uint32_t *sink, long long *cycles, int iters,
                  cudaStream_t st) {
    if (chain) probe_kernel<KIND, true><<<grid, warps * 32, 0, st>>>(src, sink, cycles, iters);
    else probe_kernel<KIND, false><<<grid, warps * 32, 0, st>>>(src, sink, cycles, iters);
}

} // namespace
} // namespace krk_cuda

using namespace krk_cuda;

extern "C" int krk_cuda_probe_issue(int kind, int warps, int iters, int chained, double *cycles_per_instr) {
    if (kind < 0 || kind >= kProbeKinds || warps < 1 || warps > 32 || iters < 1 || !cycles_per_instr) return KRK_CUDA_EARG;
    const int grid = sm_count();
    uint32_t *src = nullptr, *sink = nullptr;
    long long *cycles = nullptr;
    if (cudaMalloc(&src, 192 * 4) != cudaSuccess || cudaMalloc(&sink, (size_t)grid * 1024 * 4) != cudaSuccess ||
        cudaMalloc(&cycles, (size_t)grid * 32 * 8) != cudaSuccess) {
        cudaFree(src);
        cudaFree(sink);
        cudaFree(cycles);
        return KRK_CUDA_EDEVICE;
    }
    uint32_t h[192];
    const bool half_kind = kind == kHmmaK16 || kind == kHmmaK8 || kind == kHfma2;
    for (int i = 0; i < 192; i++)
        h[i] = half_kind ? 0x3C003C00u : kind == kBmmaK16 ? 0x3F803F80u : kind == kQmmaK32 ? 0x38383838u
               : kind == kFfma ? 0x3F800000u : 0x01020304u * (uint32_t)(i + 1);
    cudaMemcpy(src, h, sizeof h, cudaMemcpyHostToDevice);
    cudaMemset(cycles, 0, (size_t)grid * 32 * 8);
    const bool ch = chained != 0;
    for (int rep = 0; rep < 2; rep++) {   // the second pass is the measured one (the first pages the code in)
        switch (kind) {
        case kImmaK32: probe_launch<kImmaK32>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kImmaK16: probe_launch<kImmaK16>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kHmmaK16: probe_launch<kHmmaK16>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kBmmaK16: probe_launch<kBmmaK16>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kQmmaK32: probe_launch<kQmmaK32>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kDp4a: probe_launch<kDp4a>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kImad: probe_launch<kImad>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kHfma2: probe_launch<kHfma2>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kLop3: probe_launch<kLop3>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        case kFfma: probe_launch<kFfma>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        default: probe_launch<kHmmaK8>(ch, grid, warps, src, sink, cycles, iters, 0); break;
        }
    }
    note_launch(2);
    int rc = check_launch();
    if (rc == KRK_CUDA_OK && cudaDeviceSynchronize() != cudaSuccess) rc = KRK_CUDA_ELAUNCH;
    if (rc == KRK_CUDA_OK) {
        long long h_cycles[32];
        cudaMemcpy(h_cycles, cycles, sizeof h_cycles, cudaMemcpyDeviceToHost);   // the first SM's warps
        long long mx = 0;
        for (int w = 0; w < warps; w++) mx = h_cycles[w] > mx ? h_cycles[w] : mx;
        // instructions one sub-partition issued: 8 per round from each of its warps
        const double per_smsp = (double)iters * 8.0 * (double)((warps + 3) / 4);
        *cycles_per_instr = (double)mx / per_smsp;
    }
    cudaFree(src);
    cudaFree(sink);
    cudaFree(cycles);
    return rc;
}
