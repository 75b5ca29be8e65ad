// Prefill GEMM for sm_100a: Y[rows][n_out] = X[rows][n_in] . W^T with W block-quantized in HBM,
// decoded to f16 and contracted on the 5th-generation tensor cores (tcgen05.mma, f32 accumulators
// in tensor memory).
//
// Mapping. The weight tile is the MMA's A operand (128 weight rows = the 128 TMEM lanes), the
// token tile its B operand (up to 256 tokens = TMEM columns), so a weight tile is decoded once
// per 256 tokens and the accumulator D[weight row][token] is Y transposed: the epilogue reads one
// TMEM lane per thread and 32 neighbouring weight rows of one token form one coalesced 128-byte
// store.
//
// The decoded weights never touch shared memory: a decode thread owns a weight row = a TMEM lane,
// so it writes its f16 values straight into tensor memory (tcgen05.st) and the MMA takes A from
// TMEM. Shared memory then carries only the X tiles (TMA, 128-byte swizzle) and the raw quantized
// bytes, which leaves its bandwidth to the one operand the MMA still reads from it.
//
// One persistent CTA per SM, warp-specialised, everything connected by mbarriers:
//   warps 0..7   decode: two threads per weight row, 32 values each per 64-value K step. The raw blocks of
//                128 rows x 256 values (Q8_0: 128 values) arrive in shared memory by TMA: a 2-D tensor map
//                over the raw byte matrix for Q4_K / Q4_0 / Q5_K / Q8_0, eight maps (rows 8 apart) for
//                Q6_K, whose rows do not start on 16-byte boundaries; a thread takes its row's bytes into
//                registers and decodes with packed half2 arithmetic. Q5_0 / Q5_1 are staged by the decode
//                warps themselves and decoded element by element. 16 x 32-bit TMEM columns per thread and step;
//   warps 8..11  epilogue: tcgen05.ld of the accumulator (warp w%4 owns TMEM lanes 32*(w%4)..), 32 tokens
//                at a time into a [token][weight row] staging buffer in shared memory, TMA stores of Y;
//   warp 12      TMA producer of X tiles (cp.async.bulk.tensor.2d, each CTA loads its own copy);
//   warp 13      TMA producer of the raw block columns;
//   warp 14      TMEM allocation and the single thread that issues tcgen05.mma / tcgen05.commit.
// Tensor memory: columns 0..255 the accumulator, 256..511 four A stages of 64 columns (two K steps each).
//
// Same contract as gemm_wmma_kernel of the reference (src/hip/kernels/gemm.hpp:621-970): f16
// staged operands, f32 accumulation; here the output stays f32.
//
// Every mbarrier wait is bounded; a wait that gives up raises the device status word, and the CTA
// runs to its end without waiting again and frees its tensor memory.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "krk_common.cuh"

namespace krk_cuda {

namespace {

constexpr int kTileN = 128;            // weight rows per tile (MMA M)
constexpr int kMaxTileM = 256;         // tokens per tile (MMA N)
constexpr int kBK = 64;                // K values per step: one 128-byte swizzle row of f16 X, 32 TMEM columns of A
constexpr int kBStages = 4;            // X tiles in shared memory
constexpr int kAStages = 4;            // decoded weight tiles in tensor memory, two K steps (64 columns) each
constexpr int kRawStages = 3;          // raw block columns (256 values x 128 rows) in shared memory, at most
constexpr int kRawBytes = kTileN * 144;
// Formats whose 256-value row segment is a multiple of 16 bytes arrive by TMA: Q4_K (144), Q4_0 (8 x 18 = 144),
// Q5_K (176, two stages in the same area). Q8_0 arrives 128 values at a time: four 34-byte blocks = 136 bytes,
// which start 0 or 8 bytes after a 16-byte boundary, so a 144-byte box that starts on the boundary covers them.

// Q6_K's 210-byte blocks start on even addresses only, but eight rows on, the address is the same modulo 16
// (row lengths are even): the rows r = c (mod 8) of the matrix, seen from the 16-byte boundary at or before row
// c, are a tensor with a 16-byte-multiple pitch. One map per c; a stage is eight boxes of 16 rows x 224 bytes
// (the 16-byte granules that hold a block), and the 128 staged rows are in the order (c, k) <-> row c + 8k.
__host__ __device__ constexpr bool row_phased(int wt) { return wt == KRK_CUDA_Q6_K; }
constexpr int kPhases = 8;
__host__ __device__ constexpr bool tma_staged(int wt) {
    return wt == KRK_CUDA_Q4_K || wt == KRK_CUDA_Q4_0 || wt == KRK_CUDA_Q5_K || wt == KRK_CUDA_Q8_0 || wt == KRK_CUDA_Q5_0 ||
           wt == KRK_CUDA_Q5_1 || row_phased(wt);
}
// (Q5_0: eight 22-byte blocks = 176 bytes; Q5_1: eight 24-byte blocks = 192)
__host__ __device__ constexpr int raw_seg(int wt) {
    return (wt == KRK_CUDA_Q5_K || wt == KRK_CUDA_Q5_0) ? 176 : wt == KRK_CUDA_Q5_1 ? 192 : wt == KRK_CUDA_Q6_K ? 224 : 144;
}
// Which staged row and which weight row of the tile the decode thread of TMEM lane t works on. Phased formats:
// a warp's 32 lanes take the rows 32w .. 32w + 31 of the tile (so the read-out writes 32 different banks) in
// an order whose neighbouring lanes read staged rows on different banks.
__host__ __device__ constexpr int tile_row(int wt, int t) { return row_phased(wt) ? ((t & 31) >> 2) + 8 * (4 * (t >> 5) + (t & 3)) : t; }
__host__ __device__ constexpr int tile_slot(int wt, int t) { return row_phased(wt) ? 16 * ((t & 31) >> 2) + 4 * (t >> 5) + (t & 3) : t; }
struct WMaps {
    CUtensorMap m[kPhases];   // m[0] alone for the formats staged as one box
};
__host__ __device__ constexpr int raw_stages(int wt) { return raw_seg(wt) > 144 ? 2 : 3; }
constexpr int kRawArea = 2 * kTileN * 224;
static_assert(2 * kTileN * 192 <= kRawArea && kRawStages * kRawBytes <= kRawArea, "every format's stages fit the raw area");
constexpr int kDecodeThreads = 256, kEpilogueThreads = 128;   // two decode threads per weight row
constexpr int kThreads = kDecodeThreads + kEpilogueThreads + 96;
constexpr int kTmemCols = 512, kTmemA = 256;
constexpr int kYChunk = 32;            // tokens per TMA store of the read-out
constexpr int kMaxPieces = 4;          // a cut tile has about this many pieces at most
constexpr long long kWaitCycles = 4000000000LL;

struct GemmParams {
    const uint8_t *w;
    float *y;
    int64_t n_out, n_in, rows;
    int tile_m;          // tokens per tile: multiple of 16, <= 256
    int n_tiles_n, n_tiles_m;
    int row_bytes;
    int *status;
    int split_tail;        // 1: cut the tiles left after the last whole wave over the CTAs along K (needs y_tma and the counters)
    unsigned *tail_count;  // per tail tile: how many of its pieces (in K order) are in Y; zero at launch
    int y_tma;             // 1: whole tiles leave through shared memory and TMA stores (y 16-byte aligned, n_out % 4 == 0)
};

struct __align__(1024) GemmSmem {
    uint8_t b[kBStages][kMaxTileM * 128];      // X tiles, [tokens][64 f16], 128B swizzle (TMA)
    uint8_t raw[kRawArea];                     // raw block bytes, stages of [128 rows][144, 176 or 224] (TMA), or the decode warps' own staging
    float ystage[2][kYChunk][kTileN];          // accumulator read-out on its way to Y: [tokens][weight rows] (TMA store)
    unsigned long long b_full[kBStages], b_empty[kBStages];
    unsigned long long a_full[kAStages], a_empty[kAStages];
    unsigned long long raw_full[kRawStages], raw_empty[kRawStages];
    unsigned long long d_full, d_empty;
    uint32_t tmem_base;
    int gave_up;
};

// ---- PTX wrappers -------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __noinline__ void wait_slow(uint32_t bar, uint32_t parity, volatile int *gave_up, int *status) {
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 32; i++) {
            if (mbar_try_wait(bar, parity)) return;
            __nanosleep(20);
        }
        if (*gave_up) return;
        if (clock64() - t0 > kWaitCycles) {
            *gave_up = 1;
            atomicExch(status, KRK_CUDA_ETIMEOUT);
            return;
        }
    }
}
__device__ __forceinline__ void wait_phase(uint32_t bar, uint32_t parity, volatile int *gave_up, int *status) {
    if (mbar_try_wait(bar, parity)) return;
    if (*gave_up) return;
    wait_slow(bar, parity, gave_up, status);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, int x, int y, uint32_t src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// A from tensor memory (lane = row, 32-bit column = two consecutive K values), B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                   "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile of 128-byte rows in the 128-byte swizzle:
// start address >> 4 in bits 0-13, leading byte offset (unused for this layout) 1 in bits 16-29,
// stride byte offset 1024 >> 4 (eight rows) in bits 32-45, descriptor version 1 in bits 46-47,
// layout type 2 (SWIZZLE_128B) in bits 61-63.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// Instruction descriptor, kind::f16: D f32 (bits 4-5 = 1), A and B f16 (0), both K-major (0),
// N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- decode of half a weight row's K step (32 values) to f16 ---------------------------------------
// A decode thread first LOADS the raw bytes it needs (Raw), ahead of time, and later CONVERTS
// them: out[j] holds values 2j, 2j+1 (low, high half) of its 32. f16 arithmetic runs on exact
// small integers; the scale products are formed in f32 as the host decoder forms them and rounded
// to f16 once.

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

template <int WT>
struct Raw {   // formats without a packed decoder (IQ4_NL, Q2_K, Q3_K): raw bytes staged in shared memory, decoded element by element
    static constexpr int kSteps = 4;                                                       // K steps per stage
    static constexpr int kRowSeg = kSteps * kBK / block_size(WT) * block_bytes(WT);       // bytes of one row per stage
    static constexpr int kStageBytes = kTileN * kRowSeg;
    // Staging granule: with K a multiple of 256 the rows and the segments start on a multiple of it (144-byte
    // segments: 8 bytes; Q2_K's 84: 4; Q3_K's 110: 2).
    static constexpr int kGran = kRowSeg % 8 == 0 ? 8 : kRowSeg % 4 == 0 ? 4 : 2;
    static constexpr int kUnits = kStageBytes / kGran;
    static constexpr int kPer = (kUnits + kDecodeThreads - 1) / kDecodeThreads;            // loads per thread
    static constexpr int kWords = kGran == 8 ? 2 : 1;
    static_assert(kStageBytes <= kRawStages * kRawBytes / 2, "two stages must fit the raw staging area");
    uint32_t pre[kWords * kPer];   // this thread's share of the NEXT stage, on its way from global memory
    const uint8_t *stage;     // the stage being decoded, [128 rows][kRowSeg]
    // Loads of stage `ks` (K steps ks .. ks + kSteps of weight rows n0 ..): neighbouring threads take
    // neighbouring granules of a row. Rows past n_out read as zero blocks.
    __device__ __forceinline__ void fetch(const uint8_t *w, int64_t n0, int64_t n_out, int row_bytes, int ks, int tid) {
        const size_t seg = (size_t)(ks * kBK / block_size(WT)) * block_bytes(WT);
#pragma unroll
        for (int j = 0; j < kPer; j++) {
            const int i = tid + j * kDecodeThreads;
            const int rr = i / (kRowSeg / kGran), col = i - rr * (kRowSeg / kGran);
            const bool ok = i < kUnits && n0 + rr < n_out;
            const uint8_t *src = w + (size_t)(n0 + rr) * row_bytes + seg + (size_t)col * kGran;
            if constexpr (kGran == 8) {
                uint2 v = make_uint2(0u, 0u);
                if (ok) v = __ldg(reinterpret_cast<const uint2 *>(src));
                pre[2 * j] = v.x;
                pre[2 * j + 1] = v.y;
            } else if constexpr (kGran == 4) {
                pre[j] = ok ? __ldg(reinterpret_cast<const uint32_t *>(src)) : 0u;
            } else {
                pre[j] = ok ? (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(src)) : 0u;
            }
        }
    }
    __device__ __forceinline__ void stash(uint8_t *dst, int tid) {
#pragma unroll
        for (int j = 0; j < kPer; j++) {
            const int i = tid + j * kDecodeThreads;
            if (i < kUnits) {
                if constexpr (kGran == 8) reinterpret_cast<uint2 *>(dst)[i] = make_uint2(pre[2 * j], pre[2 * j + 1]);
                else if constexpr (kGran == 4) reinterpret_cast<uint32_t *>(dst)[i] = pre[j];
                else reinterpret_cast<unsigned short *>(dst)[i] = (unsigned short)pre[j];
            }
        }
        stage = dst;
    }
    __device__ __forceinline__ void convert(int j, int half, int r, uint32_t (&out)[16]) const {
        const uint8_t *row = stage + (size_t)r * kRowSeg;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int64_t k = (int64_t)j * kBK + 32 * half + 2 * i;   // relative to the stage: stages start on block boundaries
            out[i] = h2_bits(__floats2half2_rn(decode_value<WT>(row, k), decode_value<WT>(row, k + 1)));
        }
    }
};

// Q6_K: the staged slot of a row holds its 210-byte block (src/quant.cpp:491-512) `lead` bytes (even, 0..14)
// after the slot's 16-byte-aligned start. A thread (half h of its row) takes what its four chunks need into
// registers at once: for each 128-value half hf the 32 ql bytes at 64 hf + 32 h and the 32 qh bytes at
// 128 + 32 hf, each read as three 128-bit words and moved down by lead's word and half-word parts; its four
// scale pairs; d. Chunk c = 2j + h then is quad = c & 3 of half hf = j >> 1: the low (quad < 2) or high nibbles
// of those ql bytes and bit pair `quad` of the qh bytes, four quants per step.
template <>
struct Raw<KRK_CUDA_Q6_K> {
    static constexpr int kSteps = 4;
    uint32_t ql[2][8], qh[2][8], sc[4], dbits;
    int lead = 0;
    // the eight words that start `o` bytes (even) into the slot
    __device__ __forceinline__ static void window(const uint8_t *slot, int o, uint32_t (&y)[8]) {
        const uint4 *b = reinterpret_cast<const uint4 *>(slot + (o & ~15));
        const uint4 v0 = b[0], v1 = b[1], v2 = b[2];
        uint32_t x[12] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w};
        const bool by2 = (o & 8) != 0, by1 = (o & 4) != 0;
#pragma unroll
        for (int i = 0; i < 10; i++) x[i] = by2 ? x[i + 2] : x[i];
#pragma unroll
        for (int i = 0; i < 9; i++) x[i] = by1 ? x[i + 1] : x[i];
        const int sh = 8 * (o & 2);
#pragma unroll
        for (int i = 0; i < 8; i++) y[i] = __funnelshift_r(x[i], x[i + 1], sh);
    }
    __device__ __forceinline__ void load_block(const uint8_t *slot, int half, int) {
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            window(slot, lead + 64 * hf + 32 * half, ql[hf]);
            window(slot, lead + 128 + 32 * hf, qh[hf]);
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
            sc[j] = *reinterpret_cast<const unsigned short *>(slot + lead + 192 + 8 * (j >> 1) + 4 * (j & 1) + 2 * half);
        dbits = *reinterpret_cast<const unsigned short *>(slot + lead + 208);
    }
    // f16(d * scale) is formed in f32 as the host decoder forms d * scale.
    __device__ __forceinline__ void convert(int j, int half, int, uint32_t (&out)[16]) const {
        const int hf = j >> 1, nib = (j & 1) ? 4 : 0, hs = 4 * (j & 1) + 2 * half;
        const float d = __half2float(__ushort_as_half((unsigned short)dbits));
        const __half2 dl0 = __float2half2_rn(__fmul_rn(d, (float)(int8_t)(sc[j] & 0xFF)));
        const __half2 dl1 = __float2half2_rn(__fmul_rn(d, (float)(int8_t)(sc[j] >> 8)));
        const __half2 bias = __float2half2_rn(1056.0f);   // 0x6400 | q is the half 1024 + q; the quant is q - 32
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t t = ((ql[hf][i] >> nib) & 0x0F0F0F0Fu) | (((qh[hf][i] >> hs) & 0x03030303u) << 4);
            const __half2 dl = i < 4 ? dl0 : dl1;
            out[2 * i] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(t, 0x64646464u, 0x5140)), bias), dl));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(t, 0x64646464u, 0x7362)), bias), dl));
        }
    }
};

// Q4_K: one load() takes a whole 144-byte super-block = four K steps (from the TMA-staged tile in
// shared memory). K step p of the block covers chunks 2p, 2p+1: the low and the high nibbles of the
// same 32 bytes (src/quant.cpp:437-460). Thread half h converts chunk 2p+h.
template <>
struct Raw<KRK_CUDA_Q4_K> {
    static constexpr int kSteps = 4;
    uint4 hdr, q[8];
    __device__ __forceinline__ void load_block(const uint8_t *block, int, int) {
        const uint4 *b = reinterpret_cast<const uint4 *>(block);
        hdr = b[0];
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = b[1 + i];
    }
    __device__ __forceinline__ void convert(int p, int half, int, uint32_t (&out)[16]) const {
        // 6-bit scale / min of chunk c = 2p + half out of the 12 packed bytes in hdr.y, hdr.z, hdr.w
        // (src/quant.cpp:427-435)
        const int c = 2 * p + half;
        int sc, mn;
        if (c < 4) {
            sc = (hdr.y >> (8 * c)) & 63;
            mn = (hdr.z >> (8 * c)) & 63;
        } else {
            const int sh = 8 * (c - 4);
            sc = ((hdr.w >> sh) & 0xF) | (((hdr.y >> (sh + 6)) & 3) << 4);
            mn = ((hdr.w >> (sh + 4)) & 0xF) | (((hdr.z >> (sh + 6)) & 3) << 4);
        }
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
        const float dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        const __half2 dl = __float2half2_rn(__fmul_rn(d, (float)sc)), ml = __float2half2_rn(-__fmul_rn(dm, (float)mn));
        const __half2 k1024 = __float2half2_rn(1024.0f);
        const uint32_t qw[8] = {q[2 * p].x, q[2 * p].y, q[2 * p].z, q[2 * p].w, q[2 * p + 1].x, q[2 * p + 1].y, q[2 * p + 1].z, q[2 * p + 1].w};
        const int shift = 4 * half;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            // bytes 4i..4i+3 hold values 4i..4i+3 of the chunk; 0x6400 | q is the half 1024 + q
            const uint32_t t = (qw[i] >> shift) & 0x0F0F0F0Fu;
            const uint32_t v01 = __byte_perm(t, 0x64646464u, 0x5140), v23 = __byte_perm(t, 0x64646464u, 0x7362);
            out[2 * i] = h2_bits(__hfma2(__hsub2(bits_h2(v01), k1024), dl, ml));
            out[2 * i + 1] = h2_bits(__hfma2(__hsub2(bits_h2(v23), k1024), dl, ml));
        }
    }
};

// Q4_0: eight 18-byte blocks per 256 values = the same 144-byte column as Q4_K. K step p covers blocks 2p
// (thread half 0) and 2p + 1 (half 1): block 2p starts on a word of the 144 bytes, block 2p + 1 half a word
// later, so its 16 quant bytes are whole words (src/quant.cpp:331-339).
template <>
struct Raw<KRK_CUDA_Q4_0> {
    static constexpr int kSteps = 4;
    uint32_t w[36];
    __device__ __forceinline__ void load_block(const uint8_t *block, int, int) {
        const uint4 *b = reinterpret_cast<const uint4 *>(block);
#pragma unroll
        for (int i = 0; i < 9; i++) {
            const uint4 v = b[i];
            w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
        }
    }
    __device__ __forceinline__ void convert(int p, int half, int, uint32_t (&out)[16]) const {
        uint32_t q[4], dbits;
        if (half == 0) {
            dbits = w[9 * p] & 0xFFFFu;
#pragma unroll
            for (int i = 0; i < 4; i++) q[i] = __funnelshift_r(w[9 * p + i], w[9 * p + i + 1], 16);
        } else {
            dbits = w[9 * p + 4] >> 16;
#pragma unroll
            for (int i = 0; i < 4; i++) q[i] = w[9 * p + 5 + i];
        }
        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
        const __half2 bias = __float2half2_rn(1032.0f);   // 0x6400 | q is the half 1024 + q; the quant is q - 8
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // byte b of the block: value b in its low nibble, value 16 + b in its high one
            const uint32_t lo = q[i] & 0x0F0F0F0Fu, hi = (q[i] >> 4) & 0x0F0F0F0Fu;
            out[2 * i] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x5140)), bias), d2));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x7362)), bias), d2));
            out[8 + 2 * i] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x5140)), bias), d2));
            out[8 + 2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x7362)), bias), d2));
        }
    }
};

// Q5_K: the 176-byte super-block (src/quant.cpp:462-489) is Q4_K's header and nibbles plus 32 mask bytes whose
// bit c is the fifth quant bit of chunk c. K step p covers chunks 2p, 2p + 1; thread half h converts 2p + h.
template <>
struct Raw<KRK_CUDA_Q5_K> {
    static constexpr int kSteps = 4;
    uint4 hdr;
    uint32_t qh[8], q[32];
    __device__ __forceinline__ void load_block(const uint8_t *block, int, int) {
        const uint4 *b = reinterpret_cast<const uint4 *>(block);
        hdr = b[0];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint4 v = b[1 + i];
            qh[4 * i] = v.x, qh[4 * i + 1] = v.y, qh[4 * i + 2] = v.z, qh[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint4 v = b[3 + i];
            q[4 * i] = v.x, q[4 * i + 1] = v.y, q[4 * i + 2] = v.z, q[4 * i + 3] = v.w;
        }
    }
    __device__ __forceinline__ void convert(int p, int half, int, uint32_t (&out)[16]) const {
        const int c = 2 * p + half;
        int sc, mn;
        if (c < 4) {
            sc = (hdr.y >> (8 * c)) & 63;
            mn = (hdr.z >> (8 * c)) & 63;
        } else {
            const int sh = 8 * (c - 4);
            sc = ((hdr.w >> sh) & 0xF) | (((hdr.y >> (sh + 6)) & 3) << 4);
            mn = ((hdr.w >> (sh + 4)) & 0xF) | (((hdr.z >> (sh + 6)) & 3) << 4);
        }
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFF)));
        const float dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        const __half2 dl = __float2half2_rn(__fmul_rn(d, (float)sc)), ml = __float2half2_rn(-__fmul_rn(dm, (float)mn));
        const __half2 k1024 = __float2half2_rn(1024.0f);
        const int shift = 4 * half;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t t = ((q[8 * p + i] >> shift) & 0x0F0F0F0Fu) | (((qh[i] >> c) & 0x01010101u) << 4);
            const uint32_t v01 = __byte_perm(t, 0x64646464u, 0x5140), v23 = __byte_perm(t, 0x64646464u, 0x7362);
            out[2 * i] = h2_bits(__hfma2(__hsub2(bits_h2(v01), k1024), dl, ml));
            out[2 * i + 1] = h2_bits(__hfma2(__hsub2(bits_h2(v23), k1024), dl, ml));
        }
    }
};

// Four bits (a nibble's worth of fifth quant bits) spread to bit 4 of four bytes: bit m of b goes to bit 8m + 4.
__device__ __forceinline__ uint32_t spread_fifth(uint32_t b) { return (((b & 0xFu) * 0x00204081u) & 0x01010101u) << 4; }

// Q5_0: eight 22-byte blocks per 256 values (src/quant.cpp:351-364): f16 d, 32 fifth bits, 16 bytes whose low nibbles
// are quants 0..15 and whose high nibbles are quants 16..31; value = d * (q - 16). K step p covers blocks 2p (thread
// half 0: the block starts on a word of the 176 bytes) and 2p + 1 (half 1: half a word later, so its bit word and its
// quant bytes are whole words).
template <>
struct Raw<KRK_CUDA_Q5_0> {
    static constexpr int kSteps = 4;
    uint32_t w[44];
    __device__ __forceinline__ void load_block(const uint8_t *block, int, int) {
        const uint4 *b = reinterpret_cast<const uint4 *>(block);
#pragma unroll
        for (int i = 0; i < 11; i++) {
            const uint4 v = b[i];
            w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
        }
    }
    __device__ __forceinline__ void convert(int p, int half, int, uint32_t (&out)[16]) const {
        // (both candidates with constant indices, then a select: a branch on `half` would index w[] dynamically)
        const int W = 11 * p;
        uint32_t q[4];
        const uint32_t dbits = half ? (w[W + 5] >> 16) : (w[W] & 0xFFFFu);
        const uint32_t qh = half ? w[W + 6] : __funnelshift_r(w[W], w[W + 1], 16);
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = half ? w[W + 7 + i] : __funnelshift_r(w[W + 1 + i], w[W + 2 + i], 16);
        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
        const __half2 bias = __float2half2_rn(1040.0f);   // 0x6400 | q is the half 1024 + q; the quant is q - 16
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t lo = (q[i] & 0x0F0F0F0Fu) | spread_fifth(qh >> (4 * i));
            const uint32_t hi = ((q[i] >> 4) & 0x0F0F0F0Fu) | spread_fifth(qh >> (16 + 4 * i));
            out[2 * i] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x5140)), bias), d2));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x7362)), bias), d2));
            out[8 + 2 * i] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x5140)), bias), d2));
            out[8 + 2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x7362)), bias), d2));
        }
    }
};

// Q5_1: eight 24-byte blocks per 256 values (src/quant.cpp:366-379): f16 d, f16 m, 32 fifth bits, 16 quant bytes;
// value = d * q + m, q unsigned. Every field of every block is word aligned.
template <>
struct Raw<KRK_CUDA_Q5_1> {
    static constexpr int kSteps = 4;
    uint32_t w[48];
    __device__ __forceinline__ void load_block(const uint8_t *block, int, int) {
        const uint4 *b = reinterpret_cast<const uint4 *>(block);
#pragma unroll
        for (int i = 0; i < 12; i++) {
            const uint4 v = b[i];
            w[4 * i] = v.x, w[4 * i + 1] = v.y, w[4 * i + 2] = v.z, w[4 * i + 3] = v.w;
        }
    }
    __device__ __forceinline__ void convert(int p, int half, int, uint32_t (&out)[16]) const {
        // (the block's six words picked with constant indices and a select: `half` in the index would put w[] in
        // local memory)
        uint32_t b[6];
#pragma unroll
        for (int i = 0; i < 6; i++) b[i] = half ? w[12 * p + 6 + i] : w[12 * p + i];
        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)(b[0] & 0xFFFFu)));
        const __half2 m2 = __half2half2(__ushort_as_half((unsigned short)(b[0] >> 16)));
        const uint32_t qh = b[1];
        const __half2 k1024 = __float2half2_rn(1024.0f);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t qw = b[2 + i];
            const uint32_t lo = (qw & 0x0F0F0F0Fu) | spread_fifth(qh >> (4 * i));
            const uint32_t hi = ((qw >> 4) & 0x0F0F0F0Fu) | spread_fifth(qh >> (16 + 4 * i));
            out[2 * i] = h2_bits(__hfma2(__hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x5140)), k1024), d2, m2));
            out[2 * i + 1] = h2_bits(__hfma2(__hsub2(bits_h2(__byte_perm(lo, 0x64646464u, 0x7362)), k1024), d2, m2));
            out[8 + 2 * i] = h2_bits(__hfma2(__hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x5140)), k1024), d2, m2));
            out[8 + 2 * i + 1] = h2_bits(__hfma2(__hsub2(bits_h2(__byte_perm(hi, 0x64646464u, 0x7362)), k1024), d2, m2));
        }
    }
};

// Q8_0: a stage is 128 values = four 34-byte blocks (f16 d, 32 int8; src/quant.cpp:381-387) inside a 144-byte
// box that starts 0 (even stage) or 8 (odd stage) bytes before them. K step p covers blocks 2p (thread half 0)
// and 2p + 1 (half 1); a thread takes only its own two blocks, as nine words each: block 2p starts on a word,
// block 2p + 1 half a word later, so its quants are whole words.
template <>
struct Raw<KRK_CUDA_Q8_0> {
    static constexpr int kSteps = 2;
    uint32_t w[2][9];
    int odd;
    __device__ __forceinline__ void load_block(const uint8_t *box, int half, int ks) {
        odd = half;
        const uint32_t *b = reinterpret_cast<const uint32_t *>(box + 8 * ((ks >> 1) & 1) + 32 * half);
#pragma unroll
        for (int p = 0; p < 2; p++)
#pragma unroll
            for (int i = 0; i < 9; i++) w[p][i] = b[17 * p + i];
    }
    __device__ __forceinline__ void convert(int p, int, int, uint32_t (&out)[16]) const {
        uint32_t q[8], dbits;
        if (odd == 0) {
            dbits = w[p][0] & 0xFFFFu;
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = __funnelshift_r(w[p][i], w[p][i + 1], 16);
        } else {
            dbits = w[p][0] >> 16;
#pragma unroll
            for (int i = 0; i < 8; i++) q[i] = w[p][1 + i];
        }
        const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
        const __half2 bias = __float2half2_rn(1152.0f);   // q ^ 0x80 under a 0x64 high byte is the half 1024 + 128 + q
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t t = q[i] ^ 0x80808080u;
            out[2 * i] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(t, 0x64646464u, 0x5140)), bias), d2));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bits_h2(__byte_perm(t, 0x64646464u, 0x7362)), bias), d2));
        }
    }
};

// ---- the kernel ------------------------------------------------------------------------------------

// ---- work items ---------------------------------------------------------------------------------------
// Tiles are dealt to the persistent CTAs in whole waves. With split_tail set (off by default) the tiles left
// over after the last whole wave, which would keep only some SMs busy, have their K range cut into equal
// pieces over ALL CTAs instead (in units of four K steps = one super-block). The pieces of a cut tile meet in
// Y itself: piece 0 stores, piece k waits (bounded) until the tile's count says that pieces 0..k-1 are in Y and
// then adds with a TMA reduction, so the additions happen in K order and the result is the same on every run.
struct Item {
    int tile;      // tile index
    int k0, nk;    // K steps [k0, k0 + nk)
    int partial;   // 1: a piece of a cut tile (accumulate into Y), 0: the whole tile (store)
};

struct ItemIter {
    int next_full, n_full, stride;   // whole tiles: next_full, next_full + stride, ... < n_full
    int b, e, k_blocks, tail0;       // tail pieces in units of 4 K steps: [b, e) of the tail's block range
    int tail_grid;                   // CTAs that share the tail (at most kMaxPieces per tile, so the last piece's
                                     // additions stay short)
    __device__ __forceinline__ void init(int cta, int grid, int n_tiles, int k_steps, int split_tail) {
        n_full = split_tail ? (n_tiles / grid) * grid : n_tiles;
        next_full = cta;
        stride = grid;
        k_blocks = k_steps / 4;
        tail0 = n_full;
        const int tail_tiles = n_tiles - n_full;
        tail_grid = min(grid, tail_tiles * kMaxPieces);
        const long long total = (long long)tail_tiles * k_blocks;
        b = e = 0;
        if (cta < tail_grid) {
            b = (int)(total * cta / tail_grid);
            e = (int)(total * (cta + 1) / tail_grid);
        }
    }
    __device__ __forceinline__ bool next(Item &it) {
        if (next_full < n_full) {
            it.tile = next_full;
            it.k0 = 0;
            it.nk = k_blocks * 4;
            it.partial = 0;
            next_full += stride;
            return true;
        }
        if (b < e) {
            // A share that runs from the middle of one tile into the next gives its piece of the LATER tile
            // first: that piece starts the tile's sum and waits for nobody, so the chain of pieces waiting
            // for their predecessor in K order never gets longer than one tile's pieces.
            const int t_b = b / k_blocks, t_e = (e - 1) / k_blocks;
            int from = b, to = e;
            if (t_e > t_b) from = t_e * k_blocks;
            const int t = from / k_blocks, kb = from - t * k_blocks;
            const int n = to - from;
            it.tile = tail0 + t;
            it.k0 = kb * 4;
            it.nk = n * 4;
            it.partial = n != k_blocks;
            e = from;   // what is left is the earlier tile's piece (or nothing)
            return true;
        }
        return false;
    }
};

template <int WT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap x_map,
               const __grid_constant__ WMaps w_maps, const __grid_constant__ CUtensorMap y_map) {
    constexpr bool kStagedRaw = tma_staged(WT);
    constexpr int kSeg = raw_seg(WT), kNRaw = raw_stages(WT);
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    GemmSmem *sm = reinterpret_cast<GemmSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int *gave_up = &sm->gave_up;

    if (tid == 0) {
        for (int s = 0; s < kBStages; s++) {
            mbar_init(smem_u32(&sm->b_full[s]), 1);
            mbar_init(smem_u32(&sm->b_empty[s]), 1);
        }
        for (int s = 0; s < kAStages; s++) {
            mbar_init(smem_u32(&sm->a_full[s]), kDecodeThreads / 32);
            mbar_init(smem_u32(&sm->a_empty[s]), 1);
        }
        for (int s = 0; s < kRawStages; s++) {
            mbar_init(smem_u32(&sm->raw_full[s]), 1);
            mbar_init(smem_u32(&sm->raw_empty[s]), kDecodeThreads / 32);
        }
        mbar_init(smem_u32(&sm->d_full), 1);
        mbar_init(smem_u32(&sm->d_empty), kEpilogueThreads / 32);
        sm->gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 14) {
        tmem_alloc(smem_u32(&sm->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm->tmem_base;

    const int n_tiles = p.n_tiles_n * p.n_tiles_m;
    const int k_steps = (int)(p.n_in / kBK);
    ItemIter iter;
    iter.init((int)blockIdx.x, (int)gridDim.x, n_tiles, k_steps, p.split_tail);
    Item it;

    if (warp < 8) {
        // ===== decode warps: threads r and r + 128 <-> weight row r = TMEM lane r, 32 values each =====
        const int r = tid & 127, half = tid >> 7;
        const int trow = tile_row(WT, r), tslot = tile_slot(WT, r);
        const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + kTmemA + 16 * half;
        int sa = 0, sr = 0;
        uint32_t pa = 0, pr = 0;
        while (iter.next(it)) {
            const int64_t n0 = (int64_t)(it.tile / p.n_tiles_m) * kTileN;
            // Rows past n_out need no care here: their staged bytes are zero (the tensor maps fill what lies
            // outside the matrix with zeros, and fetch() does the same), and a zero block decodes to zeros.
            Raw<WT> cur;
            if constexpr (!kStagedRaw) cur.fetch(p.w, n0, p.n_out, p.row_bytes, it.k0, tid);
            for (int ks0 = it.k0; ks0 < it.k0 + it.nk; ks0 += Raw<WT>::kSteps) {
                if constexpr (kStagedRaw) {
                    wait_phase(smem_u32(&sm->raw_full[sr]), pr, gave_up, p.status);
                    if constexpr (row_phased(WT))
                        cur.lead = (int)(((size_t)trow * p.row_bytes + (size_t)(ks0 >> 2) * 210) & 15);   // n0 rows are a multiple of 16 bytes
                    cur.load_block(sm->raw + (size_t)sr * (kTileN * kSeg) + tslot * kSeg, half, ks0);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sm->raw_empty[sr]));   // the bytes are in registers now
                    if (++sr == kNRaw) {
                        sr = 0;
                        pr ^= 1;
                    }
                } else {
                    // The bytes fetched a stage ago go to the buffer nobody reads any more (the one before
                    // last); one barrier of the decode warps makes them visible, and the next stage's loads
                    // fly while this one is decoded.
                    cur.stash(sm->raw + (size_t)(sr & 1) * (kRawStages * kRawBytes / 2), tid);
                    sr++;
                    asm volatile("bar.sync 1, %0;" ::"n"(kDecodeThreads) : "memory");
                    if (ks0 + Raw<WT>::kSteps < it.k0 + it.nk)
                        cur.fetch(p.w, n0, p.n_out, p.row_bytes, ks0 + Raw<WT>::kSteps, tid);
                }
                // Two K steps share one tensor-memory stage and one hand-over to the MMA thread; the next K step
                // is converted while this one's store is in flight.
                uint32_t v[2][16];
                cur.convert(0, half, r, v[0]);
#pragma unroll
                for (int j = 0; j < Raw<WT>::kSteps; j++) {
                    if ((j & 1) == 0) {
                        wait_phase(smem_u32(&sm->a_empty[sa]), pa ^ 1, gave_up, p.status);
                        tc_fence_after();
                    }
                    tmem_st16(lane_addr + 64 * sa + 32 * (j & 1), v[j & 1]);
                    if (j + 1 < Raw<WT>::kSteps) cur.convert(j + 1, half, r, v[(j + 1) & 1]);
                    if (j & 1) {
                        tmem_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&sm->a_full[sa]));
                        if (++sa == kAStages) {
                            sa = 0;
                            pa ^= 1;
                        }
                    }
                }
            }
        }
    } else if (warp < 12) {
        // ===== epilogue warps: TMEM lane = weight row, column = token =====
        // Whole tiles and cut tiles leave the same way: the accumulator is read 32 tokens at a time, written to
        // shared memory as [token][weight row] and stored by TMA, so the accumulator is free again as soon as
        // it has been read (this read-out is not hidden behind MMAs: its length counts). Rows past the end of
        // Y are clipped by the tensor map.
        const int ew = warp - 8, et = tid - kDecodeThreads;
        const int tgrid = iter.tail_grid;
        const long long tail_total = (long long)(n_tiles - iter.n_full) * iter.k_blocks;
        const uint32_t d_addr = tmem_base + ((uint32_t)(32 * ew) << 16);
        int ybuf = 0;
        uint32_t ph = 0;
        // one chunk: registers -> staging buffer -> TMA store through `map` at (x, y)
        auto ship = [&](const uint32_t (&v)[32], const CUtensorMap *map, int x, int y, bool add) {
            if (et == 0) tma_store_wait_read<1>();   // the store that read this buffer two chunks ago is done with it
            asm volatile("bar.sync 2, %0;" ::"n"(kEpilogueThreads) : "memory");
            float *dst = &sm->ystage[ybuf][0][tile_row(WT, 32 * ew + lane)];
#pragma unroll
            for (int j = 0; j < 32; j++) dst[j * kTileN] = __uint_as_float(v[j]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 2, %0;" ::"n"(kEpilogueThreads) : "memory");
            if (et == 0) {
                if (add) tma_reduce_add_2d(map, x, y, smem_u32(sm->ystage[ybuf]));
                else tma_store_2d(map, x, y, smem_u32(sm->ystage[ybuf]));
                tma_store_commit();
            }
            ybuf ^= 1;
        };
        // one chunk straight to Y (a Y the tensor map cannot describe)
        auto put = [&](const uint32_t (&v)[32], int64_t n, int64_t m_first) {
            if (n < p.n_out) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int64_t m = m_first + j;
                    if (m < p.rows) p.y[m * p.n_out + n] = __uint_as_float(v[j]);
                }
            }
        };
        while (iter.next(it)) {
            const int64_t n0 = (int64_t)(it.tile / p.n_tiles_m) * kTileN, m0 = (int64_t)(it.tile % p.n_tiles_m) * p.tile_m;
            wait_phase(smem_u32(&sm->d_full), ph, gave_up, p.status);
            ph ^= 1;
            tc_fence_after();
            const int64_t n = n0 + tile_row(WT, 32 * ew + lane);
            if (!it.partial) {
                for (int c0 = 0; c0 < p.tile_m; c0 += kYChunk) {
                    uint32_t v[32];
                    tmem_ld32(d_addr + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (p.y_tma) ship(v, &y_map, (int)n0, (int)(m0 + c0), false);
                    else put(v, n, m0 + c0);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sm->d_empty));   // the accumulator is free again
                continue;
            }
            // ---- a piece of a cut tile: added into Y in K order ----
            // Piece k of the tile (k = how many CTAs hold earlier blocks of it) waits, bounded, until the
            // tile's count says that pieces 0..k-1 are in Y; piece 0 stores, the others add (TMA reduction in
            // L2); then the count goes up. The order of the additions is the K order whoever finishes first.
            const int t = it.tile - iter.tail0;
            const long long lo = (long long)t * iter.k_blocks, hi = lo + iter.k_blocks;
            int c_lo = (int)(lo * tgrid / tail_total);
            c_lo = max(c_lo - 1, 0);
            int k_piece = 0;
            for (int c = c_lo; c < (int)blockIdx.x; c++) {
                const long long sb = tail_total * c / tgrid, se = tail_total * (c + 1) / tgrid;
                k_piece += (max(sb, lo) < min(se, hi)) ? 1 : 0;
            }
            if (k_piece > 0) {
                if (et == 0) {
                    const long long t0 = clock64();
                    while (*reinterpret_cast<volatile unsigned *>(p.tail_count + t) < (unsigned)k_piece) {
                        __nanosleep(64);
                        if (clock64() - t0 > kWaitCycles) {
                            atomicExch(p.status, KRK_CUDA_ETIMEOUT);
                            break;
                        }
                    }
                    __threadfence();
                }
                asm volatile("bar.sync 2, %0;" ::"n"(kEpilogueThreads) : "memory");
            }
            for (int c0 = 0; c0 < p.tile_m; c0 += kYChunk) {
                uint32_t v[32];
                tmem_ld32(d_addr + (uint32_t)c0, v);
                tmem_ld_wait();
                ship(v, &y_map, (int)n0, (int)(m0 + c0), k_piece > 0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm->d_empty));
            if (et == 0) {
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // this piece is in Y
                asm volatile("fence.proxy.async;" ::: "memory");
                __threadfence();
                atomicAdd(p.tail_count + t, 1u);
            }
        }
        // the staging buffers must outlive the stores that read them
        if (et == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else if (warp == 12) {
        // ===== TMA producer of X tiles =====
        if (lane == 0) {
            int sb = 0;
            uint32_t pb = 0;
            while (iter.next(it)) {
                const int m0 = (it.tile % p.n_tiles_m) * p.tile_m;
                for (int ks = it.k0; ks < it.k0 + it.nk; ks++) {
                    wait_phase(smem_u32(&sm->b_empty[sb]), pb ^ 1, gave_up, p.status);
                    const uint32_t bar = smem_u32(&sm->b_full[sb]);
                    mbar_arrive_expect_tx(bar, (uint32_t)p.tile_m * 128u);
                    tma_load_2d(smem_u32(sm->b[sb]), &x_map, ks * kBK, m0, bar);
                    if (++sb == kBStages) {
                        sb = 0;
                        pb ^= 1;
                    }
                }
            }
        }
    } else if (warp == 13) {
        // ===== producer of raw block columns: one TMA box of 128 rows per stage, or one bulk copy per row =====
        if constexpr (row_phased(WT)) {
            if (lane == 0) {
                int sr = 0;
                uint32_t pr = 0;
                while (iter.next(it)) {
                    const int n0 = (it.tile / p.n_tiles_m) * kTileN;
                    for (int blk = it.k0 / 4; blk < (it.k0 + it.nk) / 4; blk++) {
                        wait_phase(smem_u32(&sm->raw_empty[sr]), pr ^ 1, gave_up, p.status);
                        const uint32_t bar = smem_u32(&sm->raw_full[sr]);
                        mbar_arrive_expect_tx(bar, (uint32_t)(kTileN * kSeg));
                        const uint32_t stage = smem_u32(sm->raw + (size_t)sr * (kTileN * kSeg));
                        for (int c = 0; c < kPhases; c++) {
                            // map c starts (c * row_bytes) % 16 bytes before row c; the block's granules from there
                            const int x0 = (int)((((size_t)c * p.row_bytes) & 15) + (size_t)blk * 210) & ~15;
                            // a matrix of fewer than eight rows has no row c: read outside the map, which fills zeros
                            const int y0 = c < p.n_out ? n0 / kPhases : (1 << 24);
                            tma_load_2d(stage + c * (kTileN / kPhases) * kSeg, &w_maps.m[c], x0, y0, bar);
                        }
                        if (++sr == kNRaw) {
                            sr = 0;
                            pr ^= 1;
                        }
                    }
                }
            }
        } else if (kStagedRaw && lane == 0) {
            int sr = 0;
            uint32_t pr = 0;
            while (iter.next(it)) {
                const int n0 = (it.tile / p.n_tiles_m) * kTileN;
                constexpr int kPer = Raw<WT>::kSteps;   // K steps per stage
                for (int blk = it.k0 / kPer; blk < (it.k0 + it.nk) / kPer; blk++) {
                    wait_phase(smem_u32(&sm->raw_empty[sr]), pr ^ 1, gave_up, p.status);
                    const uint32_t bar = smem_u32(&sm->raw_full[sr]);
                    mbar_arrive_expect_tx(bar, (uint32_t)(kTileN * kSeg));
                    const int x0 = WT == KRK_CUDA_Q8_0 ? 136 * blk - 8 * (blk & 1) : blk * kSeg;   // a multiple of 16
                    tma_load_2d(smem_u32(sm->raw + (size_t)sr * (kTileN * kSeg)), &w_maps.m[0], x0, n0, bar);
                    if (++sr == kNRaw) {
                        sr = 0;
                        pr ^= 1;
                    }
                }
            }
        }
    } else {
        // ===== MMA issuer =====
        if (lane == 0) {
            const uint32_t idesc = instr_desc(kTileN, p.tile_m);
            int sa = 0, sb = 0;
            uint32_t pa = 0, pb = 0, pd = 0;
            while (iter.next(it)) {
                wait_phase(smem_u32(&sm->d_empty), pd ^ 1, gave_up, p.status);   // the epilogue has drained the accumulator
                pd ^= 1;
                tc_fence_after();
                for (int ks = 0; ks < it.nk; ks++) {   // nk is even: a stage of decoded A holds two K steps
                    wait_phase(smem_u32(&sm->b_full[sb]), pb, gave_up, p.status);
                    if ((ks & 1) == 0) wait_phase(smem_u32(&sm->a_full[sa]), pa, gave_up, p.status);
                    tc_fence_after();
                    const uint64_t bdesc = smem_desc(smem_u32(sm->b[sb]));
                    const uint32_t a_tmem = tmem_base + kTmemA + 64 * sa + 32 * (ks & 1);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; kk++)   // 16 K values = 8 TMEM columns of A, 32 bytes of every B row
                        umma_f16_ts(tmem_base, a_tmem + 8 * kk, bdesc + 2 * kk, idesc, (ks | kk) ? 1u : 0u);
                    umma_commit(smem_u32(&sm->b_empty[sb]));   // a stage is free once the MMAs that read it are done
                    if (ks & 1) {
                        umma_commit(smem_u32(&sm->a_empty[sa]));
                        if (++sa == kAStages) {
                            sa = 0;
                            pa ^= 1;
                        }
                    }
                    if (++sb == kBStages) {
                        sb = 0;
                        pb ^= 1;
                    }
                }
                umma_commit(smem_u32(&sm->d_full));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 14) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

__global__ void __launch_bounds__(256) f32_to_f16_kernel(__half *__restrict__ out, const float *__restrict__ in, int64_t n) {
    // A finite activation beyond the f16 range saturates to +-65504 instead of becoming an infinity (which the
    // f32 accumulation would turn into NaN on the first cancellation): the rule of the reference's f16
    // activation stores (src/hip/krk_hip.hpp:141-202). Infinities and NaNs pass through unchanged.
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = in[i];
        out[i] = __float2half_rn(fabsf(v) <= 3.4028234e38f ? fminf(fmaxf(v, -65504.0f), 65504.0f) : v);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// Tensor map over the raw weight bytes as a [n_out][row_bytes] byte matrix, box = one Q4_K super-block
// (144 bytes) x 128 rows. For the formats that are not staged this way a 16-byte-wide box of the same
// matrix is encoded so that the kernel always receives a valid map.
bool encode_w_map(CUtensorMap *map, const uint8_t *w, int wt, int64_t n_out, int row_bytes) {
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return false;
    const bool staged = tma_staged(wt) && !row_phased(wt);   // phased formats: encode_phase_maps
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n_out};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {staged ? (cuuint32_t)raw_seg(wt) : 16u, staged ? (cuuint32_t)kTileN : 1u};
    const cuuint32_t estr[2] = {1, 1};
    if (!staged && (row_bytes % 16) != 0) {
        // never used by the kernel; describe a 16-byte row of the same buffer so that encoding succeeds
        const cuuint64_t d2[2] = {16, 1};
        const cuuint64_t s2[1] = {16};
        return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w), d2, s2, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Phased formats: map c covers the rows c, c + 8, c + 16, ... of the matrix from the 16-byte boundary at or before
// row c: inner extent = the lead bytes + one row (so nothing past a row's own end is ever read, and what the box
// holds beyond it is zero fill), pitch = eight rows, box = 224 bytes x 16 rows. A c with no row at all (fewer than
// eight rows in the matrix) repeats map 0; its staged rows are never used.
bool encode_phase_maps(WMaps *maps, const uint8_t *w, int64_t n_out, int row_bytes) {
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return false;
    const cuuint32_t box[2] = {224u, (cuuint32_t)(kTileN / kPhases)};
    const cuuint32_t estr[2] = {1, 1};
    for (int c = 0; c < kPhases; c++) {
        const int cc = c < n_out ? c : 0;
        const size_t start = (size_t)cc * row_bytes, lead = start & 15;
        const cuuint64_t dims[2] = {(cuuint64_t)(lead + row_bytes), (cuuint64_t)((n_out - cc + kPhases - 1) / kPhases)};
        const cuuint64_t strides[1] = {(cuuint64_t)kPhases * row_bytes};
        if (encode(&maps->m[c], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w + (start - lead)), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

// Tensor map over Y as a [rows][n_out] f32 matrix, box = 128 weight rows x kYChunk tokens, for the TMA stores
// of the read-out. A Y that is not 16-byte aligned with 16-byte-multiple rows cannot be described: then a
// dummy map over the first 16 bytes of the weights is encoded (never used) and the kernel stores directly.
bool encode_y_map(CUtensorMap *map, float *y, const uint8_t *w, int64_t n_out, int64_t rows, bool usable) {
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return false;
    const cuuint32_t estr[2] = {1, 1};
    if (!usable) {
        const cuuint64_t d2[2] = {16, 1};
        const cuuint64_t s2[1] = {16};
        const cuuint32_t b2[2] = {16, 1};
        return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(w), d2, s2, b2, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)n_out, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)n_out * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)kTileN, (cuuint32_t)kYChunk};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int WT>
int launch_wt(const GemmParams &p, const CUtensorMap &map, int grid, cudaStream_t st) {
    WMaps w_maps;
    CUtensorMap y_map;
    if (!encode_w_map(&w_maps.m[0], p.w, WT, p.n_out, p.row_bytes)) return KRK_CUDA_ELAUNCH;
    for (int c = 1; c < kPhases; c++) w_maps.m[c] = w_maps.m[0];
    if (row_phased(WT) && !encode_phase_maps(&w_maps, p.w, p.n_out, p.row_bytes)) return KRK_CUDA_ELAUNCH;
    if (!encode_y_map(&y_map, p.y, p.w, p.n_out, p.rows, p.y_tma != 0)) return KRK_CUDA_ELAUNCH;
    static bool configured[64] = {};
    auto kernel = gemm_tc_kernel<WT>;
    const size_t smem = sizeof(GemmSmem) + 1024;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            note_cuda_error(e);
            return KRK_CUDA_ELAUNCH;
        }
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kernel<<<grid, kThreads, smem, st>>>(p, map, w_maps, y_map);
    note_launch(1, KRK_CUDA_FAMILY_GEMM_TC);
    return check_launch();
}

} // namespace

namespace {

struct GemmPlan {
    int tile_m, n_tiles_n, n_tiles_m, grid, tail;   // tail: tiles left after the last whole wave (0 = none)
    size_t x_bytes, count_bytes;
};

int grid_bound() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
        return sms;
    (void)cudaGetLastError();
    return 148;
}

GemmPlan plan_gemm(int x_dtype, int64_t n_out, int64_t n_in, int64_t rows) {
    GemmPlan g;
    g.tile_m = rows >= kMaxTileM ? kMaxTileM : (int)((rows + 15) / 16 * 16);
    g.n_tiles_n = (int)((n_out + kTileN - 1) / kTileN);
    g.n_tiles_m = (int)((rows + g.tile_m - 1) / g.tile_m);
    const int tiles = g.n_tiles_n * g.n_tiles_m, sms = grid_bound();
    g.grid = tiles < sms ? tiles : sms;
    // Cutting the left-over tiles along K is opt-in (KRK_CUDA_GEMM_SPLIT=1, read once, in the style of the
    // reference's KRK_* A/B switches): the pieces meet in Y through ordered TMA reductions, without scratch,
    // but every extra piece pays a pipeline fill and a read-out, and measured on config 3 that eats what the
    // better balance gains (M = 512: 65.1 vs 64.9 us), so whole tiles are the default.
    static const bool split_on = [] {
        const char *e = std::getenv("KRK_CUDA_GEMM_SPLIT");
        return e && e[0] == '1';
    }();
    g.tail = (split_on && tiles >= sms) ? tiles % sms : 0;
    g.x_bytes = x_dtype == KRK_CUDA_X_F32 ? (((size_t)rows * (size_t)n_in * sizeof(__half) + 255) & ~(size_t)255) : 0;
    g.count_bytes = g.tail ? (((size_t)g.tail * sizeof(unsigned) + 255) & ~(size_t)255) : 0;
    return g;
}

} // namespace

size_t gemm_workspace_bytes(int x_dtype, int64_t n_out, int64_t n_in, int64_t rows) {
    const GemmPlan g = plan_gemm(x_dtype, n_out, n_in, rows);
    return g.x_bytes + g.count_bytes;
}

int launch_gemm_tc(float *y, const void *x, int x_dtype, const uint8_t *w, int wt, int64_t n_out, int64_t n_in,
                   int64_t rows, void *workspace, cudaStream_t st) {
    if (rows > (1 << 24) || n_out > (1 << 30) || n_in > (1 << 24)) return KRK_CUDA_ESHAPE;
    const GemmPlan g = plan_gemm(x_dtype, n_out, n_in, rows);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    const __half *xh = static_cast<const __half *>(x);
    if (x_dtype == KRK_CUDA_X_F32) {
        const int64_t n = rows * n_in;
        const int64_t want = (n + 255) / 256;
        const int cgrid = (int)(want < (int64_t)sm_count() * 8 ? want : (int64_t)sm_count() * 8);
        f32_to_f16_kernel<<<cgrid, 256, 0, st>>>(reinterpret_cast<__half *>(ws), static_cast<const float *>(x), n);
        note_launch();
        const int rc = check_launch();
        if (rc != KRK_CUDA_OK) return rc;
        xh = reinterpret_cast<const __half *>(ws);
    }
    GemmParams p{};
    p.w = w;
    p.y = y;
    p.n_out = n_out;
    p.n_in = n_in;
    p.rows = rows;
    p.tile_m = g.tile_m;
    p.n_tiles_n = g.n_tiles_n;
    p.n_tiles_m = g.n_tiles_m;
    p.row_bytes = (int)row_bytes(wt, n_in);
    p.y_tma = ((reinterpret_cast<uintptr_t>(y) & 15) == 0 && (n_out % 4) == 0) ? 1 : 0;
    p.split_tail = (g.tail && p.y_tma) ? 1 : 0;   // the pieces of a cut tile meet in Y through TMA reductions
    p.tail_count = reinterpret_cast<unsigned *>(ws + g.x_bytes);
    p.status = device_status_word();
    if (!p.status) return KRK_CUDA_EDEVICE;
    if (g.tail) {
        const cudaError_t e = cudaMemsetAsync(p.tail_count, 0, g.count_bytes, st);
        if (e != cudaSuccess) {
            note_cuda_error(e);
            return KRK_CUDA_ELAUNCH;
        }
    }

    EncodeTiledFn encode = encode_tiled();
    if (!encode) return KRK_CUDA_EDEVICE;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)n_in, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)n_in * sizeof(__half)};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)p.tile_m};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(xh), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return KRK_CUDA_ELAUNCH;

    int rc = KRK_CUDA_EDTYPE;
    KRK_DISPATCH_WT_GEMM(wt, rc = launch_wt<WT>(p, map, g.grid, st));
    return rc;
}

// ---- prefill GEMM for callers that must not allocate --------------------------------------------------
// The f32-activation form of the prefill GEMM needs an f16 copy of X. krk_cuda_gemm takes that space
// from the caller; this entry takes it from a fixed array that lives in the library's device image, so
// that a host which has already committed all device memory (an engine that sizes weights and KV cache
// against a budget at load time and allocates nothing afterwards), or which cannot tolerate the implicit
// device synchronisation of an allocation in the middle of a decode loop, can still run it.

constexpr int64_t kStaticHalves = 4ll << 20;   // rows * n_in <= 4 Mi values (8 MiB of f16), e.g. 1024 x 4096
static __device__ __align__(256) unsigned char g_static_scratch[kStaticHalves * 2 + 256];   // f16 X, then a status word
std::mutex g_static_mu;
unsigned char *g_static_addr[64] = {};   // device address of the array, per device, once looked up
int g_static_sms[64] = {};

} // namespace krk_cuda

using namespace krk_cuda;

extern "C" int krk_cuda_gemm_f32_static(void *y_f32, const void *x_f32, const void *w, int wt, int64_t n_out, int64_t n_in,
                                        int64_t rows, void *stream) {
    if (!krk_cuda_dtype_ok(wt) || !gemm_tc_takes(wt)) return KRK_CUDA_EDTYPE;
    if (n_out < 0 || rows < 0 || !krk_cuda_gemm_k_ok(wt, n_in) || n_in % 256 != 0) return KRK_CUDA_ESHAPE;
    if (rows > (1 << 24) || n_out > (1 << 30) || n_in > (1 << 24)) return KRK_CUDA_ESHAPE;
    if (n_out == 0 || rows == 0) return KRK_CUDA_OK;
    if (!y_f32 || !x_f32 || !w) return KRK_CUDA_ENULL;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x_f32) & 15) || (reinterpret_cast<uintptr_t>(y_f32) & 3))
        return KRK_CUDA_EALIGN;
    if (rows * n_in > kStaticHalves) return KRK_CUDA_ETOOBIG;   // larger than the fixed array: use krk_cuda_gemm

    // Once per device, with that device current: the device address of the array. In host code the
    // array's name is only a handle for this query, never a pointer a kernel may be given.
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return KRK_CUDA_EDEVICE;
    unsigned char *scratch = nullptr;
    int sms = 0;
    {
        // first use on this device, under a lock so that a second host thread never sees half of it
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_addr[dev]) {
            void *ptr = nullptr;
            int n_sm = 0;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess || !ptr || n_sm <= 0) {
                if (e != cudaSuccess) note_cuda_error(e);
                return KRK_CUDA_EDEVICE;
            }
            g_static_sms[dev] = n_sm;
            g_static_addr[dev] = static_cast<unsigned char *>(ptr);
        }
        scratch = g_static_addr[dev];
        sms = g_static_sms[dev];
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    __half *xh = reinterpret_cast<__half *>(scratch);
    int *status = reinterpret_cast<int *>(scratch + kStaticHalves * 2);

    // Everything that can fail on the host comes before the first launch.
    GemmParams p{};
    p.w = static_cast<const uint8_t *>(w);
    p.y = static_cast<float *>(y_f32);
    p.n_out = n_out;
    p.n_in = n_in;
    p.rows = rows;
    p.tile_m = rows >= kMaxTileM ? kMaxTileM : (int)((rows + 15) / 16 * 16);
    p.n_tiles_n = (int)((n_out + kTileN - 1) / kTileN);
    p.n_tiles_m = (int)((rows + p.tile_m - 1) / p.tile_m);
    p.row_bytes = (int)row_bytes(wt, n_in);
    // Y leaves by tensor stores only where a tensor map can describe it; otherwise element by element
    p.y_tma = ((reinterpret_cast<uintptr_t>(y_f32) & 15) == 0 && (n_out % 4) == 0) ? 1 : 0;
    p.split_tail = 0;   // cutting tiles needs counters in a workspace; this entry keeps whole tiles
    p.tail_count = nullptr;
    p.status = status;
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return KRK_CUDA_EDEVICE;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)n_in, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)n_in * sizeof(__half)};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)p.tile_m};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xh, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return KRK_CUDA_ELAUNCH;
    {
        CUtensorMap probe_map;   // the maps launch_wt will encode: refuse now rather than after the first kernel
        if (!encode_w_map(&probe_map, p.w, wt, n_out, p.row_bytes) || !encode_y_map(&probe_map, p.y, p.w, n_out, rows, p.y_tma != 0))
            return KRK_CUDA_ELAUNCH;
    }

    // Every call overwrites the part of the array it uses before reading it (the conversion kernel
    // below), so nothing of the previous call's contents is ever consumed.
    const int64_t n = rows * n_in;
    const int64_t want = (n + 255) / 256;
    const int cgrid = (int)(want < (int64_t)sms * 8 ? want : (int64_t)sms * 8);
    f32_to_f16_kernel<<<cgrid, 256, 0, st>>>(xh, static_cast<const float *>(x_f32), n);
    note_launch();
    int rc = check_launch();
    if (rc != KRK_CUDA_OK) return rc;
    const int tiles = p.n_tiles_n * p.n_tiles_m;
    const int grid = tiles < sms ? tiles : sms;
    rc = KRK_CUDA_EDTYPE;
    KRK_DISPATCH_WT_GEMM(wt, rc = launch_wt<WT>(p, map, grid, st));
    return rc;
}

extern "C" int krk_cuda_gemm_f32_static_status(void) {
    // The word behind the f16 area: 0, or the code a bounded wait of this entry's kernels left there.
    // Read and cleared through the symbol itself (copies, no allocation); synchronises the device.
    int v = 0;
    const size_t at = (size_t)kStaticHalves * 2;
    if (cudaDeviceSynchronize() != cudaSuccess) return KRK_CUDA_ELAUNCH;
    if (cudaMemcpyFromSymbol(&v, g_static_scratch, sizeof v, at) != cudaSuccess) return KRK_CUDA_EDEVICE;
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_static_scratch, &zero, sizeof zero, at);
    }
    return v;
}
